// Developer aid, compiled out unless TA_KERNEL_TRACE is defined: CTA 0 of every
// launch of an instrumented kernel records %globaltimer at its phase boundaries
// into a per-translation-unit buffer that a debug export copies out.
#pragma once
#ifdef TA_KERNEL_TRACE
#include <algorithm>
#include <cuda_runtime.h>
namespace {
__device__ unsigned long long g_trace[4096][8];
__device__ unsigned int g_trace_n;
}
#define TA_TRACE_BEGIN_IF(cond)                                               \
  unsigned int trace_rec = 0xffffffffu;                                       \
  if ((cond) && threadIdx.x == 0) trace_rec = atomicAdd(&g_trace_n, 1u) & 4095u;
#define TA_TRACE_BEGIN() TA_TRACE_BEGIN_IF(blockIdx.x == 0 && blockIdx.y == 0)
#define TA_TRACE(i)                                                           \
  if (trace_rec != 0xffffffffu) {                                             \
    unsigned long long t;                                                     \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));                     \
    g_trace[trace_rec][i] = t;                                                \
  }
#define TA_TRACE_EXPORT(name)                                                                            \
  extern "C" __attribute__((visibility("default"))) int name(unsigned long long *out, int max_recs) {   \
    unsigned int n = 0;                                                                                  \
    cudaMemcpyFromSymbol(&n, g_trace_n, sizeof(n));                                                      \
    const int recs = (int)std::min<unsigned int>(n, (unsigned int)std::min(max_recs, 4096));             \
    cudaMemcpyFromSymbol(out, g_trace, (size_t)recs * 8 * sizeof(unsigned long long));                   \
    const unsigned int zero = 0;                                                                         \
    cudaMemcpyToSymbol(g_trace_n, &zero, sizeof(zero));                                                  \
    return recs;                                                                                         \
  }
#else
#define TA_TRACE_BEGIN_IF(cond)
#define TA_TRACE_BEGIN()
#define TA_TRACE(i)
#define TA_TRACE_EXPORT(name)
#endif
