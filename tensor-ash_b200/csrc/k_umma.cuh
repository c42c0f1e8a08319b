// tcgen05 / TMA / mbarrier PTX wrappers shared by the tensor-core GEMM kernels.
// Everything is `static`-linkage device code inside namespace ta::umma.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>

#include "ta_core.hpp"

namespace ta {
namespace umma {

constexpr uint32_t WAIT_LIMIT_NS = 2000000000u;

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false when the wait gave up (flag raised by this or
// another role); callers then leave their loops.
// sleep_ns > 0 backs off between polls: for the long waits (a whole tile's main
// loop) so that idle warps do not burn issue slots and shared-memory bandwidth.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort,
                                          uint32_t sleep_ns = 0, uint32_t limit_ns = WAIT_LIMIT_NS) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (sleep_ns) __nanosleep(sleep_ns);
    if ((++spins & 63u) == 0) {
      if (*abort) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *abort = 1;
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float *v) {
  uint32_t *r = reinterpret_cast<uint32_t *>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"  // same asm block: nothing may read the registers earlier
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float *v) {
  uint32_t *r = reinterpret_cast<uint32_t *>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"  // same asm block: nothing may read the registers earlier
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// One lane of a converged warp, chosen by the hardware.  Unlike `lane == 0`, the compiler knows
// the elected region runs in exactly one thread and keeps warp-uniform operands (descriptors,
// barrier and tensor-memory addresses) on the uniform datapath, which is where the TMA and MMA
// instructions take them from.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// Shared-memory matrix descriptor (64-bit): start address, leading / stride
// byte offsets (all >> 4), descriptor version 1, swizzle mode in the top bits.
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type) {
  const uint32_t lo = ((addr >> 4) & 0x3fffu) | (((lbo_bytes >> 4) & 0x3fffu) << 16);
  const uint32_t hi = ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | (layout_type << 29);
  return ((uint64_t)hi << 32) | lo;
}
// B is N-contiguous ("MN-major").  For 32-bit operands the tensor core reads an
// MN-major tile only in the 128B-swizzle-with-32-byte-atoms layout (type 1):
// rows of 32 floats (128 B) per k, 32-byte chunks XOR-ed with (k & 3), groups of
// 4 k-rows 512 B apart (SBO), 32-column blocks BK*128 B apart (LBO).  TMA
// produces exactly that image with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.  The
// plain 128B swizzle (type 2) makes the tensor core read zeros for this case.
constexpr uint32_t LAYOUT_SW128_BASE32B = 1, LAYOUT_SW128 = 2, LAYOUT_SW64 = 4;

// cuTensorMapEncodeTiled for a rank-3 tensor (dims innermost first, box {box0, box1, 1}).
inline void encode_map3(const Context &ctx, CUtensorMap *map, CUtensorMapDataType dtype, const void *base,
                        uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes,
                        uint32_t box0, uint32_t box1, CUtensorMapSwizzle swz) {
  auto encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ctx.encode_tiled);
  if (!encode) fail("cuTensorMapEncodeTiled is unavailable in this CUDA driver");
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  const cuuint32_t box[3] = {box0, box1, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult rc = encode(map, dtype, 3, const_cast<void *>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) fail("cuTensorMapEncodeTiled failed with CUresult %d", (int)rc);
}

// Rank-4 view of a row-major [batch, K, N] operand as {group columns, K, N / group, batch}: one
// box {group, box_k, groups, 1} lands in shared memory as `groups` consecutive [box_k][group]
// blocks -- the image that one TMA per column group produces, in a single instruction.  Only for
// N % group == 0 (otherwise the last group would wrap into the next row).
inline void encode_map_grouped(const Context &ctx, CUtensorMap *map, CUtensorMapDataType dtype, const void *base,
                               uint32_t elem_bytes, uint64_t n, uint64_t k, uint64_t batch, uint64_t batch_stride_bytes,
                               uint32_t group, uint32_t box_k, uint32_t groups, CUtensorMapSwizzle swz) {
  auto encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ctx.encode_tiled);
  if (!encode) fail("cuTensorMapEncodeTiled is unavailable in this CUDA driver");
  const cuuint64_t dims[4] = {group, k, n / group, batch};
  const cuuint64_t strides[3] = {n * elem_bytes, (cuuint64_t)group * elem_bytes, batch_stride_bytes};
  const cuuint32_t box[4] = {group, box_k, groups, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult rc = encode(map, dtype, 4, const_cast<void *>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) fail("cuTensorMapEncodeTiled (grouped) failed with CUresult %d", (int)rc);
}

}  // namespace umma
}  // namespace ta
