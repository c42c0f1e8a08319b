// Decode GEMV / skinny GEMM over f16 weights: out[m, :] = epi(alpha * x'[m, :] @ W),
// M <= 8 activation rows per weight pass, W f16 either row-major [K, N] or packed
// [N/tile][K][tile] (tile 32 or 64), x f32.  HBM-bound: every weight byte is read
// exactly once with 128-bit loads and the weights are never staged.
//
// Semantics follow the reference's row kernel (shaders/matmul_row_bda_kernel.glsl):
//   * f16 weights widened exactly to f32, f32 fma accumulation (:252-259, :334-341);
//   * fused RMSNorm of A: x'[k] = x[k] * rsqrt(mean(x^2) + eps) * w[k] (:212-234);
//   * epilogue alpha -> (+C) -> bias -> act -> binary(D) (:272-276);
//   * fused store: interleaved-pair RoPE with the partner column, then C or a
//     strided scatter destination (f32 or f16), position from pos_base + *pos_ptr
//     (:143-176, :277-291).
// The reference walks K in 16 interleaved slices per workgroup; here K is split
// over the CTAs of a thread-block cluster and over the warps of a CTA in
// contiguous blocks, and every partial sum is combined in a fixed order (lane
// tree -> warp index -> cluster rank), so results are run-to-run bit-identical.
// The f64 oracle with f16-rounded weights is the parity reference (rel 2e-3).
//
// A second weight matrix sharing x can ride along (`w2`): half of the warps take
// each matrix and the epilogue stores silu(x@W) * (x@W2), the decode SwiGLU gate,
// in one launch with x read once.
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include "k_epilogue.cuh"
#include "ta_core.hpp"

namespace cg = cooperative_groups;

namespace ta {

namespace {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;

template <int MROWS, int TN>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_f16w_kernel(const GemvParams p) {
  // 16-byte loads in flight per lane: deep for few rows (pure latency hiding),
  // shallower where the accumulators need the registers
  constexpr int GEMV_UNROLL = MROWS <= 2 ? 8 : 4;
  constexpr int LPR = TN / 8;          // lanes per weight row (8 f16 per lane)
  constexpr int RPL = 32 / LPR;        // weight rows per warp-wide load
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t S = p.ksplit;
  const uint32_t rank = S > 1 ? cluster.block_rank() : 0;
  const uint32_t tile = blockIdx.x / S;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool dual = p.w2 != nullptr;
  const int nw = dual ? GEMV_WARPS / 2 : GEMV_WARPS;   // warps per matrix
  const int wi = warp % nw, mat = warp / nw;

  // K range of this CTA, in whole warp-load blocks
  const uint32_t blocks = (p.k + RPL - 1) / RPL;
  const uint32_t blocks_per = (blocks + S - 1) / S;
  const uint32_t k_lo = min(p.k, rank * blocks_per * RPL);
  const uint32_t k_hi = min(p.k, (rank + 1) * blocks_per * RPL);
  const uint32_t k_cta = k_hi - k_lo;

  // shared: xs[k_cta][MROWS] | wpart[2][nw][MROWS][TN] | cpart[2][MROWS][TN] | scale[MROWS]
  float *xs = reinterpret_cast<float *>(gemv_smem);
  float *wpart = xs + (size_t)p.k_cta_max * MROWS;
  float *cpart = wpart + 2 * GEMV_WARPS * MROWS * TN;
  float *scale = cpart + 2 * MROWS * TN;

  // ---- fused RMSNorm scale per activation row (whole K, every CTA computes it)
  if (p.norm_w) {
    for (int m = warp; m < MROWS; m += GEMV_WARPS) {
      float ss = 0.0f;
      if ((uint32_t)m < p.m)
        for (uint32_t k = lane; k < p.k; k += 32) {
          const float a = p.x[(size_t)m * p.k + k];
          ss = fmaf(a, a, ss);
        }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) scale[m] = rsqrtf(ss / (float)p.k + p.norm_eps);
    }
    __syncthreads();
  }
  // ---- stage this CTA's slice of x' as xs[k][m]
  for (uint32_t idx = threadIdx.x; idx < k_cta * MROWS; idx += GEMV_THREADS) {
    const uint32_t kk = idx / MROWS, m = idx % MROWS;
    float v = 0.0f;
    if (m < p.m) {
      v = p.x[(size_t)m * p.k + k_lo + kk];
      if (p.norm_w) v = v * scale[m] * p.norm_w[k_lo + kk];
    }
    xs[idx] = v;
  }
  __syncthreads();

  // ---- stream the weights
  const __half *__restrict__ W = static_cast<const __half *>(mat == 0 ? p.w : p.w2);
  const uint32_t col0 = tile * TN;
  const int lrow = lane / LPR, lcg = (lane % LPR) * 8;
  const bool col_ok = col0 + lcg < p.n;   // row-major weights: the last tile may be partial
  size_t base, row_stride;   // in halfs
  if (p.packed) {
    base = ((size_t)tile * p.k) * TN + lcg;
    row_stride = TN;
  } else {
    base = (size_t)col0 + lcg;
    row_stride = p.n;
  }
  float2 acc[MROWS][4];
#pragma unroll
  for (int m = 0; m < MROWS; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[m][j] = make_float2(0.f, 0.f);

  const uint32_t step = (uint32_t)nw * RPL;
  for (uint32_t kb = k_lo + (uint32_t)wi * RPL; kb < k_hi; kb += step * GEMV_UNROLL) {
    uint4 wv[GEMV_UNROLL];
#pragma unroll
    for (int u = 0; u < GEMV_UNROLL; ++u) {
      const uint32_t k = kb + u * step + lrow;
      wv[u] = make_uint4(0u, 0u, 0u, 0u);
      if (k < k_hi && col_ok) wv[u] = __ldcs(reinterpret_cast<const uint4 *>(W + base + (size_t)k * row_stride));
    }
#pragma unroll
    for (int u = 0; u < GEMV_UNROLL; ++u) {
      const uint32_t k = kb + u * step + lrow;
      if (k < k_hi) {
        const __half2 *h = reinterpret_cast<const __half2 *>(&wv[u]);
        float2 w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = __half22float2(h[j]);
        const float *xr = xs + (size_t)(k - k_lo) * MROWS;
        float xm[MROWS];
        if constexpr (MROWS >= 4) {
#pragma unroll
          for (int m4 = 0; m4 < MROWS / 4; ++m4) {
            const float4 t = reinterpret_cast<const float4 *>(xr)[m4];
            xm[4 * m4] = t.x; xm[4 * m4 + 1] = t.y; xm[4 * m4 + 2] = t.z; xm[4 * m4 + 3] = t.w;
          }
        } else if constexpr (MROWS == 2) {
          const float2 t = *reinterpret_cast<const float2 *>(xr);
          xm[0] = t.x; xm[1] = t.y;
        } else {
          xm[0] = xr[0];
        }
#pragma unroll
        for (int m = 0; m < MROWS; ++m) {
          const float xv = xm[m];
          const float2 x2 = make_float2(xv, xv);
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[m][j] = __ffma2_rn(x2, w[j], acc[m][j]);
        }
      }
    }
  }

  // ---- fixed-order reduction: lanes sharing a column group, then warps, then cluster ranks
#pragma unroll
  for (int m = 0; m < MROWS; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int o = 16; o >= LPR; o >>= 1) {
        acc[m][j].x += __shfl_xor_sync(0xffffffffu, acc[m][j].x, o);
        acc[m][j].y += __shfl_xor_sync(0xffffffffu, acc[m][j].y, o);
      }
  if (lane < LPR) {
#pragma unroll
    for (int m = 0; m < MROWS; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float *dst = wpart + (((size_t)mat * GEMV_WARPS + wi) * MROWS + m) * TN + lcg + 2 * j;
        dst[0] = acc[m][j].x;
        dst[1] = acc[m][j].y;
      }
  }
  __syncthreads();
  const int nmat = dual ? 2 : 1;
  for (int idx = threadIdx.x; idx < nmat * MROWS * TN; idx += GEMV_THREADS) {
    const int mt = idx / (MROWS * TN), rem = idx % (MROWS * TN);
    float s = 0.0f;
    for (int w = 0; w < nw; ++w) s += wpart[((size_t)mt * GEMV_WARPS + w) * MROWS * TN + rem];
    cpart[idx] = s;
  }
  if (S > 1) cluster.sync(); else __syncthreads();

  if (rank == 0) {
    float *fin = wpart;   // reuse: final pre-store values [MROWS][TN]
    for (int idx = threadIdx.x; idx < MROWS * TN; idx += GEMV_THREADS) {
      float g = 0.0f, u = 0.0f;
      for (uint32_t r = 0; r < S; ++r) {
        const float *rp = S > 1 ? cluster.map_shared_rank(cpart, r) : cpart;
        g += rp[idx];
        if (dual) u += rp[MROWS * TN + idx];
      }
      float v = p.alpha == 1.0f ? g : p.alpha * g;
      if (dual) v = epi_activate(v, 2) * u;
      fin[idx] = v;
    }
    __syncthreads();
    const uint32_t pos = p.pos_base + (p.pos_ptr ? *p.pos_ptr : 0u);
    for (int idx = threadIdx.x; idx < MROWS * TN; idx += GEMV_THREADS) {
      const uint32_t m = idx / TN, c = col0 + idx % TN;
      if (m >= p.m || c >= p.n) continue;
      const size_t ci = (size_t)m * p.n + c;
      float v = fin[idx];
      if (p.store_kind == 0) {
        if (p.accumulate) v += p.c[ci];
        v = epi_apply(v, p.bias != nullptr, p.bias ? p.bias[c] : 0.0f, p.act, p.binary,
                      p.d ? p.d[ci] : 0.0f, p.beta);
        p.c[ci] = v;
      } else {
        if (p.store_kind != 2) {   // rope with the partner column (c ^ 1)
          const float partner = fin[idx ^ 1];
          const uint32_t dim = c % p.head_dim;
          const float *cs = p.table + ((size_t)pos * (p.head_dim / 2) + dim / 2) * 2;
          v = (dim & 1u) == 0u ? fmaf(v, cs[0], -partner * cs[1]) : fmaf(partner, cs[1], v * cs[0]);
        }
        if (p.store_kind == 1) {
          p.c[ci] = v;
        } else {
          const size_t di = (size_t)pos * p.pos_scale + (size_t)(c / p.head_dim) * p.stride_head +
                            (size_t)(c % p.head_dim) * p.stride_dim;
          if (p.dst_f16) reinterpret_cast<__half *>(p.dst)[di] = __float2half_rn(v);
          else reinterpret_cast<float *>(p.dst)[di] = v;
        }
      }
    }
  }
  if (S > 1) cluster.sync();   // remote partials stay mapped until rank 0 has read them
}

size_t gemv_smem_bytes(uint32_t k_cta_max, int mrows, int tn) {
  return ((size_t)k_cta_max * mrows + 2 * (size_t)GEMV_WARPS * mrows * tn + 2 * (size_t)mrows * tn + mrows) *
             sizeof(float) + 16;
}

template <int MROWS, int TN>
void launch_t(GemvParams p, uint32_t tiles, cudaStream_t stream) {
  const size_t smem = gemv_smem_bytes(p.k_cta_max, MROWS, TN);
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    TA_CUDA(cudaFuncSetAttribute(gemv_f16w_kernel<MROWS, TN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 200 * 1024));
    attr_done[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * p.ksplit, 1, 1);
  cfg.blockDim = dim3(GEMV_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.ksplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TA_CUDA(cudaLaunchKernelEx(&cfg, gemv_f16w_kernel<MROWS, TN>, p));
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

}  // namespace

bool gemv_f16w_supported(uint32_t m, uint32_t n, uint32_t k, bool packed, uint32_t tile_n) {
  if (m == 0 || m > 8) return false;
  if (packed) return (tile_n == 32 || tile_n == 64) && n % tile_n == 0;
  (void)k;
  return n % 8 == 0;   // 16-byte loads of row-major rows
}

void launch_gemv_f16w(GemvParams p, int sm_count, cudaStream_t stream) {
  const uint32_t tn = p.packed ? p.tile_n : 32;
  const uint32_t tiles = (p.n + tn - 1) / tn;
  const int mrows = p.m <= 1 ? 1 : p.m <= 2 ? 2 : p.m <= 4 ? 4 : 8;
  // K split over a cluster: fill the machine, keep every
  // CTA's x slice inside shared memory, never split below 256 rows.
  const uint64_t per_sm = mrows == 1 ? 5 : mrows == 2 ? 4 : mrows == 4 ? 3 : 2;   // resident CTAs (registers)
  const uint64_t slots = per_sm * (uint64_t)sm_count;
  uint32_t best_s = 0;
  double best_eff = -1.0;
  for (uint32_t s : {1u, 2u, 4u, 8u}) {
    if (s > 1 && p.k / s < 256) break;
    const uint32_t rpl = 32 / (tn / 8);
    const uint32_t k_cta = (((p.k + rpl - 1) / rpl + s - 1) / s) * rpl;
    if (gemv_smem_bytes(k_cta, mrows, (int)tn) > 196 * 1024) continue;
    const double waves = (double)tiles * s / (double)slots;
    const double eff = waves / (double)(uint64_t)(waves + 0.999999);
    if (eff > best_eff + 0.02) {
      best_eff = eff;
      best_s = s;
    }
  }
  if (!best_s) fail("GEMV: K = %u with %u rows does not fit shared memory at any cluster split", p.k, p.m);
  p.ksplit = best_s;
  {
    const uint32_t rpl = 32 / (tn / 8);
    p.k_cta_max = (((p.k + rpl - 1) / rpl + best_s - 1) / best_s) * rpl;
  }
#define TA_GEMV_CASE(MR)                                             \
  if (mrows == MR) {                                                 \
    if (tn == 64) launch_t<MR, 64>(p, tiles, stream);                \
    else launch_t<MR, 32>(p, tiles, stream);                         \
    return;                                                          \
  }
  TA_GEMV_CASE(1)
  TA_GEMV_CASE(2)
  TA_GEMV_CASE(4)
  TA_GEMV_CASE(8)
#undef TA_GEMV_CASE
}

}  // namespace ta
