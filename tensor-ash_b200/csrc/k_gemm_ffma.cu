// SIMT FFMA GEMM tiles: the any-shape, any-alignment FP32 route, its f16-weight
// sibling, and the stage-1 / reduce kernels of deterministic two-stage split-K.
//
// Arithmetic follows the reference's default FP32 shader
// (shaders/matmul_bda_v4_kernel.glsl:296-323): every output element is one
// thread's fmaf chain over k ascending, f16 B is widened exactly to f32 while
// staging (:124-146), and the fused epilogue runs at the store (:377-451).
// Split-K stage 1 partitions K as shaders/matmul_splitk2_kernel.glsl:138-142
// and plain-stores alpha*partial into plane (batch*S + split) (:197-215);
// the reduce sums planes s = 0..S-1 in order
// (shaders/matmul_f32_splitk2_reduce.comp:54-59), which is what makes the
// route bit-stable from run to run.
#include <cuda_fp16.h>

#include "k_epilogue.cuh"
#include "ta_core.hpp"

#include <mutex>

namespace ta {

// K elements staged per step: 16, and 64 for the 64 x 64 split-K stage-1 tile, whose CTAs walk a
// long K range of a skinny problem: 256-byte row segments of A per step instead of 64-byte ones
// and a quarter of the barriers.
template <int BM, int BN, bool SPLITK>
constexpr int ffma_bk() { return (SPLITK && BM == 64 && BN == 64) ? 64 : 16; }

template <int BM, int BN, int TM, int TN, bool B_F16, bool SPLITK>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_ffma_kernel(GemmParams p, float *__restrict__ scratch) {
  constexpr int NT = (BM / TM) * (BN / TN);
  constexpr int TX = BN / TN;
  constexpr int FFMA_BK = ffma_bk<BM, BN, SPLITK>();
  static_assert(TN % 4 == 0 && TM % 4 == 0, "micro tile is built from float4 strips");
  __shared__ __align__(16) float As[FFMA_BK][BM + 4];
  __shared__ __align__(16) float Bs[FFMA_BK][BN + 4];

  const int tid = threadIdx.x;
  const int tx = tid % TX, ty = tid / TX;
  const uint32_t block_col = blockIdx.x, block_row = blockIdx.y;
  uint32_t batch = blockIdx.z, split = 0;
  uint32_t k_lo = 0, k_hi = p.k;
  if (SPLITK) {
    split = blockIdx.z % p.splits;
    batch = blockIdx.z / p.splits;
    const uint32_t per = p.k / p.splits, rem = p.k % p.splits;
    k_lo = split * per + min(split, rem);
    k_hi = k_lo + per + (split < rem ? 1u : 0u);
  }

  const float *__restrict__ A = (const float *)p.a + (size_t)batch * p.stride_a;
  const size_t b_off = (size_t)batch * p.stride_b;
  const float *__restrict__ Bf = (const float *)p.b + b_off;
  const __half *__restrict__ Bh = (const __half *)p.b + b_off;

  const uint32_t row0 = block_row * BM, col0 = block_col * BN;

  // Column strips of 4: strip s covers cols (s * TX + tx) * 4 .. +3, so a warp's
  // float4 reads of Bs are contiguous (no bank conflicts).
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  const bool a_vec = (p.k % 4 == 0) && ((p.stride_a % 4) == 0) && (k_lo % 4 == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.a) & 15) == 0);
  const bool b_vec = !B_F16 && (p.n % 4 == 0) && ((p.stride_b % 4) == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.b) & 15) == 0);

  // Software pipeline: the global loads of the tiles two K steps ahead are in flight (in two
  // register sets) while the current tile is multiplied out of shared memory, so a CTA with a long
  // K range (split-K stage 1, deep-K shapes) is not one exposed global round trip per 16 k.  The
  // arithmetic per output element is unchanged: one fmaf chain over k ascending.
  constexpr int A_ITERS = BM * (FFMA_BK / 4) / NT, B_ITERS = FFMA_BK * (BN / 4) / NT;
  static_assert(A_ITERS * NT == BM * (FFMA_BK / 4) && B_ITERS * NT == FFMA_BK * (BN / 4), "tile loads must divide evenly");
  float4 a_pre[2][A_ITERS], b_pre[2][B_ITERS];

  auto load_tile = [&](float4 (&ar)[A_ITERS], float4 (&br)[B_ITERS], uint32_t k0) {
#pragma unroll
    for (int it = 0; it < A_ITERS; ++it) {
      const int idx = tid + it * NT;
      const int r = idx / (FFMA_BK / 4), kq = (idx % (FFMA_BK / 4)) * 4;
      const uint32_t gr = row0 + r, gk = k0 + kq;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (gr < p.m && gk < k_hi) {
        const float *src = A + (size_t)gr * p.k + gk;
        if (a_vec && gk + 4 <= k_hi) {
          const float4 t = *reinterpret_cast<const float4 *>(src);
          v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (gk + q < k_hi) v[q] = src[q];
        }
      }
      ar[it] = make_float4(v[0], v[1], v[2], v[3]);
    }
#pragma unroll
    for (int it = 0; it < B_ITERS; ++it) {
      const int idx = tid + it * NT;
      const int kk = idx / (BN / 4), cq = (idx % (BN / 4)) * 4;
      const uint32_t gk = k0 + kk, gc = col0 + cq;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (gk < k_hi) {
        const size_t off = (size_t)gk * p.n + gc;
        if (B_F16) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (gc + q < p.n) v[q] = __half2float(Bh[off + q]);
        } else if (b_vec && gc + 4 <= p.n) {
          const float4 t = *reinterpret_cast<const float4 *>(Bf + off);
          v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (gc + q < p.n) v[q] = Bf[off + q];
        }
      }
      br[it] = make_float4(v[0], v[1], v[2], v[3]);
    }
  };
  // registers -> shared memory: A transposed into As[kk][row], B as is
  auto store_tile = [&](const float4 (&ar)[A_ITERS], const float4 (&br)[B_ITERS]) {
#pragma unroll
    for (int it = 0; it < A_ITERS; ++it) {
      const int idx = tid + it * NT;
      const int r = idx / (FFMA_BK / 4), kq = (idx % (FFMA_BK / 4)) * 4;
      As[kq][r] = ar[it].x; As[kq + 1][r] = ar[it].y; As[kq + 2][r] = ar[it].z; As[kq + 3][r] = ar[it].w;
    }
#pragma unroll
    for (int it = 0; it < B_ITERS; ++it) {
      const int idx = tid + it * NT;
      const int kk = idx / (BN / 4), cq = (idx % (BN / 4)) * 4;
      *reinterpret_cast<float4 *>(&Bs[kk][cq]) = br[it];
    }
  };
  auto multiply_tile = [&]() {
#pragma unroll
    for (int kk = 0; kk < FFMA_BK; ++kk) {
      float a_reg[TM], b_reg[TN];
#pragma unroll
      for (int i = 0; i < TM; i += 4) {
        const float4 t = *reinterpret_cast<const float4 *>(&As[kk][ty * TM + i]);
        a_reg[i] = t.x; a_reg[i + 1] = t.y; a_reg[i + 2] = t.z; a_reg[i + 3] = t.w;
      }
#pragma unroll
      for (int s = 0; s < TN / 4; ++s) {
        const float4 t = *reinterpret_cast<const float4 *>(&Bs[kk][(s * TX + tx) * 4]);
        b_reg[s * 4] = t.x; b_reg[s * 4 + 1] = t.y; b_reg[s * 4 + 2] = t.z; b_reg[s * 4 + 3] = t.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a_reg[i], b_reg[j], acc[i][j]);
    }
  };

  load_tile(a_pre[0], b_pre[0], k_lo);
  load_tile(a_pre[1], b_pre[1], k_lo + FFMA_BK);
  for (uint32_t k0 = k_lo; k0 < k_hi; k0 += 2 * FFMA_BK) {
    store_tile(a_pre[0], b_pre[0]);
    __syncthreads();
    load_tile(a_pre[0], b_pre[0], k0 + 2 * FFMA_BK);
    multiply_tile();
    __syncthreads();
    if (k0 + FFMA_BK >= k_hi) break;
    store_tile(a_pre[1], b_pre[1]);
    __syncthreads();
    load_tile(a_pre[1], b_pre[1], k0 + 3 * FFMA_BK);
    multiply_tile();
    __syncthreads();
  }

  // ---- store
  const size_t mn = (size_t)p.m * p.n;
  float *__restrict__ out;
  if (SPLITK) out = scratch + ((size_t)batch * p.splits + split) * mn;
  else out = p.c + (size_t)batch * p.stride_c;
  const float *__restrict__ D = p.d ? p.d + (size_t)batch * p.stride_c : nullptr;
  const float *__restrict__ bias = p.bias ? p.bias + (size_t)batch * p.bias_stride : nullptr;
  const bool alpha_is_one = p.alpha == 1.0f;

  // one dispatch on the activation per tile; the store loop is compiled per activation
  epi_dispatch_act(SPLITK ? 0u : p.act, [&](auto act_tag) {
    constexpr uint32_t ACT = decltype(act_tag)::value;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      const uint32_t gr = row0 + ty * TM + i;
      if (gr >= p.m) continue;
#pragma unroll
      for (int s = 0; s < TN / 4; ++s) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t gc = col0 + (s * TX + tx) * 4 + q;
          if (gc >= p.n) continue;
          const size_t idx = (size_t)gr * p.n + gc;
          float v = acc[i][s * 4 + q];
          if (!alpha_is_one) v = p.alpha * v;
          if (!SPLITK) {
            if (p.accumulate) v += out[idx];
            v = epi_apply_t<ACT>(v, bias != nullptr, bias ? bias[gc] : 0.0f, p.binary, D ? D[idx] : 0.0f, p.beta);
          }
          out[idx] = v;
        }
      }
    }
  });
}

template <int BM, int BN, int TM, int TN, bool SPLITK>
static void launch_ffma_t(const GemmParams &p, float *scratch, cudaStream_t stream) {
  dim3 grid((p.n + BN - 1) / BN, (p.m + BM - 1) / BM, p.batch * (SPLITK ? p.splits : 1u));
  dim3 block((BM / TM) * (BN / TN));
  if (grid.y > 65535 || grid.z > 65535) fail("GEMM grid exceeds launch limits (M tiles %u, batch %u)", grid.y, grid.z);
  if (p.b_f16) gemm_ffma_kernel<BM, BN, TM, TN, true, SPLITK><<<grid, block, 0, stream>>>(p, scratch);
  else gemm_ffma_kernel<BM, BN, TM, TN, false, SPLITK><<<grid, block, 0, stream>>>(p, scratch);
  TA_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

// The two degenerate shapes of the SIMT family (the reference's col_bda and outer_bda kernels,
// src/pipeline/catalog.rs:272-281, chosen there only when N == 1 / K == 1, pipeline/mod.rs:530-531):
// a 64 x 64 tile would spend 63 of its 64 columns (or its whole K loop) on padding.
//
// N == 1: C[b, m] = epi(alpha * A[b, m, :] . B[b, :, 0]); one warp per row, lanes stride k with
// coalesced loads, each lane one fmaf chain over its k ascending, then a fixed xor-shuffle tree.
template <bool B_F16>
__global__ void __launch_bounds__(256)
gemm_col_kernel(GemmParams p) {
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row = blockIdx.x * 8 + warp, batch = blockIdx.y;
  if (row >= p.m) return;
  const float *__restrict__ a = (const float *)p.a + (size_t)batch * p.stride_a + (size_t)row * p.k;
  const float *__restrict__ bf = (const float *)p.b + (size_t)batch * p.stride_b;
  const __half *__restrict__ bh = (const __half *)p.b + (size_t)batch * p.stride_b;
  float acc = 0.0f;
  for (uint32_t k = lane; k < p.k; k += 32) acc = fmaf(a[k], B_F16 ? __half2float(bh[k]) : bf[k], acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    const size_t idx = (size_t)batch * p.stride_c + row;
    float v = p.alpha == 1.0f ? acc : p.alpha * acc;
    if (p.accumulate) v += p.c[idx];
    const float bias = p.bias ? p.bias[(size_t)batch * p.bias_stride] : 0.0f;
    const float d = p.d ? p.d[idx] : 0.0f;
    epi_dispatch_act(p.act, [&](auto act_tag) {
      v = epi_apply_t<decltype(act_tag)::value>(v, p.bias != nullptr, bias, p.binary, d, p.beta);
    });
    p.c[idx] = v;
  }
}

// K == 1: C[b, m, n] = epi(alpha * A[b, m] * B[b, n]); VEC consecutive outputs per thread (four
// with 16-byte accesses when N, the strides and the bases allow), rows of C coalesced.
template <bool B_F16, int VEC>
__global__ void __launch_bounds__(256)
gemm_outer_kernel(GemmParams p) {
  const uint32_t col = (blockIdx.x * 256 + threadIdx.x) * VEC, row = blockIdx.y, batch = blockIdx.z;
  if (col >= p.n) return;
  const float av = ((const float *)p.a)[(size_t)batch * p.stride_a + row];
  const size_t idx = (size_t)batch * p.stride_c + (size_t)row * p.n + col;
  float bv[VEC], cv[VEC], dv[VEC], biasv[VEC], v[VEC];
  if constexpr (VEC == 4) {
    const float4 t = *reinterpret_cast<const float4 *>((const float *)p.b + (size_t)batch * p.stride_b + col);
    bv[0] = t.x; bv[1] = t.y; bv[2] = t.z; bv[3] = t.w;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 c4 = p.accumulate ? *reinterpret_cast<const float4 *>(p.c + idx) : z;
    const float4 d4 = p.d ? *reinterpret_cast<const float4 *>(p.d + idx) : z;
    const float4 b4 = p.bias ? *reinterpret_cast<const float4 *>(p.bias + (size_t)batch * p.bias_stride + col) : z;
    cv[0] = c4.x; cv[1] = c4.y; cv[2] = c4.z; cv[3] = c4.w;
    dv[0] = d4.x; dv[1] = d4.y; dv[2] = d4.z; dv[3] = d4.w;
    biasv[0] = b4.x; biasv[1] = b4.y; biasv[2] = b4.z; biasv[3] = b4.w;
  } else {
    bv[0] = B_F16 ? __half2float(((const __half *)p.b)[(size_t)batch * p.stride_b + col])
                  : ((const float *)p.b)[(size_t)batch * p.stride_b + col];
    cv[0] = p.accumulate ? p.c[idx] : 0.0f;
    dv[0] = p.d ? p.d[idx] : 0.0f;
    biasv[0] = p.bias ? p.bias[(size_t)batch * p.bias_stride + col] : 0.0f;
  }
  epi_dispatch_act(p.act, [&](auto act_tag) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      float x = fmaf(av, bv[j], 0.0f);
      if (p.alpha != 1.0f) x *= p.alpha;
      if (p.accumulate) x += cv[j];
      v[j] = epi_apply_t<decltype(act_tag)::value>(x, p.bias != nullptr, biasv[j], p.binary, dv[j], p.beta);
    }
  });
  if constexpr (VEC == 4) *reinterpret_cast<float4 *>(p.c + idx) = make_float4(v[0], v[1], v[2], v[3]);
  else p.c[idx] = v[0];
}

// M <= 32 rows over f32 weights (the reference's row_bda shape, widened: the 64 x 64 tile takes
// 215 us for 9..32 rows of 4096 x 4096; f16 weights have their own GEMV).  grid.z walks groups of MR rows:
// a CTA owns 32 columns (so that 4096 columns already fill 128 SMs), 8 column quads x 32 k slices;
// thread (slice, quad) walks k = slice, slice + 32, ... with 16-byte loads of B rows (a warp reads
// four full 128-byte row segments, eight loads in flight per thread) and keeps MR x 4 sums; the 32
// slices are added in slice order through shared memory.
constexpr uint32_t ROWS_QUADS = 8, ROWS_SLICES = 256 / ROWS_QUADS, ROWS_COLS = ROWS_QUADS * 4;
template <int MR>
__global__ void __launch_bounds__(256)
gemm_rows_f32_kernel(GemmParams p) {
  constexpr int RB = MR < 8 ? MR : 8;   // rows reduced per pass through shared memory
  __shared__ float red[ROWS_SLICES][RB][ROWS_COLS + 4];
  const uint32_t quad = threadIdx.x % ROWS_QUADS, slice = threadIdx.x / ROWS_QUADS;
  const uint32_t col = blockIdx.x * ROWS_COLS + quad * 4, batch = blockIdx.y;
  const uint32_t m0 = blockIdx.z * MR, rows = p.m - m0;   // rows of this group that exist (may exceed MR)
  const float *__restrict__ A = (const float *)p.a + (size_t)batch * p.stride_a + (size_t)m0 * p.k;
  const float *__restrict__ B = (const float *)p.b + (size_t)batch * p.stride_b;
  float acc[MR][4];
#pragma unroll
  for (int m = 0; m < MR; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[m][j] = 0.0f;
  const bool vec = (p.n & 3u) == 0 && (p.stride_b & 3u) == 0 && (reinterpret_cast<uintptr_t>(p.b) & 15u) == 0;
  // 16-byte loads of A as well (four consecutive k per step) when K and the A strides allow: the
  // scalar loads of A, not the stream of B, otherwise keep the load pipe busy (eight rows: 82 -> 32 us
  // at 4096 x 4096).
  const bool kvec = vec && (p.k & 3u) == 0 && (p.stride_a & 3u) == 0 && (reinterpret_cast<uintptr_t>(p.a) & 15u) == 0;
  if (col < p.n && kvec) {
#pragma unroll 2
    for (uint32_t k = slice * 4; k < p.k; k += ROWS_SLICES * 4) {
      float4 w[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) w[r] = *reinterpret_cast<const float4 *>(B + (size_t)(k + r) * p.n + col);
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const float4 x = (uint32_t)m < rows ? *reinterpret_cast<const float4 *>(A + (size_t)m * p.k + k)
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
        const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          acc[m][0] = fmaf(xs[r], w[r].x, acc[m][0]);
          acc[m][1] = fmaf(xs[r], w[r].y, acc[m][1]);
          acc[m][2] = fmaf(xs[r], w[r].z, acc[m][2]);
          acc[m][3] = fmaf(xs[r], w[r].w, acc[m][3]);
        }
      }
    }
  } else if (col < p.n) {
#pragma unroll 8
    for (uint32_t k = slice; k < p.k; k += ROWS_SLICES) {
      float w[4] = {0.f, 0.f, 0.f, 0.f};
      const float *src = B + (size_t)k * p.n + col;
      if (vec && col + 4 <= p.n) {
        const float4 t = *reinterpret_cast<const float4 *>(src);
        w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
      } else {
        for (uint32_t j = 0; j < 4 && col + j < p.n; ++j) w[j] = src[j];
      }
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const float x = (uint32_t)m < rows ? A[(size_t)m * p.k + k] : 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[m][j] = fmaf(x, w[j], acc[m][j]);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < MR; h += RB) {
    if (h) __syncthreads();
#pragma unroll
    for (int m = 0; m < RB; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) red[slice][m][quad * 4 + j] = acc[h + m][j];
    __syncthreads();
    // thread -> (row, column) of the tile; slices added in ascending order
    for (uint32_t i = threadIdx.x; i < (uint32_t)RB * ROWS_COLS; i += 256) {
      const uint32_t m = i / ROWS_COLS, c = i % ROWS_COLS, gc = blockIdx.x * ROWS_COLS + c;
      if (h + m >= rows || gc >= p.n) continue;
      float v = 0.0f;
#pragma unroll
      for (uint32_t sidx = 0; sidx < ROWS_SLICES; ++sidx) v += red[sidx][m][c];
      const size_t idx = (size_t)batch * p.stride_c + (size_t)(m0 + h + m) * p.n + gc;
      if (p.alpha != 1.0f) v *= p.alpha;
      if (p.accumulate) v += p.c[idx];
      const float bias = p.bias ? p.bias[(size_t)batch * p.bias_stride + gc] : 0.0f;
      const float d = p.d ? p.d[idx] : 0.0f;
      epi_dispatch_act(p.act, [&](auto act_tag) {
        v = epi_apply_t<decltype(act_tag)::value>(v, p.bias != nullptr, bias, p.binary, d, p.beta);
      });
      p.c[idx] = v;
    }
  }
}

void launch_gemm_ffma(const GemmParams &p, uint32_t tile, cudaStream_t stream) {
  if (p.n == 1 && p.batch <= 65535) {
    dim3 grid((p.m + 7) / 8, p.batch);
    if (p.b_f16) gemm_col_kernel<true><<<grid, 256, 0, stream>>>(p);
    else gemm_col_kernel<false><<<grid, 256, 0, stream>>>(p);
    TA_CUDA(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return;
  }
  if (p.k == 1 && p.m <= 65535 && p.batch <= 65535) {
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(p.b) | reinterpret_cast<uintptr_t>(p.c) |
                           reinterpret_cast<uintptr_t>(p.d) | reinterpret_cast<uintptr_t>(p.bias);
    const bool vec = !p.b_f16 && p.n % 4 == 0 && p.stride_b % 4 == 0 && p.stride_c % 4 == 0 && p.bias_stride % 4 == 0 &&
                     (ptrs & 15) == 0;
    dim3 grid((p.n + (vec ? 1023 : 255)) / (vec ? 1024 : 256), p.m, p.batch);
    if (vec) gemm_outer_kernel<false, 4><<<grid, 256, 0, stream>>>(p);
    else if (p.b_f16) gemm_outer_kernel<true, 1><<<grid, 256, 0, stream>>>(p);
    else gemm_outer_kernel<false, 1><<<grid, 256, 0, stream>>>(p);
    TA_CUDA(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return;
  }
  if (p.m <= 32 && !p.b_f16 && p.n >= 64 && p.k >= 64 && p.batch <= 65535) {
    const uint32_t mr = p.m == 1 ? 1 : p.m <= 4 ? 4 : p.m <= 8 ? 8 : 16;
    dim3 grid((p.n + ROWS_COLS - 1) / ROWS_COLS, p.batch, (p.m + mr - 1) / mr);
    if (mr == 1) gemm_rows_f32_kernel<1><<<grid, 256, 0, stream>>>(p);
    else if (mr == 4) gemm_rows_f32_kernel<4><<<grid, 256, 0, stream>>>(p);
    else if (mr == 8) gemm_rows_f32_kernel<8><<<grid, 256, 0, stream>>>(p);
    else gemm_rows_f32_kernel<16><<<grid, 256, 0, stream>>>(p);
    TA_CUDA(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return;
  }
  if (tile >= 128) launch_ffma_t<128, 128, 8, 8, false>(p, nullptr, stream);
  else launch_ffma_t<64, 64, 4, 4, false>(p, nullptr, stream);
}

// Stage 1 for skinny deep-K problems (M x N small, K long, f32 B).  The reference's 64 x 64 stage-1
// tile (src/executor/splitk2.rs:36-42) with a 4 x 4 micro tile gives such a problem
// tiles x splits x 8 warps: 512 warps at M = N = 64, S = 64, i.e. 3.5 per SM, and the kernel idles on
// shared-memory latency (ncu: 5 % of warp slots occupied, issue slots 27 % busy, FMA pipe 16 %).  Here a CTA of 256 threads
// owns a 32 x 32 tile with a 2 x 2 micro tile: four times the threads for the same chains.  Every
// output element is still one thread's fmaf chain over its split's k range in ascending order, so
// the planes are bit-identical to the 64 x 64 tile's.
constexpr int SKINNY_T = 32, SKINNY_BK = 32;

__global__ void __launch_bounds__(256)
splitk2_skinny_kernel(GemmParams p, float *__restrict__ scratch) {
  __shared__ __align__(16) float As[SKINNY_BK][SKINNY_T + 2];
  __shared__ __align__(16) float Bs[SKINNY_BK][SKINNY_T];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const uint32_t split = blockIdx.z % p.splits, batch = blockIdx.z / p.splits;
  const uint32_t per = p.k / p.splits, rem = p.k % p.splits;
  const uint32_t k_lo = split * per + min(split, rem), k_hi = k_lo + per + (split < rem ? 1u : 0u);
  const float *__restrict__ A = (const float *)p.a + (size_t)batch * p.stride_a;
  const float *__restrict__ B = (const float *)p.b + (size_t)batch * p.stride_b;
  const uint32_t row0 = blockIdx.y * SKINNY_T, col0 = blockIdx.x * SKINNY_T;
  const bool a_vec = (p.k % 4 == 0) && ((p.stride_a % 4) == 0) && (k_lo % 4 == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.a) & 15) == 0);
  const bool b_vec = (p.n % 4 == 0) && ((p.stride_b % 4) == 0) && ((reinterpret_cast<uintptr_t>(p.b) & 15) == 0);
  // one float4 of A (row ar, k offset akq) and one of B (k offset bk, column bcq) per thread and K step
  const int ar = tid >> 3, akq = (tid & 7) * 4, bk = tid >> 3, bcq = (tid & 7) * 4;

  auto load_a = [&](uint32_t k0) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    const uint32_t gr = row0 + ar, gk = k0 + akq;
    if (gr < p.m && gk < k_hi) {
      const float *src = A + (size_t)gr * p.k + gk;
      if (a_vec && gk + 4 <= k_hi) {
        v = *reinterpret_cast<const float4 *>(src);
      } else {
        v.x = src[0];
        if (gk + 1 < k_hi) v.y = src[1];
        if (gk + 2 < k_hi) v.z = src[2];
        if (gk + 3 < k_hi) v.w = src[3];
      }
    }
    return v;
  };
  auto load_b = [&](uint32_t k0) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    const uint32_t gk = k0 + bk, gc = col0 + bcq;
    if (gk < k_hi && gc < p.n) {
      const float *src = B + (size_t)gk * p.n + gc;
      if (b_vec && gc + 4 <= p.n) {
        v = *reinterpret_cast<const float4 *>(src);
      } else {
        v.x = src[0];
        if (gc + 1 < p.n) v.y = src[1];
        if (gc + 2 < p.n) v.z = src[2];
        if (gc + 3 < p.n) v.w = src[3];
      }
    }
    return v;
  };
  auto store_tile = [&](const float4 &a, const float4 &b) {
    As[akq][ar] = a.x; As[akq + 1][ar] = a.y; As[akq + 2][ar] = a.z; As[akq + 3][ar] = a.w;
    *reinterpret_cast<float4 *>(&Bs[bk][bcq]) = b;
  };
  float acc00 = 0.f, acc01 = 0.f, acc10 = 0.f, acc11 = 0.f;
  auto multiply_tile = [&]() {
#pragma unroll
    for (int kk = 0; kk < SKINNY_BK; ++kk) {
      const float2 a = *reinterpret_cast<const float2 *>(&As[kk][ty * 2]);
      const float2 b = *reinterpret_cast<const float2 *>(&Bs[kk][tx * 2]);
      acc00 = fmaf(a.x, b.x, acc00); acc01 = fmaf(a.x, b.y, acc01);
      acc10 = fmaf(a.y, b.x, acc10); acc11 = fmaf(a.y, b.y, acc11);
    }
  };
  // loads run two K steps ahead of the multiply (a ring of two register sets; four measured the
  // same, the kernel is bound by shared-memory operand traffic, not by the global round trip)
  constexpr int DIST = 2;
  float4 a_pre[DIST], b_pre[DIST];
#pragma unroll
  for (int d = 0; d < DIST; ++d) {
    a_pre[d] = load_a(k_lo + d * SKINNY_BK);
    b_pre[d] = load_b(k_lo + d * SKINNY_BK);
  }
  for (uint32_t k0 = k_lo; k0 < k_hi; k0 += DIST * SKINNY_BK) {
#pragma unroll
    for (int d = 0; d < DIST; ++d) {
      if (k0 + d * SKINNY_BK >= k_hi) break;
      store_tile(a_pre[d], b_pre[d]);
      __syncthreads();
      a_pre[d] = load_a(k0 + (DIST + d) * SKINNY_BK);
      b_pre[d] = load_b(k0 + (DIST + d) * SKINNY_BK);
      multiply_tile();
      __syncthreads();
    }
  }
  float *__restrict__ out = scratch + ((size_t)batch * p.splits + split) * ((size_t)p.m * p.n);
  const bool alpha_is_one = p.alpha == 1.0f;
  const float r[2][2] = {{acc00, acc01}, {acc10, acc11}};
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint32_t gr = row0 + ty * 2 + i, gc = col0 + tx * 2 + j;
      if (gr < p.m && gc < p.n) out[(size_t)gr * p.n + gc] = alpha_is_one ? r[i][j] : p.alpha * r[i][j];
    }
}

void launch_splitk2_stage1(const GemmParams &p, uint32_t tile, float *scratch, cudaStream_t stream) {
  if (tile >= 128) {
    launch_ffma_t<128, 128, 8, 8, true>(p, scratch, stream);
    return;
  }
  const uint64_t ctas64 = (uint64_t)((p.m + 63) / 64) * ((p.n + 63) / 64) * p.batch * p.splits;
  static const int sms = [] {
    int dev = 0, n = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }();
  const uint64_t grid_z = (uint64_t)p.batch * p.splits;
  // measured on M = 64, K = 65536: faster than the 64 x 64 tile up to 64 of its CTAs (N = 64: 165 us
  // against 359 at S = 8, 51 against 63 at S = 64; N = 256: 171 against 363 at S = 8), slower from
  // 128 on (2 x 2 micro tiles read four times the shared-memory operands per FMA)
  if (!p.b_f16 && ctas64 * 2 <= (uint64_t)sms && grid_z <= 65535) {
    dim3 grid((p.n + SKINNY_T - 1) / SKINNY_T, (p.m + SKINNY_T - 1) / SKINNY_T, (unsigned)grid_z);
    if (grid.y <= 65535) {
      splitk2_skinny_kernel<<<grid, 256, 0, stream>>>(p, scratch);
      TA_CUDA(cudaGetLastError());
      g_launches.fetch_add(1, std::memory_order_relaxed);
      return;
    }
  }
  launch_ffma_t<64, 64, 4, 4, true>(p, scratch, stream);
}

// One thread per 4 consecutive outputs; planes added in split order starting
// from 0.0f (shaders/matmul_f32_splitk2_reduce.comp:44-75).
__global__ void splitk2_reduce_kernel(const float *__restrict__ scratch, float *__restrict__ c,
                                      uint64_t total, uint64_t mn, uint32_t splits) {
  const uint64_t base = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (base >= total) return;
  if ((mn & 3) == 0 && base + 4 <= total) {
    const uint64_t b = base / mn, e = base % mn;
    const float *src = scratch + b * splits * mn + e;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    uint32_t s = 0;
    for (; s + 8 <= splits; s += 8) {   // eight plane loads in flight, added in plane order
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldcg(reinterpret_cast<const float4 *>(src + (uint64_t)(s + u) * mn));
#pragma unroll
      for (int u = 0; u < 8; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
    }
    for (; s < splits; ++s) {
      const float4 v = __ldcg(reinterpret_cast<const float4 *>(src + (uint64_t)s * mn));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4 *>(c + base) = acc;
  } else {
    for (uint32_t lane = 0; lane < 4; ++lane) {
      const uint64_t i = base + lane;
      if (i >= total) break;
      const uint64_t b = i / mn, e = i % mn;
      const float *src = scratch + b * splits * mn + e;
      float acc = 0.0f;
      for (uint32_t s = 0; s < splits; ++s) acc += src[(uint64_t)s * mn];
      c[i] = acc;
    }
  }
}

void launch_splitk2_reduce(const float *scratch, float *c, uint64_t total, uint64_t mn,
                           uint32_t splits, cudaStream_t stream) {
  const uint64_t threads = (total + 3) / 4;
  const uint32_t blocks = (uint32_t)((threads + 255) / 256);
  splitk2_reduce_kernel<<<blocks, 256, 0, stream>>>(scratch, c, total, mn, splits);
  TA_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

// Reduce for many planes over few outputs (the tensor-core stage 1 writes about one plane per SM):
// a block of 256 threads owns 32 float4 outputs; thread (g, e) adds the planes of group g
// (planes [g P/8, (g+1) P/8), in plane order, eight loads in flight) for output e, then thread
// (0, e) adds the eight group sums in group order.  The order depends on the plane count only, so
// two runs are bit-identical.  Launched with programmatic stream serialization: the grid may be
// resident while stage 1 still runs and waits for it here.
constexpr int RW_GROUPS = 8, RW_COLS = 32;

__global__ void __launch_bounds__(RW_GROUPS * RW_COLS)
splitk2_reduce_wide_kernel(const float *__restrict__ scratch, float *__restrict__ c, uint64_t total, uint64_t mn,
                           uint32_t planes) {
  __shared__ float4 part[RW_GROUPS][RW_COLS];
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int e = threadIdx.x % RW_COLS, g = threadIdx.x / RW_COLS;
  const uint64_t base = ((uint64_t)blockIdx.x * RW_COLS + e) * 4;   // mn % 4 == 0: a float4 never straddles a batch
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (base < total) {
    const uint64_t b = base / mn, off = base % mn;
    const uint32_t per = (planes + RW_GROUPS - 1) / RW_GROUPS;
    const uint32_t p0 = min(planes, (uint32_t)g * per), p1 = min(planes, p0 + per);
    const float *src = scratch + b * planes * mn + off;
    uint32_t s = p0;
    for (; s + 8 <= p1; s += 8) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldcg(reinterpret_cast<const float4 *>(src + (uint64_t)(s + u) * mn));
#pragma unroll
      for (int u = 0; u < 8; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
    }
    for (; s < p1; ++s) {
      const float4 v = __ldcg(reinterpret_cast<const float4 *>(src + (uint64_t)s * mn));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
  }
  part[g][e] = acc;
  __syncthreads();
  if (g == 0 && base < total) {
    float4 r = part[0][e];
#pragma unroll
    for (int q = 1; q < RW_GROUPS; ++q) { r.x += part[q][e].x; r.y += part[q][e].y; r.z += part[q][e].z; r.w += part[q][e].w; }
    *reinterpret_cast<float4 *>(c + base) = r;
  }
}

void launch_splitk2_reduce_wide(const float *scratch, float *c, uint64_t total, uint64_t mn, uint32_t planes,
                                cudaStream_t stream) {
  if (mn % 4) fail("internal: wide split-K reduce needs M*N to be a multiple of 4");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((total / 4 + RW_COLS - 1) / RW_COLS), 1, 1);
  cfg.blockDim = dim3(RW_GROUPS * RW_COLS, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TA_CUDA(cudaLaunchKernelEx(&cfg, splitk2_reduce_wide_kernel, scratch, c, total, mn, planes));
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

// ---------------------------------------------------------------------------
// Split-K2 without any allocation: the partial planes live in a fixed array
// that is part of the loaded module (4 MiB per GPU that loads the library, held
// until the process exits).
//
// `g_splitk2_static` is a device symbol.  On the host its name is only a
// stand-in, never a device address, so the address kernels receive is fetched
// with cudaGetSymbolAddress: once per device, with that device current, on the
// first call made for it.  Stage 1 plain-stores every element of every plane
// it uses before the reduce reads them, so nothing has to start at zero; what a
// previous call left behind is simply overwritten.  All calls share the one
// array: two calls whose kernels overlap on the GPU race on it.
// ---------------------------------------------------------------------------
static __device__ __align__(256) float g_splitk2_static[SPLITK2_STATIC_MAX_FLOATS];

namespace {
std::mutex g_static_mu;
float *g_static_ptr[64] = {};  // per device ordinal, filled on first use
}  // namespace

void launch_splitk2_static(const GemmParams &p, cudaStream_t stream) {
  const uint64_t need = (uint64_t)p.splits * p.m * p.n;
  if (p.batch != 1) fail("split-K2 on the static scratch handles one matrix per call (batch %u)", p.batch);
  if (need > SPLITK2_STATIC_MAX_FLOATS)
    fail("split-K2 on the static scratch needs splits*M*N = %llu floats, more than the fixed %llu "
         "(4 MiB); use ta_matmul_split_k2, which sizes its own scratch",
         (unsigned long long)need, (unsigned long long)SPLITK2_STATIC_MAX_FLOATS);
  int dev = -1;
  TA_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) fail("unsupported CUDA device ordinal %d", dev);
  float *scratch;
  {
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[dev]) {
      void *sym = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&sym, g_splitk2_static);
      if (e != cudaSuccess || !sym)
        fail("cudaGetSymbolAddress for the static split-K2 scratch failed on device %d: %s", dev,
             cudaGetErrorString(e));
      g_static_ptr[dev] = static_cast<float *>(sym);
    }
    scratch = g_static_ptr[dev];
  }
  const uint32_t tile = (p.m >= 128 && p.n >= 128) ? 128 : 64;  // same stage-1 tile rule as the executor
  launch_splitk2_stage1(p, tile, scratch, stream);
  launch_splitk2_reduce(scratch, p.c, (uint64_t)p.m * p.n, (uint64_t)p.m * p.n, p.splits, stream);
}

}  // namespace ta
