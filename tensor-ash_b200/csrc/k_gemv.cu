// Decode GEMV / skinny GEMM over f16 weights: out[m, :] = epi(alpha * x'[m, :] @ W),
// M <= 8 activation rows per weight pass, W f16 either row-major [K, N] or packed
// [N/tile][K][tile] (tile 32 or 64), x f32.  HBM-bound: every weight byte is read
// exactly once with 128-bit streaming loads and never staged.
//
// Semantics follow the reference's row kernel (shaders/matmul_row_bda_kernel.glsl):
//   * f16 weights widened exactly to f32, f32 fma accumulation (:252-259, :334-341);
//   * fused RMSNorm of A: x'[k] = x[k] * rsqrt(mean(x^2) + eps) * w[k] (:212-234); the
//     per-row factor rsqrt(...) is applied to the finished dot products instead of to
//     every element (same value up to f32 rounding order);
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
// Latency structure (a decode step is a chain of ~100 such launches over a few MB
// each, so the chain latency matters as much as the bandwidth):
//   * weights first: a CTA issues the 16-byte loads of its first pass before
//     anything else, and only then waits for the previous kernel in the stream
//     (programmatic dependent launch, `griddepcontrol.wait`).  Weights never
//     depend on earlier kernels, so their HBM latency hides behind the tail of the
//     producer of x.  Everything that reads x or writes memory comes after the wait;
//   * passes are double-buffered in registers: the loads of pass i+1 are in flight
//     while pass i is multiplied;
//   * cluster ranks push their partial tile straight into rank 0's shared memory
//     (distributed shared memory stores) and leave; rank 0 alone waits, sums in
//     rank order and runs the epilogue;
//   * up to three GEMVs that share x (q, k, v projections) ride in one launch as
//     segments of the tile range, each with its own epilogue and store.
//
// A second weight matrix sharing x can ride along (`w2`): half of the warps take
// each matrix and the epilogue stores silu(x@W) * (x@W2), the decode SwiGLU gate
// (and x@W2 itself when `c2` is set), in one launch with x read once.
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "k_epilogue.cuh"
#include "k_umma.cuh"
#include "ta_core.hpp"

namespace cg = cooperative_groups;

namespace ta {

namespace {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;

constexpr int XS_PRE = 6;   // slice elements per thread fetched in the single activation round trip

template <int MROWS>
struct GemvCfg {
  static constexpr int U = 4;   // 16-byte loads per lane per pass (two passes in flight)
};

constexpr int RING_STAGES = 4;             // bulk-copy ring: stages of one pass (16 KiB) each
constexpr int RING_STAGE_BYTES = 16384;

// BULK: packed weights only.  One thread streams the CTA's contiguous tile slice into a
// shared-memory ring with bulk asynchronous copies (cp.async.bulk + mbarrier transaction
// counts), four passes ahead and starting before the dependency wait; the warps read their
// 16-byte pieces from the ring instead of from global memory.  In-flight bytes per SM then
// depend on shared memory (64 KiB per CTA), not on registers.
// Three to eight rows over shapes the tensor-memory kernel (k_gemv_umma.cu) takes go there instead.
// PEER: the launch takes part in a tensor-parallel exchange fused into it.  Pull: the activation x
// is not read from memory but summed, in rank order, from what every rank pushed into this rank's
// exchange buffer at the launch's exchange point; every element is a (value, flag) pair and a reader
// spins (bounded) on the pair itself until it carries this submission's flag.  The first column
// tile also writes the sum to x_out for later readers.  Push: a segment's outputs go to every
// rank's buffer as such pairs instead of C.  No extra launch, no fence, no counter.
__device__ __forceinline__ uint2 *peer_slot(const PeerLink &l, uint32_t owner, uint32_t slot, uint32_t src) {
  return reinterpret_cast<uint2 *>(l.buf[owner] + PEER_X_DATA_OFF) + ((size_t)slot * PEER_MAX_WORLD + src) * PEER_MAX_FLOATS;
}
// One pushed element: the value once its flag is this submission's.  `dead` is the caller's
// give-up state: after one wait has run out no later element waits again.
__device__ __forceinline__ float peer_pair_load(const uint2 *p, uint32_t flag, uint64_t limit_ns, uint32_t *status, bool &dead) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  if (v.y != flag && !dead) {
    const uint64_t t0 = umma::global_timer_ns();
    uint32_t spins = 0;
    for (;;) {
      asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
      if (v.y == flag) break;
      if ((++spins & 255u) == 0 && umma::global_timer_ns() - t0 > limit_ns) {
        if (status) atomicOr(status, 4u);     // reported by the host; the sums are then invalid
        dead = true;
        break;
      }
    }
  }
  return __uint_as_float(v.x);
}

// EB pushed elements at once: the pairs of RB ranks per element are requested together and a poll
// re-requests every pair that is still missing before it looks at any, so a pull costs one L2 round
// trip per poll, not one per (element, rank).  The sum runs in rank order.
template <int EB, int RB>
__device__ __forceinline__ void peer_pull_sum(const PeerLink &pl, uint32_t flag, const size_t (&off)[EB], const bool (&on)[EB],
                                              float (&out)[EB], uint32_t *status, bool &dead) {
#pragma unroll
  for (int e = 0; e < EB; ++e) out[e] = 0.0f;
  for (uint32_t r0 = 0; r0 < pl.world; r0 += RB) {
    uint2 v[EB][RB];
    const uint2 *src[RB];
#pragma unroll
    for (int j = 0; j < RB; ++j) src[j] = peer_slot(pl, pl.rank, pl.pull_slot, min(r0 + j, pl.world - 1));
#pragma unroll
    for (int e = 0; e < EB; ++e)
#pragma unroll
      for (int j = 0; j < RB; ++j) v[e][j] = make_uint2(0u, ~flag);
    const uint64_t t0 = umma::global_timer_ns();
    uint32_t spins = 0;
    for (;;) {
#pragma unroll
      for (int e = 0; e < EB; ++e)
#pragma unroll
        for (int j = 0; j < RB; ++j)
          if (on[e] && r0 + j < pl.world && v[e][j].y != flag)
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v[e][j].x), "=r"(v[e][j].y) : "l"(src[j] + off[e]) : "memory");
      bool all = true;
#pragma unroll
      for (int e = 0; e < EB; ++e)
#pragma unroll
        for (int j = 0; j < RB; ++j) all = all && (!on[e] || r0 + j >= pl.world || v[e][j].y == flag);
      if (all || dead) break;
      if ((++spins & 255u) == 0 && umma::global_timer_ns() - t0 > pl.limit_ns) {
        if (status) atomicOr(status, 4u);     // reported by the host; the sums are then invalid
        dead = true;
        break;
      }
    }
#pragma unroll
    for (int e = 0; e < EB; ++e)
#pragma unroll
      for (int j = 0; j < RB; ++j)
        if (r0 + j < pl.world) out[e] += __uint_as_float(v[e][j].x);
  }
}

template <int MROWS, int TN, bool BULK, bool PEER = false, bool WIDE = false>
// Three CTAs per SM for one and two rows (85 registers): at four (64 registers) the two prefetched
// weight passes did not fit beside the staged activation, part of them went to local memory before
// the dependency wait and came back from L2 after it, 1.3 us per launch of a decode step
// (0.94 -> 0.83 ms per token).
// WIDE (exchange variant only): two CTAs per SM (128 registers) for launches that fit one wave at
// that residency; a pull then requests four elements x four ranks per poll instead of two x two
// (4 GPUs: 0.733 against 0.786 ms per token; on 2 GPUs, whose launches need three per SM, 0.894 against 0.789).
__global__ void __launch_bounds__(GEMV_THREADS, MROWS <= 2 ? ((PEER && WIDE) ? 2 : 3) : (MROWS == 4 ? 3 : 2))
gemv_f16w_kernel(const __grid_constant__ GemvGroup g) {
  static_assert(!PEER || !BULK, "the exchange variant is built for the register-streamed path");
  constexpr int U = GemvCfg<MROWS>::U;
  constexpr int LPR = TN / 8;                    // lanes per weight row (8 f16 per lane)
  constexpr int RPL = 32 / LPR;                  // weight rows per warp-wide load
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t S = g.ksplit;
  const uint32_t rank = S > 1 ? cluster.block_rank() : 0;
  const uint32_t tile_all = blockIdx.x / S;
  int si = 0;
  while (si + 1 < (int)g.nseg && tile_all >= g.tile_end[si]) ++si;
  const GemvParams &p = g.seg[si];
  const uint32_t tile = tile_all - (si ? g.tile_end[si - 1] : 0u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool dual = p.w2 != nullptr;
  const int nw = dual ? GEMV_WARPS / 2 : GEMV_WARPS;   // warps per matrix
  const int wi = warp % nw, mat = warp / nw;

  // K range of this CTA
  const uint32_t k_lo = min(p.k, rank * g.k_cta), k_hi = min(p.k, k_lo + g.k_cta);
  const uint32_t k_len = k_hi - k_lo;
  const uint32_t rows_per_pass = (uint32_t)nw * RPL * U;
  const uint32_t passes = (k_len + rows_per_pass - 1) / rows_per_pass;

  // shared: xs[k_cta][MROWS] | wpart[WARPS][MROWS][TN] | cpart[S][2][MROWS][TN] | red[WARPS][MROWS] | scale[MROWS]
  // BULK prepends: ring[RING_STAGES][16 KiB] | full barriers | abort flag (128 bytes reserved)
  constexpr size_t RING_BYTES = BULK ? (size_t)RING_STAGES * RING_STAGE_BYTES + 128 : 0;
  float *xs = reinterpret_cast<float *>(gemv_smem + RING_BYTES);
  float *wpart = xs + (size_t)(g.k_cta + 8) * MROWS;
  float *cpart = wpart + GEMV_WARPS * MROWS * TN;
  float *red = cpart + (size_t)S * 2 * MROWS * TN;
  float *scale = red + GEMV_WARPS * MROWS;

  // ---- weight addressing
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
  auto load_pass = [&](uint4 (&wv)[U], uint32_t pass) {
    const uint32_t k0 = k_lo + pass * rows_per_pass + (uint32_t)wi * RPL + lrow;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t k = k0 + u * nw * RPL;
      wv[u] = make_uint4(0u, 0u, 0u, 0u);
      if (k < k_hi && col_ok) wv[u] = __ldcs(reinterpret_cast<const uint4 *>(W + base + (size_t)k * row_stride));
    }
  };
  // ---- BULK: ring bookkeeping.  Stage s holds pass p (p % RING_STAGES == s): rows_per_pass rows
  // of matrix 0, then (dual) the same rows of matrix 1, each row TN halves, rows contiguous.
  const uint32_t ring_base = umma::smem_u32(gemv_smem);
  const uint32_t bar_base = ring_base + RING_STAGES * RING_STAGE_BYTES;
  volatile uint32_t *ring_abort = reinterpret_cast<volatile uint32_t *>(gemv_smem + RING_STAGES * RING_STAGE_BYTES + 64);
  auto issue_pass = [&](uint32_t pass) {   // one thread
    const uint32_t stage = pass % RING_STAGES;
    const uint32_t row0 = k_lo + pass * rows_per_pass;
    const uint32_t rows = min(rows_per_pass, k_hi - row0);
    const uint32_t bytes = rows * TN * 2;
    const uint32_t bar = bar_base + 8u * stage;
    umma::mbar_arrive_expect_tx(bar, bytes * (dual ? 2u : 1u));
    for (int mt = 0; mt < (dual ? 2 : 1); ++mt) {
      const __half *src = static_cast<const __half *>(mt == 0 ? p.w : p.w2) + ((size_t)tile * p.k + row0) * TN;
      const uint32_t dst = ring_base + stage * RING_STAGE_BYTES + mt * (rows_per_pass * TN * 2);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
    }
  };
  auto ring_pass = [&](uint4 (&wv)[U], uint32_t pass) {   // every thread, after the stage's barrier
    const uint32_t stage = pass % RING_STAGES;
    const uint8_t *sp = gemv_smem + stage * RING_STAGE_BYTES + mat * (rows_per_pass * TN * 2);
    const uint32_t r0 = (uint32_t)wi * RPL + lrow, kk0 = pass * rows_per_pass + r0;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t r = r0 + u * nw * RPL;
      wv[u] = make_uint4(0u, 0u, 0u, 0u);
      if (kk0 + u * nw * RPL < k_len) wv[u] = *reinterpret_cast<const uint4 *>(sp + ((size_t)r * TN + lcg) * 2);
    }
  };

  uint4 wa[U], wb[U];
  if constexpr (BULK) {
    if (threadIdx.x == 0) {
      for (int st = 0; st < RING_STAGES; ++st) umma::mbar_init(bar_base + 8u * st, 1);
      *ring_abort = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      for (uint32_t ps = 0; ps < passes && ps < (uint32_t)RING_STAGES; ++ps) issue_pass(ps);
    }
  } else {
    if (passes > 0) load_pass(wa, 0);
    if (passes > 1) load_pass(wb, 1);
  }
  // the position cell is written by the host before the launch, never by a kernel:
  // fetch it now (it may live in host memory) so its latency hides behind the weights
  uint32_t pos = p.pos_base;
  if (p.pos_ptr && rank == 0 && p.store_kind != 0) pos += *p.pos_ptr;
  // a position the rope table or the scatter destination does not hold: every access that uses it
  // is skipped and the host is told (status bit 3)
  const bool pos_bad = p.store_kind != 0 && rank == 0 && pos >= p.pos_limit;
  if (pos_bad) {
    if (threadIdx.x == 0 && g.status) atomicOr(g.status, 8u);
    pos = 0;
  }
  uint32_t pull_flag = 0;   // what every element of this submission's push carries
  if constexpr (PEER)       // the use counts were staged by the submission's first stream operation, long before this launch
    if (g.peer.pull_point1) pull_flag = peer_flag_of(g.peer.expect_base[g.peer.pull_point1 - 1], g.peer.pull_point1);
  // also independent of earlier kernels: the norm weights of the first slice elements
  // and this thread's rope table entry; epilogue operands (D, bias, old C) follow the wait
  // (the norm weights wait in the thread's own xs slots, not in registers: the prefetched weight
  // passes need those across the dependency wait)
#pragma unroll
  for (int it = 0; it < XS_PRE; ++it) {
    const uint32_t idx = threadIdx.x + it * GEMV_THREADS, kk = idx / MROWS;
    if (idx < k_len * MROWS) xs[idx] = (p.norm_w && kk < k_len) ? p.norm_w[k_lo + kk] : 1.0f;
  }
  const uint32_t e_m = threadIdx.x / TN, e_c = col0 + threadIdx.x % TN;
  const bool e_valid = rank == 0 && threadIdx.x < MROWS * TN && e_m < p.m && e_c < p.n;
  const size_t e_ci = (size_t)e_m * p.n + e_c;
  float pre_d = 0.0f, pre_bias = 0.0f, pre_c = 0.0f;
  float2 pre_cs = make_float2(1.0f, 0.0f);
  if (e_valid && (p.store_kind == 1 || p.store_kind == 3))
    pre_cs = *reinterpret_cast<const float2 *>(p.table + ((size_t)pos * (p.head_dim / 2) + (e_c % p.head_dim) / 2) * 2);

  // ---- cluster hand-over: the partial tiles of ranks 1.. reach rank 0 as asynchronous
  // shared-memory stores that count their bytes on a barrier in rank 0's shared memory (one hop, no
  // fence, no cluster barrier on the way).  The barrier is armed here, before the dependency
  // wait, and one cluster barrier makes it known to the other ranks while everybody idles.
  const uint32_t cbar = (umma::smem_u32(scale + MROWS) + 7u) & ~7u;
  __shared__ uint32_t cbar_abort;
  if (S > 1 && g.handoff_async) {
    if (rank == 0 && threadIdx.x == 0) {
      cbar_abort = 0;
      umma::mbar_init(cbar, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      umma::mbar_arrive_expect_tx(cbar, (S - 1u) * (uint32_t)((dual ? 2 : 1) * MROWS * TN * 4));
    }
    cluster.sync();
  }

  // ---- everything below may depend on the previous kernel in the stream
  if (g.pdl) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }

  // ---- activations: one L2 round trip.  The first slice elements of every thread
  // and (rank 0) the whole rows for the RMSNorm sum of squares are requested back
  // to back; nothing consumes a value before every request is out.
  // x'[k] = x[k] * s * w[k] with one scalar s per row, so s factors out of the dot
  // product: the slice is staged as x[k] * w[k] and rank 0 multiplies the finished
  // sums by s.  Only rank 0 needs s, and nothing waits for it before the epilogue.
  const bool pull = PEER && g.peer.pull_point1 != 0;
  bool peer_dead = false;
  // x[m, k]: from memory, or the rank-ordered sum of the pushed partial rows
  auto xval = [&](uint32_t m, uint32_t k) -> float {
    if constexpr (PEER) {
      if (pull) {
        const size_t off[1] = {(size_t)m * p.k + k};
        const bool on[1] = {true};
        float out[1];
        peer_pull_sum<1, (WIDE ? 4 : 2)>(g.peer, pull_flag, off, on, out, g.status, peer_dead);
        return out[0];
      }
    }
    return p.x[(size_t)m * p.k + k];
  };
  const uint32_t stage_n = k_len * MROWS;
  float xv[XS_PRE];
  bool xv_pulled = false;
  if constexpr (PEER) {
    if (pull) {   // two slice elements per poll
      xv_pulled = true;
#pragma unroll
      for (int it = 0; it < XS_PRE; it += 2) {
        size_t off[2];
        bool on[2];
        float out[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t idx = threadIdx.x + (it + e) * GEMV_THREADS, kk = idx / MROWS, m = idx % MROWS;
          on[e] = idx < stage_n && m < p.m;
          off[e] = on[e] ? (size_t)m * p.k + k_lo + kk : 0;
        }
        if (on[0] || on[1]) peer_pull_sum<2, (WIDE ? 4 : 2)>(g.peer, pull_flag, off, on, out, g.status, peer_dead);
        xv[it] = on[0] ? out[0] : 0.0f;
        xv[it + 1] = on[1] ? out[1] : 0.0f;
      }
    }
  }
  if (!xv_pulled) {
#pragma unroll
    for (int it = 0; it < XS_PRE; ++it) {
      const uint32_t idx = threadIdx.x + it * GEMV_THREADS, kk = idx / MROWS, m = idx % MROWS;
      xv[it] = (idx < stage_n && m < p.m) ? xval(m, k_lo + kk) : 0.0f;
    }
  }
  if constexpr (PEER) {
    // the first column tile leaves the summed activation where later launches expect x
    if (pull && g.peer.x_out && tile_all == 0) {
#pragma unroll
      for (int it = 0; it < XS_PRE; ++it) {
        const uint32_t idx = threadIdx.x + it * GEMV_THREADS, kk = idx / MROWS, m = idx % MROWS;
        if (idx < stage_n && m < p.m) g.peer.x_out[(size_t)m * p.k + k_lo + kk] = xv[it];
      }
      for (uint32_t idx = threadIdx.x + XS_PRE * GEMV_THREADS; idx < stage_n; idx += GEMV_THREADS) {
        const uint32_t kk = idx / MROWS, m = idx % MROWS;
        if (m < p.m) g.peer.x_out[(size_t)m * p.k + k_lo + kk] = xval(m, k_lo + kk);
      }
    }
  }
  if (e_valid && p.store_kind == 0) {
    if (p.d) pre_d = p.d[e_ci];
    if (p.bias) pre_bias = p.bias[e_c];
    if (p.accumulate) pre_c = p.c[e_ci];
  }
  if (p.norm_w && rank == 0) {
    float ss[MROWS];
#pragma unroll
    for (int m = 0; m < MROWS; ++m) {
      ss[m] = 0.0f;
      if ((uint32_t)m < p.m && pull) {
        if constexpr (PEER) {   // NE row elements per poll (registers), squares added in k order
          constexpr int NE = WIDE ? 4 : 2;
          for (uint32_t k0 = threadIdx.x; k0 < p.k; k0 += NE * GEMV_THREADS) {
            size_t off[NE];
            bool on[NE];
            float out[NE];
#pragma unroll
            for (int e = 0; e < NE; ++e) {
              const uint32_t k = k0 + e * GEMV_THREADS;
              on[e] = k < p.k;
              off[e] = on[e] ? (size_t)m * p.k + k : 0;
            }
            peer_pull_sum<NE, NE>(g.peer, pull_flag, off, on, out, g.status, peer_dead);
#pragma unroll
            for (int e = 0; e < NE; ++e)
              if (on[e]) ss[m] = fmaf(out[e], out[e], ss[m]);
          }
        }
      } else if ((uint32_t)m < p.m) {
        const float *xr = p.x + (size_t)m * p.k;
        if ((p.k & 3u) == 0 && (reinterpret_cast<uintptr_t>(xr) & 15u) == 0) {
          for (uint32_t k = threadIdx.x * 4; k < p.k; k += GEMV_THREADS * 4) {
            const float4 a = *reinterpret_cast<const float4 *>(xr + k);
            ss[m] = fmaf(a.x, a.x, ss[m]); ss[m] = fmaf(a.y, a.y, ss[m]);
            ss[m] = fmaf(a.z, a.z, ss[m]); ss[m] = fmaf(a.w, a.w, ss[m]);
          }
        } else {
          for (uint32_t k = threadIdx.x; k < p.k; k += GEMV_THREADS) ss[m] = fmaf(xr[k], xr[k], ss[m]);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], o);
      if (lane == 0) red[warp * MROWS + m] = ss[m];
    }
  }
  // ---- stage this CTA's slice of x (times the norm weight) as xs[k][m]
#pragma unroll
  for (int it = 0; it < XS_PRE; ++it) {
    const uint32_t idx = threadIdx.x + it * GEMV_THREADS;
    if (idx < stage_n) xs[idx] = xv[it] * xs[idx];
  }
  if constexpr (MROWS >= 4) {
    // many rows: walk k within a row so that global reads are contiguous (the first
    // XS_PRE * 256 / MROWS k of every row are staged above)
    const uint32_t kk_done = (XS_PRE * GEMV_THREADS) / MROWS;
#pragma unroll
    for (int m = 0; m < MROWS; ++m) {
      const bool row = (uint32_t)m < p.m;
      for (uint32_t kk = kk_done + threadIdx.x; kk < k_len; kk += GEMV_THREADS) {
        float v = row ? xval(m, k_lo + kk) : 0.0f;
        if (row && p.norm_w) v *= p.norm_w[k_lo + kk];
        xs[(size_t)kk * MROWS + m] = v;
      }
    }
  } else {
    for (uint32_t idx = threadIdx.x + XS_PRE * GEMV_THREADS; idx < stage_n; idx += GEMV_THREADS) {
      const uint32_t kk = idx / MROWS, m = idx % MROWS;
      float v = 0.0f;
      if (m < p.m) {
        v = xval(m, k_lo + kk);
        if (p.norm_w) v *= p.norm_w[k_lo + kk];
      }
      xs[idx] = v;
    }
  }
  __syncthreads();
  if (p.norm_w && rank == 0 && threadIdx.x < MROWS) {
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w) s += red[w * MROWS + threadIdx.x];
    scale[threadIdx.x] = rsqrtf(s / (float)p.k + p.norm_eps);   // read after the reduction barriers below
  }

  {
    // ---- stream the weights: pass i multiplies while pass i+1 is in flight
    float2 acc[MROWS][4];
  #pragma unroll
    for (int m = 0; m < MROWS; ++m)
  #pragma unroll
      for (int j = 0; j < 4; ++j) acc[m][j] = make_float2(0.f, 0.f);

    auto mul_pass = [&](const uint4 (&wv)[U], uint32_t pass) {
      const uint32_t kk0 = pass * rows_per_pass + (uint32_t)wi * RPL + lrow;
  #pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t kk = kk0 + u * nw * RPL;
        if (kk < k_len) {
          const __half2 *h = reinterpret_cast<const __half2 *>(&wv[u]);
          float2 w[4];
  #pragma unroll
          for (int j = 0; j < 4; ++j) w[j] = __half22float2(h[j]);
          const float *xr = xs + (size_t)kk * MROWS;
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
            const float2 x2 = make_float2(xm[m], xm[m]);
  #pragma unroll
            for (int j = 0; j < 4; ++j) acc[m][j] = __ffma2_rn(x2, w[j], acc[m][j]);
          }
        }
      }
    };
    if constexpr (BULK) {
      bool ring_ok = true;
      for (uint32_t pass = 0; pass < passes; ++pass) {
        if (ring_ok) ring_ok = umma::mbar_wait(bar_base + 8u * (pass % RING_STAGES), (pass / RING_STAGES) & 1u, ring_abort);
        if (ring_ok) {
          ring_pass(wa, pass);
          mul_pass(wa, pass);
        }
        if (pass + RING_STAGES < passes) {
          __syncthreads();   // every warp is done with the stage before it is refilled
          if (threadIdx.x == 0 && ring_ok) issue_pass(pass + RING_STAGES);
        }
      }
      if (!ring_ok && threadIdx.x == 0 && g.status) atomicOr(g.status, 1u);   // bounded wait ran out: the host call fails
    } else {
      for (uint32_t pass = 0; pass < passes; pass += 2) {
        mul_pass(wa, pass);
        if (pass + 2 < passes) load_pass(wa, pass + 2);
        if (pass + 1 < passes) {
          mul_pass(wb, pass + 1);
          if (pass + 3 < passes) load_pass(wb, pass + 3);
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
      for (int m = 0; m < MROWS; ++m) {
        float *dst = wpart + ((size_t)warp * MROWS + m) * TN + lcg;
        reinterpret_cast<float4 *>(dst)[0] = make_float4(acc[m][0].x, acc[m][0].y, acc[m][1].x, acc[m][1].y);
        reinterpret_cast<float4 *>(dst)[1] = make_float4(acc[m][2].x, acc[m][2].y, acc[m][3].x, acc[m][3].y);
      }
    }

  }
  __syncthreads();
  const int nmat = dual ? 2 : 1;
  if (S > 1 && g.handoff_async) {
    uint32_t rdst = 0, rbar = 0;
    if (rank != 0) {
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rdst) : "r"(umma::smem_u32(cpart + (size_t)rank * 2 * MROWS * TN)), "r"(0u));
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(cbar), "r"(0u));
    }
    for (int idx = threadIdx.x; idx < nmat * MROWS * TN; idx += GEMV_THREADS) {
      const int mt = idx / (MROWS * TN), rem = idx % (MROWS * TN);
      float s = 0.0f;
      for (int w = 0; w < nw; ++w) s += wpart[((size_t)(mt * nw + w)) * MROWS * TN + rem];
      if (rank == 0) cpart[idx] = s;
      else
        asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(rdst + (uint32_t)idx * 4u),
                     "r"(__float_as_uint(s)), "r"(rbar) : "memory");
    }
    if (rank != 0) return;
    // every thread of rank 0 waits (bounded) for the other ranks' bytes
    if (!umma::mbar_wait(cbar, 0, &cbar_abort) && threadIdx.x == 0 && g.status) atomicOr(g.status, 1u);
    __syncthreads();
  } else {
  float *cdst = S > 1 ? cluster.map_shared_rank(cpart, 0) : cpart;   // rank 0's buffer
  for (int idx = threadIdx.x; idx < nmat * MROWS * TN; idx += GEMV_THREADS) {
    const int mt = idx / (MROWS * TN), rem = idx % (MROWS * TN);
    float s = 0.0f;
    for (int w = 0; w < nw; ++w) s += wpart[((size_t)(mt * nw + w)) * MROWS * TN + rem];
    cdst[(size_t)rank * 2 * MROWS * TN + idx] = s;
  }
  if (S > 1) {
    cluster.barrier_arrive();          // release: the pushed partials are visible to rank 0 after its wait
    if (rank != 0) return;
    cluster.barrier_wait();
  } else {
    __syncthreads();
  }
  }

  // ---- rank 0: sum ranks in order, epilogue, store
  float *fin = wpart;   // reuse: final pre-store values [MROWS][TN]
  float *fin2 = wpart + MROWS * TN;
  for (int idx = threadIdx.x; idx < MROWS * TN; idx += GEMV_THREADS) {
    float gsum = 0.0f, usum = 0.0f;
    for (uint32_t r = 0; r < S; ++r) {
      const float *rp = cpart + (size_t)r * 2 * MROWS * TN;
      gsum += rp[idx];
      if (dual) usum += rp[MROWS * TN + idx];
    }
    if (p.norm_w) {
      const float sc = scale[idx / TN];
      gsum *= sc;
      usum *= sc;
    }
    float v = p.alpha == 1.0f ? gsum : p.alpha * gsum;
    if (dual) {
      v = epi_activate(v, 2) * usum;
      fin2[idx] = usum;
    }
    fin[idx] = v;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < MROWS * TN; idx += GEMV_THREADS) {
    const uint32_t m = idx / TN, c = col0 + idx % TN;
    if (m >= p.m || c >= p.n) continue;
    const bool first = idx == (int)threadIdx.x && idx < GEMV_THREADS;   // operands prefetched above
    const size_t ci = (size_t)m * p.n + c;
    float v = fin[idx];
    if (dual && p.c2) p.c2[ci] = fin2[idx];
    if (p.store_kind == 0) {
      if (p.accumulate) v += first ? pre_c : p.c[ci];
      const float bv = p.bias ? (first ? pre_bias : p.bias[c]) : 0.0f;
      const float dv = p.d ? (first ? pre_d : p.d[ci]) : 0.0f;
      v = epi_apply(v, p.bias != nullptr, bv, p.act, p.binary, dv, p.beta);
      bool pushed = false;
      if constexpr (PEER) {
        if (p.push_point1) {     // this rank's partial row into every rank's buffer (its own included)
          const uint32_t flag = peer_flag_of(g.peer.expect_base[p.push_point1 - 1], p.push_point1);
          for (uint32_t r = 0; r < g.peer.world; ++r)
            asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(peer_slot(g.peer, r, p.push_slot, g.peer.rank) + ci),
                         "r"(__float_as_uint(v)), "r"(flag) : "memory");
          pushed = true;
        }
      }
      if (!pushed) p.c[ci] = v;
    } else if (!pos_bad) {
      if (p.store_kind != 2) {   // rope with the partner column (c ^ 1)
        const float partner = fin[idx ^ 1];
        const uint32_t dim = c % p.head_dim;
        float2 cs = pre_cs;
        if (!first) cs = *reinterpret_cast<const float2 *>(p.table + ((size_t)pos * (p.head_dim / 2) + dim / 2) * 2);
        v = (dim & 1u) == 0u ? fmaf(v, cs.x, -partner * cs.y) : fmaf(partner, cs.y, v * cs.x);
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

size_t gemv_smem_bytes(uint32_t k_cta, int mrows, int tn, uint32_t s, bool bulk = false) {
  return ((size_t)(k_cta + 8) * mrows + (size_t)GEMV_WARPS * mrows * tn + (size_t)s * 2 * mrows * tn +
          (size_t)GEMV_WARPS * mrows + mrows) * sizeof(float) + 16 +
         (bulk ? (size_t)RING_STAGES * RING_STAGE_BYTES + 128 : 0);
}

bool pdl_enabled() { return tunables().pdl; }

template <int MROWS, int TN, bool BULK, bool PEER = false, bool WIDE = false>
void launch_t(GemvGroup &g, uint32_t tiles, cudaStream_t stream) {
  const size_t smem = gemv_smem_bytes(g.k_cta, MROWS, TN, g.ksplit, BULK);
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    TA_CUDA(cudaFuncSetAttribute(gemv_f16w_kernel<MROWS, TN, BULK, PEER, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 200 * 1024));
    attr_done[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * g.ksplit, 1, 1);
  cfg.blockDim = dim3(GEMV_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  attr[na].id = cudaLaunchAttributeClusterDimension;
  attr[na].val.clusterDim.x = g.ksplit;
  attr[na].val.clusterDim.y = 1;
  attr[na].val.clusterDim.z = 1;
  ++na;
  if (g.pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  TA_CUDA(cudaLaunchKernelEx(&cfg, gemv_f16w_kernel<MROWS, TN, BULK, PEER, WIDE>, g));
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

}  // namespace

bool gemv_f16w_supported(uint32_t m, uint32_t n, uint32_t k, bool packed, uint32_t tile_n) {
  if (m == 0 || m > 8) return false;
  if (packed) return (tile_n == 32 || tile_n == 64) && n % tile_n == 0;
  (void)k;
  return n % 8 == 0;   // 16-byte loads of row-major rows
}

// Segments must agree on everything the CTA geometry depends on.
bool gemv_f16w_groupable(const GemvParams &a, const GemvParams &b) {
  const uint32_t ta = a.packed ? a.tile_n : 32, tb = b.packed ? b.tile_n : 32;
  return a.x == b.x && a.m == b.m && a.k == b.k && a.norm_w == b.norm_w && a.norm_eps == b.norm_eps &&
         ta == tb && !a.w2 == !b.w2;
}

static bool bulk_possible(const GemvParams *segs, int nseg) {
  for (int i = 0; i < nseg; ++i)
    if (!segs[i].packed || (reinterpret_cast<uintptr_t>(segs[i].w) & 15u) ||
        (segs[i].w2 && (reinterpret_cast<uintptr_t>(segs[i].w2) & 15u)))
      return false;
  return true;
}

// Rows from which a lone GEMV (or SwiGLU pair) goes to the tensor-memory kernel when its shape
// and the slot's workspace allow: 3 by default; the experiment switch gemv_umma forces it on for
// every row count (1) or off (0).
bool gemv_routes_to_umma(const GemvParams &p) {
  const int force = tunables().gemv_umma;
  if (force == 0) return false;
  return (force == 1 || p.m >= 3) && gemv_umma_eligible(p);
}

void launch_gemv_f16w_group(const Context &ctx, const GemvParams *segs, int nseg, bool pdl, const GemvWorkspace &ws,
                            cudaStream_t stream, const PeerLink *peer) {
  if (nseg < 1 || nseg > GEMV_MAX_SEGS) fail("GEMV group of %d segments (1..%d)", nseg, GEMV_MAX_SEGS);
  const int sm_count = ctx.sm_count;
  uint32_t *status = ws.status;
  if (peer && (segs[0].m != 1 || peer->world < 2 || peer->world > PEER_MAX_WORLD))
    fail("internal: the fused tensor-parallel exchange is built for single-row GEMVs on 2..%u ranks", PEER_MAX_WORLD);
  if (!peer && nseg == 1 && gemv_routes_to_umma(segs[0]) && ws.scratch && ws.counters &&
      ws.scratch_bytes >= gemv_umma_scratch_bytes(segs[0].n, segs[0].k, segs[0].w2 != nullptr, sm_count)) {
    launch_gemv_umma(ctx, segs[0], static_cast<float *>(ws.scratch), ws.scratch_bytes, ws.counters, status, pdl, stream);
    return;
  }
  GemvGroup g{};
  const GemvParams &p0 = segs[0];
  const uint32_t tn = p0.packed ? p0.tile_n : 32;
  uint32_t tiles = 0;
  for (int i = 0; i < nseg; ++i) {
    if (i && !gemv_f16w_groupable(p0, segs[i])) fail("GEMV group: segment %d does not share x / K / tile with segment 0", i);
    g.seg[i] = segs[i];
    tiles += (segs[i].n + tn - 1) / tn;
    g.tile_end[i] = tiles;
  }
  g.nseg = (uint32_t)nseg;
  g.pdl = (pdl && pdl_enabled()) ? 1u : 0u;
  g.status = status;
  if (peer) g.peer = *peer;
  const int mrows = p0.m <= 1 ? 1 : p0.m <= 2 ? 2 : p0.m <= 4 ? 4 : 8;
  const uint32_t u = 4;
  const uint32_t rpl = 32 / (tn / 8);
  const uint32_t nw = p0.w2 ? GEMV_WARPS / 2 : GEMV_WARPS;
  const uint32_t rows_per_pass = nw * rpl * u;
  // K split over a cluster: about one and a half CTAs per SM.  With three resident
  // per SM that is one wave for this launch and leaves room for the early CTAs of
  // the next launch, which prefetch their weights while this one finishes.  Never
  // split below one pass of rows.
  bool bulk = !peer && bulk_possible(segs, nseg);   // bulk-copy ring: packed tiles (contiguous per CTA), 16-byte aligned bases
  uint64_t weight_bytes = 0;
  for (int i = 0; i < nseg; ++i) weight_bytes += (uint64_t)segs[i].k * segs[i].n * 2 * (segs[i].w2 ? 2 : 1);
  if (p0.m > 2) bulk = false;   // more rows: the staged x slice and the accumulators need the space
  // The asynchronous hand-over arms its barrier behind one cluster barrier at CTA start: free while a
  // resident CTA waits for the launch before it (the few-MB matrices of a decode step: 0.973 -> 0.937 ms
  // per token), a cost per CTA when a long stream runs in several waves (4096 x 11008: 56.8 -> 58.7 us)
  g.handoff_async = (tunables().gemv_handoff && weight_bytes < (64ull << 20)) ? 1u : 0u;
  // measured: the ring wins on long streams (4096 x 11008: 3.8 -> 4.8 TB/s) and is neutral to
  // slightly slower on the few-MB matrices of a decode step, which are latency-bound
  if (weight_bytes < (64ull << 20)) bulk = false;
  if (tunables().gemv_bulk >= 0) bulk = !peer && tunables().gemv_bulk != 0 && p0.m <= 2 && bulk_possible(segs, nseg);
  uint32_t best_s = 1;
  if (weight_bytes >= (64ull << 20) && mrows <= 2) {
    // Large matrices stream: about eight passes per CTA amortise its prologue and epilogue
    // while several CTAs per SM overlap them (measured best on 4096 x 11008 and the llama MLP).
    const uint32_t want_k = 8 * rows_per_pass;
    for (uint32_t s : {1u, 2u, 4u, 8u}) {
      best_s = s;
      if (p0.k / s <= want_k + want_k / 2) break;
    }
  } else {
    for (uint32_t s : {1u, 2u, 4u, 8u}) {
      if (s > 1 && p0.k / s < rows_per_pass) break;
      const uint32_t k_cta = (p0.k + s - 1) / s;
      if (gemv_smem_bytes(k_cta, mrows, (int)tn, s, bulk) > 160 * 1024) continue;
      best_s = s;
      // the staged x slice (k_cta x rows floats) must leave room for several CTAs per SM
      if (s < 8 && gemv_smem_bytes(k_cta, mrows, (int)tn, s) > 40 * 1024 && p0.k / (2 * s) >= rows_per_pass) continue;
      // small matrices: 1.5 CTAs per SM; from 16 MB up more CTAs keep more of the stream in flight
      const uint64_t want2 = weight_bytes >= (16ull << 20) ? 6ull : 3ull;   // CTAs per SM, doubled
      if ((uint64_t)tiles * s * 2 >= want2 * (uint64_t)sm_count) break;
      if (s < 8 && (uint64_t)tiles * s * 2 * 2 > 6ull * (uint64_t)sm_count) break;   // the next split would not fit one wave (three CTAs per SM)
    }
  }
  {   // experiment switch: force the cluster split
    const uint32_t v = (uint32_t)std::max(0, tunables().gemv_ksplit);
    if ((v == 1 || v == 2 || v == 4 || v == 8) && p0.k / v >= rows_per_pass) best_s = v;
  }
  g.ksplit = best_s;
  g.k_cta = (p0.k + best_s - 1) / best_s;
  if (gemv_smem_bytes(g.k_cta, mrows, (int)tn, best_s, bulk) > 196 * 1024)
    fail("GEMV: K = %u with %u rows does not fit shared memory at any cluster split", p0.k, p0.m);
#define TA_GEMV_CASE(MR)                                                          \
  if (mrows == MR) {                                                              \
    if (bulk) {                                                                   \
      if (tn == 64) launch_t<MR, 64, true>(g, tiles, stream);                     \
      else launch_t<MR, 32, true>(g, tiles, stream);                              \
    } else {                                                                      \
      if (tn == 64) launch_t<MR, 64, false>(g, tiles, stream);                    \
      else launch_t<MR, 32, false>(g, tiles, stream);                             \
    }                                                                             \
    return;                                                                       \
  }
  if (peer) {
    // four ranks and more, one wave at two CTAs per SM: the variant with the wider pulls (on 2 GPUs it
    // measured 0.807 against 0.792 ms per token for the launches that fit, so two ranks never take it)
    const bool wide = peer->world >= 4 && (uint64_t)tiles * best_s <= 2ull * (uint64_t)sm_count && tunables().gemv_peer_wide;
    if (wide) {
      if (tn == 64) launch_t<1, 64, false, true, true>(g, tiles, stream);
      else launch_t<1, 32, false, true, true>(g, tiles, stream);
    } else {
      if (tn == 64) launch_t<1, 64, false, true, false>(g, tiles, stream);
      else launch_t<1, 32, false, true, false>(g, tiles, stream);
    }
    return;
  }
  TA_GEMV_CASE(1)
  TA_GEMV_CASE(2)
  TA_GEMV_CASE(4)
  TA_GEMV_CASE(8)
#undef TA_GEMV_CASE
}

uint32_t gemv_f16w_tiles(const GemvParams *segs, int nseg) {
  const uint32_t tn = segs[0].packed ? segs[0].tile_n : 32;
  uint32_t tiles = 0;
  for (int i = 0; i < nseg; ++i) tiles += (segs[i].n + tn - 1) / tn;
  return tiles;
}

void launch_gemv_f16w(const Context &ctx, GemvParams p, const GemvWorkspace &ws, cudaStream_t stream) {
  launch_gemv_f16w_group(ctx, &p, 1, true, ws, stream);
}

}  // namespace ta
