// Skinny f16-weight GEMM for 3..8 activation rows on the 5th-generation tensor cores:
//     out[m, :] = epi(alpha * x'[m, :] @ W),   W f16 [K, N] row-major or packed [N/t][K][t]
// the M > 1 form of the reference's row kernel (shaders/matmul_row_bda_kernel.glsl:186-404:
// f16 weights widened exactly, f32 accumulation, fused RMSNorm of A :212-234, epilogue
// alpha -> (+C) -> bias -> act -> binary(D) :272-276) and of its SwiGLU pair
// (tools/llama-ash/src/model/forward/mod.rs:194-206).  HBM-bound: every weight byte is read once.
//
// The weights never pass through registers.  TMA streams them into a deep shared-memory ring
// exactly as they lie in memory ([k][column], column-contiguous); the tensor core reads them from
// there as the A operand of tcgen05.mma kind::f16 (M = 128 weight columns, "MN-major" shared-memory
// descriptor) with the activations as the B operand (N = 16) and the sums in tensor memory.
// Bytes in flight per SM are what the ring holds (8 x 16 KiB), independent of registers.
//
// x is an f32 operand and the tensor core multiplies f16: each CTA scales its K slice of every row
// by a power of two so that the largest magnitude lies in [0.5, 1) (exact, undone on the sums), then
// splits v = hi + lo with hi = f16(v), lo = f16(v - hi) and hands the tensor core 16 "columns":
// rows 0-7 the hi parts, rows 8-15 the lo parts of the 8 activation rows.  One MMA per 16 k covers
// both; the epilogue adds the two halves.  About 22 bits of x enter the products, the weights are
// used exactly as stored, accumulation is f32: inside the f16-weight tolerance (2e-3) by orders of
// magnitude, and no activation range is excluded.
//
// Work split: the grid is S teams; team s owns K boxes [s KB/S, (s+1) KB/S) of 64 rows and keeps
// that slice of x resident in shared memory; the CTAs of a team share out the column groups
// (128 columns; with a second matrix sharing x: 64 columns of each) and walk them back to back, the
// ring never draining between groups.  A CTA's partial sums go to a scratch record (group, slice);
// the CTA that takes the last ticket of a group adds the S records in slice order -- a fixed order,
// so results are run-to-run bit-identical whichever CTA comes last -- and runs the epilogue.
//
// Warps: 0-3 drain tensor memory / finish groups, 4 issues TMA (it starts before the dependency
// wait: weights never depend on the producer of x), 5 owns tensor memory and issues the MMAs.
// Every wait is bounded; a timeout raises the abort flag, all roles leave, status bit 0 is set.
#include <cuda_fp16.h>

#include <algorithm>

#include "k_epilogue.cuh"
#include "k_umma.cuh"
#include "ta_core.hpp"

namespace ta {

namespace {

using namespace umma;

constexpr int GU_THREADS = 192;
constexpr int GU_BOX_K = 64;                         // weight rows per ring stage
constexpr int GU_STAGE_BYTES = GU_BOX_K * 128 * 2;   // 128 columns of f16: 16 KiB
constexpr int GU_STAGES = 8;
constexpr int GU_XS_MAX_K = 2048;                    // resident x slice: 16 rows x 2048 halves = 64 KiB
constexpr int GU_XS_BYTES = GU_XS_MAX_K * 16 * 2;
constexpr int GU_REC_FLOATS = 8 * 128 + 8;           // scratch record: 8 rows x 128 sums, then 8 sums of squares
constexpr uint32_t GU_MAX_GROUPS = 4094;             // ticket words [0, 4094), then the finish cursor and the exit count
constexpr uint32_t GU_CURSOR = 4094, GU_DONE = 4095;
constexpr int GU_MISC_BYTES = 1024;                  // barriers, tensor-memory slot, flags, per-row scalars
constexpr int GU_SMEM_BYTES = GU_STAGES * GU_STAGE_BYTES + GU_XS_BYTES + GU_MISC_BYTES + 1024;

struct GemvUmmaParams {
  GemvParams p;
  uint32_t groups, team_size, teams;   // column groups; CTAs per team; K slices
  uint32_t boxes;                      // K boxes of 64 rows in all
  uint32_t dual;                       // second matrix sharing x (64 + 64 columns per group)
  uint32_t pdl;
  float *scratch;
  uint32_t *counters;                  // one ticket word per group, zero between launches
  uint32_t *status;
};

// BLK32: packed tiles of 32 columns (64-byte rows, 64-byte swizzle, four blocks per stage);
// otherwise 64-column blocks (packed tiles of 64 or row-major weights; 128-byte swizzle, two blocks).
template <bool BLK32>
__global__ void __launch_bounds__(GU_THREADS, 1)
gemv_umma_kernel(const __grid_constant__ GemvUmmaParams g, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_w2) {
  extern __shared__ uint8_t smem_raw[];
  const GemvParams &p = g.p;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t xs_base = smem_base + GU_STAGES * GU_STAGE_BYTES;
  uint8_t *xs_gen = smem_gen + GU_STAGES * GU_STAGE_BYTES;
  const uint32_t bar_base = xs_base + GU_XS_BYTES;
  uint8_t *misc = xs_gen + GU_XS_BYTES;
  auto full = [&](int s) { return bar_base + 8u * s; };
  auto empty = [&](int s) { return bar_base + 8u * (GU_STAGES + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (2 * GU_STAGES + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (2 * GU_STAGES + 2 + b); };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(misc + 8 * (2 * GU_STAGES + 4));
  volatile uint32_t *abort_flag = tmem_slot + 1;
  volatile uint32_t *ticket_slot = tmem_slot + 2;
  float *unscale = reinterpret_cast<float *>(misc + 256);    // [8] 2^e per row: undoes the staging scale
  float *ssq = unscale + 8;                                   // [8] sum of squares of this slice, per row
  float *red_max = ssq + 8;                                   // [5 warps][8]
  float *red_ss = red_max + 40;                               // [5 warps][8]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GU_STAGES; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 128);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 5) tmem_alloc(smem_u32((const void *)tmem_slot), 32);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // this CTA: K slice `slice` (boxes [box_lo, box_hi)), column groups rank, rank + team_size, ...
  const uint32_t slice = blockIdx.x % g.teams, rank = blockIdx.x / g.teams;
  const uint32_t box_lo = (uint32_t)(((uint64_t)slice * g.boxes) / g.teams);
  const uint32_t box_hi = (uint32_t)(((uint64_t)(slice + 1) * g.boxes) / g.teams);
  const uint32_t k_lo = box_lo * GU_BOX_K, k_hi = min(p.k, box_hi * GU_BOX_K);
  const uint32_t cols_per_group = g.dual ? 64u : 128u;
  constexpr uint32_t BLK_COLS = BLK32 ? 32u : 64u;
  constexpr uint32_t BLK_BYTES = GU_BOX_K * BLK_COLS * 2;     // one [64 rows][BLK_COLS] block

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    // weights depend on no earlier kernel: no dependency wait here; the trigger lets the next
    // kernel in the stream be scheduled as soon as every warp of the grid has issued it
    if (g.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (uint32_t grp = rank; ok && grp < g.groups; grp += g.team_size) {
      for (uint32_t box = box_lo; box < box_hi; ++box) {
        ok = mbar_wait(empty(stage), phase ^ 1u, abort_flag);
        if (!ok) break;
        if (elect_one()) {
          const uint32_t dst = smem_base + stage * GU_STAGE_BYTES;
          const int k0 = (int)(box * GU_BOX_K);
          mbar_arrive_expect_tx(full(stage), GU_STAGE_BYTES);
          if (p.packed) {
            // map {tile columns, K, tiles}: one box brings the group's consecutive tiles, block after block
            const int tiles_per_mat = (int)(cols_per_group / BLK_COLS);
            tma_load_3d(dst, &map_w, full(stage), 0, k0, (int)grp * tiles_per_mat);
            if (g.dual) tma_load_3d(dst + GU_STAGE_BYTES / 2, &map_w2, full(stage), 0, k0, (int)grp * tiles_per_mat);
          } else {
            // row-major map {N, K, 1}: one box per 64-column block
            const int c0 = (int)(grp * cols_per_group);
            if (g.dual) {
              tma_load_3d(dst, &map_w, full(stage), c0, k0, 0);
              tma_load_3d(dst + BLK_BYTES, &map_w2, full(stage), c0, k0, 0);
            } else {
              tma_load_3d(dst, &map_w, full(stage), c0, k0, 0);
              tma_load_3d(dst + BLK_BYTES, &map_w, full(stage), c0 + 64, k0, 0);
            }
          }
        }
        __syncwarp();
        if (++stage == GU_STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // ---- everything below may depend on the previous kernel in the stream (x, scratch, tickets)
    if (g.pdl) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    // ------------------------------------------------------------ stage the x slice (160 threads)
    // One round trip: every thread requests its share of the slice (two runs of 8 consecutive k, all
    // 8 rows) before anything is consumed, keeps x * norm weight in registers, and converts from
    // there once the row maxima are known.
    const int st = warp < 4 ? threadIdx.x : threadIdx.x - 32;      // 0..159
    const int swarp = st >> 5;
    const uint32_t k_len = k_hi > k_lo ? k_hi - k_lo : 0u;
    const uint32_t k_pad = (k_len + 31u) & ~31u;                    // whole 32-k blocks are written
    const bool vec = (p.k & 3u) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15u) == 0 &&
                     (!p.norm_w || (reinterpret_cast<uintptr_t>(p.norm_w) & 15u) == 0);
    constexpr int OCT = GU_XS_MAX_K / 8 / 160 + 1;                  // runs of 8 k per thread (2)
    static_assert(OCT * 160 * 8 >= GU_XS_MAX_K, "the staging threads must cover the largest slice");
    float xr[OCT][8][8];
    float mx[8], ss[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) { mx[m] = 0.0f; ss[m] = 0.0f; }
#pragma unroll
    for (int i = 0; i < OCT; ++i) {
      const uint32_t kk = (uint32_t)(st + 160 * i) * 8u;
      float w8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) w8[j] = 1.0f;
      if (p.norm_w && kk < k_len) {
        if (vec && kk + 8 <= k_len) {
          const float4 a = *reinterpret_cast<const float4 *>(p.norm_w + k_lo + kk);
          const float4 b = *reinterpret_cast<const float4 *>(p.norm_w + k_lo + kk + 4);
          w8[0] = a.x; w8[1] = a.y; w8[2] = a.z; w8[3] = a.w; w8[4] = b.x; w8[5] = b.y; w8[6] = b.z; w8[7] = b.w;
        } else {
          for (uint32_t j = 0; j < 8 && kk + j < k_len; ++j) w8[j] = p.norm_w[k_lo + kk + j];
        }
      }
#pragma unroll
      for (int m = 0; m < 8; ++m) {
#pragma unroll
        for (int j = 0; j < 8; ++j) xr[i][m][j] = 0.0f;
        if ((uint32_t)m < p.m && kk < k_len) {
          const float *src = p.x + (size_t)m * p.k + k_lo + kk;
          if (vec && kk + 8 <= k_len) {
            const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 4);
            xr[i][m][0] = a.x; xr[i][m][1] = a.y; xr[i][m][2] = a.z; xr[i][m][3] = a.w;
            xr[i][m][4] = b.x; xr[i][m][5] = b.y; xr[i][m][6] = b.z; xr[i][m][7] = b.w;
          } else {
            for (uint32_t j = 0; j < 8 && kk + j < k_len; ++j) xr[i][m][j] = src[j];
          }
        }
      }
      // rows at or beyond p.m are skipped from here on: their operand rows stay unwritten, and the
      // output columns they produce are never read
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        if ((uint32_t)m >= p.m) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float x = xr[i][m][j];
          ss[m] = fmaf(x, x, ss[m]);            // the RMSNorm statistic is over x itself
          const float v = x * w8[j];
          xr[i][m][j] = v;
          mx[m] = fmaxf(mx[m], fabsf(v));
        }
      }
    }
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      if ((uint32_t)m >= p.m) continue;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mx[m] = fmaxf(mx[m], __shfl_xor_sync(0xffffffffu, mx[m], o));
        ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], o);
      }
      if (lane == 0) {
        red_max[swarp * 8 + m] = mx[m];
        red_ss[swarp * 8 + m] = ss[m];
      }
    }
    asm volatile("bar.sync 1, 160;" ::: "memory");
    if (st < 8 && (uint32_t)st < p.m) {
      float rmx = 0.0f, rss = 0.0f;
      for (int w = 0; w < 5; ++w) {       // warp order: a fixed sum
        rmx = fmaxf(rmx, red_max[w * 8 + st]);
        rss += red_ss[w * 8 + st];
      }
      // power of two e with rmx * 2^-e in [0.5, 1); zero, denormal and huge rows stay finite
      int e = (int)((__float_as_uint(rmx) >> 23) & 0xffu) - 126;
      if (rmx == 0.0f) e = 0;
      e = max(-125, min(125, e));
      unscale[st] = __uint_as_float((uint32_t)(127 + e) << 23);
      ssq[st] = rss;
    }
    asm volatile("bar.sync 1, 160;" ::: "memory");
    // hi / lo halves into the K-major, 64-byte-swizzled image the tensor core reads: a block of 32 k is
    // 16 rows (0-7 hi, 8-15 lo) x 64 bytes, 16-byte chunk c of row r stored at chunk c ^ ((r >> 1) & 3)
#pragma unroll
    for (int i = 0; i < OCT; ++i) {
      const uint32_t kk = (uint32_t)(st + 160 * i) * 8u;
      if (kk < k_pad) {
        const uint32_t blk = kk >> 5, chunk = (kk & 31u) >> 3;
        uint8_t *base = xs_gen + (size_t)blk * 1024;
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          if ((uint32_t)m >= p.m) continue;
          const float sc = 1.0f / unscale[m];   // exact: a power of two
          uint32_t hi[4], lo[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float v0 = xr[i][m][2 * j] * sc, v1 = xr[i][m][2 * j + 1] * sc;
            const __half2 h = __floats2half2_rn(v0, v1);
            const float2 hf = __half22float2(h);
            const __half2 l = __floats2half2_rn(v0 - hf.x, v1 - hf.y);
            hi[j] = *reinterpret_cast<const uint32_t *>(&h);
            lo[j] = *reinterpret_cast<const uint32_t *>(&l);
          }
          const uint32_t r_hi = m, r_lo = m + 8;
          *reinterpret_cast<uint4 *>(base + r_hi * 64 + ((chunk ^ ((r_hi >> 1) & 3u)) << 4)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          *reinterpret_cast<uint4 *>(base + r_lo * 64 + ((chunk ^ ((r_lo >> 1) & 3u)) << 4)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> the tensor core's reads
    asm volatile("bar.sync 1, 160;" ::: "memory");

    if (warp == 5) {
      // ---------------------------------------------------------- MMA issuer
      // D f32 | A, B f16 | A MN-major (columns contiguous), B K-major | N = 16 | M = 128
      const uint32_t idesc = (1u << 4) | (1u << 15) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
      uint32_t stage = 0, phase = 0, acc_it = 0;
      bool ok = true;
      for (uint32_t grp = rank; ok && grp < g.groups; grp += g.team_size, ++acc_it) {
        const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
        ok = mbar_wait(acc_empty(buf), acc_phase ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * 16u;
        for (uint32_t box = box_lo; box < box_hi; ++box) {
          ok = mbar_wait(full(stage), phase, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_base + stage * GU_STAGE_BYTES;
          // A: [k][columns] blocks; 8-k groups 8 rows apart (SBO), column blocks BLK_BYTES apart (LBO);
          // 16 k further = 16 rows further.  B: 64-byte rows, 8-row groups 512 B apart; 16 k = 32 bytes.
          const uint64_t da0 = BLK32 ? make_desc(a_base, BLK_BYTES, 512, LAYOUT_SW64)
                                     : make_desc(a_base, BLK_BYTES, 1024, LAYOUT_SW128);
          const uint32_t kk0 = (box - box_lo) * GU_BOX_K;                 // slice offset of this box
          const uint64_t db0 = make_desc(xs_base + (kk0 >> 5) * 1024u, 16, 512, LAYOUT_SW64);
          const uint32_t steps = min((uint32_t)(GU_BOX_K / 16), (k_hi - (k_lo + kk0) + 15u) / 16u);   // K % 16 == 0
          if (elect_one()) {
#pragma unroll
            for (uint32_t t = 0; t < GU_BOX_K / 16; ++t) {
              if (t < steps) {
                const uint64_t da = da0 + (uint64_t)(t * (BLK32 ? 64u : 128u));          // 16 rows of 64 / 128 bytes, in 16-byte units
                const uint64_t db = db0 + (uint64_t)((t >> 1) * 64u + (t & 1u) * 2u);    // next 32-k block: 1 KiB; odd step: +32 B
                mma_f16(d_tmem, da, db, idesc, (box != box_lo || t != 0u) ? 1u : 0u);
              }
            }
            tc_commit(empty(stage));
            if (box + 1 == box_hi) tc_commit(acc_full(buf));
          }
          __syncwarp();
          if (++stage == GU_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    } else {
      // ---------------------------------------------------------- drain + finish (warps 0-3)
      // Draining and finishing are decoupled.  A drained group costs a record and a ticket, nothing
      // else; complete groups are finished in group order by whichever CTA claims them from a cursor:
      // without waiting between two drains (a claim succeeds only on a complete group), and with a
      // bounded wait once the CTA's own groups are drained.  So the finishing work is spread over all
      // CTAs instead of falling on the slowest slice, and no drain waits behind a finish.
      uint32_t acc_it = 0;
      bool ok = true;
      const uint32_t tid = threadIdx.x;                    // 0..127 = weight column within the group
      uint32_t *cursor = g.counters + GU_CURSOR, *done = g.counters + GU_DONE;

      auto finish_group = [&](uint32_t grp) {
        const float *grp_rec = g.scratch + (size_t)grp * g.teams * GU_REC_FLOATS;
        const uint32_t col = grp * cols_per_group + (g.dual ? (tid & 63u) : tid);
        if (col >= p.n || (g.dual && tid >= 64)) return;
        // records of four or eight slices are requested together (slices in order: a fixed sum), the
        // epilogue operands of all rows with the first of them: one to three L2 round trips per group
        float s0[8], s1[8], ssum[8], oldc[8], dv[8];
        const float bv = p.bias ? p.bias[col] : 0.0f;
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          const bool live = (uint32_t)m < p.m;
          const size_t ci = (size_t)m * p.n + col;
          s0[m] = 0.0f; s1[m] = 0.0f; ssum[m] = 0.0f;
          oldc[m] = (live && p.accumulate) ? p.c[ci] : 0.0f;
          dv[m] = (live && p.d) ? p.d[ci] : 0.0f;
        }
        if (p.m <= 4) {
          // up to four live rows: eight slices per batch fit the registers
          for (uint32_t sl0 = 0; sl0 < g.teams; sl0 += 8) {
            float a[8][4], b[8][4], q[8][4];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const float *r = grp_rec + (size_t)(sl0 + u) * GU_REC_FLOATS;
              const bool have = sl0 + u < g.teams;
#pragma unroll
              for (int m = 0; m < 4; ++m) {
                const bool live = have && (uint32_t)m < p.m;
                a[u][m] = live ? __ldcg(r + m * 128 + tid) : 0.0f;
                b[u][m] = (live && g.dual) ? __ldcg(r + m * 128 + 64 + tid) : 0.0f;
                q[u][m] = (live && p.norm_w) ? __ldcg(r + 8 * 128 + m) : 0.0f;
              }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
              for (int m = 0; m < 4; ++m) { s0[m] += a[u][m]; s1[m] += b[u][m]; ssum[m] += q[u][m]; }
          }
        } else {
          for (uint32_t sl0 = 0; sl0 < g.teams; sl0 += 4) {
            float a[4][8], b[4][8], q[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float *r = grp_rec + (size_t)(sl0 + u) * GU_REC_FLOATS;
              const bool have = sl0 + u < g.teams;
#pragma unroll
              for (int m = 0; m < 8; ++m) {
                const bool live = have && (uint32_t)m < p.m;
                a[u][m] = live ? __ldcg(r + m * 128 + tid) : 0.0f;
                b[u][m] = (live && g.dual) ? __ldcg(r + m * 128 + 64 + tid) : 0.0f;
                q[u][m] = (live && p.norm_w) ? __ldcg(r + 8 * 128 + m) : 0.0f;
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
              for (int m = 0; m < 8; ++m) { s0[m] += a[u][m]; s1[m] += b[u][m]; ssum[m] += q[u][m]; }
          }
        }
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          if ((uint32_t)m >= p.m) break;
          float v0 = s0[m], v1 = s1[m];
          if (p.norm_w) {
            const float rs = rsqrtf(ssum[m] / (float)p.k + p.norm_eps);
            v0 *= rs;
            v1 *= rs;
          }
          const size_t ci = (size_t)m * p.n + col;
          float o = p.alpha == 1.0f ? v0 : p.alpha * v0;
          if (g.dual) {
            o = epi_activate(o, 2) * v1;
            if (p.c2) p.c2[ci] = v1;
          }
          if (p.accumulate) o += oldc[m];
          o = epi_apply(o, p.bias != nullptr, bv, p.act, p.binary, dv[m], p.beta);
          p.c[ci] = o;
        }
      };
      // claim the next group in order; `block`: wait (bounded) for it to be complete, else take it only
      // if it already is.  Returns the group or ~0u.  Thread 0 decides, all 128 threads learn it.
      auto claim = [&](bool block) -> uint32_t {
        if (tid == 0) {
          uint32_t got = ~0u;
          if (block) {
            const uint32_t c = atomicAdd(cursor, 1u);
            if (c < g.groups) {
              const uint64_t t0 = global_timer_ns();
              uint32_t seen = 0, spins = 0;
              for (;;) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(g.counters + c) : "memory");
                if (seen >= g.teams) { got = c; break; }
                if ((++spins & 63u) == 0 && (*abort_flag || global_timer_ns() - t0 > WAIT_LIMIT_NS)) {
                  *abort_flag = 1;
                  break;
                }
              }
            }
          } else {
            uint32_t c, seen = 0;
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(c) : "l"(cursor) : "memory");
            if (c < g.groups) {
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(g.counters + c) : "memory");
              if (seen >= g.teams && atomicCAS(cursor, c, c + 1u) == c) got = c;
            }
          }
          *ticket_slot = got;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        const uint32_t got = *ticket_slot;
        asm volatile("bar.sync 2, 128;" ::: "memory");       // the slot may be rewritten after this
        return got;
      };
      auto finish_claimed = [&](uint32_t grp) {
        __threadfence();                                       // the acquire of thread 0, for all threads
        finish_group(grp);
        if (tid == 0) g.counters[grp] = 0u;                    // every slice has arrived: ready for the next launch
      };

      for (uint32_t grp = rank; ok && grp < g.groups; grp += g.team_size, ++acc_it) {
        const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
        ok = mbar_wait(acc_full(buf), acc_phase, abort_flag, 128);
        if (!ok) break;
        tc_fence_after();
        float v[16];
        tmem_ld16(tmem_base + buf * 16u + ((uint32_t)(warp * 32) << 16), v);
        tc_fence_before();
        mbar_arrive(acc_empty(buf));
        float *rec = g.scratch + ((size_t)grp * g.teams + slice) * GU_REC_FLOATS;
#pragma unroll
        for (int m = 0; m < 8; ++m)
          if ((uint32_t)m < p.m) rec[m * 128 + tid] = (v[m] + v[8 + m]) * unscale[m];
        if (tid < 8) rec[8 * 128 + tid] = ssq[tid];
        __threadfence();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (tid == 0) atomicAdd(&g.counters[grp], 1u);
        const uint32_t ready = claim(false);
        if (ready != ~0u) finish_claimed(ready);
      }
      // own groups drained: help until every group has been claimed
      while (ok) {
        const uint32_t grp = claim(true);
        if (grp == ~0u) break;
        finish_claimed(grp);
      }
      // the last CTA to leave puts the cursor back (claims beyond the last group overshoot it)
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (tid == 0 && atomicAdd(done, 1u) == gridDim.x - 1) {
        *cursor = 0u;
        *done = 0u;
      }
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(100000);   // let copies / MMAs in flight land
    if (threadIdx.x == 0 && g.status) atomicOr(g.status, 1u);
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
}

// Teams (K slices) and team size: fewest ring stages on the critical path,
//   rounds * boxes per slice (+ half a box per round for the drain and the ticket),
// subject to the x slice fitting shared memory; ties go to fewer slices (fewer records to add).
void choose_split(uint32_t groups, uint32_t boxes, int sm_count, uint32_t *teams, uint32_t *team_size) {
  uint64_t best_cost = ~0ull;
  *teams = 1;
  *team_size = 1;
  const uint32_t max_s = std::min<uint32_t>(boxes, std::min<uint32_t>(64u, (uint32_t)sm_count));
  for (uint32_t s = 1; s <= max_s; ++s) {
    const uint32_t per = (boxes + s - 1) / s;
    if ((uint64_t)per * GU_BOX_K > GU_XS_MAX_K) continue;
    const uint32_t ts = std::max<uint32_t>(1, std::min<uint32_t>(groups, (uint32_t)sm_count / s));
    const uint32_t rounds = (groups + ts - 1) / ts;
    const uint64_t cost = (uint64_t)rounds * (2 * per + 1);
    if (cost < best_cost) {
      best_cost = cost;
      *teams = s;
      *team_size = ts;
    }
  }
}

}  // namespace

size_t gemv_umma_scratch_bytes(uint32_t n, uint32_t k, bool dual, int sm_count) {
  const uint32_t groups = (n + (dual ? 63u : 127u)) / (dual ? 64u : 128u);
  const uint32_t boxes = (k + GU_BOX_K - 1) / GU_BOX_K;
  uint32_t teams, team_size;
  choose_split(groups, boxes, sm_count, &teams, &team_size);
  return (size_t)groups * teams * GU_REC_FLOATS * sizeof(float);
}

// Shapes this kernel takes: plain epilogue (no fused RoPE / scatter store), K a multiple of 16 (the
// tensor core's k step; a partial step would multiply rows of the next packed tile), 16-byte
// aligned weights, at most 4094 column groups (one ticket word each).
bool gemv_umma_eligible(const GemvParams &p) {
  if (p.m == 0 || p.m > 8 || p.store_kind != 0) return false;
  if (p.k % 16 || p.k < 64) return false;
  if (reinterpret_cast<uintptr_t>(p.w) & 15u) return false;
  if (p.w2 && (reinterpret_cast<uintptr_t>(p.w2) & 15u)) return false;
  if (p.packed) {
    if ((p.tile_n != 32 && p.tile_n != 64) || p.n % p.tile_n) return false;
  } else if (p.n % 8) {
    return false;
  }
  const uint32_t cols = p.w2 ? 64u : 128u;
  if ((p.n + cols - 1) / cols > GU_MAX_GROUPS) return false;
  if (((uint64_t)(p.k + GU_BOX_K - 1) / GU_BOX_K) > 64ull * (GU_XS_MAX_K / GU_BOX_K)) return false;   // x slice at 64 teams
  return true;
}

void launch_gemv_umma(const Context &ctx, const GemvParams &p, float *scratch, size_t scratch_bytes, uint32_t *counters,
                      uint32_t *status, bool pdl, cudaStream_t stream) {
  if (!gemv_umma_eligible(p)) fail("internal: tensor-memory GEMV launched on an ineligible problem");
  GemvUmmaParams g{};
  g.p = p;
  g.dual = p.w2 ? 1u : 0u;
  g.groups = (p.n + (g.dual ? 63u : 127u)) / (g.dual ? 64u : 128u);
  g.boxes = (p.k + GU_BOX_K - 1) / GU_BOX_K;
  choose_split(g.groups, g.boxes, ctx.sm_count, &g.teams, &g.team_size);
  const size_t need = (size_t)g.groups * g.teams * GU_REC_FLOATS * sizeof(float);
  if (!scratch || scratch_bytes < need)
    fail("internal: tensor-memory GEMV needs %zu bytes of scratch, the slot holds %zu", need, scratch_bytes);
  g.scratch = scratch;
  g.counters = counters + ATTN_DECODE_MAX_KV_HEADS;
  g.status = status;
  g.pdl = (pdl && tunables().pdl) ? 1u : 0u;

  const bool blk32 = p.packed && p.tile_n == 32;
  CUtensorMap maps[2];
  for (int i = 0; i < (g.dual ? 2 : 1); ++i) {
    const void *w = i == 0 ? p.w : p.w2;
    if (p.packed) {
      // packed [N/t][K][t]: dims {t, K, N/t}; a box holds the group's consecutive tiles
      const uint32_t per_mat_cols = g.dual ? 64u : 128u, depth = per_mat_cols / p.tile_n;
      auto encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ctx.encode_tiled);
      if (!encode) fail("cuTensorMapEncodeTiled is unavailable in this CUDA driver");
      const cuuint64_t dims[3] = {p.tile_n, p.k, p.n / p.tile_n};
      const cuuint64_t strides[2] = {(cuuint64_t)p.tile_n * 2, (cuuint64_t)p.k * p.tile_n * 2};
      const cuuint32_t box[3] = {p.tile_n, GU_BOX_K, depth};
      const cuuint32_t estr[3] = {1, 1, 1};
      const CUresult rc = encode(&maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(w), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, blk32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (rc != CUDA_SUCCESS) fail("cuTensorMapEncodeTiled (packed weights) failed with CUresult %d", (int)rc);
    } else {
      encode_map3(ctx, &maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, w, p.n, p.k, 1, (uint64_t)p.n * 2,
                  (uint64_t)p.n * p.k * 2, 64, GU_BOX_K, CU_TENSOR_MAP_SWIZZLE_128B);
    }
  }
  if (!g.dual) maps[1] = maps[0];

  static bool attr_set[2][64] = {};
  if (!attr_set[blk32][ctx.device & 63]) {
    if (blk32) TA_CUDA(cudaFuncSetAttribute(gemv_umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GU_SMEM_BYTES));
    else TA_CUDA(cudaFuncSetAttribute(gemv_umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GU_SMEM_BYTES));
    attr_set[blk32][ctx.device & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(g.teams * g.team_size, 1, 1);
  cfg.blockDim = dim3(GU_THREADS, 1, 1);
  cfg.dynamicSmemBytes = GU_SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g.pdl ? 1 : 0;
  if (blk32) TA_CUDA(cudaLaunchKernelEx(&cfg, gemv_umma_kernel<true>, g, maps[0], maps[1]));
  else TA_CUDA(cudaLaunchKernelEx(&cfg, gemv_umma_kernel<false>, g, maps[0], maps[1]));
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

}  // namespace ta
