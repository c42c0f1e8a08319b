// Fused attention kernels.
//
// flash_prefill_kernel: causal prefill attention with online softmax, the math
// of shaders/attention_flash_kernel.glsl:82-177 in the reference:
//   out[h, i, :] = softmax_j(scale * q[h, i, :] . Kt[kv, :, j]) @ V[kv, j, :],
//   j < min(kv_len, pos_base + i + 1), kv = h / group; a row that sees no
//   position is left untouched.  q/out f32 with (head, row) strides so head-major
//   [H, T, dh] and token-major [T, H*dh] both work; Kt [H_kv, dh, T_max] and
//   V [H_kv, T_max, dh] in f32 or f16.
// Each query row is owned by a pair of adjacent lanes (each half of the head
// dim); the half dots meet through one xor-shuffle; the running (m, l, acc)
// state lives in registers; K/V tiles of 32 positions are staged in shared
// memory; tiles past the CTA's causal frontier are skipped.
//
// attn_decode_kernel: split-K decode attention (shaders/attention_decode_kernel.glsl:89-170
// and shaders/op_attn_decode_combine.comp:42-74 in one launch), described at the kernel.
// The valid length may come from a host-visible cell (kv_len + *pos), read on the
// device, so a captured graph serves every position.
#include <cuda_fp16.h>

#include "ta_core.hpp"

namespace ta {

namespace {

constexpr float NEG_BIG = -3.402823466e38f;

__device__ __forceinline__ float kv_load(const void *base, size_t idx, bool f16) {
  return f16 ? __half2float(static_cast<const __half *>(base)[idx]) : static_cast<const float *>(base)[idx];
}

// ------------------------------------------------------------------ prefill
template <int DH>
__global__ void __launch_bounds__(128)
flash_prefill_kernel(const FlashParams p) {
  constexpr int BQ = 64, BK = 32, DHS = DH / 2;
  __shared__ float Ksh[DH * BK];   // [d][j]
  __shared__ float Vsh[BK * DH];   // [j][d]
  const uint32_t head = blockIdx.y, tid = threadIdx.x;
  const uint32_t q0 = blockIdx.x * BQ;
  const uint32_t row = q0 + tid / 2, half_id = tid & 1u, d0 = half_id * DHS;
  const bool live = row < p.t_q;
  const uint32_t kv_head = head / p.group;
  const size_t q_base = (size_t)head * p.q_head_stride + (size_t)min(row, p.t_q - 1) * p.q_row_stride + d0;
  const size_t kt_base = (size_t)kv_head * DH * p.t_max, v_base = (size_t)kv_head * p.t_max * DH;

  const uint32_t valid_row = live ? (uint32_t)min((uint64_t)p.kv_len, (uint64_t)p.pos_base + row + 1u) : 0u;
  const uint32_t last_row = min(q0 + BQ, p.t_q) - 1u;
  const uint32_t valid_max = (uint32_t)min((uint64_t)p.kv_len, (uint64_t)p.pos_base + last_row + 1u);
  const uint32_t num_tiles = (valid_max + BK - 1) / BK;

  float qreg[DHS];
#pragma unroll
  for (int d = 0; d < DHS; ++d) qreg[d] = p.q[q_base + d];
  float m = NEG_BIG, l = 0.0f, acc[DHS];
#pragma unroll
  for (int d = 0; d < DHS; ++d) acc[d] = 0.0f;

  for (uint32_t tile = 0; tile < num_tiles; ++tile) {
    const uint32_t k0 = tile * BK;
    for (uint32_t i = tid; i < DH * BK; i += 128) {
      const uint32_t d = i / BK, j = i % BK, pos = k0 + j;
      Ksh[i] = pos < p.t_max ? kv_load(p.kt, kt_base + (size_t)d * p.t_max + pos, p.kv_f16) : 0.0f;
    }
    for (uint32_t i = tid; i < BK * DH; i += 128) {
      const uint32_t j = i / DH, d = i % DH, pos = k0 + j;
      Vsh[i] = (pos < p.t_max && pos < p.kv_len) ? kv_load(p.v, v_base + (size_t)pos * DH + d, p.kv_f16) : 0.0f;
    }
    __syncthreads();

    float s[BK];
#pragma unroll
    for (int j = 0; j < BK; ++j) s[j] = 0.0f;
#pragma unroll
    for (int d = 0; d < DHS; ++d) {
      const float qd = qreg[d];
      const float4 *krow = reinterpret_cast<const float4 *>(&Ksh[(d0 + d) * BK]);
#pragma unroll
      for (int j4 = 0; j4 < BK / 4; ++j4) {
        const float4 kk = krow[j4];
        s[4 * j4] = fmaf(qd, kk.x, s[4 * j4]);
        s[4 * j4 + 1] = fmaf(qd, kk.y, s[4 * j4 + 1]);
        s[4 * j4 + 2] = fmaf(qd, kk.z, s[4 * j4 + 2]);
        s[4 * j4 + 3] = fmaf(qd, kk.w, s[4 * j4 + 3]);
      }
    }
    float tile_max = NEG_BIG;
#pragma unroll
    for (int j = 0; j < BK; ++j) {
      s[j] += __shfl_xor_sync(0xffffffffu, s[j], 1);   // the other half of the head dim
      s[j] = (k0 + j) < valid_row ? s[j] * p.scale : NEG_BIG;
      tile_max = fmaxf(tile_max, s[j]);
    }
    if (tile_max > -3.0e38f) {
      const float m_new = fmaxf(m, tile_max);
      const float corr = expf(m - m_new);
      l *= corr;
#pragma unroll
      for (int d = 0; d < DHS; ++d) acc[d] *= corr;
#pragma unroll
      for (int j = 0; j < BK; ++j) {
        const float pj = expf(s[j] - m_new);
        l += pj;
        const float4 *vrow = reinterpret_cast<const float4 *>(&Vsh[j * DH + d0]);
#pragma unroll
        for (int d4 = 0; d4 < DHS / 4; ++d4) {
          const float4 vv = vrow[d4];
          acc[4 * d4] = fmaf(pj, vv.x, acc[4 * d4]);
          acc[4 * d4 + 1] = fmaf(pj, vv.y, acc[4 * d4 + 1]);
          acc[4 * d4 + 2] = fmaf(pj, vv.z, acc[4 * d4 + 2]);
          acc[4 * d4 + 3] = fmaf(pj, vv.w, acc[4 * d4 + 3]);
        }
      }
      m = m_new;
    }
    __syncthreads();
  }

  if (live && valid_row > 0) {
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    float *o = p.out + (size_t)head * p.o_head_stride + (size_t)row * p.o_row_stride + d0;
#pragma unroll
    for (int d = 0; d < DHS; ++d) o[d] = acc[d] * inv;
  }
}

// ------------------------------------------------------------------ prefill, tensor cores
// The f16-operand route of the reference (its coopmat2 flash kernels round Q*scale, K, V and
// the softmax weights through f16 and accumulate in f32, tests/correctness/flash.rs:481-485):
// mma.sync m16n8k16 for S = (Q*scale) K^T and O = P V, online softmax in registers.
// A warp group = 4 warps x 16 query rows; K/V tiles of 64 positions arrive through cp.async into the
// group's own ring of shared-memory stages (Kt rows [d][pos], V rows [pos][d], 16-byte padded) and
// reach the B fragments with ldmatrix.trans.  f16 caches with dh = 64 only.
//
// A CTA holds NG warp groups over the SAME 64 query rows; group g walks tiles g, g + NG, ... and the
// groups' (max, sum, accumulator) triples meet through shared memory at the end, group 0 first, so the
// result does not depend on timing.  The kernel is a chain of dependent steps per query block (the
// causal block of the last 64 rows of a 512-token prompt walks 8 tiles while the first walks one), and
// each step is latency, not throughput: two groups halve the longest chain and double the warps a
// scheduler can pick from.
constexpr int FM_BQ = 64, FM_BKV = 64, FM_DH = 64, FM_PAD = 8, FM_LD = FM_BKV + FM_PAD;
constexpr int FM_TILE_HALVES = FM_DH * FM_LD;                         // one K or V tile
constexpr int FM_STAGES_TOTAL = 4;                                    // stages of a CTA, split between its groups
constexpr int FM_SMEM_BYTES = FM_STAGES_TOTAL * 2 * FM_TILE_HALVES * 2;   // 73 728 bytes of dynamic shared memory
constexpr float FM_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *smem_row) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_src) : "memory");
}

template <int NG>
__global__ void __launch_bounds__(128 * NG, 2)
flash_prefill_mma_kernel(const FlashParams p) {
  constexpr int STAGES = FM_STAGES_TOTAL / NG;               // of one group
  static_assert(STAGES >= 2, "a group needs a stage to fill while it reads another");
  static_assert(NG == 1 || NG == 2, "one named barrier per group: 1 and 2");
  extern __shared__ __align__(16) __half fm_smem[];          // per group and stage: K tile [d][pos], then V tile [pos][d]
  const uint32_t grp = threadIdx.x >> 7, tid = threadIdx.x & 127u, warp = tid >> 5, lane = tid & 31;
  __half *const grp_smem = fm_smem + (size_t)grp * STAGES * 2 * FM_TILE_HALVES;
  auto Ksh = [&](int b) { return grp_smem + (size_t)b * 2 * FM_TILE_HALVES; };
  auto Vsh = [&](int b) { return grp_smem + (size_t)b * 2 * FM_TILE_HALVES + FM_TILE_HALVES; };
  // the 128 threads of a group meet on a barrier of their own: the groups never wait for one another inside the loop
  auto group_sync = [&]() {
    if (NG == 1) __syncthreads();
    else if (grp == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
    else asm volatile("bar.sync 2, 128;" ::: "memory");
  };
  TA_CHAIN_ENTER();
  const uint32_t head = blockIdx.y;
  const uint32_t g = lane >> 2, t = lane & 3;
  const uint32_t q0 = blockIdx.x * FM_BQ;
  const uint32_t kv_head = head / p.group;
  const __half *kt = static_cast<const __half *>(p.kt) + (size_t)kv_head * FM_DH * p.t_max;
  const __half *vv = static_cast<const __half *>(p.v) + (size_t)kv_head * p.t_max * FM_DH;

  const uint32_t row_a = q0 + warp * 16 + g, row_b = row_a + 8;   // this thread's two query rows
  const uint32_t valid_a = row_a < p.t_q ? (uint32_t)min((uint64_t)p.kv_len, (uint64_t)p.pos_base + row_a + 1u) : 0u;
  const uint32_t valid_b = row_b < p.t_q ? (uint32_t)min((uint64_t)p.kv_len, (uint64_t)p.pos_base + row_b + 1u) : 0u;
  // a tile that ends at or before this bound is visible to every row of the warp: no masking there
  const uint32_t warp_min_valid = __reduce_min_sync(0xffffffffu, min(valid_a, valid_b));
  const uint32_t last_row = min(q0 + FM_BQ, p.t_q) - 1u;
  const uint32_t valid_max = (uint32_t)min((uint64_t)p.kv_len, (uint64_t)p.pos_base + last_row + 1u);
  const uint32_t num_tiles = (valid_max + FM_BKV - 1) / FM_BKV;
  // this group's tiles: grp, grp + NG, ...
  const uint32_t my_tiles = num_tiles > grp ? (num_tiles - grp + NG - 1) / NG : 0u;

  auto load_tile = [&](uint32_t tile, int buf) {
    const uint32_t k0 = tile * FM_BKV;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const uint32_t i = tid + it * 128, r = i >> 3, c8 = (i & 7u) * 8u;
      // K: row r = head dim d, 8 positions k0 + c8..; V: row r = position k0 + r, 8 dims c8..
      __half *kd = Ksh(buf) + r * FM_LD + c8;
      __half *vd = Vsh(buf) + r * FM_LD + c8;
      if (k0 + c8 + 8 <= p.t_max) cp_async16(kd, kt + (size_t)r * p.t_max + k0 + c8);
      else *reinterpret_cast<uint4 *>(kd) = make_uint4(0u, 0u, 0u, 0u);
      // rows at or beyond kv_len get probability 0: they must be zeros, not whatever the cache holds
      // there (0 x Inf or 0 x NaN from a never-written row would poison the whole output row)
      if (k0 + r < p.t_max && k0 + r < p.kv_len) cp_async16(vd, vv + (size_t)(k0 + r) * FM_DH + c8);
      else *reinterpret_cast<uint4 *>(vd) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // look-ahead of STAGES - 1 tiles; a group is committed per tile slot whether or not a tile is left,
  // so that "all but the newest STAGES - 1 groups" always means "this tile has landed"
#pragma unroll
  for (uint32_t i = 0; i < (uint32_t)STAGES - 1; ++i) {
    if (i < my_tiles) load_tile(grp + i * NG, (int)i);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }

  // Q * scale as f16 A fragments: 4 steps of 16 head dims
  uint32_t qf[4][4];
  {
    const size_t off_a = (size_t)head * p.q_head_stride + (size_t)min(row_a, p.t_q - 1) * p.q_row_stride;
    const size_t off_b = (size_t)head * p.q_head_stride + (size_t)min(row_b, p.t_q - 1) * p.q_row_stride;
    const bool la = row_a < p.t_q, lb = row_b < p.t_q;
    // two consecutive head dims of a row, from f32 or (io16) f16 storage
    auto q2 = [&](size_t off, int d, bool live) {
      if (!live) return make_float2(0.f, 0.f);
      if (p.io_f16) return __half22float2(*reinterpret_cast<const __half2 *>(reinterpret_cast<const __half *>(p.q) + off + d));
      return *reinterpret_cast<const float2 *>(p.q + off + d);
    };
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int d0 = 16 * s + 2 * t;
      const float2 a0 = q2(off_a, d0, la), b0 = q2(off_b, d0, lb), a1 = q2(off_a, d0 + 8, la), b1 = q2(off_b, d0 + 8, lb);
      qf[s][0] = pack_h2(a0.x * p.scale, a0.y * p.scale);
      qf[s][1] = pack_h2(b0.x * p.scale, b0.y * p.scale);
      qf[s][2] = pack_h2(a1.x * p.scale, a1.y * p.scale);
      qf[s][3] = pack_h2(b1.x * p.scale, b1.y * p.scale);
    }
  }

  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[j][i] = 0.0f;
  float m_a = NEG_BIG, m_b = NEG_BIG, l_a = 0.0f, l_b = 0.0f;   // l: this thread's share of the row sum

  // ldmatrix row addressing: lane -> matrix lane / 8, row lane % 8
  const uint32_t lm = lane >> 3, lr = lane & 7;

  for (uint32_t step = 0; step < my_tiles; ++step) {
    const int buf = (int)(step % STAGES);
    // the stage refilled here held the tile of the step before, whose reads ended at the barrier that closed it
    if (step + STAGES - 1 < my_tiles) load_tile(grp + (step + STAGES - 1) * NG, (int)((step + STAGES - 1) % STAGES));
    else asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 1) : "memory");
    group_sync();
    const uint32_t k0 = (grp + step * NG) * FM_BKV;

    // ---- S = (Q*scale) K^T : 8 blocks of 8 positions
    float sc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[j][i] = 0.0f;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {   // position blocks 2jp, 2jp+1
        uint32_t b[4];
        // matrices: (d 16s..+7, blk 2jp), (d 16s+8.., blk 2jp), (d 16s.., blk 2jp+1), (d 16s+8.., blk 2jp+1)
        ldmatrix_x4_trans(b, Ksh(buf) + (16 * s + (lm & 1u) * 8 + lr) * FM_LD + (2 * jp + (lm >> 1)) * 8);
        mma_f16_16816(sc[2 * jp], qf[s], b[0], b[1]);
        mma_f16_16816(sc[2 * jp + 1], qf[s], b[2], b[3]);
      }
    }
    // ---- mask (only a tile that reaches past some row's visible range), running max, probabilities
    const bool masked = k0 + FM_BKV > warp_min_valid;   // the same for the whole warp
    if (masked) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t pos = k0 + 8 * j + 2 * t;
        sc[j][0] = pos < valid_a ? sc[j][0] : NEG_BIG;
        sc[j][1] = pos + 1 < valid_a ? sc[j][1] : NEG_BIG;
        sc[j][2] = pos < valid_b ? sc[j][2] : NEG_BIG;
        sc[j][3] = pos + 1 < valid_b ? sc[j][3] : NEG_BIG;
      }
    }
    float mx_a = NEG_BIG, mx_b = NEG_BIG;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mx_a = fmaxf(mx_a, fmaxf(sc[j][0], sc[j][1]));
      mx_b = fmaxf(mx_b, fmaxf(sc[j][2], sc[j][3]));
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    // exp(x - m) as 2^(x log2e - m log2e): one fused multiply-add and one ex2 per weight (the weights
    // are rounded to f16 next, far coarser than the approximation); 1 while nothing is visible yet
    const float corr_a = ex2_approx((m_a - mn_a) * FM_LOG2E), corr_b = ex2_approx((m_b - mn_b) * FM_LOG2E);
    m_a = mn_a;
    m_b = mn_b;
    l_a *= corr_a;
    l_b *= corr_b;
    const float nml_a = -mn_a * FM_LOG2E, nml_b = -mn_b * FM_LOG2E;
    uint32_t pf[4][4];   // P as A fragments: 4 steps of 16 positions
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p0 = ex2_approx(fmaf(sc[j][0], FM_LOG2E, nml_a));
      float p1 = ex2_approx(fmaf(sc[j][1], FM_LOG2E, nml_a));
      float p2 = ex2_approx(fmaf(sc[j][2], FM_LOG2E, nml_b));
      float p3 = ex2_approx(fmaf(sc[j][3], FM_LOG2E, nml_b));
      if (masked) {   // a masked score against a row maximum that is itself "nothing visible" is not a number
        p0 = sc[j][0] > -3.0e38f ? p0 : 0.0f;
        p1 = sc[j][1] > -3.0e38f ? p1 : 0.0f;
        p2 = sc[j][2] > -3.0e38f ? p2 : 0.0f;
        p3 = sc[j][3] > -3.0e38f ? p3 : 0.0f;
      }
      l_a += p0 + p1;
      l_b += p2 + p3;
      pf[j >> 1][(j & 1) * 2] = pack_h2(p0, p1);
      pf[j >> 1][(j & 1) * 2 + 1] = pack_h2(p2, p3);
      o[j][0] *= corr_a; o[j][1] *= corr_a;
      o[j][2] *= corr_b; o[j][3] *= corr_b;
    }
    // ---- O += P V : 4 steps of 16 positions x 8 blocks of 8 head dims
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {   // head-dim blocks 2jp, 2jp+1
        uint32_t b[4];
        // matrices: (pos 16ks..+7, dblk 2jp), (pos 16ks+8.., dblk 2jp), (pos 16ks.., dblk 2jp+1), (pos 16ks+8.., 2jp+1)
        ldmatrix_x4_trans(b, Vsh(buf) + (16 * ks + (lm & 1u) * 8 + lr) * FM_LD + (2 * jp + (lm >> 1)) * 8);
        mma_f16_16816(o[2 * jp], pf[ks], b[0], b[1]);
        mma_f16_16816(o[2 * jp + 1], pf[ks], b[2], b[3]);
      }
    }
    group_sync();   // the buffer is refilled by the load issued in the next step
  }

  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

  if (NG > 1) {
    // groups 1.. hand (o, m, l) to group 0 through the stage memory, [value][thread] so that a warp's
    // accesses are consecutive; group 0 folds them in group order
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();   // every group is done with its stages
    float *xch = reinterpret_cast<float *>(fm_smem);
    constexpr int XW = 36;   // 32 accumulators, 2 maxima, 2 sums
    if (grp > 0) {
      float *mine = xch + (size_t)(grp - 1) * XW * 128 + tid;
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) mine[(j * 4 + i) * 128] = o[j][i];
      mine[32 * 128] = m_a;
      mine[33 * 128] = m_b;
      mine[34 * 128] = l_a;
      mine[35 * 128] = l_b;
    }
    __syncthreads();
    if (grp > 0) return;
#pragma unroll
    for (int og = 1; og < NG; ++og) {
      const float *theirs = xch + (size_t)(og - 1) * XW * 128 + tid;
      const float tm_a = theirs[32 * 128], tm_b = theirs[33 * 128];
      const float mn_a = fmaxf(m_a, tm_a), mn_b = fmaxf(m_b, tm_b);
      const float ca = ex2_approx((m_a - mn_a) * FM_LOG2E), cb = ex2_approx((m_b - mn_b) * FM_LOG2E);
      const float ta = ex2_approx((tm_a - mn_a) * FM_LOG2E), tb = ex2_approx((tm_b - mn_b) * FM_LOG2E);
      l_a = l_a * ca + theirs[34 * 128] * ta;
      l_b = l_b * cb + theirs[35 * 128] * tb;
      m_a = mn_a;
      m_b = mn_b;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j][0] = o[j][0] * ca + theirs[(j * 4 + 0) * 128] * ta;
        o[j][1] = o[j][1] * ca + theirs[(j * 4 + 1) * 128] * ta;
        o[j][2] = o[j][2] * cb + theirs[(j * 4 + 2) * 128] * tb;
        o[j][3] = o[j][3] * cb + theirs[(j * 4 + 3) * 128] * tb;
      }
    }
  }

  const float inv_a = l_a > 0.0f ? 1.0f / l_a : 0.0f, inv_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;
  auto store_row = [&](uint32_t row, float inv, int lo) {
    const size_t off = (size_t)head * p.o_head_stride + (size_t)row * p.o_row_stride;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float x = o[j][lo] * inv, y = o[j][lo + 1] * inv;
      if (p.io_f16) {
        *reinterpret_cast<__half2 *>(reinterpret_cast<__half *>(p.out) + off + 8 * j + 2 * t) = __floats2half2_rn(x, y);
      } else {
        *reinterpret_cast<float2 *>(p.out + off + 8 * j + 2 * t) = make_float2(x, y);
        if (p.out16)   // token-major output also as the f16 A of the projection that follows
          *reinterpret_cast<__half2 *>(static_cast<__half *>(p.out16) + (size_t)head * p.o_head_stride +
                                       (size_t)row * p.out16_row_stride + 8 * j + 2 * t) = __floats2half2_rn(x, y);
      }
    }
  };
  if (valid_a > 0) store_row(row_a, inv_a, 0);
  if (valid_b > 0) store_row(row_b, inv_b, 2);
}

// ------------------------------------------------------------------ decode
// One CTA per (chunk, kv head), 128 threads = 8 query rows x 16 lanes.  A chunk
// is walked in tiles of 64 positions whose loads are issued up front (one round trip
// of latency per tile), thread (r, c) computes the four scores j = 4c..4c+3 of
// row r, the tile's max / sum meet through xor-shuffles inside the 16-lane
// group, probabilities go through shared memory, and thread (r, c) accumulates
// the four output dims d = 4c..4c+3.  Partials [kv_heads, chunks, group, dh+2]
// (acc, m, l) go to caller scratch.  The last CTA of a kv head to finish (a
// ticket counter, reset for the next launch) weighs every chunk by exp(m_i - max m)
// and sums in chunk order, so the result does not depend on which CTA that is.
// When the slot lends its pair region the partials travel as flagged (value, flag)
// pairs instead and the CTA of chunk 0 combines (no fence, no ticket); with 16-byte
// f16 cache rows that route runs attn_decode_pairs_kernel, a warp per query row.
// All routes add in the same order and give the same bits.
constexpr int DEC_DH = 64, DEC_LANES = 16, DEC_THREADS = 128, DEC_BP = 64;

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// The combine of the flagged hand-over, run by 128 threads (row = query row, lane = one of sixteen)
// of the CTA of chunk 0: polls the pairs of every live chunk (bounded), weighs and sums them in
// chunk order, writes the kv head's output rows and advances its launch count.
__device__ __forceinline__ void attn_decode_combine_pairs(const AttnDecodeParams &p, uint4 *pair_rows, uint32_t kv_head, uint32_t row,
                                                          uint32_t lane, uint32_t kv_len, uint32_t chunk_size, uint32_t pair_flag) {
  if (row >= p.group) return;
  constexpr uint32_t ROW_V4 = (DEC_DH + 2) / 2;
  auto ld_pair = [](const uint4 *src) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
    return v;
  };
  const uint32_t live_chunks = chunk_size ? min(p.num_chunks, (kv_len + chunk_size - 1) / chunk_size) : 0u;
  const uint32_t half_mask = 0xffffu << (16u * (row & 1u));   // the sixteen lanes of this row
  const uint4 *rbase = pair_rows + (size_t)row * ROW_V4;
  constexpr size_t CSTEP = 8u * ROW_V4;
  const uint64_t t_begin = global_timer_ns();
  bool gave_up = false;
  // a pair is there when both of its flags are set.  A poll re-requests EVERY pair that is not
  // there yet before it looks at any (one L2 round trip per poll, whatever the number missing),
  // bounded at about a second.
  auto there = [&](const uint4 &v) { return v.y == pair_flag && v.w == pair_flag; };
  float num[4] = {0.f, 0.f, 0.f, 0.f}, l_total = 0.0f;
  constexpr int MAXB = ATTN_DECODE_MAX_CHUNKS / 16;
  uint4 ml[MAXB], pa[16], pb[16];   // this lane's (max, sum) pair per batch of sixteen chunks; a batch's sums
#pragma unroll
  for (int b = 0; b < MAXB; ++b) ml[b] = make_uint4(__float_as_uint(NEG_BIG), 0u, 0u, 0u);
  auto poll_batch = [&](uint32_t c0, bool with_ml) {
#pragma unroll
    for (int u = 0; u < 16; ++u) pa[u] = pb[u] = make_uint4(0u, 0u, 0u, 0u);
    uint32_t spins = 0;
    for (;;) {
      if (with_ml) {
#pragma unroll
        for (int b = 0; b < MAXB; ++b) {
          const uint32_t c = 16u * b + lane;
          if (c < live_chunks && !there(ml[b])) ml[b] = ld_pair(rbase + c * CSTEP + DEC_DH / 2);
        }
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const uint32_t c = c0 + u;
        if (c < live_chunks) {
          if (!there(pa[u])) pa[u] = ld_pair(rbase + c * CSTEP + lane * 2);
          if (!there(pb[u])) pb[u] = ld_pair(rbase + c * CSTEP + lane * 2 + 1);
        }
      }
      bool all = true;
      if (with_ml) {
#pragma unroll
        for (int b = 0; b < MAXB; ++b) all = all && (16u * b + lane >= live_chunks || there(ml[b]));
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) all = all && (c0 + u >= live_chunks || (there(pa[u]) && there(pb[u])));
      if (all) break;
      if ((++spins & 63u) == 0 && global_timer_ns() - t_begin > 1000000000ull) {
        gave_up = true;
        break;
      }
    }
  };
  poll_batch(0, true);
  float m_star = NEG_BIG, w_l[MAXB], l_l[MAXB];
#pragma unroll
  for (int b = 0; b < MAXB; ++b) m_star = fmaxf(m_star, 16u * b + lane < live_chunks ? __uint_as_float(ml[b].x) : NEG_BIG);
#pragma unroll
  for (int off = DEC_LANES / 2; off >= 1; off >>= 1) m_star = fmaxf(m_star, __shfl_xor_sync(half_mask, m_star, off, 16));
#pragma unroll
  for (int b = 0; b < MAXB; ++b) {
    w_l[b] = 16u * b + lane < live_chunks ? expf(__uint_as_float(ml[b].x) - m_star) : 0.0f;
    l_l[b] = __uint_as_float(ml[b].z);
  }
#pragma unroll
  for (int b = 0; b < MAXB; ++b) {
    if (16u * b < live_chunks) {   // the same for the sixteen lanes of the row
      if (b > 0) poll_batch(16u * b, false);
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        // past the live count: weight 0 (from the lane that holds no chunk) times the zeros of an unfetched pair
        const float w = __shfl_sync(half_mask, w_l[b], u, 16), lc = __shfl_sync(half_mask, l_l[b], u, 16);
        l_total = fmaf(lc, w, l_total);
        num[0] = fmaf(__uint_as_float(pa[u].x), w, num[0]); num[1] = fmaf(__uint_as_float(pa[u].z), w, num[1]);
        num[2] = fmaf(__uint_as_float(pb[u].x), w, num[2]); num[3] = fmaf(__uint_as_float(pb[u].z), w, num[3]);
      }
    }
  }
  if (gave_up && p.status) atomicOr(p.status, 1u);
  const float inv = l_total > 0.0f ? 1.0f / l_total : 0.0f;
  float *o = p.out + ((size_t)kv_head * p.group + row) * DEC_DH + lane * 4;
  *reinterpret_cast<float4 *>(o) = make_float4(num[0] * inv, num[1] * inv, num[2] * inv, num[3] * inv);
  if (row == 0 && lane == 0) p.pair_seq[kv_head] = pair_flag;   // the next launch on this slot tags with the next count
}

__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_kernel(const AttnDecodeParams p) {
  // f16 caches with 16-byte rows (the decode graph's case): a thread keeps ITS K values in registers
  // (row r, positions 4 lane..4 lane + 3, all 64 head dims: 64 eight-byte loads, issued before the
  // dependency wait), V rows sit in shared memory as f16, q as [d][row] and the weights as
  // [position][row], so that a warp's shared-memory reads are one or two wavefronts.  Any other
  // cache goes through f32 tiles in shared memory.  Both routes add in the same order.
  __shared__ __align__(16) float Ksh[DEC_DH * DEC_BP];   // [d][j], f32 route only
  __shared__ __align__(16) float Vsh[DEC_BP * DEC_DH];   // [j][d] f32, or (f16 route) [j][64 halves] in its first half
  __shared__ __align__(16) float Qsh[DEC_DH * 8];        // [d][row]
  __shared__ __align__(16) float Psh[DEC_BP * 8];        // [j][row]
  __shared__ uint32_t last_flag;
  const uint32_t chunk = blockIdx.x, kv_head = blockIdx.y, tid = threadIdx.x;
  const uint32_t row = tid / DEC_LANES, lane = tid % DEC_LANES;
  const bool live = row < p.group;

  // the position cell is host-written before the launch: read it ahead of the dependency wait
  uint32_t kv_len = p.kv_len + (p.pos_ptr ? *p.pos_ptr : 0u);
  if (kv_len > p.t_max || kv_len < p.kv_len) {   // a position the cache does not hold: stay inside it and report
    if (tid == 0 && chunk == 0 && kv_head == 0 && p.status) atomicOr(p.status, 8u);
    kv_len = p.t_max;
  }
  // positions per chunk, a multiple of 8 so that f16 K rows start on 16 bytes: one whole tile when the
  // grid can cover the current length that way (the fewest live chunks, each a single tile), else an
  // even split
  const uint32_t chunk_size = (uint64_t)p.num_chunks * DEC_BP >= kv_len ? (uint32_t)DEC_BP
                                                                        : ((((kv_len + p.num_chunks - 1) / p.num_chunks) + 7u) & ~7u);
  const uint32_t p0 = min(kv_len, chunk * chunk_size), p1 = min(p0 + chunk_size, kv_len);
  const size_t kt_base = (size_t)kv_head * DEC_DH * p.t_max, v_base = (size_t)kv_head * p.t_max * DEC_DH;
  const bool vec16 = p.kv_f16 && (p.t_max % 8u) == 0 &&
                     (reinterpret_cast<uintptr_t>(p.kt) & 15u) == 0 && (reinterpret_cast<uintptr_t>(p.v) & 15u) == 0;

  uint2 kreg[DEC_DH];   // f16 route: K[d][t0 + 4 lane .. + 3]
  uint4 vraw[4];        // f16 route: 64 position rows x 8 groups of 8 dims, four groups per thread
  auto load_tile = [&](uint32_t t0, uint32_t n) {
    const __half *kcol = static_cast<const __half *>(p.kt) + kt_base + t0 + lane * 4u;
    const bool k_ok = lane * 4u < n;   // a group may run past kv_len inside t_max (a multiple of 8): masked at the scores
#pragma unroll
    for (int d = 0; d < DEC_DH; ++d)
      kreg[d] = k_ok ? *reinterpret_cast<const uint2 *>(kcol + (size_t)d * p.t_max) : make_uint2(0u, 0u);
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const uint32_t i = tid + it * DEC_THREADS, j = i >> 3, dg = (i & 7u) * 8u;
      vraw[it] = make_uint4(0u, 0u, 0u, 0u);
      if (j < n)
        vraw[it] = *reinterpret_cast<const uint4 *>(static_cast<const __half *>(p.v) + v_base + (size_t)(t0 + j) * DEC_DH + dg);
    }
  };
  // The launch before this one may only have appended position kv_len - 1 (the planner
  // sets prefetch_kv when that holds): every other position is read before the wait.
  const uint32_t n_first = min((uint32_t)DEC_BP, p1 - p0);
  const bool newest_here = kv_len > 0 && kv_len - 1 >= p0 && kv_len - 1 < p0 + n_first;
  const bool early = vec16 && n_first > 0 && p.prefetch_kv;
  if (early) load_tile(p0, n_first);   // in the chunk of the newest position that one column / row is stale: re-read below
  // the launch count of this kv head was last written by the attention launch before this one on
  // the slot, which ended launches ago
  uint32_t pair_flag = 0;
  if (p.pairs) {
    pair_flag = __ldcg(p.pair_seq + kv_head) + 1u;
    if (pair_flag == 0u) pair_flag = 1u;   // zero is what untouched pairs hold
  }

  if (p.pdl) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }
  // q: group x 64 floats, one float4 per thread (requested before the late tile loads), staged as [d][row]
  float4 qv = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool q_vec = (reinterpret_cast<uintptr_t>(p.q) & 15u) == 0;
  if (q_vec) {
    if (tid * 4 < p.group * DEC_DH) qv = *reinterpret_cast<const float4 *>(p.q + (size_t)kv_head * p.group * DEC_DH + tid * 4);
  }
  if (vec16 && n_first > 0 && !early) load_tile(p0, n_first);
  if (early && newest_here) {
    // the appended position, now that its writer has finished: the K column group that holds it
    // (the threads of one lane index) and its V row, from L2 instead of a whole tile from memory
    const uint32_t jn = kv_len - 1u - p0;
    if (lane == (jn >> 2)) {
      const __half *kcol = static_cast<const __half *>(p.kt) + kt_base + p0 + lane * 4u;
#pragma unroll
      for (int d = 0; d < DEC_DH; ++d) kreg[d] = __ldcg(reinterpret_cast<const uint2 *>(kcol + (size_t)d * p.t_max));   // past L1, which may hold the line as it was
    }
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const uint32_t i = tid + it * DEC_THREADS, j = i >> 3, dg = (i & 7u) * 8u;
      if (j == jn) vraw[it] = __ldcg(reinterpret_cast<const uint4 *>(static_cast<const __half *>(p.v) + v_base + (size_t)(p0 + j) * DEC_DH + dg));
    }
  }
  if (q_vec) {
    if (tid * 4 < p.group * DEC_DH) {
      const uint32_t qr = (tid * 4) / DEC_DH, qd = (tid * 4) % DEC_DH;
      Qsh[(qd + 0) * 8 + qr] = qv.x; Qsh[(qd + 1) * 8 + qr] = qv.y;
      Qsh[(qd + 2) * 8 + qr] = qv.z; Qsh[(qd + 3) * 8 + qr] = qv.w;
    }
  } else {
    for (uint32_t i = tid; i < p.group * DEC_DH; i += DEC_THREADS) Qsh[(i % DEC_DH) * 8 + i / DEC_DH] = p.q[(size_t)kv_head * p.group * DEC_DH + i];
  }

  float m_run = NEG_BIG, l_run = 0.0f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  __half *Vh = reinterpret_cast<__half *>(Vsh);

  for (uint32_t t0 = p0; t0 < p1; t0 += DEC_BP) {
    const uint32_t n = min((uint32_t)DEC_BP, p1 - t0);
    if (vec16) {
      if (t0 != p0) load_tile(t0, n);
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const uint32_t i = tid + it * DEC_THREADS;   // row i / 8, group i % 8: 16 bytes at halves [8 i, 8 i + 8)
        *reinterpret_cast<uint4 *>(Vh + (size_t)i * 8) = vraw[it];
      }
    } else {
      for (uint32_t i = tid; i < DEC_DH * DEC_BP; i += DEC_THREADS) {
        const uint32_t d = i / DEC_BP, j = i % DEC_BP;
        Ksh[i] = j < n ? kv_load(p.kt, kt_base + (size_t)d * p.t_max + t0 + j, p.kv_f16) : 0.0f;
      }
      for (uint32_t i = tid; i < DEC_BP * DEC_DH; i += DEC_THREADS) {
        const uint32_t j = i / DEC_DH, d = i % DEC_DH;
        Vsh[i] = j < n ? kv_load(p.v, v_base + (size_t)(t0 + j) * DEC_DH + d, p.kv_f16) : 0.0f;
      }
    }
    __syncthreads();

    float s[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
      if (vec16) {
        // eight q values are requested while the eight before them are used: with K filling the
        // register file the compiler does not move these loads ahead on its own
        float qn[8], qc[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) qn[u] = Qsh[u * 8 + row];
#pragma unroll
        for (int d0 = 0; d0 < DEC_DH; d0 += 8) {
#pragma unroll
          for (int u = 0; u < 8; ++u) qc[u] = qn[u];
          if (d0 + 8 < DEC_DH) {
#pragma unroll
            for (int u = 0; u < 8; ++u) qn[u] = Qsh[(d0 + 8 + u) * 8 + row];
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const float2 k01 = __half22float2(*reinterpret_cast<const __half2 *>(&kreg[d0 + u].x));
            const float2 k23 = __half22float2(*reinterpret_cast<const __half2 *>(&kreg[d0 + u].y));
            s[0] = fmaf(qc[u], k01.x, s[0]); s[1] = fmaf(qc[u], k01.y, s[1]);
            s[2] = fmaf(qc[u], k23.x, s[2]); s[3] = fmaf(qc[u], k23.y, s[3]);
          }
        }
      } else {
#pragma unroll 16
        for (int d = 0; d < DEC_DH; ++d) {
          const float qd = Qsh[d * 8 + row];
          const float4 kk = *reinterpret_cast<const float4 *>(&Ksh[d * DEC_BP + lane * 4]);
          s[0] = fmaf(qd, kk.x, s[0]); s[1] = fmaf(qd, kk.y, s[1]);
          s[2] = fmaf(qd, kk.z, s[2]); s[3] = fmaf(qd, kk.w, s[3]);
        }
      }
    }
    float tmax = NEG_BIG;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      s[q] = (lane * 4 + q) < n ? s[q] * p.scale : NEG_BIG;
      tmax = fmaxf(tmax, s[q]);
    }
#pragma unroll
    for (int off = DEC_LANES / 2; off >= 1; off >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
    const float m_new = fmaxf(m_run, tmax);
    const float corr = expf(m_run - m_new);
    float lsum = 0.0f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float pe = (lane * 4 + q) < n ? expf(s[q] - m_new) : 0.0f;
      lsum += pe;
      Psh[(lane * 4 + q) * 8 + row] = pe;
    }
#pragma unroll
    for (int off = DEC_LANES / 2; off >= 1; off >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
    l_run = l_run * corr + lsum;
    m_run = m_new;
    __syncthreads();
    if (live) {
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[q] *= corr;
      // whole groups of eight positions with their loads issued together: rows at or past n hold
      // weight 0 and (staged from zeroed registers) value 0, so they add nothing
      for (uint32_t j0 = 0; j0 < n; j0 += 8) {
        float pj[8];
        float4 vv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          pj[u] = Psh[(j0 + u) * 8 + row];
          if (vec16) {
            const uint2 h = *reinterpret_cast<const uint2 *>(Vh + (size_t)(j0 + u) * DEC_DH + lane * 4);
            const float2 v01 = __half22float2(*reinterpret_cast<const __half2 *>(&h.x));
            const float2 v23 = __half22float2(*reinterpret_cast<const __half2 *>(&h.y));
            vv[u] = make_float4(v01.x, v01.y, v23.x, v23.y);
          } else {
            vv[u] = *reinterpret_cast<const float4 *>(&Vsh[(j0 + u) * DEC_DH + lane * 4]);
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          acc[0] = fmaf(pj[u], vv[u].x, acc[0]); acc[1] = fmaf(pj[u], vv[u].y, acc[1]);
          acc[2] = fmaf(pj[u], vv[u].z, acc[2]); acc[3] = fmaf(pj[u], vv[u].w, acc[3]);
        }
      }
    }
    __syncthreads();
  }

  const uint32_t stride = DEC_DH + 2;
  if (p.pairs) {
    // ---- flagged hand-over through the slot's pair region.  Every partial value travels as an
    // 8-byte (value, flag) pair, two pairs per 16-byte store, flag = this kv head's launch count + 1:
    // a reader knows a value is this launch's by looking at it, so no fence and no ticket lie
    // between a chunk's stores and the combine.  The CTA of chunk 0 combines: it polls (bounded)
    // the pairs themselves, lane u of a row fetching the (max, sum) of chunk u, every lane the four
    // sums of its head dims for sixteen chunks at once, adds with the arithmetic of the ticket route
    // below and advances the count.  Every CTA of the grid is resident or will be (none waits for
    // the combiner), so the poll cannot starve its producers.
    constexpr uint32_t ROW_V4 = (DEC_DH + 2) / 2;   // 33 sixteen-byte pieces per row
    uint4 *pair_rows = reinterpret_cast<uint4 *>(p.pairs) + (size_t)kv_head * p.num_chunks * 8u * ROW_V4;
    auto st_pair = [&](uint4 *dst, float a, float b) {
      asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(__float_as_uint(a)), "r"(pair_flag),
                   "r"(__float_as_uint(b)), "r"(pair_flag) : "memory");
    };
    if (live && p0 < p1) {
      uint4 *dst = pair_rows + ((size_t)chunk * 8u + row) * ROW_V4;
      st_pair(dst + lane * 2, acc[0], acc[1]);
      st_pair(dst + lane * 2 + 1, acc[2], acc[3]);
      if (lane == 0) st_pair(dst + DEC_DH / 2, m_run, l_run);
    }
    if (chunk != 0 || !live) return;
    attn_decode_combine_pairs(p, pair_rows, kv_head, row, lane, kv_len, chunk_size, pair_flag);
    return;
  }
  if (live) {
    float *dst = p.scratch + (((size_t)kv_head * p.num_chunks + chunk) * p.group + row) * stride;
    dst[lane * 4] = acc[0]; dst[lane * 4 + 1] = acc[1]; dst[lane * 4 + 2] = acc[2]; dst[lane * 4 + 3] = acc[3];
    if (lane == 0) {
      dst[DEC_DH] = m_run;
      dst[DEC_DH + 1] = l_run;
    }
  }
  // ---- the last CTA of this kv head combines (shaders/op_attn_decode_combine.comp:42-74)
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const uint32_t ticket = atomicAdd(&p.counters[kv_head], 1u);
    last_flag = ticket == p.num_chunks - 1 ? 1u : 0u;
    if (last_flag) p.counters[kv_head] = 0u;   // ready for the next launch on this stream
  }
  __syncthreads();
  if (!last_flag || !live) return;
  __threadfence();
  const float *base = p.scratch + ((size_t)kv_head * p.num_chunks * p.group + row) * stride;
  const size_t chunk_step = (size_t)p.group * stride;
  // chunks past the valid length hold nothing; partials come from other CTAs: L2 loads
  const uint32_t live_chunks = chunk_size ? min(p.num_chunks, (kv_len + chunk_size - 1) / chunk_size) : 0u;
  // the reference's combine: the maximum over the chunks, one weight exp(m_i - m*) per chunk, sums
  // in chunk order.  Sixteen chunks' partials are requested together under a fixed trip count (a
  // loop bounded by the live count keeps each load behind the arithmetic of the chunk before: one
  // L2 round trip per chunk); up to sixteen live chunks that is the only round trip.
  float m_star = NEG_BIG, l_total = 0.0f, num[4] = {0.f, 0.f, 0.f, 0.f};
  float m_c[16], l_c[16];
  float2 a_c[16], b_c[16];
  auto load_batch = [&](uint32_t c0) {
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const uint32_t i = min(c0 + u, live_chunks - 1);   // past the end: the last chunk again, weight 0 below
      m_c[u] = __ldcg(&base[i * chunk_step + DEC_DH]);
      l_c[u] = __ldcg(&base[i * chunk_step + DEC_DH + 1]);
      // rows are dh + 2 floats long: 8-byte aligned, not 16
      a_c[u] = __ldcg(reinterpret_cast<const float2 *>(&base[i * chunk_step + lane * 4]));
      b_c[u] = __ldcg(reinterpret_cast<const float2 *>(&base[i * chunk_step + lane * 4 + 2]));
    }
  };
  auto add_batch = [&](uint32_t c0) {
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const float w = c0 + u < live_chunks ? expf(m_c[u] - m_star) : 0.0f;
      l_total = fmaf(l_c[u], w, l_total);
      num[0] = fmaf(a_c[u].x, w, num[0]); num[1] = fmaf(a_c[u].y, w, num[1]);
      num[2] = fmaf(b_c[u].x, w, num[2]); num[3] = fmaf(b_c[u].y, w, num[3]);
    }
  };
  if (live_chunks > 0) {
    load_batch(0);
#pragma unroll
    for (int u = 0; u < 16; ++u) m_star = fmaxf(m_star, m_c[u]);
    for (uint32_t i = 16; i < live_chunks; ++i) m_star = fmaxf(m_star, __ldcg(&base[i * chunk_step + DEC_DH]));
    add_batch(0);
    for (uint32_t c0 = 16; c0 < live_chunks; c0 += 16) {
      load_batch(c0);
      add_batch(c0);
    }
  }
  const float inv = l_total > 0.0f ? 1.0f / l_total : 0.0f;
  float *o = p.out + ((size_t)kv_head * p.group + row) * DEC_DH + lane * 4;
  *reinterpret_cast<float4 *>(o) = make_float4(num[0] * inv, num[1] * inv, num[2] * inv, num[3] * inv);
}


// The decode graph's case as its own kernel: f16 caches with 16-byte rows and the flagged hand-over,
// 256 threads = 8 query rows x 32 lanes (a warp per row).  A lane owns TWO positions of a tile (all
// 64 head dims of K in 64 registers) and two output dims, half of what a lane of the 128-thread
// kernel above carries, so the score loop and the P V loop are half as long.  Every sum runs in
// the order of that kernel (scores over d, outputs over positions, the tile's weight sum as
// ((p0 + p1) + p2) + p3 per group of four positions and then the same tree), so the two kernels
// agree bit for bit; the combine is the same code on the first 128 threads.
constexpr int DP_THREADS = 256;

__global__ void __launch_bounds__(DP_THREADS)
attn_decode_pairs_kernel(const AttnDecodeParams p) {
  __shared__ __align__(16) __half Vh[DEC_BP * DEC_DH];   // [j][64 halves]
  __shared__ __align__(16) float Qsh[DEC_DH * 8];        // [d][row]
  __shared__ __align__(16) float Psh[DEC_BP * 8];        // [j][row]
  const uint32_t chunk = blockIdx.x, kv_head = blockIdx.y, tid = threadIdx.x;
  const uint32_t row = tid >> 5, l32 = tid & 31u, c = l32 >> 1, h = l32 & 1u;
  const bool live = row < p.group;
  const uint32_t pos_in = 4u * c + 2u * h;   // this lane's two positions inside a tile

  uint32_t kv_len = p.kv_len + (p.pos_ptr ? *p.pos_ptr : 0u);
  if (kv_len > p.t_max || kv_len < p.kv_len) {   // a position the cache does not hold: stay inside it and report
    if (tid == 0 && chunk == 0 && kv_head == 0 && p.status) atomicOr(p.status, 8u);
    kv_len = p.t_max;
  }
  const uint32_t chunk_size = (uint64_t)p.num_chunks * DEC_BP >= kv_len ? (uint32_t)DEC_BP
                                                                        : ((((kv_len + p.num_chunks - 1) / p.num_chunks) + 7u) & ~7u);
  const uint32_t p0 = min(kv_len, chunk * chunk_size), p1 = min(p0 + chunk_size, kv_len);
  const size_t kt_base = (size_t)kv_head * DEC_DH * p.t_max, v_base = (size_t)kv_head * p.t_max * DEC_DH;

  uint32_t kreg[DEC_DH];   // K[d][t0 + pos_in], K[d][t0 + pos_in + 1]
  uint4 vraw[2];           // 64 position rows x 8 groups of 8 dims, two groups per thread
  auto load_tile = [&](uint32_t t0, uint32_t n) {
    const __half *kcol = static_cast<const __half *>(p.kt) + kt_base + t0 + pos_in;
    const bool k_ok = pos_in < n;   // a pair may run past kv_len inside t_max (a multiple of 8): masked at the scores
#pragma unroll
    for (int d = 0; d < DEC_DH; ++d) kreg[d] = k_ok ? *reinterpret_cast<const uint32_t *>(kcol + (size_t)d * p.t_max) : 0u;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const uint32_t i = tid + it * DP_THREADS, j = i >> 3, dg = (i & 7u) * 8u;
      vraw[it] = make_uint4(0u, 0u, 0u, 0u);
      if (j < n) vraw[it] = *reinterpret_cast<const uint4 *>(static_cast<const __half *>(p.v) + v_base + (size_t)(t0 + j) * DEC_DH + dg);
    }
  };
  const uint32_t n_first = min((uint32_t)DEC_BP, p1 - p0);
  const bool newest_here = kv_len > 0 && kv_len - 1 >= p0 && kv_len - 1 < p0 + n_first;
  const bool early = n_first > 0 && p.prefetch_kv;
  if (early) load_tile(p0, n_first);
  uint32_t pair_flag = __ldcg(p.pair_seq + kv_head) + 1u;
  if (pair_flag == 0u) pair_flag = 1u;

  if (p.pdl) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }
  float4 qv = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool q_vec = (reinterpret_cast<uintptr_t>(p.q) & 15u) == 0;
  if (q_vec) {
    if (tid * 4 < p.group * DEC_DH) qv = *reinterpret_cast<const float4 *>(p.q + (size_t)kv_head * p.group * DEC_DH + tid * 4);
  }
  if (n_first > 0 && !early) load_tile(p0, n_first);
  if (early && newest_here) {   // the appended position: its K pair column and its V row, past L1
    const uint32_t jn = kv_len - 1u - p0;
    if ((pos_in >> 1) == (jn >> 1)) {
      const __half *kcol = static_cast<const __half *>(p.kt) + kt_base + p0 + pos_in;
#pragma unroll
      for (int d = 0; d < DEC_DH; ++d) kreg[d] = __ldcg(reinterpret_cast<const uint32_t *>(kcol + (size_t)d * p.t_max));
    }
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const uint32_t i = tid + it * DP_THREADS, j = i >> 3, dg = (i & 7u) * 8u;
      if (j == jn) vraw[it] = __ldcg(reinterpret_cast<const uint4 *>(static_cast<const __half *>(p.v) + v_base + (size_t)(p0 + j) * DEC_DH + dg));
    }
  }
  if (q_vec) {
    if (tid * 4 < p.group * DEC_DH) {
      const uint32_t qr = (tid * 4) / DEC_DH, qd = (tid * 4) % DEC_DH;
      Qsh[(qd + 0) * 8 + qr] = qv.x; Qsh[(qd + 1) * 8 + qr] = qv.y;
      Qsh[(qd + 2) * 8 + qr] = qv.z; Qsh[(qd + 3) * 8 + qr] = qv.w;
    }
  } else {
    for (uint32_t i = tid; i < p.group * DEC_DH; i += DP_THREADS) Qsh[(i % DEC_DH) * 8 + i / DEC_DH] = p.q[(size_t)kv_head * p.group * DEC_DH + i];
  }

  float m_run = NEG_BIG, l_run = 0.0f, acc[2] = {0.f, 0.f};
  for (uint32_t t0 = p0; t0 < p1; t0 += DEC_BP) {
    const uint32_t n = min((uint32_t)DEC_BP, p1 - t0);
    if (t0 != p0) load_tile(t0, n);
#pragma unroll
    for (int it = 0; it < 2; ++it) *reinterpret_cast<uint4 *>(Vh + (size_t)(tid + it * DP_THREADS) * 8) = vraw[it];
    __syncthreads();

    float s[2] = {0.f, 0.f};
    {
      float qn[8], qc[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) qn[u] = Qsh[u * 8 + row];
#pragma unroll
      for (int d0 = 0; d0 < DEC_DH; d0 += 8) {
#pragma unroll
        for (int u = 0; u < 8; ++u) qc[u] = qn[u];
        if (d0 + 8 < DEC_DH) {
#pragma unroll
          for (int u = 0; u < 8; ++u) qn[u] = Qsh[(d0 + 8 + u) * 8 + row];
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float2 k01 = __half22float2(*reinterpret_cast<const __half2 *>(&kreg[d0 + u]));
          s[0] = fmaf(qc[u], k01.x, s[0]);
          s[1] = fmaf(qc[u], k01.y, s[1]);
        }
      }
    }
    float tmax = NEG_BIG;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      s[q] = (pos_in + q) < n ? s[q] * p.scale : NEG_BIG;
      tmax = fmaxf(tmax, s[q]);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
    const float m_new = fmaxf(m_run, tmax);
    const float corr = expf(m_run - m_new);
    float pe[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      pe[q] = (pos_in + q) < n ? expf(s[q] - m_new) : 0.0f;
      Psh[(pos_in + q) * 8 + row] = pe[q];
    }
    // the weight sum of four positions as ((p0 + p1) + p2) + p3, then the tree over the groups of four
    const float pair_sum = pe[0] + pe[1];
    const float below = __shfl_xor_sync(0xffffffffu, pair_sum, 1);     // on the odd lane: p0 + p1 of its group
    float lsum = (below + pe[0]) + pe[1];                              // valid on the odd lane
    lsum = __shfl_sync(0xffffffffu, lsum, l32 | 1u);
#pragma unroll
    for (int off = 16; off >= 2; off >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
    l_run = l_run * corr + lsum;
    m_run = m_new;
    __syncthreads();
    acc[0] *= corr;
    acc[1] *= corr;
    for (uint32_t j0 = 0; j0 < n; j0 += 8) {   // rows at or past n hold weight 0 and value 0
      float pj[8];
      float2 vv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        pj[u] = Psh[(j0 + u) * 8 + row];
        vv[u] = __half22float2(*reinterpret_cast<const __half2 *>(Vh + (size_t)(j0 + u) * DEC_DH + pos_in));
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        acc[0] = fmaf(pj[u], vv[u].x, acc[0]);
        acc[1] = fmaf(pj[u], vv[u].y, acc[1]);
      }
    }
    __syncthreads();
  }

  constexpr uint32_t ROW_V4 = (DEC_DH + 2) / 2;
  uint4 *pair_rows = reinterpret_cast<uint4 *>(p.pairs) + (size_t)kv_head * p.num_chunks * 8u * ROW_V4;
  auto st_pair = [&](uint4 *dst, float a, float b) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(__float_as_uint(a)), "r"(pair_flag),
                 "r"(__float_as_uint(b)), "r"(pair_flag) : "memory");
  };
  if (live && p0 < p1) {
    uint4 *dst = pair_rows + ((size_t)chunk * 8u + row) * ROW_V4;
    st_pair(dst + l32, acc[0], acc[1]);          // dims 2 l32, 2 l32 + 1
    if (l32 == 0) st_pair(dst + DEC_DH / 2, m_run, l_run);
  }
  if (chunk != 0 || tid >= 128u) return;
  attn_decode_combine_pairs(p, pair_rows, kv_head, tid >> 4, tid & 15u, kv_len, chunk_size, pair_flag);
}

inline void launched() {
  TA_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

}  // namespace

// The tensor-core route: f16 caches, head dim 64, 16-byte-aligned rows, at least 32 query rows
// (short prefills keep f32 operands), and not pinned to the f32 kernel by the caller.
bool flash_prefill_mma_eligible(const FlashParams &p) {
  return !p.simt && p.kv_f16 && p.dh == 64 && (p.t_q >= 32 || p.io_f16) && (p.t_max % 8u) == 0 &&
         (reinterpret_cast<uintptr_t>(p.kt) & 15u) == 0 && (reinterpret_cast<uintptr_t>(p.v) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(p.q) & 7u) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 7u) == 0 &&
         (p.q_row_stride % 2u) == 0 && (p.q_head_stride % 2u) == 0 && (p.o_row_stride % 2u) == 0 &&
         (p.o_head_stride % 2u) == 0;
}

void launch_flash_prefill(const FlashParams &p, cudaStream_t stream) {
  dim3 grid((p.t_q + 63) / 64, p.heads);
  if (flash_prefill_mma_eligible(p)) {
    // two warp groups per query block unless the experiment switch asks for one
    const bool two = tunables().flash_groups != 1;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
      TA_CUDA(cudaFuncSetAttribute(flash_prefill_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, FM_SMEM_BYTES));
      TA_CUDA(cudaFuncSetAttribute(flash_prefill_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, FM_SMEM_BYTES));
      attr_set[dev & 63] = true;
    }
    if (two) launch_chained(flash_prefill_mma_kernel<2>, grid, dim3(256), (size_t)FM_SMEM_BYTES, stream, p);
    else launch_chained(flash_prefill_mma_kernel<1>, grid, dim3(128), (size_t)FM_SMEM_BYTES, stream, p);
    launched();
    return;
  }
  if (p.out16) fail("internal: the f16 mirror of an attention output was planned on a problem the tensor-core kernel does not take");
  if (p.io_f16)
    fail("run_flash_attention: f16 q/out need the tensor-core kernel (f16 caches, dh 64, T_max %% 8 == 0, "
         "even strides, 16-byte aligned caches)");
  if (p.dh == 64) flash_prefill_kernel<64><<<grid, 128, 0, stream>>>(p);
  else if (p.dh == 128) flash_prefill_kernel<128><<<grid, 128, 0, stream>>>(p);
  else fail("run_flash_attention: head dim %u is not supported (64 or 128)", p.dh);
  launched();
}

void launch_attn_decode(const AttnDecodeParams &p, cudaStream_t stream) {
  if (!p.counters) fail("run_attn_decode: internal: no ticket counters");
  if (p.kv_heads > ATTN_DECODE_MAX_KV_HEADS)
    fail("run_attn_decode: %u kv heads exceed the %u ticket counters", p.kv_heads, ATTN_DECODE_MAX_KV_HEADS);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.num_chunks, p.kv_heads, 1);
  cfg.blockDim = dim3(DEC_THREADS, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  const bool rows16 = p.kv_f16 && (p.t_max % 8u) == 0 && (reinterpret_cast<uintptr_t>(p.kt) & 15u) == 0 &&
                      (reinterpret_cast<uintptr_t>(p.v) & 15u) == 0;
  if (p.pairs && rows16 && tunables().attn_wide) {   // the decode graph's case: a warp per query row
    cfg.blockDim = dim3(DP_THREADS, 1, 1);
    TA_CUDA(cudaLaunchKernelEx(&cfg, attn_decode_pairs_kernel, p));
  } else {
    TA_CUDA(cudaLaunchKernelEx(&cfg, attn_decode_kernel, p));
  }
  launched();
}

}  // namespace ta
