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
// attn_decode_stage1_kernel / attn_decode_combine_kernel: split-K decode
// attention (shaders/attention_decode_kernel.glsl:89-170 and
// shaders/op_attn_decode_combine.comp:42-74): one CTA per (chunk, kv head), 8 q
// rows x 16 lanes, lanes stride the chunk's positions with private online
// softmax state, a xor-shuffle butterfly merges the 16 lane states exactly, and
// partials [kv_heads, chunks, group, dh + 2] go to caller scratch.  The combine
// rescales every chunk to the global max and sums in chunk order.  The valid
// length may come from a host-visible cell (kv_len + *pos), read on the device,
// so a captured graph serves every position.
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
      Vsh[i] = pos < p.t_max ? kv_load(p.v, v_base + (size_t)pos * DH + d, p.kv_f16) : 0.0f;
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

// ------------------------------------------------------------------ decode, stage 1
constexpr int DEC_DH = 64, DEC_LANES = 16, DEC_THREADS = 128;

__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_stage1_kernel(const AttnDecodeParams p) {
  __shared__ float Qsh[8 * DEC_DH];
  const uint32_t chunk = blockIdx.x, kv_head = blockIdx.y, tid = threadIdx.x;
  const uint32_t row = tid / DEC_LANES, lane = tid % DEC_LANES;
  const bool live = row < p.group;
  for (uint32_t i = tid; i < p.group * DEC_DH; i += DEC_THREADS) Qsh[i] = p.q[(size_t)kv_head * p.group * DEC_DH + i];
  __syncthreads();

  const uint32_t kv_len = p.kv_len + (p.pos_ptr ? *p.pos_ptr : 0u);
  const uint32_t chunk_size = (kv_len + p.num_chunks - 1) / p.num_chunks;
  const uint32_t p0 = min(kv_len, chunk * chunk_size), p1 = min(p0 + chunk_size, kv_len);
  const size_t kt_base = (size_t)kv_head * DEC_DH * p.t_max, v_base = (size_t)kv_head * p.t_max * DEC_DH;

  float m = NEG_BIG, l = 0.0f, acc[DEC_DH];
#pragma unroll
  for (int d = 0; d < DEC_DH; ++d) acc[d] = 0.0f;

  if (live) {
    const float *qr = &Qsh[row * DEC_DH];
    for (uint32_t pos = p0 + lane; pos < p1; pos += DEC_LANES) {
      float s = 0.0f;
      if (p.kv_f16) {
        const __half *kt = static_cast<const __half *>(p.kt) + kt_base + pos;
#pragma unroll 16
        for (int d = 0; d < DEC_DH; ++d) s = fmaf(qr[d], __half2float(kt[(size_t)d * p.t_max]), s);
      } else {
        const float *kt = static_cast<const float *>(p.kt) + kt_base + pos;
#pragma unroll 16
        for (int d = 0; d < DEC_DH; ++d) s = fmaf(qr[d], kt[(size_t)d * p.t_max], s);
      }
      s *= p.scale;
      const float m_new = fmaxf(m, s);
      const float corr = expf(m - m_new), pe = expf(s - m_new);
      l = l * corr + pe;
      if (p.kv_f16) {
        const uint4 *vv = reinterpret_cast<const uint4 *>(static_cast<const __half *>(p.v) + v_base + (size_t)pos * DEC_DH);
#pragma unroll
        for (int d8 = 0; d8 < DEC_DH / 8; ++d8) {
          const uint4 raw = vv[d8];
          const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = __half22float2(h[q]);
            acc[d8 * 8 + 2 * q] = fmaf(pe, f.x, acc[d8 * 8 + 2 * q] * corr);
            acc[d8 * 8 + 2 * q + 1] = fmaf(pe, f.y, acc[d8 * 8 + 2 * q + 1] * corr);
          }
        }
      } else {
        const float4 *vv = reinterpret_cast<const float4 *>(static_cast<const float *>(p.v) + v_base + (size_t)pos * DEC_DH);
#pragma unroll
        for (int d4 = 0; d4 < DEC_DH / 4; ++d4) {
          const float4 f = vv[d4];
          acc[4 * d4] = fmaf(pe, f.x, acc[4 * d4] * corr);
          acc[4 * d4 + 1] = fmaf(pe, f.y, acc[4 * d4 + 1] * corr);
          acc[4 * d4 + 2] = fmaf(pe, f.z, acc[4 * d4 + 2] * corr);
          acc[4 * d4 + 3] = fmaf(pe, f.w, acc[4 * d4 + 3] * corr);
        }
      }
      m = m_new;
    }
  }
  // exact butterfly merge of the 16 lane states of each row (xor 8, 4, 2, 1 stays inside the group)
#pragma unroll
  for (int off = DEC_LANES / 2; off >= 1; off >>= 1) {
    const float m_o = __shfl_xor_sync(0xffffffffu, m, off);
    const float l_o = __shfl_xor_sync(0xffffffffu, l, off);
    const float m_new = fmaxf(m, m_o);
    const float c_self = expf(m - m_new), c_other = expf(m_o - m_new);
    l = l * c_self + l_o * c_other;
#pragma unroll
    for (int d = 0; d < DEC_DH; ++d) {
      const float a_o = __shfl_xor_sync(0xffffffffu, acc[d], off);
      acc[d] = acc[d] * c_self + a_o * c_other;
    }
    m = m_new;
  }
  if (live) {
    float *dst = p.scratch + (((size_t)kv_head * p.num_chunks + chunk) * p.group + row) * (DEC_DH + 2);
#pragma unroll
    for (int d = 0; d < DEC_DH; ++d)
      if ((d % DEC_LANES) == (int)lane) dst[d] = acc[d];
    if (lane == 0) {
      dst[DEC_DH] = m;
      dst[DEC_DH + 1] = l;
    }
  }
}

// ------------------------------------------------------------------ decode, combine
__global__ void __launch_bounds__(64)
attn_decode_combine_kernel(const AttnDecodeParams p) {
  const uint32_t row_id = blockIdx.x, tid = threadIdx.x;
  const uint32_t kv_head = row_id / p.group, row = row_id % p.group;
  const uint32_t stride = DEC_DH + 2;
  const float *base = p.scratch + ((size_t)kv_head * p.num_chunks * p.group + row) * stride;
  const size_t chunk_step = (size_t)p.group * stride;
  float m_star = NEG_BIG;
  for (uint32_t i = 0; i < p.num_chunks; ++i) m_star = fmaxf(m_star, base[i * chunk_step + DEC_DH]);
  float w[32], l_total = 0.0f;
  for (uint32_t i = 0; i < p.num_chunks; ++i) {
    w[i] = expf(base[i * chunk_step + DEC_DH] - m_star);
    l_total = fmaf(base[i * chunk_step + DEC_DH + 1], w[i], l_total);
  }
  const float inv = l_total > 0.0f ? 1.0f / l_total : 0.0f;
  for (uint32_t d = tid; d < DEC_DH; d += 64) {
    float num = 0.0f;
    for (uint32_t i = 0; i < p.num_chunks; ++i) num = fmaf(base[i * chunk_step + d], w[i], num);
    p.out[(size_t)row_id * DEC_DH + d] = num * inv;
  }
}

inline void launched() {
  TA_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

}  // namespace

void launch_flash_prefill(const FlashParams &p, cudaStream_t stream) {
  dim3 grid((p.t_q + 63) / 64, p.heads);
  if (p.dh == 64) flash_prefill_kernel<64><<<grid, 128, 0, stream>>>(p);
  else if (p.dh == 128) flash_prefill_kernel<128><<<grid, 128, 0, stream>>>(p);
  else fail("run_flash_attention: head dim %u is not supported (64 or 128)", p.dh);
  launched();
}

void launch_attn_decode(const AttnDecodeParams &p, cudaStream_t stream) {
  attn_decode_stage1_kernel<<<dim3(p.num_chunks, p.kv_heads), DEC_THREADS, 0, stream>>>(p);
  launched();
  attn_decode_combine_kernel<<<p.kv_heads * p.group, 64, 0, stream>>>(p);
  launched();
}

}  // namespace ta
