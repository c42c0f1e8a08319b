// Non-GEMM model ops behind ta_softmax_rows / ta_rms_norm / ta_layer_norm /
// ta_rope / ta_copy_strided.  Semantics follow the reference shaders:
//   masked row softmax   shaders/op_softmax_f32_row.comp:30-91 (masked columns store exactly 0)
//   RMS / LayerNorm      shaders/op_rmsnorm_body.glsl:60-168 (one workgroup per row)
//   interleaved RoPE     shaders/op_rope_body.glsl:100-134 (r0 = fma(x0,c,-x1*s), r1 = fma(x0,s,x1*c))
//   3-D strided copy     shaders/op_copy_strided_body.glsl:40-98
// All are bandwidth-trivial next to the GEMMs; one block per row, fixed-order
// tree reductions so results do not depend on scheduling.
#include <cuda_fp16.h>

#include "k_umma.cuh"
#include "ta_core.hpp"

namespace ta {

namespace {

constexpr int ROW_THREADS = 256;

__device__ __forceinline__ float block_reduce(float v, bool is_max, float *sh) {
  // fixed-order: warp shuffle tree, then the first warp folds the warp results
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : v + other;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = (lane < ROW_THREADS / 32) ? sh[lane] : (is_max ? -INFINITY : 0.0f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, r, o);
    r = is_max ? fmaxf(r, other) : r + other;
  }
  return r;
}

__global__ void __launch_bounds__(ROW_THREADS)
softmax_rows_kernel(const float *__restrict__ in, float *__restrict__ out, uint32_t cols,
                    float scale, uint32_t mask_kind, uint32_t valid_or_prefix,
                    uint32_t rows_per_group) {
  __shared__ float sh[32];
  const uint32_t row = blockIdx.x;
  uint32_t valid = cols;
  if (mask_kind == 1) valid = min(valid_or_prefix, cols);
  else if (mask_kind == 2) {
    const uint64_t v = (uint64_t)valid_or_prefix + (rows_per_group ? row % rows_per_group : 0u) + 1u;
    valid = (uint32_t)min((uint64_t)cols, v);
  }
  const float *x = in + (size_t)row * cols;
  float *y = out + (size_t)row * cols;
  float mx = -INFINITY;
  for (uint32_t j = threadIdx.x; j < valid; j += ROW_THREADS) mx = fmaxf(mx, x[j] * scale);
  mx = block_reduce(mx, true, sh);
  float sum = 0.0f;
  for (uint32_t j = threadIdx.x; j < valid; j += ROW_THREADS) sum += expf(x[j] * scale - mx);
  sum = block_reduce(sum, false, sh);
  const float inv = 1.0f / sum;
  for (uint32_t j = threadIdx.x; j < cols; j += ROW_THREADS)
    y[j] = j < valid ? expf(x[j] * scale - mx) * inv : 0.0f;
}

__global__ void __launch_bounds__(ROW_THREADS)
norm_rows_kernel(const float *__restrict__ in, const float *__restrict__ w,
                 const float *__restrict__ b, float *__restrict__ out, uint32_t cols, float eps,
                 bool layer_norm, __half *__restrict__ out16, uint32_t pitch16) {
  TA_CHAIN_ENTER();
  __shared__ float sh[32];
  const float *x = in + (size_t)blockIdx.x * cols;
  float *y = out + (size_t)blockIdx.x * cols;
  float mean = 0.0f;
  if (layer_norm) {
    float s = 0.0f;
    for (uint32_t j = threadIdx.x; j < cols; j += ROW_THREADS) s += x[j];
    mean = block_reduce(s, false, sh) / (float)cols;
  }
  float ss = 0.0f;
  for (uint32_t j = threadIdx.x; j < cols; j += ROW_THREADS) {
    const float d = x[j] - mean;
    ss += d * d;
  }
  ss = block_reduce(ss, false, sh);
  const float inv = rsqrtf(ss / (float)cols + eps);
  // the row may be normalised in place: every read of x[j] happens before the write of y[j]
  __half *y16 = out16 ? out16 + (size_t)blockIdx.x * pitch16 : nullptr;
  for (uint32_t j = threadIdx.x; j < cols; j += ROW_THREADS) {
    const float v = (x[j] - mean) * inv * w[j];
    const float r = layer_norm ? v + b[j] : v;
    y[j] = r;
    if (y16) y16[j] = __float2half_rn(r);   // the f16 copy a tensor-core GEMM reading this row next takes as its A
  }
  if (y16)
    for (uint32_t j = cols + threadIdx.x; j < pitch16; j += ROW_THREADS) y16[j] = __float2half_rn(0.0f);
}

__global__ void rope_kernel(const float *__restrict__ in, const float *__restrict__ table,
                            float *__restrict__ out, uint32_t tokens, uint32_t heads,
                            uint32_t head_dim, uint32_t rot_dim, uint32_t pos_base) {
  // one thread per pair of lanes (pass-through lanes beyond rot_dim are copied as pairs too)
  const uint32_t half_dim = head_dim / 2;
  const uint64_t total = (uint64_t)tokens * heads * half_dim;
  const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const uint32_t i = (uint32_t)(idx % half_dim);
  const uint64_t vec = idx / half_dim;
  const uint32_t t = (uint32_t)(vec / heads);
  const size_t base = (size_t)vec * head_dim + 2 * i;
  const float x0 = in[base], x1 = in[base + 1];
  if (2 * i < rot_dim) {
    const float *cs = table + ((size_t)(pos_base + t) * (rot_dim / 2) + i) * 2;
    const float c = cs[0], s = cs[1];
    out[base] = fmaf(x0, c, -x1 * s);
    out[base + 1] = fmaf(x0, s, x1 * c);
  } else {
    out[base] = x0;
    out[base + 1] = x1;
  }
}

__global__ void rope_tail_kernel(const float *__restrict__ in, float *__restrict__ out,
                                 uint64_t vecs, uint32_t head_dim) {
  // odd head_dim: the last lane has no partner and passes through
  const uint64_t v = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (v < vecs) out[v * head_dim + head_dim - 1] = in[v * head_dim + head_dim - 1];
}

__device__ __forceinline__ float cvt_load(float v) { return v; }
__device__ __forceinline__ float cvt_load(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T cvt_store(float v);
template <> __device__ __forceinline__ float cvt_store<float>(float v) { return v; }
template <> __device__ __forceinline__ __half cvt_store<__half>(float v) { return __float2half_rn(v); }

struct CopyArgs {
  uint32_t extent[3], src_off, src_strides[3], dst_off, dst_strides[3];
};

template <typename TS, typename TD>
__global__ void copy_strided_kernel(const TS *__restrict__ src, TD *__restrict__ dst, CopyArgs a) {
  const uint64_t total = (uint64_t)a.extent[0] * a.extent[1] * a.extent[2];
  const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const uint32_t x = (uint32_t)(idx % a.extent[0]);
  const uint32_t y = (uint32_t)((idx / a.extent[0]) % a.extent[1]);
  const uint32_t z = (uint32_t)(idx / ((uint64_t)a.extent[0] * a.extent[1]));
  const size_t s = (size_t)a.src_off + (size_t)x * a.src_strides[0] + (size_t)y * a.src_strides[1] +
                   (size_t)z * a.src_strides[2];
  const size_t d = (size_t)a.dst_off + (size_t)x * a.dst_strides[0] + (size_t)y * a.dst_strides[1] +
                   (size_t)z * a.dst_strides[2];
  dst[d] = cvt_store<TD>(cvt_load(src[s]));
}

// out = a + beta*b (mode 0) or silu(a)*b (mode 1); out may alias either input
// (shaders/op_binary_body.glsl:60-100).
__global__ void binary_kernel(const float *a, const float *b, float *out, uint32_t n, uint32_t mode,
                              float beta) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float x = a[i], y = b[i];
  out[i] = mode == 0 ? fmaf(beta, y, x) : (x / (1.0f + expf(-x))) * y;
}

// Greedy pick over one row: the maximum, ties resolved to the LARGEST index
// (the rule of shaders/op_argmax_f32.comp:44-75).  One block of 1024 threads;
// 16-byte loads when the row is aligned, (value, index) pairs folded through
// warp shuffles and one shared-memory hop.  NaNs never win (comparisons are false).
struct ArgBest {
  float v;
  uint32_t i;
};
__device__ __forceinline__ void arg_fold(ArgBest &b, float v, uint32_t i) {
  if (v > b.v || (v == b.v && i > b.i)) {
    b.v = v;
    b.i = i;
  }
}
constexpr int ARGMAX_THREADS = 1024;
__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_kernel(const float *__restrict__ in, uint32_t n, uint32_t *result) {
  __shared__ float sval[ARGMAX_THREADS / 32];
  __shared__ uint32_t sidx[ARGMAX_THREADS / 32];
  const uint32_t tid = threadIdx.x;
  ArgBest best{-INFINITY, 0u};
  uint32_t done = 0;
  if ((reinterpret_cast<uintptr_t>(in) & 15u) == 0) {
    const uint32_t n4 = n / 4;
    const float4 *in4 = reinterpret_cast<const float4 *>(in);
    for (uint32_t q = tid; q < n4; q += ARGMAX_THREADS) {
      const float4 v = in4[q];
      arg_fold(best, v.x, 4 * q);
      arg_fold(best, v.y, 4 * q + 1);
      arg_fold(best, v.z, 4 * q + 2);
      arg_fold(best, v.w, 4 * q + 3);
    }
    done = n4 * 4;
  }
  for (uint32_t i = done + tid; i < n; i += ARGMAX_THREADS) arg_fold(best, in[i], i);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best.v, off);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, best.i, off);
    arg_fold(best, ov, oi);
  }
  if ((tid & 31u) == 0) {
    sval[tid >> 5] = best.v;
    sidx[tid >> 5] = best.i;
  }
  __syncthreads();
  if (tid < 32) {
    best.v = sval[tid];
    best.i = sidx[tid];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best.v, off);
      const uint32_t oi = __shfl_xor_sync(0xffffffffu, best.i, off);
      arg_fold(best, ov, oi);
    }
    if (tid == 0) *result = best.i;
  }
}

// Row gather by token id read on the device, id clamped to vocab-1
// (shaders/op_embed_gather.comp:60-90).  grid (ceil(embd/1024), n_tokens), four columns per
// thread.  The id list usually lives in host-mapped memory: one thread per block fetches the id
// (one PCIe read per block instead of one per warp -- 32 K reads made the 512-row prefill gather
// take 107 us) and the block shares it.
template <typename TT>
__global__ void embed_gather_kernel(const uint32_t *__restrict__ tokens, const TT *__restrict__ table,
                                    float *__restrict__ out, uint32_t embd, uint32_t vocab) {
  __shared__ uint32_t token_s;
  const uint32_t t = blockIdx.y;
  if (threadIdx.x == 0) token_s = min(tokens[t], vocab - 1u);
  __syncthreads();
  const uint32_t i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= embd) return;
  const TT *__restrict__ src = table + (size_t)token_s * embd + i;
  float *__restrict__ dst = out + (size_t)t * embd + i;
  if (i + 4 <= embd && (embd & 3u) == 0) {
    float4 v;
    if constexpr (sizeof(TT) == 2) {
      const uint2 raw = *reinterpret_cast<const uint2 *>(src);   // rows are 8-byte aligned when embd % 4 == 0
      const __half2 a = *reinterpret_cast<const __half2 *>(&raw.x), b = *reinterpret_cast<const __half2 *>(&raw.y);
      v = make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    } else {
      v = *reinterpret_cast<const float4 *>(src);
    }
    *reinterpret_cast<float4 *>(dst) = v;
  } else {
    for (uint32_t j = 0; j < 4 && i + j < embd; ++j) dst[j] = cvt_load(src[j]);
  }
}

// RoPE + strided scatter of [T, H, dh] activations (shaders/op_rope_body.glsl
// scatter variant): every element, rotated or pass-through, is written to
// dst_off + pos*pos_scale + t*s0 + h*s1 + d*s2.
template <typename TD>
__global__ void rope_scatter_kernel(const float *__restrict__ in, const float *__restrict__ table,
                                    TD *__restrict__ dst, uint32_t tokens, uint32_t heads, uint32_t head_dim,
                                    uint32_t rot_dim, uint32_t pos_base, uint32_t dst_off, uint32_t s0,
                                    uint32_t s1, uint32_t s2, uint32_t pos_scale,
                                    const uint32_t *__restrict__ pos_ptr) {
  const uint32_t half_dim = head_dim / 2;
  const uint64_t total = (uint64_t)tokens * heads * half_dim;
  const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const uint32_t i = (uint32_t)(idx % half_dim);
  const uint64_t vec = idx / half_dim;
  const uint32_t t = (uint32_t)(vec / heads), h = (uint32_t)(vec % heads);
  const uint32_t p = pos_ptr ? *pos_ptr : 0u;
  const size_t base = (size_t)vec * head_dim + 2 * i;
  float r0 = in[base], r1 = in[base + 1];
  if (2 * i < rot_dim) {
    const float *cs = table + ((size_t)(pos_base + p + t) * (rot_dim / 2) + i) * 2;
    const float x0 = r0, x1 = r1;
    r0 = fmaf(x0, cs[0], -x1 * cs[1]);
    r1 = fmaf(x0, cs[1], x1 * cs[0]);
  }
  const size_t d = (size_t)dst_off + (size_t)p * pos_scale + (size_t)t * s0 + (size_t)h * s1 + (size_t)(2 * i) * s2;
  dst[d] = cvt_store<TD>(r0);
  dst[d + s2] = cvt_store<TD>(r1);
}

// Fused wide-prefill QKV pack (ExecOp::PrefillQkvPack / run_prefill_qkv_pack of the reference,
// src/executor/elementwise/flash.rs:255-330, here with f32 activations): from one
// concatenated row [T, H*dh + 2*H_kv*dh] it writes RoPE(q) head-major [H, T, dh], RoPE(k)
// into the Kt cache [H_kv, dh, T_max] at positions pos_base + t and v into the V cache
// [H_kv, T_max, dh].  One thread per interleaved pair; the rotation is the rope kernel's.
template <typename TKV>
__global__ void prefill_qkv_pack_kernel(const float *__restrict__ qkv, const float *__restrict__ table,
                                        float *__restrict__ q, TKV *__restrict__ kt, TKV *__restrict__ v,
                                        uint32_t tokens, uint32_t heads, uint32_t kv_heads, uint32_t head_dim,
                                        uint32_t rot_dim, uint32_t pos_base, uint32_t t_max) {
  TA_CHAIN_ENTER();
  const uint32_t half_dim = head_dim / 2, all_heads = heads + 2 * kv_heads;
  const uint64_t total = (uint64_t)tokens * all_heads * half_dim;
  const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const uint32_t i = (uint32_t)(idx % half_dim);
  const uint64_t vec = idx / half_dim;
  const uint32_t t = (uint32_t)(vec / all_heads), h = (uint32_t)(vec % all_heads);
  const size_t src = (size_t)t * all_heads * head_dim + (size_t)h * head_dim + 2 * i;
  float r0 = qkv[src], r1 = qkv[src + 1];
  const bool is_v = h >= heads + kv_heads;
  if (!is_v && 2 * i < rot_dim) {
    const float *cs = table + ((size_t)(pos_base + t) * (rot_dim / 2) + i) * 2;
    const float x0 = r0, x1 = r1;
    r0 = fmaf(x0, cs[0], -x1 * cs[1]);
    r1 = fmaf(x0, cs[1], x1 * cs[0]);
  }
  if (h < heads) {
    float *dst = q + ((size_t)h * tokens + t) * head_dim + 2 * i;
    dst[0] = r0;
    dst[1] = r1;
  } else if (!is_v) {
    const uint32_t kh = h - heads;
    TKV *dst = kt + ((size_t)kh * head_dim + 2 * i) * t_max + pos_base + t;
    dst[0] = cvt_store<TKV>(r0);
    dst[t_max] = cvt_store<TKV>(r1);
  } else {
    const uint32_t kh = h - heads - kv_heads;
    TKV *dst = v + ((size_t)kh * t_max + pos_base + t) * head_dim + 2 * i;
    dst[0] = cvt_store<TKV>(r0);
    dst[1] = cvt_store<TKV>(r1);
  }
}

inline void launched() {
  TA_CUDA(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

}  // namespace

void launch_softmax_rows(const float *in, float *out, uint32_t rows, uint32_t cols, float scale,
                         uint32_t mask_kind, uint32_t valid_or_prefix, uint32_t rows_per_group,
                         cudaStream_t stream) {
  softmax_rows_kernel<<<rows, ROW_THREADS, 0, stream>>>(in, out, cols, scale, mask_kind,
                                                        valid_or_prefix, rows_per_group);
  launched();
}

void launch_rms_norm(const float *in, const float *w, float *out, uint32_t rows, uint32_t cols,
                     float eps, cudaStream_t stream, void *out16, uint32_t pitch16) {
  launch_chained(norm_rows_kernel, dim3(rows), dim3(ROW_THREADS), 0, stream, in, w, (const float *)nullptr, out, cols, eps, false,
                 static_cast<__half *>(out16), pitch16);
  launched();
}

void launch_layer_norm(const float *in, const float *w, const float *b, float *out, uint32_t rows,
                       uint32_t cols, float eps, cudaStream_t stream) {
  launch_chained(norm_rows_kernel, dim3(rows), dim3(ROW_THREADS), 0, stream, in, w, b, out, cols, eps, true,
                 (__half *)nullptr, 0u);
  launched();
}

void launch_rope(const float *in, const float *table, float *out, uint32_t tokens, uint32_t heads,
                 uint32_t head_dim, uint32_t rot_dim, uint32_t pos_base, cudaStream_t stream) {
  const uint64_t total = (uint64_t)tokens * heads * (head_dim / 2);
  rope_kernel<<<(uint32_t)((total + 255) / 256), 256, 0, stream>>>(in, table, out, tokens, heads,
                                                                   head_dim, rot_dim, pos_base);
  launched();
  if (head_dim & 1u) {
    const uint64_t vecs = (uint64_t)tokens * heads;
    rope_tail_kernel<<<(uint32_t)((vecs + 255) / 256), 256, 0, stream>>>(in, out, vecs, head_dim);
    launched();
  }
}

void launch_copy_strided(const void *src, bool src_f16, void *dst, bool dst_f16, const uint32_t extent[3],
                         uint32_t src_off, const uint32_t src_strides[3], uint32_t dst_off,
                         const uint32_t dst_strides[3], cudaStream_t stream) {
  CopyArgs a;
  for (int i = 0; i < 3; ++i) {
    a.extent[i] = extent[i];
    a.src_strides[i] = src_strides[i];
    a.dst_strides[i] = dst_strides[i];
  }
  a.src_off = src_off;
  a.dst_off = dst_off;
  const uint64_t total = (uint64_t)extent[0] * extent[1] * extent[2];
  const uint32_t blocks = (uint32_t)((total + 255) / 256);
  if (!src_f16 && !dst_f16)
    copy_strided_kernel<<<blocks, 256, 0, stream>>>((const float *)src, (float *)dst, a);
  else if (!src_f16 && dst_f16)
    copy_strided_kernel<<<blocks, 256, 0, stream>>>((const float *)src, (__half *)dst, a);
  else if (src_f16 && dst_f16)
    copy_strided_kernel<<<blocks, 256, 0, stream>>>((const __half *)src, (__half *)dst, a);
  else
    copy_strided_kernel<<<blocks, 256, 0, stream>>>((const __half *)src, (float *)dst, a);
  launched();
}

void launch_binary(const float *a, const float *b, float *out, uint32_t n, uint32_t mode, float beta,
                   cudaStream_t stream) {
  binary_kernel<<<(n + 255) / 256, 256, 0, stream>>>(a, b, out, n, mode, beta);
  launched();
}

void launch_argmax(const float *in, uint32_t n, uint32_t *result, cudaStream_t stream) {
  argmax_kernel<<<1, ARGMAX_THREADS, 0, stream>>>(in, n, result);
  launched();
}

void launch_embed_gather(const uint32_t *tokens, uint32_t n_tokens, const void *table, bool table_f16,
                         float *out, uint32_t embd, uint32_t vocab, cudaStream_t stream) {
  dim3 grid((embd + 1023) / 1024, n_tokens);
  if (table_f16) embed_gather_kernel<<<grid, 256, 0, stream>>>(tokens, (const __half *)table, out, embd, vocab);
  else embed_gather_kernel<<<grid, 256, 0, stream>>>(tokens, (const float *)table, out, embd, vocab);
  launched();
}

void launch_rope_scatter(const float *in, const float *table, void *dst, bool dst_f16, uint32_t tokens,
                         uint32_t heads, uint32_t head_dim, uint32_t rot_dim, uint32_t pos_base,
                         uint32_t dst_off, const uint32_t strides[3], uint32_t pos_scale,
                         const uint32_t *pos_ptr, cudaStream_t stream) {
  const uint64_t total = (uint64_t)tokens * heads * (head_dim / 2);
  const uint32_t blocks = (uint32_t)((total + 255) / 256);
  if (dst_f16)
    rope_scatter_kernel<<<blocks, 256, 0, stream>>>(in, table, (__half *)dst, tokens, heads, head_dim, rot_dim,
                                                    pos_base, dst_off, strides[0], strides[1], strides[2],
                                                    pos_scale, pos_ptr);
  else
    rope_scatter_kernel<<<blocks, 256, 0, stream>>>(in, table, (float *)dst, tokens, heads, head_dim, rot_dim,
                                                    pos_base, dst_off, strides[0], strides[1], strides[2],
                                                    pos_scale, pos_ptr);
  launched();
}

void launch_prefill_qkv_pack(const float *qkv, const float *table, float *q, void *kt, void *v, bool kv_f16,
                             uint32_t tokens, uint32_t heads, uint32_t kv_heads, uint32_t head_dim,
                             uint32_t rot_dim, uint32_t pos_base, uint32_t t_max, cudaStream_t stream) {
  const uint64_t total = (uint64_t)tokens * (heads + 2 * kv_heads) * (head_dim / 2);
  const uint32_t blocks = (uint32_t)((total + 255) / 256);
  if (kv_f16)
    launch_chained(prefill_qkv_pack_kernel<__half>, dim3(blocks), dim3(256), 0, stream, qkv, table, q, (__half *)kt, (__half *)v,
                   tokens, heads, kv_heads, head_dim, rot_dim, pos_base, t_max);
  else
    launch_chained(prefill_qkv_pack_kernel<float>, dim3(blocks), dim3(256), 0, stream, qkv, table, q, (float *)kt, (float *)v,
                   tokens, heads, kv_heads, head_dim, rot_dim, pos_base, t_max);
  launched();
}

// Self-test of the bounded-wait machinery every tensor-core kernel here relies on: one warp waits,
// through the same helper and status word those kernels use, on a barrier that nothing ever
// completes.  After `limit_ns` the wait gives up, the kernel raises status bit 0 and returns
// normally, so the host call fails with the bounded-wait message and the context stays usable.
// Nothing faults, traps or spins without limit.
__global__ void bounded_wait_probe_kernel(uint32_t *status, uint32_t limit_ns) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    umma::mbar_init(umma::smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const bool ok = umma::mbar_wait(umma::smem_u32(&bar), 0, &abort_flag, 64, limit_ns);
  __syncthreads();
  if (!ok && threadIdx.x == 0) atomicOr(status, 1u);
}

void launch_bounded_wait_probe(uint32_t *status, uint32_t limit_ns, cudaStream_t stream) {
  bounded_wait_probe_kernel<<<1, 32, 0, stream>>>(status, limit_ns);
  launched();
}

}  // namespace ta
