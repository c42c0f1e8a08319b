/*
 * tensor_ash.h -- C ABI of the B200-native tensor-ash GEMM path.
 *
 * PART 1 restates, declaration for declaration, the C interface of the
 * reference project (its include/tensor_ash.h, lines cited per item as
 * "ref h:LINE"; the Rust implementation it binds is cited as "ref capi/...").
 * A program compiled against the reference header links against this library
 * unchanged: same type names, field order, enum values, function signatures,
 * status convention (0 / -1, pointer / NULL, message in ta_last_error()).
 *
 * PART 2 adds entry points for hot-path functions the reference exposes only
 * through its Rust API (split-K2, packed / normed-A / fused-store ops,
 * flash and decode attention, mixed op graphs, position/token cells).  They
 * are additive: nothing in PART 1 changes shape.
 *
 * Every function clears the calling thread's error string on entry.  Handles
 * are heap objects; destroying NULL is a no-op.  A tensor handed to an
 * executor must come from the executor's own context.
 */
#ifndef TENSOR_ASH_H
#define TENSOR_ASH_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ===================================================================== */
/* PART 1 -- the reference C ABI                                         */
/* ===================================================================== */

/* Opaque handles (ref h:11-14; ref capi/src/handles.rs:6-44). */
typedef struct ta_context ta_context;
typedef struct ta_executor ta_executor;
typedef struct ta_tensor ta_tensor;
typedef struct ta_prepared ta_prepared;

/* Result of one submission (ref h:16-22; ref capi/src/api/matmul.rs:86-102).
 * gpu_time_ns is device time between two events on the launch stream;
 * tflops is NaN when has_gpu_time is 0 or the time is 0. */
typedef struct ta_run_stats {
  uint32_t has_gpu_time;
  uint64_t gpu_time_ns;
  size_t n_calls;
  uint64_t total_flops;
  double tflops;
} ta_run_stats;

/* C = alpha * A @ B (+ C when accumulate != 0)  (ref h:24-30). */
typedef struct ta_matmul_call {
  const ta_tensor *a;
  const ta_tensor *b;
  const ta_tensor *c;
  float alpha;
  uint32_t accumulate;
} ta_matmul_call;

/* ta_epilogue.activation (ref h:32-38). */
enum {
  TA_ACTIVATION_NONE = 0,
  TA_ACTIVATION_RELU = 1,
  TA_ACTIVATION_SILU = 2, /* x / (1 + exp(-x)) */
  TA_ACTIVATION_GELU = 3  /* 0.5 x (1 + tanh(k0 (x + 0.044715 x^3))) */
};

/* ta_epilogue.binary_kind (ref h:40-45). */
enum {
  TA_BINARY_NONE = 0,
  TA_BINARY_ADD_SCALED = 1, /* out = act + beta * D */
  TA_BINARY_MUL = 2         /* out = act * D        */
};

/* Fused epilogue, applied on the accumulator drain in this order:
 * alpha*acc (+C_old) -> +bias -> activation -> binary with D  (ref h:47-59).
 * All-zero means none.  bias is [N] or [B, N]; d is non-NULL iff
 * binary_kind != 0 and has exactly C's shape. */
typedef struct ta_epilogue {
  const ta_tensor *bias;
  uint32_t activation;
  uint32_t binary_kind;
  const ta_tensor *d;
  float beta;
} ta_epilogue;

/* One GEMM with its epilogue (ref h:61-65). */
typedef struct ta_matmul_op {
  ta_matmul_call call;
  ta_epilogue epilogue;
} ta_matmul_op;

/* ta_softmax_rows mask_kind (ref h:67-76). */
enum {
  TA_SOFTMAX_MASK_FULL = 0,
  TA_SOFTMAX_MASK_PREFIX = 1, /* columns >= valid_or_prefix store 0 */
  TA_SOFTMAX_MASK_CAUSAL = 2  /* row i sees valid_or_prefix + (i % rows_per_group) + 1 columns */
};

/* Rotary geometry (ref h:78-88): rot_dim even, 2 <= rot_dim <= head_dim. */
typedef struct ta_rope_desc {
  uint32_t heads;
  uint32_t head_dim;
  uint32_t rot_dim;
  uint32_t pos_base;
} ta_rope_desc;

/* 3-D strided copy, strides and offsets in elements (ref h:90-98). */
typedef struct ta_copy_desc {
  uint32_t extent[3];
  uint32_t src_offset;
  uint32_t src_strides[3];
  uint32_t dst_offset;
  uint32_t dst_strides[3];
} ta_copy_desc;

/* Route report (ref h:100-108).  kernel is interned for the process lifetime. */
typedef struct ta_dispatch_info {
  const char *kernel;
  uint32_t tile[3];
  uint32_t has_split_k2;
  uint32_t split_k2_splits;
} ta_dispatch_info;

/* ref h:110-111; ref capi/src/api/lifecycle.rs:11-21.  Version "2.0.0". */
const char *ta_version(void);
const char *ta_last_error(void);

/* ref h:113-116.  device_preference: NULL/"auto", or "index:N" for CUDA
 * device N (the reference's adapter-kind names are accepted and mean auto). */
ta_context *ta_context_create(uint32_t enable_validation, const char *device_preference);
void ta_context_destroy(ta_context *ctx);

/* ref h:118-120: 0 for NULL, 1 on every CUDA device this library runs on. */
uint32_t ta_context_supports_f16(const ta_context *ctx);
uint32_t ta_context_supports_bda(const ta_context *ctx);

/* ref h:122-135; ref capi/src/api/lifecycle.rs:60-127.  n_slots = concurrent
 * submissions (one CUDA stream each); kernel_selection NULL/"auto" or any
 * registry name / alias (ML_KERNEL syntax). */
ta_executor *ta_executor_create(const ta_context *ctx, size_t n_slots,
                                uint32_t max_calls_per_submit, const char *kernel_selection);
ta_executor *ta_executor_create_v2(const ta_context *ctx, size_t n_slots,
                                   uint32_t max_calls_per_submit, const char *kernel_selection,
                                   uint32_t tune);
void ta_executor_destroy(ta_executor *exec);

/* ref h:137-153; ref capi/src/api/tensor.rs.  rank >= 1, every dim > 0;
 * contents uninitialised.  f16 tensors keep the float host API. */
ta_tensor *ta_tensor_create(const ta_context *ctx, const uint32_t *shape, size_t rank);
ta_tensor *ta_tensor_create_on_executor(const ta_executor *exec, const uint32_t *shape,
                                        size_t rank);
ta_tensor *ta_tensor_create_f16(const ta_context *ctx, const uint32_t *shape, size_t rank);
ta_tensor *ta_tensor_create_f16_on_executor(const ta_executor *exec, const uint32_t *shape,
                                            size_t rank);
void ta_tensor_destroy(ta_tensor *tensor);
uint64_t ta_tensor_len(const ta_tensor *tensor);        /* elements; 0 for NULL */
uint64_t ta_tensor_size_bytes(const ta_tensor *tensor); /* f16 rounded up to 16 B */
uint32_t ta_tensor_is_f16(const ta_tensor *tensor);

/* ref h:155-158; ref src/executor/transfer.rs:21-84.  Host side is float;
 * f16 tensors round to nearest-even on upload and widen on download.
 * len may be below capacity; above it the call fails. */
int ta_upload(const ta_executor *exec, const ta_tensor *dst, const float *src, size_t len);
int ta_download(const ta_executor *exec, const ta_tensor *src, float *dst, size_t len);

/* ref h:160-164; ref src/executor/dispatch.rs:31-85. */
int ta_matmul(const ta_executor *exec, const ta_tensor *a, const ta_tensor *b, const ta_tensor *c,
              float alpha, uint32_t accumulate, ta_run_stats *stats);
int ta_matmul_batch(const ta_executor *exec, const ta_matmul_call *calls, size_t n_calls,
                    ta_run_stats *stats);

/* Host-resident batched matmul: C[b] = epilogue(alpha * A[b] @ B) with A, D, bias and C in HOST
 * memory.  One call replaces the reference's ta_upload x3 + ta_run_ops + ta_download sequence
 * (ref src/executor/transfer.rs:21-84, dispatch.rs:87-188): the planes are cut into chunks and the
 * host->device copies of chunk i+1, the GEMM of chunk i and the device->host copy of chunk i-1
 * run at the same time on three streams, so a PCIe-bound call costs about max(bytes in, bytes out)
 * instead of their sum plus the compute.  Every chunk runs the kernel the tensor path would pick for it, so
 * results are bit-identical to that path applied chunk by chunk.  For the
 * copies to overlap the host buffers must be page-locked (ta_pinned_alloc, or memory the caller
 * pinned); pageable memory works but serialises.  One such call at a time per executor; others
 * wait.  stats->gpu_time_ns spans the first upload to the last download. */
typedef struct ta_host_batched_matmul {
  uint32_t batch, m, n, k;
  const float *a;          /* host [batch, M, K] */
  const ta_tensor *b;      /* device [K, N] f32 or f16, shared by all planes; NULL when b_host is set */
  const float *b_host;     /* host [K, N] f32, uploaded once per call; NULL when b is set */
  float *c;                /* host [batch, M, N], written */
  const float *bias;       /* host [N] (bias_per_batch 0) or [batch, N] (1); NULL: none */
  uint32_t bias_per_batch;
  const float *d;          /* host [batch, M, N] operand of the binary stage; NULL iff binary is NONE */
  uint32_t activation;     /* ta_activation */
  uint32_t binary;         /* ta_binary */
  float alpha, beta;
  uint32_t chunk_batch;    /* planes per pipeline stage; 0: the library chooses (about batch / 16) */
} ta_host_batched_matmul;
int ta_run_matmul_host_batched(const ta_executor *exec, const ta_host_batched_matmul *desc,
                               ta_run_stats *stats);

/* Page-locked host memory for the call above (cudaHostAlloc / cudaFreeHost); NULL on failure. */
void *ta_pinned_alloc(size_t bytes);
void ta_pinned_free(void *ptr);

/* ref h:166-175; ref src/executor/dispatch.rs:87-188.  ta_run_ops: independent
 * ops, one submission.  ta_run_op_graph: later ops may read earlier outputs. */
int ta_run_ops(const ta_executor *exec, const ta_matmul_op *ops, size_t n_ops,
               ta_run_stats *stats);
int ta_run_op_graph(const ta_executor *exec, const ta_matmul_op *ops, size_t n_ops,
                    ta_run_stats *stats);

/* Model ops (ref h:177-209; ref capi/src/api/elementwise.rs).  Operands f32.
 * In place is allowed except for ta_copy_strided (src != dst). */
int ta_softmax_rows(const ta_executor *exec, const ta_tensor *input, const ta_tensor *output,
                    float scale, uint32_t mask_kind, uint32_t valid_or_prefix,
                    uint32_t rows_per_group, ta_run_stats *stats);
int ta_rms_norm(const ta_executor *exec, const ta_tensor *input, const ta_tensor *weight,
                const ta_tensor *output, float eps, ta_run_stats *stats);
int ta_layer_norm(const ta_executor *exec, const ta_tensor *input, const ta_tensor *weight,
                  const ta_tensor *bias, const ta_tensor *output, float eps, ta_run_stats *stats);
int ta_rope(const ta_executor *exec, const ta_tensor *input, const ta_tensor *table,
            const ta_tensor *output, const ta_rope_desc *desc, ta_run_stats *stats);
int ta_copy_strided(const ta_executor *exec, const ta_tensor *src, const ta_tensor *dst,
                    const ta_copy_desc *desc, ta_run_stats *stats);

/* Prepared replay (ref h:211-233; ref src/executor/prepared.rs:46-353).  The
 * op batch is validated, routed and captured once (a CUDA graph) and replayed
 * per call.  The executor and every referenced tensor must outlive the handle;
 * one submission in flight per handle; destroy waits for in-flight work. */
ta_prepared *ta_prepared_create(const ta_executor *exec, const ta_matmul_op *ops, size_t n_ops,
                                uint32_t as_graph);
int ta_prepared_run(ta_prepared *prepared, ta_run_stats *stats);
int ta_prepared_submit(ta_prepared *prepared);
int ta_prepared_wait(ta_prepared *prepared, ta_run_stats *stats);
void ta_prepared_destroy(ta_prepared *prepared);

/* ref h:235-244; ref capi/src/api/diagnostics.rs. */
int ta_dispatch_info_for(const ta_executor *exec, uint32_t batch, uint32_t m, uint32_t n,
                         uint32_t k, uint32_t b_f16, ta_dispatch_info *out);
int ta_tune_shape(const ta_executor *exec, uint32_t batch, uint32_t m, uint32_t n, uint32_t k);

/* ===================================================================== */
/* PART 2 -- additive entry points for the rest of the hot path          */
/* ===================================================================== */

/* Deterministic two-stage split-K: partial planes to executor scratch, then a
 * fixed-order plane sum; no atomics, run-to-run bit-identical.  Replaces
 * Executor::run_matmuls_split_k2 (ref src/executor/reduction.rs:21-70).
 * splits == 0 picks the default (ref src/executor/splitk2.rs:94-122); splits
 * <= 1 after that runs the plain route; accumulate is rejected. */
int ta_matmul_split_k2(const ta_executor *exec, const ta_matmul_call *calls, size_t n_calls,
                       uint32_t splits, ta_run_stats *stats);

/* Split-K2 for callers that must not allocate.  No counterpart in the reference.
 *
 * Some callers cannot call cudaMalloc when they need a GEMM: code running
 * inside a memory-pool or framework allocator callback, a real-time or
 * fault-handling path where the allocator's device-wide synchronisation is not
 * allowed, or a process whose device memory was budgeted completely at start-up.
 * ta_matmul_split_k2 grows its executor's scratch with cudaMalloc on first use;
 * this entry point instead keeps the partial planes in a fixed 4 MiB array
 * inside the library's device image (present on every GPU that loads the
 * library, until the process exits) and calls no cudaMalloc, cudaFree or any
 * other allocating routine.
 *
 * C[M,N] = alpha * A[M,K] @ B[K,N], row-major f32, one matrix per call, on the
 * SIMT stage-1 kernel (one sequential fma chain per output and split) and the
 * plane-order reduce: bit-identical to ta_matmul_split_k2 on an executor whose
 * kernel selection names that stage 1 ("split_k2_m64n64" / "split_k2_m128n128";
 * an "auto" executor may take its tensor-core stage 1, equal within rounding).
 * a, b, c are device pointers on the CURRENT CUDA device; the caller owns them.
 * Limits: splits >= 2, splits <= K, splits * M * N <=
 * TA_SPLIT_K2_NOALLOC_MAX_FLOATS; anything larger is rejected with -1 and a
 * message.  The call enqueues on `stream` (NULL = default stream) and then
 * synchronises that stream: it returns after the two kernels have finished.
 *
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress) and, if nothing of the library ran on that device
 * before, pays the CUDA runtime's lazy load of the library's device code, which
 * may reserve device memory of its own; make that first call at start-up.
 * Later calls allocate nothing (cudaMemGetInfo reads the same before and
 * after them).
 * Every call uses the same array and leaves its partials there: nothing needs
 * clearing between calls (each plane element is stored before it is read), but
 * two calls that overlap on the GPU, from any thread or stream, race. */
#define TA_SPLIT_K2_NOALLOC_MAX_FLOATS (1u << 20)
int ta_split_k2_noalloc(const float *a, const float *b, float *c, uint32_t m, uint32_t n,
                        uint32_t k, uint32_t splits, float alpha, void *stream);

/* ta_store_desc.kind: fused store of an M == 1 f16-weight GEMV
 * (ref src/matmul/api.rs:120-250, MatmulStore / MatmulStoreDesc). */
enum {
  TA_STORE_NONE = 0,
  TA_STORE_ROPE = 1,        /* rotate pairs, write to C */
  TA_STORE_SCATTER = 2,     /* write to dst at pos*pos_scale + head*stride_head + d*stride_dim */
  TA_STORE_ROPE_SCATTER = 3 /* rotate, then scatter */
};

typedef struct ta_pos_cell ta_pos_cell; /* 4-byte host-visible cell, see ta_pos_cell_create */

typedef struct ta_store_desc {
  uint32_t kind;
  uint32_t head_dim;
  uint32_t pos_base;    /* position when pos_cell is NULL */
  uint32_t pos_scale;   /* elements per position in dst */
  uint32_t stride_head; /* elements between heads in dst */
  uint32_t stride_dim;  /* elements between lanes of a head in dst */
  const ta_tensor *table; /* rope (cos, sin) table [T_max, head_dim/2, 2]; kinds 1 and 3 */
  const ta_tensor *dst;   /* scatter destination (f32 or f16); kinds 2 and 3 */
  const ta_pos_cell *pos_cell; /* optional: position = pos_base + *cell, read on the device at run time */
} ta_store_desc;

/* ta_matmul_op plus the fields the reference keeps Rust-only
 * (ref capi/src/api/ops.rs:63-68 sets them to "none"):
 *   packed_b      B is [N/tile][K][tile] f16 (ref src/matmul/api.rs:317-344);
 *   normed_weight fused RMSNorm of A: a'[k] = a[k] * rsqrt(mean(a^2)+eps) * w[k]
 *                 (ref src/matmul/resolution.rs:217-247);
 *   store         fused RoPE / scatter store. */
typedef struct ta_matmul_op_ex {
  ta_matmul_op op;
  uint32_t packed_b;
  const ta_tensor *normed_weight;
  float normed_eps;
  ta_store_desc store;
} ta_matmul_op_ex;

int ta_run_ops_ex(const ta_executor *exec, const ta_matmul_op_ex *ops, size_t n_ops,
                  uint32_t as_graph, ta_run_stats *stats);

/* One launch computing silu(x @ Wg) * (x @ Wup) for packed f16 weights that
 * share x: the decode SwiGLU gate.  The reference issues this as an `up` GEMV
 * followed by a `gate` GEMV whose Mul epilogue reads `up`
 * (ref tools/llama-ash/src/model/forward/mod.rs:194-206); arithmetic per
 * output is the same, x is read once.  x [M, K] f32 (M <= 8), wg/wup packed
 * f16 [K, N], out [M, N] f32.  normed_weight may be NULL. */
int ta_swiglu_gemv(const ta_executor *exec, const ta_tensor *x, const ta_tensor *wg,
                   const ta_tensor *wup, const ta_tensor *out, const ta_tensor *normed_weight,
                   float normed_eps, ta_run_stats *stats);

/* Packed-weight helpers (ref src/matmul/api.rs:317-344,
 * ref src/pipeline/routing.rs:10-41).  Host-only; no device is touched. */
int ta_pack_f16w_row_tiles(const float *src, float *dst, size_t k, size_t n, size_t tile_n);
uint32_t ta_f16w_row_tile_n(uint32_t k, uint32_t n);

/* Raw binary16 upload into an f16 tensor (ref src/executor/transfer.rs:44-62). */
int ta_upload_f16(const ta_executor *exec, const ta_tensor *dst, const uint16_t *src, size_t len);

/* A second handle over the same device memory under another shape with the
 * same element count (ref src/tensor.rs:96-112).  Destroy both handles; the
 * memory is released with the last one. */
ta_tensor *ta_tensor_alias_with_shape(const ta_tensor *tensor, const uint32_t *shape, size_t rank);

/* Causal prefill flash attention (ref src/executor/elementwise/flash.rs:26-253,
 * FlashAttentionDesc ref src/executor/elementwise/mod.rs:162-184).
 * kt [H_kv, dh, T_max], v [H_kv, T_max, dh] (f32 or f16, same dtype), dh 64 or
 * 128; q/out f32, head-major [H, T_q, dh] or token-major [T_q, H*dh]; heads, T_q
 * and dh come from the tensor shapes, H must be a multiple of H_kv.
 * Row i attends positions < min(kv_len, pos_base + i + 1); a row that sees no
 * position is left untouched. */
typedef struct ta_flash_desc {
  uint32_t kv_len;               /* valid K/V positions in the caches, <= T_max */
  uint32_t pos_base;             /* absolute position of query row 0 */
  float scale;                   /* 1/sqrt(dh) for standard attention */
  uint32_t token_major_heads;    /* 0: q is [H, T_q, dh]; H > 0: q is token-major [T_q, H*dh] */
  uint32_t out_token_major_heads;/* 0: out follows q; H > 0: out is [T_q, H*dh] whatever q is */
  uint32_t simt;                 /* 1: pin the f32-operand kernel (run_flash_attention_simt in the reference);
                                  * 0: f16 caches with head dim 64 and >= 32 query rows take the tensor-core
                                  * kernel, which rounds Q*scale and the softmax weights through f16 */
} ta_flash_desc;

int ta_flash_attention(const ta_executor *exec, const ta_tensor *q, const ta_tensor *kt,
                       const ta_tensor *v, const ta_tensor *out, const ta_flash_desc *desc,
                       ta_run_stats *stats);

/* Split-K decode attention, two launches (ref src/executor/elementwise/attn.rs:27-185,
 * AttnDecodeDesc ref src/executor/elementwise/mod.rs:202-237).  q/out
 * [H_kv, group, dh] f32 (dh = 64, group <= 8, both from the shapes); kt/v as for
 * ta_flash_attention; scratch f32 with at least kv_heads * chunks * group *
 * (dh + 2) elements, chunks = ta_attn_decode_num_chunks(kv_len), or
 * TA_ATTN_DECODE_MAX_CHUNKS with a pos_cell. */
#define TA_ATTN_DECODE_MAX_CHUNKS 32u

typedef struct ta_attn_decode_desc {
  uint32_t kv_len;  /* valid positions, 1..T_max; with pos_cell: kv_len + *cell (record kv_len = 1) */
  float scale;
  const ta_pos_cell *pos_cell; /* optional; fixes the chunk grid at TA_ATTN_DECODE_MAX_CHUNKS */
} ta_attn_decode_desc;

uint32_t ta_attn_decode_num_chunks(uint32_t kv_len);
int ta_attn_decode(const ta_executor *exec, const ta_tensor *q, const ta_tensor *kt,
                   const ta_tensor *v, const ta_tensor *scratch, const ta_tensor *out,
                   const ta_attn_decode_desc *desc, ta_run_stats *stats);

/* 4-byte host-visible cells read or written by kernels in replayed graphs
 * (ref src/executor/cells.rs:51-201: PosBuffer, HostU32Buffer). */
ta_pos_cell *ta_pos_cell_create(const ta_context *ctx);
void ta_pos_cell_destroy(ta_pos_cell *cell);
int ta_pos_cell_set(ta_pos_cell *cell, uint32_t value);
int ta_pos_cell_get(const ta_pos_cell *cell, uint32_t *value);

/* Token-id list in host-visible memory, read by gather kernels on the device
 * (ref src/executor/cells.rs:140-201, TokenIdBuffer). */
typedef struct ta_token_ids ta_token_ids;
ta_token_ids *ta_token_ids_create(const ta_context *ctx, uint32_t capacity);
void ta_token_ids_destroy(ta_token_ids *ids);
int ta_token_ids_set(ta_token_ids *ids, const uint32_t *tokens, uint32_t n); /* n <= capacity */

/* Mixed op graphs: matmuls and model ops in one submission or one prepared
 * replay (ref src/executor/graph_ops.rs:27-161 ExecOp, :249-353 run_exec_ops /
 * prepare_exec_ops).  Later ops may read what earlier ops wrote.  Operand slots
 * by kind (unused slots stay zero):
 *   MATMUL            mm
 *   RMS_NORM          in0 input, in1 weight, out; f0 = eps
 *   LAYER_NORM        in0 input, in1 weight, in2 bias, out; f0 = eps
 *   SOFTMAX_ROWS      in0 input, out; f0 = scale; u0 mask kind, u1 valid/prefix, u2 rows per group
 *   ROPE              in0 input, in1 table, out; rope
 *   ROPE_SCATTER      in0 input, in1 table, out = dst (f32/f16); rope; dst_offset, dst_strides
 *                     per (token, head, dim), pos_scale; cell = position added to
 *                     rope.pos_base and (times pos_scale) to dst_offset
 *   COPY_STRIDED      in0 src, out dst (any f32/f16 pairing); copy
 *   BINARY            in0 a, in1 b, out; u0 = 0: a + f0*b, 1: silu(a)*b
 *   ATTN_DECODE       in0 q, in1 kt, in2 v, in3 scratch, out; attn
 *   FLASH_ATTN        in0 q, in1 kt, in2 v, out; flash
 *   ARGMAX            in0 input; cell receives the index (ties keep the largest index)
 *   EMBED_GATHER      cell = token id word; in0 table [vocab, embd] (f32/f16), out [embd]
 *   EMBED_GATHER_ROWS tokens; in0 table, out [n, embd]
 *   ALL_REDUCE        out = f32 tensor summed in place over the ranks of comm
 *   ALL_GATHER        in0 [n] f32 of every rank -> out [world * n] in rank order; comm
 *   PREFILL_QKV_PACK  in0 qkv [T, H*dh + 2*H_kv*dh] f32, in1 rope table, out q [H, T, dh] f32 (RoPE),
 *                     in2 kt cache [H_kv, dh, T_max] (RoPE'd k at positions rope.pos_base + t),
 *                     in3 v cache [H_kv, T_max, dh]; caches f32 or f16; rope = {H, dh, rot_dim,
 *                     pos_base}, u0 = H_kv (run_prefill_qkv_pack in the reference)
 *   ARGMAX_SHARDED    in0 = this rank's column slice of a row, u0 = global index of in0[0], comm, cell: every rank
 *                     receives the index of the maximum over all ranks' slices (ties keep the largest index);
 *                     one launch per rank, the ranks exchange one (value, index) pair each over peer memory.
 *                     Needs a communicator with peer access; no counterpart in the reference.
 * Inside a graph, `row-parallel GEMV (M = 1) -> ALL_REDUCE of its output -> GEMV reading that output`
 * runs as two launches: the first pushes its partial row to every rank, the second sums the
 * ranks' rows in rank order while it stages its activation; the tensor holds the sum afterwards. */
enum {
  TA_EXEC_MATMUL = 0, TA_EXEC_RMS_NORM, TA_EXEC_LAYER_NORM, TA_EXEC_SOFTMAX_ROWS, TA_EXEC_ROPE,
  TA_EXEC_ROPE_SCATTER, TA_EXEC_COPY_STRIDED, TA_EXEC_BINARY, TA_EXEC_ATTN_DECODE, TA_EXEC_FLASH_ATTN,
  TA_EXEC_ARGMAX, TA_EXEC_EMBED_GATHER, TA_EXEC_EMBED_GATHER_ROWS, TA_EXEC_ALL_REDUCE, TA_EXEC_ALL_GATHER,
  TA_EXEC_PREFILL_QKV_PACK, TA_EXEC_ARGMAX_SHARDED
};

/* Communicator for tensor-parallel graphs: one rank per process and GPU, NCCL over
 * NVLink underneath (bound at run time; creating a communicator fails with a
 * message where NCCL is absent).  No counterpart in the reference, which is
 * single-device.  Rank 0 makes an id with ta_comm_unique_id, every rank receives
 * the same 128 bytes out of band (e.g. a torch.distributed broadcast) and calls
 * ta_comm_create collectively.  world == 1 needs no id (NULL) and no NCCL. */
typedef struct ta_comm ta_comm;
#define TA_COMM_ID_BYTES 128
int ta_comm_unique_id(uint8_t out[TA_COMM_ID_BYTES]);
ta_comm *ta_comm_create(const ta_context *ctx, uint32_t rank, uint32_t world, const uint8_t *id);
void ta_comm_destroy(ta_comm *comm);
/* Small all-reduces of the group travel as peer stores with flags; a rank waits on the device for
 * its peers' flags at most this long (default 10 s: ranks of one job drift by whole milliseconds
 * while one still loads weights), then the kernel returns, the call fails (-1, "... wait for a peer
 * rank ...") and the context stays usable.  After such a failure every rank calls ta_comm_resync
 * (collective: two NCCL meetings around zeroing the flags) before the next exchange. */
int ta_comm_set_wait_limit_ns(ta_comm *comm, uint64_t limit_ns);
int ta_comm_resync(ta_comm *comm);
uint32_t ta_comm_rank(const ta_comm *comm);
uint32_t ta_comm_world(const ta_comm *comm);

typedef struct ta_exec_op {
  uint32_t kind;
  ta_matmul_op_ex mm;
  const ta_tensor *in0, *in1, *in2, *in3, *out;
  float f0;
  uint32_t u0, u1, u2;
  ta_rope_desc rope;
  ta_copy_desc copy;
  uint32_t dst_offset, dst_strides[3], pos_scale;
  ta_flash_desc flash;
  ta_attn_decode_desc attn;
  const ta_pos_cell *cell;
  const ta_token_ids *tokens;
  const struct ta_comm *comm;      /* TA_EXEC_ALL_REDUCE (in place on `out`), TA_EXEC_ALL_GATHER (in0 -> out) */
} ta_exec_op;

int ta_run_exec_ops(const ta_executor *exec, const ta_exec_op *ops, size_t n_ops, ta_run_stats *stats);
/* Prepared replay of a mixed graph; the handle works with ta_prepared_run /
 * _submit / _wait / _destroy and carries the same lifetime contract. */
ta_prepared *ta_prepared_create_exec(const ta_executor *exec, const ta_exec_op *ops, size_t n_ops);

/* Registry and routing introspection (ref src/pipeline/catalog.rs:10-41,129-376).
 * Host-only. */
size_t ta_kernel_spec_count(void);
/* Fills name/tile for registry entry `index`; -1 when out of range. */
int ta_kernel_spec_at(size_t index, ta_dispatch_info *out);
/* Resolves an ML_KERNEL-style name or alias to a registry index; -2 for
 * "auto", -1 (with an error message) for an unknown name. */
int ta_kernel_selection_parse(const char *name);

/* Shape resolution exactly as a matmul call would do it
 * (ref src/matmul/resolution.rs:16-76,421-441), without touching a device.
 * Shapes are rank-2/3 arrays.  On success fills out[0..8] =
 * {m, n, k, batch, stride_a, stride_b, stride_c, flops_lo32, flops_hi32}. */
int ta_resolve_shapes(const uint32_t *a, size_t a_rank, const uint32_t *b, size_t b_rank,
                      const uint32_t *c, size_t c_rank, uint32_t out[9]);

/* Split-K heuristics (ref src/executor/splitk2.rs:48-122).  Host-only.
 * ta_heuristic_splits returns 0 when the shape stays data-parallel. */
uint32_t ta_default_num_k_splits(uint32_t batch, uint32_t m, uint32_t n, uint32_t k,
                                 uint32_t tile_m, uint32_t tile_n);
uint32_t ta_heuristic_splits(uint32_t batch, uint32_t m, uint32_t n, uint32_t k);

/* Measured tuner, additions (ref src/executor/tuning.rs:18-344, src/pipeline/tuning.rs:60-199).
 * ta_tune_shape (PART 1) tunes an f32 shape; ta_tune_shape_f16w the same shape with f16-storage B
 * (the reference keys winners by (B, M, N, K, b_f16), src/pipeline/tuning.rs:33-45). */
int ta_tune_shape_f16w(const ta_executor *exec, uint32_t batch, uint32_t m, uint32_t n, uint32_t k);
/* Host-only tuner arithmetic, as the reference pins it in src/executor/tuning.rs:319-374:
 * ta_tune_median: median of n u64 samples, the middle pair's mean rounded down when n is even;
 *   returns 0 with *out set, 1 when n == 0 (no median), -1 on a null argument.
 * ta_tune_candidate_at: index of the candidate measured at position `offset` of `round` for a list
 *   of `len` candidates (round 0 = warm-up in index order; measured rounds alternate direction). */
int ta_tune_median(const uint64_t *samples, size_t n, uint64_t *out);
size_t ta_tune_candidate_at(size_t len, uint32_t round, size_t offset);
/* Tuned-winner store: path of the store for a device name under $XDG_CACHE_HOME (or ~/.cache), and
 * load-then-save of a store file: reads `in_path` with the loader the executor uses (a stale
 * header discards the file, malformed lines are skipped, `splitk2=S` needs 2 <= S <= 65535,
 * `bf16` marks f16-storage B), reports the entries kept and, when out_path is not NULL, writes
 * them back sorted by shape.  Host-only. */
int ta_tune_store_path(const char *device_name, char *buf, size_t cap);
int ta_tune_store_rewrite(const char *in_path, const char *out_path, size_t *n_entries);

/* Experiment switches: the library reads ONE environment variable, TA_EXPERIMENT, a comma-separated
 * list of name=value pairs (see INTEGRATION.md for the names), once per process.
 * ta_experiment_check parses a string the same way and reports an unknown name (-1). Host-only. */
int ta_experiment_check(const char *spec);

/* Self-test of the bounded device-side waits: launches one warp that waits, with the helper and the
 * status word every tensor-core kernel of the library uses, on a barrier nothing completes.  After
 * limit_ns (1 .. 1e9) the wait gives up and the kernel returns normally; the call then fails (-1)
 * with the library's "gave up on a bounded device-side wait" message and the executor and context
 * remain usable.  No counterpart in the reference (its chain kernel spins without a limit,
 * ref shaders/matmul_gemv_chain_kernel.glsl:93-132). */
int ta_selftest_bounded_wait(const ta_executor *exec, uint32_t limit_ns);

/* The kernel the heuristic stage of the routing order (explicit selection > tuned winner > heuristic,
 * ref src/pipeline/mod.rs:259-360) picks for a plain shape on a device of sm_count SMs: a name of the
 * kernel registry (static storage).  weights_f16 != 0 selects the f16-storage B family.  Host-only. */
const char *ta_heuristic_kernel(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, int weights_f16,
                                int sm_count);

/* Software conversions (ref src/dtype.rs:42-112): round-to-nearest-even encode and IEEE binary16
 * decode, bit-exact with the reference on every pattern except subnormal halves, where the
 * reference's decode (dtype.rs:93-99) normalises one bit too far and this one returns the IEEE
 * value the device's own f16 loads see.  Host-only. */
uint16_t ta_f32_to_f16_bits(float value);
float ta_f16_bits_to_f32(uint16_t bits);

/* Interop for callers that own device memory or streams themselves: the raw
 * CUDA device pointer of a tensor and the CUDA device ordinal of a context. */
void *ta_tensor_device_ptr(const ta_tensor *tensor);
int ta_context_device_index(const ta_context *ctx);
/* Device name as the driver reports it (valid while the context lives); "" for NULL. */
const char *ta_context_device_name(const ta_context *ctx);

/* Kernels launched by this library on the calling process since load; a
 * caller can difference it around a region to count launches. */
uint64_t ta_kernel_launch_count(void);

#ifdef __cplusplus
}
#endif

#endif /* TENSOR_ASH_H */
