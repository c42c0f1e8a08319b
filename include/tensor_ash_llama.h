/*
 * tensor_ash_llama.h -- llama-architecture runner built only on library ops.
 *
 * Counterpart of the reference's tools/llama-ash (model/mod.rs:59-190,
 * model/forward/{mod,prefill,decode}.rs): the same op graphs -- prefill through
 * one mixed graph with fused causal attention, greedy decode through one
 * prepared (record-once, replay-many) graph whose position comes from a 4-byte
 * cell and whose next token is chosen and embedded on the device.  Weights come
 * from an F32 / F16 GGUF file (ta_llama_load_gguf) or are random-initialised from
 * a seed (the benchmark configuration is random-init).
 */
#ifndef TENSOR_ASH_LLAMA_H
#define TENSOR_ASH_LLAMA_H

#include "tensor_ash.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ta_llama ta_llama;

typedef struct ta_llama_config {
  uint32_t layers;    /* 22 */
  uint32_t embd;      /* 2048 */
  uint32_t heads;     /* 32 */
  uint32_t kv_heads;  /* 4 */
  uint32_t head_dim;  /* 64 (heads * head_dim == embd) */
  uint32_t ffn;       /* 5632 */
  uint32_t vocab;     /* 32000 */
  uint32_t t_max;     /* KV-cache capacity in positions */
  float rms_eps;      /* 1e-5 */
  float rope_theta;   /* 1e4 */
  float weight_sigma; /* weights ~ N(0, sigma), rounded to f16; 0.02 */
  float norm_jitter;  /* norm weights = 1 + jitter * u, u uniform [-1,1); 0 gives all ones */
  uint64_t seed;
} ta_llama_config;

/* Weight tensors are generated on the host in chunks of 2^20 elements; chunk c
 * of tensor id t uses the documented LCG + Box-Muller stream with seed
 * (seed * 1000003 + t) * 4096 + c, so a checker can rebuild any tensor.
 * Tensor ids: 0 token embedding [vocab, embd]; 1 output norm; 2 lm_head
 * [embd, vocab]; per layer L (base = 16 + 16*L): +0 attn_norm, +1 wq, +2 wk,
 * +3 wv, +4 wo, +5 ffn_norm, +6 w_gate, +7 w_up, +8 w_down (all [n_in, n_out]). */
ta_llama *ta_llama_create_random(const ta_executor *exec, const ta_llama_config *cfg);

/* Tensor-parallel shard of the same model on the rank of `comm` (NULL or world 1: the whole
 * model).  Column-parallel wq / wk / wv (by head; a kv head is shared by neighbouring ranks
 * when there are more ranks than kv heads), w_gate, w_up (by MLP column) and lm_head (by
 * vocabulary column); row-parallel wo and w_down, whose partial sums are all-reduced (sum,
 * f32) -- the one exchange step per projection.  Rank 0 folds the residual into its partial
 * sum.  Every rank ends a step with the same logits and the same greedy token.  `comm`
 * must outlive the model; all ranks must call prefill / decode in step. */
ta_llama *ta_llama_create_random_tp(const ta_executor *exec, const ta_llama_config *cfg, const ta_comm *comm);
/* The same runner on the weights of an F32 / F16 GGUF file of the llama architecture
 * (ref tools/llama-ash/src/gguf.rs, model/load.rs:14-255): geometry from the llama.* metadata,
 * vocabulary from token_embd.weight, t_max clamped to llama.context_length; linear weights are
 * transposed to [n_in, n_out] and stored f16, norm weights must be f32, a missing output.weight
 * ties the head to the embeddings, quantized tensor types are refused.  `comm` as above (NULL:
 * one GPU).  weight_sigma / norm_jitter / seed of the reported config are zero. */
ta_llama *ta_llama_load_gguf(const ta_executor *exec, const char *path, uint32_t t_max, const ta_comm *comm);
int ta_llama_get_config(const ta_llama *model, ta_llama_config *out);
void ta_llama_destroy(ta_llama *model);

/* GGUF v2 / v3 inspection, host only (ref tools/llama-ash/src/gguf.rs:62-284).  Scalar and string
 * metadata are kept, arrays are walked and dropped.  ta_gguf_meta_kind: 0 u64, 1 i64, 2 f64,
 * 3 bool, 4 string, 5 skipped array, -1 absent.  ta_gguf_meta_u64 accepts unsigned and
 * non-negative signed values; ta_gguf_meta_f64 returns `fallback` for an absent key.
 * ta_gguf_tensor_info: ne[] in file order (ne[0] fastest), ggml type 0 = F32, 1 = F16, offset
 * relative to the data section.  ta_gguf_read_f32 widens f16 exactly and refuses other types. */
typedef struct ta_gguf ta_gguf;
ta_gguf *ta_gguf_open(const char *path);
void ta_gguf_close(ta_gguf *file);
int ta_gguf_meta_kind(const ta_gguf *file, const char *key);
int ta_gguf_meta_u64(const ta_gguf *file, const char *key, uint64_t *out);
int ta_gguf_meta_f64(const ta_gguf *file, const char *key, double fallback, double *out);
int ta_gguf_meta_str(const ta_gguf *file, const char *key, char *buf, size_t cap);
int ta_gguf_tensor_info(const ta_gguf *file, const char *name, uint64_t ne[4], uint32_t *n_dims,
                        uint32_t *ggml_type, uint64_t *offset);
int ta_gguf_read_f32(ta_gguf *file, const char *name, float *out, size_t len);
uint64_t ta_gguf_data_start(const ta_gguf *file);

/* Forget the KV cache: the next prefill starts at position 0. */
int ta_llama_reset(ta_llama *model);

/* Prefill n prompt tokens at the current position (one graph submission);
 * *next_token receives the greedy next token. */
int ta_llama_prefill(ta_llama *model, const uint32_t *tokens, uint32_t n, uint32_t *next_token,
                     ta_run_stats *stats);

/* Greedy decode of n tokens starting from `first_token` (normally the token the
 * prefill returned): each step is one replay of the prepared decode graph, one
 * 4-byte position write and one 4-byte token read.  out_tokens[i] is the token
 * chosen after consuming step i's input.  stats sums the device time. */
int ta_llama_decode(ta_llama *model, uint32_t first_token, uint32_t n, uint32_t *out_tokens,
                    ta_run_stats *stats);

/* One decode step with the device time of every launch measured separately (CUDA events around each
 * launch; the reference's LLAMA_ASH_BREAKDOWN=1 table, ref tools/llama-ash/src/main.rs:161-193,
 * whose per-dispatch times come from its per-op mode).  The step consumes `token` at the current
 * position like ta_llama_decode(model, token, 1, ..).  rows[0 .. min(cap, *n_rows)) receive one row per
 * op class, largest first; class names are static strings in the reference's vocabulary
 * (qkv_matmul, attn_decode, o_proj_mm, ffn_up_mm = the fused up + gate launch, ffn_down_mm,
 * lm_head_mm) plus argmax, embed_gather, all_reduce, all_gather.  *n_launches = launches of the step. */
typedef struct ta_llama_breakdown_row {
  const char *op_class;
  uint64_t gpu_ns;
  uint32_t calls;
} ta_llama_breakdown_row;
int ta_llama_decode_breakdown(ta_llama *model, uint32_t token, ta_llama_breakdown_row *rows, size_t cap,
                              size_t *n_rows, size_t *n_launches, uint32_t *next_token);

/* Logits of the most recent step ([vocab] floats), for margin checks. */
int ta_llama_logits(ta_llama *model, float *out, size_t len);

/* Current position (tokens in the KV cache) and weight bytes this rank reads per decoded token. */
uint32_t ta_llama_position(const ta_llama *model);
uint64_t ta_llama_weight_bytes_per_token(const ta_llama *model);

#ifdef __cplusplus
}
#endif

#endif /* TENSOR_ASH_LLAMA_H */
