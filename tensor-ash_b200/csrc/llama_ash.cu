// llama-architecture runner on library ops only: the prefill and decode op graphs
// of the reference's tools/llama-ash (model/forward/prefill.rs:89-291,
// forward/decode.rs:52-98,172-246, forward/mod.rs:50-87,134-328, model/load.rs:144-255).
//
// Weights live as f16 [n_in, n_out]; decode uses packed row tiles for q/k/v, gate,
// up and lm_head, row-major for o and down, exactly the reference's split.  KV
// caches are f16: Kt [H_kv, dh, T_max] and V [H_kv, T_max, dh] per layer.
//
// Decode is ONE prepared graph per model: per layer three packed GEMVs with the
// attention RMSNorm fused into A and RoPE / KV-append fused into the store, the
// split-K decode attention, o-projection + residual, up, gate (SiLU * up), down
// + residual; then lm_head with the final norm fused, argmax into a host-visible
// word, and the next token's embedding row gathered on the device.  A step is
// one position write, one graph launch and one token read.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <array>
#include <memory>
#include <string>
#include <thread>

#pragma GCC visibility push(default)
#include "../../include/tensor_ash_llama.h"
#pragma GCC visibility pop
#include "gguf.hpp"
#include "ta_handles.hpp"

namespace {

// ---- deterministic weight streams: the LCG of the reference's test fixtures
// (tools/test-support/src/lib.rs:9-18) with Box-Muller on top, per 2^20-element chunk.
inline uint64_t lcg_seed(uint64_t seed) { return (seed * 0x9E3779B97F4A7C15ull) | 1ull; }
inline uint64_t lcg_step(uint64_t s) { return s * 6364136223846793005ull + 1442695040888963407ull; }

void fill_normal_chunk(float *out, size_t n, uint64_t seed, double sigma) {
  uint64_t s = lcg_seed(seed);
  const double two_pi = 6.283185307179586476925286766559;
  for (size_t i = 0; i < n; i += 2) {
    s = lcg_step(s);
    const double u1 = ((double)(uint32_t)(s >> 40) + 1.0) / 16777216.0;
    s = lcg_step(s);
    const double u2 = (double)(uint32_t)(s >> 40) / 16777216.0;
    const double r = std::sqrt(-2.0 * std::log(u1));
    out[i] = (float)(sigma * r * std::cos(two_pi * u2));
    if (i + 1 < n) out[i + 1] = (float)(sigma * r * std::sin(two_pi * u2));
  }
}

void fill_uniform_chunk(float *out, size_t n, uint64_t seed) {
  uint64_t s = lcg_seed(seed);
  for (size_t i = 0; i < n; ++i) {
    s = lcg_step(s);
    out[i] = (float)(uint32_t)(s >> 40) / (float)(1u << 24) * 2.0f - 1.0f;
  }
}

constexpr size_t CHUNK = 1u << 20;

uint64_t chunk_seed(uint64_t seed, uint32_t tensor_id, size_t chunk) {
  return (seed * 1000003ull + tensor_id) * 4096ull + chunk;
}

// Generates tensor `id` (n elements) as f16 bits, in parallel over chunks.
std::vector<uint16_t> gen_weight_f16(uint64_t seed, uint32_t id, size_t n, double sigma) {
  std::vector<uint16_t> bits(n);
  const size_t chunks = (n + CHUNK - 1) / CHUNK;
  const unsigned nt = std::max(1u, std::min(32u, std::thread::hardware_concurrency()));
  std::vector<std::thread> pool;
  for (unsigned t = 0; t < nt; ++t)
    pool.emplace_back([&, t]() {
      std::vector<float> tmp(CHUNK);
      for (size_t c = t; c < chunks; c += nt) {
        const size_t off = c * CHUNK, len = std::min(CHUNK, n - off);
        fill_normal_chunk(tmp.data(), len, chunk_seed(seed, id, c), sigma);
        for (size_t i = 0; i < len; ++i) bits[off + i] = f32_to_f16_bits(tmp[i]);
      }
    });
  for (auto &th : pool) th.join();
  return bits;
}

// [K, N] -> packed [N/tile][K][tile] on raw f16 bits (src/matmul/api.rs:317-344)
std::vector<uint16_t> pack_bits(const std::vector<uint16_t> &src, size_t k, size_t n, size_t tile) {
  std::vector<uint16_t> out(src.size());
  const size_t tiles = n / tile;
  for (size_t t = 0; t < tiles; ++t)
    for (size_t kk = 0; kk < k; ++kk)
      memcpy(&out[(t * k + kk) * tile], &src[kk * n + t * tile], tile * 2);
  return out;
}

// columns [c0, c0 + w) of a row-major [rows, cols] matrix
std::vector<uint16_t> slice_cols(const std::vector<uint16_t> &src, size_t rows, size_t cols, size_t c0, size_t w) {
  std::vector<uint16_t> out(rows * w);
  for (size_t r = 0; r < rows; ++r) memcpy(&out[r * w], &src[r * cols + c0], w * 2);
  return out;
}
// rows [r0, r0 + h) of a row-major [rows, cols] matrix
std::vector<uint16_t> slice_rows(const std::vector<uint16_t> &src, size_t cols, size_t r0, size_t h) {
  return std::vector<uint16_t>(src.begin() + r0 * cols, src.begin() + (r0 + h) * cols);
}

// Where a model's weights come from.  Linear weights are handed over as f16 bits in the
// [n_in, n_out] layout every GEMM / GEMV here reads; ids follow include/tensor_ash_llama.h
// (0 embedding, 1 output norm, 2 lm_head, 16 + 16 L + {0 attn_norm, 1 wq, 2 wk, 3 wv, 4 wo,
// 5 ffn_norm, 6 w_gate, 7 w_up, 8 w_down}).
struct WeightSource {
  virtual ~WeightSource() = default;
  virtual std::vector<uint16_t> linear(uint32_t id, uint32_t n_in, uint32_t n_out) = 0;
  virtual std::vector<uint16_t> embedding_f16(uint32_t vocab, uint32_t embd) = 0;
  virtual bool embedding_is_f32() const { return false; }
  virtual std::vector<float> embedding_f32(uint32_t, uint32_t) { return {}; }
  virtual std::vector<float> norm(uint32_t id, uint32_t n) = 0;
};

struct RandomSource : WeightSource {
  uint64_t seed;
  double sigma;
  float jitter;
  RandomSource(uint64_t s, double sg, float j) : seed(s), sigma(sg), jitter(j) {}
  std::vector<uint16_t> linear(uint32_t id, uint32_t n_in, uint32_t n_out) override {
    return gen_weight_f16(seed, id, (size_t)n_in * n_out, sigma);
  }
  std::vector<uint16_t> embedding_f16(uint32_t vocab, uint32_t embd) override {
    return gen_weight_f16(seed, 0, (size_t)vocab * embd, sigma);
  }
  std::vector<float> norm(uint32_t id, uint32_t n) override {
    std::vector<float> w(n, 1.0f);
    if (jitter != 0.0f) {
      std::vector<float> u(n);
      fill_uniform_chunk(u.data(), u.size(), chunk_seed(seed, id, 0));
      for (size_t i = 0; i < w.size(); ++i) w[i] = 1.0f + jitter * u[i];
    }
    return w;
  }
};

// GGUF tensors (tools/llama-ash/src/model/load.rs:104-232): a linear weight `y = W x` is stored
// with ne = [n_in, n_out], i.e. n_out rows of n_in values, and is transposed to [n_in, n_out];
// f32 payloads round to f16 (nearest even), f16 payloads are taken bit for bit.  A file without
// output.weight ties the lm_head to the embedding table.
struct GgufSource : WeightSource {
  GgufFile &g;
  explicit GgufSource(GgufFile &file) : g(file) {}
  static std::string name_of(uint32_t id) {
    if (id == 1) return "output_norm.weight";
    if (id == 2) return "output.weight";
    const uint32_t layer = (id - 16) / 16, part = (id - 16) % 16;
    static const char *parts[9] = {"attn_norm", "attn_q", "attn_k", "attn_v", "attn_output",
                                   "ffn_norm", "ffn_gate", "ffn_up", "ffn_down"};
    if (id < 16 || part > 8) fail("internal error: no GGUF tensor for weight id %u", id);
    return "blk." + std::to_string(layer) + "." + parts[part] + ".weight";
  }
  static std::vector<uint16_t> transposed(const std::vector<uint16_t> &src, size_t rows, size_t cols) {
    std::vector<uint16_t> out(src.size());   // [rows, cols] -> [cols, rows], blocked for the cache
    constexpr size_t B = 64;
    for (size_t r0 = 0; r0 < rows; r0 += B)
      for (size_t c0 = 0; c0 < cols; c0 += B)
        for (size_t r = r0; r < std::min(rows, r0 + B); ++r)
          for (size_t c = c0; c < std::min(cols, c0 + B); ++c) out[c * rows + r] = src[r * cols + c];
    return out;
  }
  std::vector<uint16_t> linear(uint32_t id, uint32_t n_in, uint32_t n_out) override {
    if (id == 2 && !g.has_tensor("output.weight"))   // tied head: embedding [vocab, embd] -> [embd, vocab]
      return transposed(embedding_f16(n_out, n_in), n_out, n_in);
    const std::string name = name_of(id);
    const GgufTensorInfo &ti = g.info(name);
    if (ti.ne != std::vector<uint64_t>{n_in, n_out})
      fail("%s: ne [%s] != expected [%u, %u]", name.c_str(), ne_str(ti).c_str(), n_in, n_out);
    return transposed(g.read_f16_bits(name), n_out, n_in);
  }
  std::vector<uint16_t> embedding_f16(uint32_t, uint32_t) override { return g.read_f16_bits("token_embd.weight"); }
  bool embedding_is_f32() const override { return g.info("token_embd.weight").ggml_type == GGML_TYPE_F32; }
  std::vector<float> embedding_f32(uint32_t, uint32_t) override { return g.read_f32("token_embd.weight"); }
  std::vector<float> norm(uint32_t id, uint32_t n) override {
    const std::string name = name_of(id);
    const GgufTensorInfo &ti = g.info(name);
    if (ti.ne != std::vector<uint64_t>{n} || ti.ggml_type != GGML_TYPE_F32)
      fail("%s: expected f32 [%u], got ne [%s] type %u", name.c_str(), n, ne_str(ti).c_str(), ti.ggml_type);
    return g.read_f32(name);
  }
  static std::string ne_str(const GgufTensorInfo &ti) {
    std::string s;
    for (size_t i = 0; i < ti.ne.size(); ++i) s += (i ? ", " : "") + std::to_string(ti.ne[i]);
    return s;
  }
};

struct Layer {
  Tensor attn_norm, ffn_norm;
  Tensor wq_p, wk_p, wv_p, w_qkv, wo, w_gate, w_up, w_gate_p, w_up_p, w_down;
  Tensor kt_cache, v_cache;
};

struct PrefillScratch {
  Tensor x_a, x_b, xn, qkv, q, k, v, attn_flat, o, on, up, gate, last, last_n;
};

}  // namespace

struct ta_llama {
  std::shared_ptr<Context> ctx;
  Executor *exec = nullptr;
  ta_llama_config cfg{};
  // tensor-parallel shard of this rank (world 1: the whole model)
  const Comm *comm = nullptr;
  uint32_t rank = 0, world = 1;
  uint32_t heads_l = 0, kv_l = 0, kv_first = 0, q_w = 0, kv_w = 0, ffn_l = 0, vocab_l = 0;
  std::vector<Layer> layers;
  Tensor embd, output_norm, lm_head, lm_head_p, rope_table;
  // decode scratch (t = 1)
  Tensor x_a, x_b, q, k, v, attn, o, up, gate, logits, logits_l, attn_partials;
  PosCell pos_cell, token_cell;
  TokenIds token_ids;
  std::unique_ptr<PreparedOps> decode_graph;
  std::unique_ptr<PrefillScratch> prefill_full;
  bool logits_stale = false;   // sharded decode: `logits` holds the last gathered row, not the last step's
  bool pos_last_decode = false;   // the most recent step was a decode step (not a prefill)
  uint32_t pos = 0;
  ~ta_llama();
};

namespace {

Tensor make(const std::shared_ptr<Context> &ctx, std::initializer_list<uint32_t> shape, DType dt) {
  std::vector<uint32_t> s(shape);
  return Tensor::uninit_device(ctx, s.data(), s.size(), dt);
}

Tensor upload_bits(ta_llama &m, const std::vector<uint16_t> &bits, uint32_t rows, uint32_t cols) {
  Tensor t = make(m.ctx, {rows, cols}, DType::F16);
  m.exec->upload_f16(bits.data(), bits.size(), t);
  return t;
}

Tensor norm_weight(ta_llama &m, WeightSource &src, uint32_t id) {
  const std::vector<float> w = src.norm(id, m.cfg.embd);
  Tensor t = make(m.ctx, {m.cfg.embd}, DType::F32);
  m.exec->upload(w.data(), w.size(), t);
  return t;
}

void make_pinned_cell(const std::shared_ptr<Context> &ctx, PosCell &c) {
  c.ctx = ctx;
  TA_CUDA(cudaHostAlloc((void **)&c.host, sizeof(uint32_t), cudaHostAllocMapped));
  TA_CUDA(cudaHostGetDevicePointer((void **)&c.device, c.host, 0));
  *c.host = 0;
}

}  // namespace

ta_llama::~ta_llama() {
  decode_graph.reset();   // waits for in-flight work before the tensors go away
  if (ctx) cudaSetDevice(ctx->device);
  if (pos_cell.host) cudaFreeHost(pos_cell.host);
  if (token_cell.host) cudaFreeHost(token_cell.host);
  if (token_ids.host) cudaFreeHost(token_ids.host);
}

// ------------------------------------------------------------------ construction
namespace {

void build_model(ta_llama &m, WeightSource &src) {
  const ta_llama_config &c = m.cfg;
  if (!c.layers || !c.embd || !c.heads || !c.kv_heads || !c.head_dim || !c.ffn || !c.vocab || !c.t_max)
    fail("ta_llama_create: every config dimension must be non-zero");
  if (c.heads * c.head_dim != c.embd) fail("ta_llama_create: heads * head_dim must equal embd");
  if (c.heads % c.kv_heads || c.heads / c.kv_heads > 8) fail("ta_llama_create: GQA group must be 1..8");
  if (c.head_dim != 64) fail("ta_llama_create: head_dim must be 64 (decode attention variant)");
  const uint32_t kv_dim = c.kv_heads * c.head_dim;
  // Tensor-parallel shard (world 1 keeps everything): query heads and the MLP width split
  // evenly; kv heads split, or are shared by W / kv_heads neighbouring ranks when there are
  // more ranks than kv heads; the lm_head splits by vocabulary columns.  Column-parallel:
  // wq, wk, wv, w_gate, w_up, lm_head.  Row-parallel (partial sums, all-reduced): wo, w_down.
  const uint32_t W = m.world, R = m.rank;
  if (c.heads % W) fail("ta_llama_create: %u heads do not split over %u ranks", c.heads, W);
  if (c.kv_heads % W && W % c.kv_heads) fail("ta_llama_create: %u kv heads do not map onto %u ranks", c.kv_heads, W);
  if (c.ffn % W || c.vocab % W) fail("ta_llama_create: ffn %u / vocab %u do not split over %u ranks", c.ffn, c.vocab, W);
  m.heads_l = c.heads / W;
  m.kv_l = c.kv_heads >= W ? c.kv_heads / W : 1;
  m.kv_first = (uint32_t)(((uint64_t)R * c.kv_heads) / W);
  m.q_w = m.heads_l * c.head_dim;
  m.kv_w = m.kv_l * c.head_dim;
  m.ffn_l = c.ffn / W;
  m.vocab_l = c.vocab / W;
  if (m.heads_l % m.kv_l || m.heads_l / m.kv_l > 8) fail("ta_llama_create: local GQA group must be 1..8");
  const uint32_t n_qkv = m.q_w + 2 * m.kv_w;
  for (uint32_t n : {c.embd, kv_dim, c.ffn, c.vocab, m.q_w, m.kv_w, m.ffn_l, m.vocab_l})
    if (n % 32) fail("ta_llama_create: projection widths must be multiples of 32 (got %u)", n);
  auto tile = [](uint32_t k, uint32_t n) { return f16w_row_tile_n(k, n); };
  const size_t q0 = (size_t)R * m.q_w, kv0 = (size_t)m.kv_first * c.head_dim, f0 = (size_t)R * m.ffn_l,
               v0 = (size_t)R * m.vocab_l;

  {  // token embedding [vocab, embd] (replicated), final norm, lm_head columns [embd, vocab_l]
    if (src.embedding_is_f32()) {   // an f32 model file keeps its embedding rows in f32 (model/load.rs:205-214)
      const std::vector<float> e = src.embedding_f32(c.vocab, c.embd);
      m.embd = make(m.ctx, {c.vocab, c.embd}, DType::F32);
      m.exec->upload(e.data(), e.size(), m.embd);
    } else {
      m.embd = upload_bits(m, src.embedding_f16(c.vocab, c.embd), c.vocab, c.embd);
    }
    m.output_norm = norm_weight(m, src, 1);
    auto h = slice_cols(src.linear(2, c.embd, c.vocab), c.embd, c.vocab, v0, m.vocab_l);
    m.lm_head = upload_bits(m, h, c.embd, m.vocab_l);
    m.lm_head_p = upload_bits(m, pack_bits(h, c.embd, m.vocab_l, tile(c.embd, m.vocab_l)), c.embd, m.vocab_l);
  }
  m.layers.resize(c.layers);
  for (uint32_t li = 0; li < c.layers; ++li) {
    Layer &L = m.layers[li];
    const uint32_t base = 16 + 16 * li;
    L.attn_norm = norm_weight(m, src, base + 0);
    L.ffn_norm = norm_weight(m, src, base + 5);
    auto wq = slice_cols(src.linear(base + 1, c.embd, c.embd), c.embd, c.embd, q0, m.q_w);
    auto wk = slice_cols(src.linear(base + 2, c.embd, kv_dim), c.embd, kv_dim, kv0, m.kv_w);
    auto wv = slice_cols(src.linear(base + 3, c.embd, kv_dim), c.embd, kv_dim, kv0, m.kv_w);
    L.wq_p = upload_bits(m, pack_bits(wq, c.embd, m.q_w, tile(c.embd, m.q_w)), c.embd, m.q_w);
    L.wk_p = upload_bits(m, pack_bits(wk, c.embd, m.kv_w, tile(c.embd, m.kv_w)), c.embd, m.kv_w);
    L.wv_p = upload_bits(m, pack_bits(wv, c.embd, m.kv_w, tile(c.embd, m.kv_w)), c.embd, m.kv_w);
    {  // concatenated [embd, q_w + 2 kv_w] for the prefill GEMM
      std::vector<uint16_t> cat((size_t)c.embd * n_qkv);
      for (uint32_t r = 0; r < c.embd; ++r) {
        memcpy(&cat[(size_t)r * n_qkv], &wq[(size_t)r * m.q_w], (size_t)m.q_w * 2);
        memcpy(&cat[(size_t)r * n_qkv + m.q_w], &wk[(size_t)r * m.kv_w], (size_t)m.kv_w * 2);
        memcpy(&cat[(size_t)r * n_qkv + m.q_w + m.kv_w], &wv[(size_t)r * m.kv_w], (size_t)m.kv_w * 2);
      }
      L.w_qkv = upload_bits(m, cat, c.embd, n_qkv);
    }
    L.wo = upload_bits(m, slice_rows(src.linear(base + 4, c.embd, c.embd), c.embd, q0, m.q_w),
                       m.q_w, c.embd);
    auto wg = slice_cols(src.linear(base + 6, c.embd, c.ffn), c.embd, c.ffn, f0, m.ffn_l);
    auto wu = slice_cols(src.linear(base + 7, c.embd, c.ffn), c.embd, c.ffn, f0, m.ffn_l);
    L.w_gate = upload_bits(m, wg, c.embd, m.ffn_l);
    L.w_up = upload_bits(m, wu, c.embd, m.ffn_l);
    L.w_gate_p = upload_bits(m, pack_bits(wg, c.embd, m.ffn_l, tile(c.embd, m.ffn_l)), c.embd, m.ffn_l);
    L.w_up_p = upload_bits(m, pack_bits(wu, c.embd, m.ffn_l, tile(c.embd, m.ffn_l)), c.embd, m.ffn_l);
    L.w_down = upload_bits(m, slice_rows(src.linear(base + 8, c.ffn, c.embd), c.embd, f0, m.ffn_l),
                           m.ffn_l, c.embd);
    L.kt_cache = make(m.ctx, {m.kv_l, c.head_dim, c.t_max}, DType::F16);
    L.v_cache = make(m.ctx, {m.kv_l, c.t_max, c.head_dim}, DType::F16);
    TA_CUDA(cudaMemset(L.kt_cache.ptr(), 0, L.kt_cache.size_bytes()));
    TA_CUDA(cudaMemset(L.v_cache.ptr(), 0, L.v_cache.size_bytes()));
  }
  {  // rope table [t_max, dh/2, 2], angles in f64 (model/load.rs:243-253)
    const uint32_t half = c.head_dim / 2;
    std::vector<float> table((size_t)c.t_max * half * 2);
    for (uint32_t p = 0; p < c.t_max; ++p)
      for (uint32_t i = 0; i < half; ++i) {
        const double theta = (double)p / std::pow((double)c.rope_theta, 2.0 * i / (double)c.head_dim);
        table[((size_t)p * half + i) * 2] = (float)std::cos(theta);
        table[((size_t)p * half + i) * 2 + 1] = (float)std::sin(theta);
      }
    m.rope_table = make(m.ctx, {c.t_max, half, 2}, DType::F32);
    m.exec->upload(table.data(), table.size(), m.rope_table);
  }
  // decode scratch
  m.x_a = make(m.ctx, {1, c.embd}, DType::F32);
  m.x_b = make(m.ctx, {1, c.embd}, DType::F32);
  m.q = make(m.ctx, {1, m.q_w}, DType::F32);
  m.k = make(m.ctx, {1, m.kv_w}, DType::F32);
  m.v = make(m.ctx, {1, m.kv_w}, DType::F32);
  m.attn = make(m.ctx, {1, m.q_w}, DType::F32);
  m.o = make(m.ctx, {1, c.embd}, DType::F32);
  m.up = make(m.ctx, {1, m.ffn_l}, DType::F32);
  m.gate = make(m.ctx, {1, m.ffn_l}, DType::F32);
  m.logits = make(m.ctx, {1, c.vocab}, DType::F32);
  m.logits_l = make(m.ctx, {1, m.vocab_l}, DType::F32);
  m.attn_partials = make(m.ctx, {m.kv_l * ATTN_DECODE_MAX_CHUNKS * (m.heads_l / m.kv_l) * (c.head_dim + 2)}, DType::F32);
  make_pinned_cell(m.ctx, m.pos_cell);
  make_pinned_cell(m.ctx, m.token_cell);
  m.token_ids.ctx = m.ctx;
  m.token_ids.capacity = c.t_max;
  TA_CUDA(cudaHostAlloc((void **)&m.token_ids.host, (size_t)c.t_max * 4, cudaHostAllocMapped));
  TA_CUDA(cudaHostGetDevicePointer((void **)&m.token_ids.device, m.token_ids.host, 0));
}

ExecOp mm_op(const Tensor &a, const Tensor &b, const Tensor &c) {
  ExecOp o;
  o.kind = ExecKind::Matmul;
  o.mm.call = MatmulCall{&a, &b, &c, 1.0f, false};
  return o;
}

// forward/mod.rs:134-227 push_mlp_ops; residual adds and the SiLU gate ride the
// GEMM epilogues at every width (every kernel family here fuses them).
ExecOp all_reduce_op(ta_llama &m, const Tensor &t) {
  ExecOp o;
  o.kind = ExecKind::AllReduce;
  o.out = &t;
  o.comm = m.comm;
  return o;
}

void push_mlp_ops(ta_llama &m, std::vector<ExecOp> &ops, Layer &L, bool decode, const Tensor &attn_flat,
                  const Tensor &o, const Tensor &on, const Tensor &up, const Tensor &gate, const Tensor &x_in,
                  const Tensor &x_out) {
  const float eps = m.cfg.rms_eps;
  const bool tp = m.world > 1;
  // Row-parallel projections produce partial sums: rank 0 alone folds the residual in,
  // so the all-reduced sum holds it exactly once.
  const bool add_residual = m.rank == 0;
  ExecOp op = mm_op(attn_flat, L.wo, o);
  if (add_residual) {
    op.mm.epilogue.binary = BinaryKind::AddScaled;
    op.mm.epilogue.d = &x_in;
    op.mm.epilogue.beta = 1.0f;
  }
  ops.push_back(op);
  if (tp) ops.push_back(all_reduce_op(m, o));
  if (decode) {
    ExecOp u = mm_op(o, L.w_up_p, up);
    u.mm.packed_b = true; u.mm.normed_weight = &L.ffn_norm; u.mm.normed_eps = eps;
    ops.push_back(u);
    ExecOp g = mm_op(o, L.w_gate_p, gate);
    g.mm.packed_b = true; g.mm.normed_weight = &L.ffn_norm; g.mm.normed_eps = eps;
    g.mm.epilogue.activation = Activation::Silu;
    g.mm.epilogue.binary = BinaryKind::Mul;
    g.mm.epilogue.d = &up;
    ops.push_back(g);
  } else {
    ExecOp n;
    n.kind = ExecKind::RmsNorm;
    n.in0 = &o; n.in1 = &L.ffn_norm; n.out = &on; n.f0 = eps;
    ops.push_back(n);
    ops.push_back(mm_op(on, L.w_up, up));
    ExecOp g = mm_op(on, L.w_gate, gate);
    g.mm.epilogue.activation = Activation::Silu;
    g.mm.epilogue.binary = BinaryKind::Mul;
    g.mm.epilogue.d = &up;
    ops.push_back(g);
  }
  ExecOp d = mm_op(gate, L.w_down, x_out);
  if (add_residual) {
    d.mm.epilogue.binary = BinaryKind::AddScaled;
    d.mm.epilogue.d = &o;
    d.mm.epilogue.beta = 1.0f;
  }
  ops.push_back(d);
  if (tp) ops.push_back(all_reduce_op(m, x_out));
}

// lm_head on one normed row; sharded ranks gather their logit slices (rank order =
// vocabulary order) so that every rank takes the same argmax over the whole vocabulary.
void push_head_ops(ta_llama &m, std::vector<ExecOp> &ops, ExecOp head, bool decode) {
  if (m.world == 1) {
    head.mm.call.c = &m.logits;
    ops.push_back(head);
  } else if (decode && m.comm->fused_exchange_ready()) {
    // every rank folds its own slice and the ranks exchange one (value, index) pair each: no
    // gather of the vocabulary on the token path (ta_llama_logits gathers on demand)
    head.mm.call.c = &m.logits_l;
    ops.push_back(head);
    ExecOp am;
    am.kind = ExecKind::ArgmaxSharded;
    am.in0 = &m.logits_l; am.cell = &m.token_cell; am.comm = m.comm; am.u0 = m.rank * m.vocab_l;
    ops.push_back(am);
    m.logits_stale = true;
    return;
  } else {
    head.mm.call.c = &m.logits_l;
    ops.push_back(head);
    ExecOp ag;
    ag.kind = ExecKind::AllGather;
    ag.in0 = &m.logits_l; ag.out = &m.logits; ag.comm = m.comm;
    ops.push_back(ag);
  }
  ExecOp am;
  am.kind = ExecKind::Argmax;
  am.in0 = &m.logits; am.cell = &m.token_cell;
  ops.push_back(am);
}

// forward/decode.rs:172-246 decode_ops + forward/mod.rs:316-328 decode_close_ops,
// position-relative (pos_base 0 + *pos_cell).
// Op class of every entry of decode_ops(), in the reference's vocabulary for its
// LLAMA_ASH_BREAKDOWN table (tools/llama-ash/src/model/forward/*.rs `note(class, ..)`), plus the
// classes this runner has on top (collectives, argmax and the embedding gather run on the device).
std::vector<const char *> decode_op_classes(ta_llama &m) {
  std::vector<const char *> cls;
  const bool tp = m.world > 1;
  for (size_t l = 0; l < m.layers.size(); ++l) {
    for (int i = 0; i < 3; ++i) cls.push_back("qkv_matmul");
    cls.push_back("attn_decode");
    cls.push_back("o_proj_mm");
    if (tp) cls.push_back("all_reduce");
    cls.push_back("ffn_up_mm");
    cls.push_back("ffn_gate_mm");
    cls.push_back("ffn_down_mm");
    if (tp) cls.push_back("all_reduce");
  }
  cls.push_back("lm_head_mm");
  if (tp && !m.comm->fused_exchange_ready()) cls.push_back("all_gather");
  cls.push_back("argmax");
  cls.push_back("embed_gather");
  return cls;
}

std::vector<ExecOp> decode_ops(ta_llama &m) {
  const ta_llama_config &c = m.cfg;
  const float eps = c.rms_eps;
  const uint32_t dh = c.head_dim, t_max = c.t_max;
  std::vector<ExecOp> ops;
  const Tensor *x_in = &m.x_a, *x_out = &m.x_b;
  for (Layer &L : m.layers) {
    auto gemv = [&](const Tensor &w, const Tensor &out) {
      ExecOp o = mm_op(*x_in, w, out);
      o.mm.packed_b = true; o.mm.normed_weight = &L.attn_norm; o.mm.normed_eps = eps;
      o.mm.store.head_dim = dh; o.mm.store.pos_cell = &m.pos_cell;
      return o;
    };
    ExecOp q = gemv(L.wq_p, m.q);
    q.mm.store.kind = StoreKind::Rope; q.mm.store.table = &m.rope_table;
    ops.push_back(q);
    ExecOp k = gemv(L.wk_p, m.k);
    k.mm.store.kind = StoreKind::RopeScatter; k.mm.store.table = &m.rope_table; k.mm.store.dst = &L.kt_cache;
    k.mm.store.pos_scale = 1; k.mm.store.stride_head = dh * t_max; k.mm.store.stride_dim = t_max;
    ops.push_back(k);
    ExecOp v = gemv(L.wv_p, m.v);
    v.mm.store.kind = StoreKind::Scatter; v.mm.store.dst = &L.v_cache;
    v.mm.store.pos_scale = dh; v.mm.store.stride_head = t_max * dh; v.mm.store.stride_dim = 1;
    ops.push_back(v);
    ExecOp a;
    a.kind = ExecKind::AttnDecode;
    a.in0 = &m.q; a.in1 = &L.kt_cache; a.in2 = &L.v_cache; a.in3 = &m.attn_partials; a.out = &m.attn;
    a.attn.kv_len = 1; a.attn.scale = 1.0f / std::sqrt((float)dh); a.attn.pos_cell = &m.pos_cell;
    ops.push_back(a);
    push_mlp_ops(m, ops, L, true, m.attn, m.o, m.o, m.up, m.gate, *x_in, *x_out);
    std::swap(x_in, x_out);
  }
  ExecOp head = mm_op(*x_in, m.lm_head_p, m.logits);
  head.mm.packed_b = true; head.mm.normed_weight = &m.output_norm; head.mm.normed_eps = eps;
  push_head_ops(m, ops, head, true);
  ExecOp eg;
  eg.kind = ExecKind::EmbedGather;
  eg.cell = &m.token_cell; eg.in0 = &m.embd; eg.out = &m.x_a;
  ops.push_back(eg);
  return ops;
}

}  // namespace

// ------------------------------------------------------------------ prefill
namespace {


// Prefill activations are allocated once for t_max rows; a call works on
// views of their first n rows (same buffer, shorter shape).
PrefillScratch prefill_view(ta_llama &m, uint32_t n);

ExecOp copy_op(const Tensor &src, const Tensor &dst, std::array<uint32_t, 3> extent, uint32_t src_off,
               std::array<uint32_t, 3> ss, uint32_t dst_off, std::array<uint32_t, 3> ds) {
  ExecOp o;
  o.kind = ExecKind::CopyStrided;
  o.in0 = &src; o.out = &dst; o.src_offset = src_off; o.dst_offset = dst_off;
  for (int i = 0; i < 3; ++i) {
    o.extent[i] = extent[i];
    o.src_strides[i] = ss[i];
    o.strides[i] = ds[i];
  }
  return o;
}

// forward/prefill.rs:89-291 (f32 activations, fused QKV pack, fused flash).
std::vector<ExecOp> prefill_ops(ta_llama &m, PrefillScratch &s, uint32_t t, uint32_t pos_base) {
  const ta_llama_config &c = m.cfg;
  const uint32_t heads = m.heads_l, kv = m.kv_l, dh = c.head_dim, embd = c.embd;
  std::vector<ExecOp> ops;
  {
    ExecOp g;
    g.kind = ExecKind::EmbedGatherRows;
    g.tokens = &m.token_ids; g.in0 = &m.embd; g.out = &s.x_a;
    ops.push_back(g);
  }
  const Tensor *x_in = &s.x_a, *x_out = &s.x_b;
  for (Layer &L : m.layers) {
    ExecOp n;
    n.kind = ExecKind::RmsNorm;
    n.in0 = x_in; n.in1 = &L.attn_norm; n.out = &s.xn; n.f0 = c.rms_eps;
    ops.push_back(n);
    ops.push_back(mm_op(s.xn, L.w_qkv, s.qkv));
    {  // one launch: RoPE(q) head-major, RoPE(k) and v into the caches (forward/prefill.rs wide path)
      ExecOp pk;
      pk.kind = ExecKind::PrefillQkvPack;
      pk.in0 = &s.qkv; pk.in1 = &m.rope_table; pk.out = &s.q; pk.in2 = &L.kt_cache; pk.in3 = &L.v_cache;
      pk.heads = heads; pk.u0 = kv; pk.head_dim = dh; pk.rot_dim = dh; pk.pos_base = pos_base;
      ops.push_back(pk);
    }
    ExecOp f;
    f.kind = ExecKind::FlashAttn;
    f.in0 = &s.q; f.in1 = &L.kt_cache; f.in2 = &L.v_cache; f.out = &s.attn_flat;
    f.flash.kv_len = pos_base + t; f.flash.pos_base = pos_base; f.flash.scale = 1.0f / std::sqrt((float)dh);
    f.flash.out_token_major_heads = heads;   // head-major q, token-major out: Wo-ready
    ops.push_back(f);
    push_mlp_ops(m, ops, L, false, s.attn_flat, s.o, s.on, s.up, s.gate, *x_in, *x_out);
    std::swap(x_in, x_out);
  }
  // final norm + lm_head on the last row (forward/mod.rs:231-270), then argmax
  ops.push_back(copy_op(*x_in, s.last, {embd, 1, 1}, (t - 1) * embd, {1, 0, 0}, 0, {1, 0, 0}));
  ExecOp n;
  n.kind = ExecKind::RmsNorm;
  n.in0 = &s.last; n.in1 = &m.output_norm; n.out = &s.last_n; n.f0 = c.rms_eps;
  ops.push_back(n);
  push_head_ops(m, ops, mm_op(s.last_n, m.lm_head, m.logits), false);
  return ops;
}

PrefillScratch prefill_view(ta_llama &m, uint32_t n) {
  const ta_llama_config &c = m.cfg;
  const uint32_t kv_dim = m.kv_w;
  PrefillScratch &full = *m.prefill_full;
  if (full.x_a.shape.empty()) {
    auto f32 = [&](uint32_t cols) { return make(m.ctx, {c.t_max, cols}, DType::F32); };
    full.x_a = f32(c.embd); full.x_b = f32(c.embd); full.xn = f32(c.embd);
    full.qkv = f32(m.q_w + 2 * kv_dim);
    full.q = f32(m.q_w); full.k = f32(kv_dim); full.v = f32(kv_dim);
    full.attn_flat = f32(m.q_w); full.o = f32(c.embd); full.on = f32(c.embd);
    full.up = f32(m.ffn_l); full.gate = f32(m.ffn_l);
    full.last = make(m.ctx, {1, c.embd}, DType::F32);
    full.last_n = make(m.ctx, {1, c.embd}, DType::F32);
  }
  auto rows = [&](const Tensor &t, uint32_t cols) {   // the first n rows of a [t_max, cols] buffer
    Tensor v;
    v.buf = t.buf;
    v.shape = {n, cols};
    v.dtype = t.dtype;
    return v;
  };
  PrefillScratch s;
  s.x_a = rows(full.x_a, c.embd); s.x_b = rows(full.x_b, c.embd); s.xn = rows(full.xn, c.embd);
  s.qkv = rows(full.qkv, m.q_w + 2 * kv_dim);
  s.q = rows(full.q, m.q_w); s.k = rows(full.k, kv_dim); s.v = rows(full.v, kv_dim);
  s.q.shape = {m.heads_l, n, c.head_dim};   // head-major [H, T, dh] over the same n * q_w floats
  s.attn_flat = rows(full.attn_flat, m.q_w); s.o = rows(full.o, c.embd); s.on = rows(full.on, c.embd);
  s.up = rows(full.up, m.ffn_l); s.gate = rows(full.gate, m.ffn_l);
  s.last = full.last; s.last_n = full.last_n;
  return s;
}

int guarded(const std::function<void()> &f) {
  ta_set_last_error("");
  try {
    f();
    return 0;
  } catch (const std::exception &e) {
    ta_set_last_error(e.what());
  } catch (...) {
    ta_set_last_error("panic crossed tensor-ash C ABI boundary");
  }
  return -1;
}

void write_stats(ta_run_stats *out, const RunStats &st) {
  if (!out) return;
  out->has_gpu_time = st.gpu_time_ns ? 1u : 0u;
  out->gpu_time_ns = st.gpu_time_ns.value_or(0);
  out->n_calls = st.n_calls;
  out->total_flops = st.total_flops;
  const auto tf = st.tflops();
  out->tflops = tf ? *tf : std::nan("");
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

ta_llama *ta_llama_create_random(const ta_executor *exec, const ta_llama_config *cfg) {
  return ta_llama_create_random_tp(exec, cfg, nullptr);
}

ta_llama *ta_llama_create_random_tp(const ta_executor *exec, const ta_llama_config *cfg, const ta_comm *comm) {
  ta_llama *m = nullptr;
  const int rc = guarded([&]() {
    if (!exec) fail("ta_llama_create_random: exec is null");
    if (!cfg) fail("ta_llama_create_random: cfg is null");
    m = new ta_llama;
    m->prefill_full.reset(new PrefillScratch);
    if (comm) {
      if (comm->comm->ctx.get() != exec->ctx.get()) fail("ta_llama_create_random_tp: comm belongs to a different context");
      m->comm = comm->comm.get();
      m->rank = comm->comm->rank;
      m->world = comm->comm->world;
    }
    m->ctx = exec->ctx;
    m->exec = exec->exec.get();
    m->cfg = *cfg;
    m->ctx->make_current();
    RandomSource src(cfg->seed, cfg->weight_sigma, cfg->norm_jitter);
    build_model(*m, src);
  });
  if (rc != 0) {
    delete m;
    return nullptr;
  }
  return m;
}

// ------------------------------------------------------------------ GGUF inspection (host only)
struct ta_gguf {
  std::unique_ptr<GgufFile> file;
};

ta_gguf *ta_gguf_open(const char *path) {
  ta_gguf *h = nullptr;
  const int rc = guarded([&]() {
    if (!path) fail("ta_gguf_open: path is null");
    h = new ta_gguf;
    h->file.reset(new GgufFile(path));
  });
  if (rc != 0) {
    delete h;
    return nullptr;
  }
  return h;
}

void ta_gguf_close(ta_gguf *file) {
  ta_set_last_error("");
  delete file;
}

int ta_gguf_meta_kind(const ta_gguf *file, const char *key) {
  int kind = -1;
  guarded([&]() {
    if (!file || !key) fail("ta_gguf_meta_kind: file or key is null");
    if (const GgufValue *v = file->file->find(key)) kind = (int)v->kind;
  });
  return kind;
}

int ta_gguf_meta_u64(const ta_gguf *file, const char *key, uint64_t *out) {
  return guarded([&]() {
    if (!file || !key || !out) fail("ta_gguf_meta_u64: null argument");
    *out = file->file->require_u64(key);
  });
}

int ta_gguf_meta_f64(const ta_gguf *file, const char *key, double fallback, double *out) {
  return guarded([&]() {
    if (!file || !key || !out) fail("ta_gguf_meta_f64: null argument");
    *out = file->file->f64_or(key, fallback);
  });
}

int ta_gguf_meta_str(const ta_gguf *file, const char *key, char *buf, size_t cap) {
  return guarded([&]() {
    if (!file || !key || !buf || !cap) fail("ta_gguf_meta_str: null argument");
    const GgufValue *v = file->file->find(key);
    if (!v || v->kind != GgufValue::Str) fail("GGUF metadata missing string key %s", key);
    if (v->s.size() + 1 > cap) fail("ta_gguf_meta_str: value of %zu bytes does not fit %zu", v->s.size(), cap);
    memcpy(buf, v->s.c_str(), v->s.size() + 1);
  });
}

int ta_gguf_tensor_info(const ta_gguf *file, const char *name, uint64_t ne[4], uint32_t *n_dims,
                        uint32_t *ggml_type, uint64_t *offset) {
  return guarded([&]() {
    if (!file || !name || !ne || !n_dims) fail("ta_gguf_tensor_info: null argument");
    const GgufTensorInfo &ti = file->file->info(name);
    *n_dims = (uint32_t)ti.ne.size();
    for (size_t i = 0; i < 4; ++i) ne[i] = i < ti.ne.size() ? ti.ne[i] : 1;
    if (ggml_type) *ggml_type = ti.ggml_type;
    if (offset) *offset = ti.offset;
  });
}

int ta_gguf_read_f32(ta_gguf *file, const char *name, float *out, size_t len) {
  return guarded([&]() {
    if (!file || !name || !out) fail("ta_gguf_read_f32: null argument");
    const std::vector<float> v = file->file->read_f32(name);
    if (v.size() != len) fail("ta_gguf_read_f32: tensor %s has %zu elements, buffer holds %zu", name, v.size(), len);
    memcpy(out, v.data(), len * 4);
  });
}

uint64_t ta_gguf_data_start(const ta_gguf *file) { return file ? file->file->data_start() : 0; }

// tools/llama-ash/src/model/load.rs:14-120: architecture and geometry from the metadata, the
// vocabulary from the embedding tensor, t_max clamped to the model's context length.
ta_llama *ta_llama_load_gguf(const ta_executor *exec, const char *path, uint32_t t_max, const ta_comm *comm) {
  ta_llama *m = nullptr;
  const int rc = guarded([&]() {
    if (!exec) fail("ta_llama_load_gguf: exec is null");
    if (!path) fail("ta_llama_load_gguf: path is null");
    if (!t_max) fail("ta_llama_load_gguf: t_max must be non-zero");
    GgufFile g(path);
    const GgufValue *arch = g.find("general.architecture");
    if (!arch || arch->kind != GgufValue::Str) fail("GGUF missing general.architecture");
    if (arch->s != "llama") fail("unsupported architecture %s (want llama)", arch->s.c_str());
    ta_llama_config c{};
    c.layers = (uint32_t)g.require_u64("llama.block_count");
    c.embd = (uint32_t)g.require_u64("llama.embedding_length");
    c.heads = (uint32_t)g.require_u64("llama.attention.head_count");
    uint64_t kvh = c.heads;
    g.get_u64("llama.attention.head_count_kv", &kvh);
    c.kv_heads = (uint32_t)kvh;
    c.ffn = (uint32_t)g.require_u64("llama.feed_forward_length");
    const uint32_t ctx_len = (uint32_t)g.require_u64("llama.context_length");
    c.rms_eps = (float)g.f64_or("llama.attention.layer_norm_rms_epsilon", 1e-5);
    c.rope_theta = (float)g.f64_or("llama.rope.freq_base", 10000.0);
    if (!c.heads || c.embd % c.heads) fail("bad head geometry (embd %u, heads %u)", c.embd, c.heads);
    if (!c.kv_heads || c.heads % c.kv_heads) fail("heads must divide by kv_heads (%u / %u)", c.heads, c.kv_heads);
    c.head_dim = c.embd / c.heads;
    c.t_max = std::min(t_max, ctx_len);
    const GgufTensorInfo &ei = g.info("token_embd.weight");
    if (ei.ne.size() != 2 || ei.ne[0] != c.embd)
      fail("token_embd.weight ne [%s] does not match embd %u", GgufSource::ne_str(ei).c_str(), c.embd);
    c.vocab = (uint32_t)ei.ne[1];
    m = new ta_llama;
    m->prefill_full.reset(new PrefillScratch);
    if (comm) {
      if (comm->comm->ctx.get() != exec->ctx.get()) fail("ta_llama_load_gguf: comm belongs to a different context");
      m->comm = comm->comm.get();
      m->rank = comm->comm->rank;
      m->world = comm->comm->world;
    }
    m->ctx = exec->ctx;
    m->exec = exec->exec.get();
    m->cfg = c;
    m->ctx->make_current();
    GgufSource src(g);
    build_model(*m, src);
  });
  if (rc != 0) {
    delete m;
    return nullptr;
  }
  return m;
}

int ta_llama_get_config(const ta_llama *model, ta_llama_config *out) {
  return guarded([&]() {
    if (!model) fail("ta_llama_get_config: model is null");
    if (!out) fail("ta_llama_get_config: out is null");
    *out = model->cfg;
  });
}

void ta_llama_destroy(ta_llama *model) {
  ta_set_last_error("");
  delete model;
}

int ta_llama_reset(ta_llama *model) {
  return guarded([&]() {
    if (!model) fail("ta_llama_reset: model is null");
    model->pos = 0;
  });
}

int ta_llama_prefill(ta_llama *model, const uint32_t *tokens, uint32_t n, uint32_t *next_token,
                     ta_run_stats *stats) {
  return guarded([&]() {
    if (!model) fail("ta_llama_prefill: model is null");
    if (!tokens || n == 0) fail("ta_llama_prefill: prefill needs at least one token");
    ta_llama &m = *model;
    const ta_llama_config &c = m.cfg;
    if (m.pos + n > c.t_max) fail("ta_llama_prefill: KV cache overflow (%u + %u > %u)", m.pos, n, c.t_max);
    m.ctx->make_current();
    PrefillScratch s = prefill_view(m, n);
    memcpy(m.token_ids.host, tokens, (size_t)n * 4);
    m.token_ids.len = n;
    const RunStats st = m.exec->run_exec_ops(prefill_ops(m, s, n, m.pos));
    m.pos += n;
    m.pos_last_decode = false;
    if (next_token) *next_token = *(volatile uint32_t *)m.token_cell.host;
    write_stats(stats, st);
  });
}

int ta_llama_decode(ta_llama *model, uint32_t first_token, uint32_t n, uint32_t *out_tokens,
                    ta_run_stats *stats) {
  return guarded([&]() {
    if (!model) fail("ta_llama_decode: model is null");
    ta_llama &m = *model;
    if (n && !out_tokens) fail("ta_llama_decode: out_tokens is null");
    if (m.pos + n > m.cfg.t_max) fail("ta_llama_decode: KV cache overflow (%u + %u > %u)", m.pos, n, m.cfg.t_max);
    m.ctx->make_current();
    RunStats total;
    total.gpu_time_ns = 0;
    if (n == 0) { write_stats(stats, total); return; }
    // first input embedding: gather on the device from the token word
    *(volatile uint32_t *)m.token_cell.host = first_token;
    m.exec->embed_gather(m.token_cell, m.embd, m.x_a);
    if (!m.decode_graph) m.decode_graph = prepare_exec_ops(*m.exec, decode_ops(m));   // records only
    for (uint32_t i = 0; i < n; ++i) {
      *(volatile uint32_t *)m.pos_cell.host = m.pos;
      const RunStats st = m.decode_graph->run();
      out_tokens[i] = *(volatile uint32_t *)m.token_cell.host;
      m.pos += 1;
      m.pos_last_decode = true;
      *total.gpu_time_ns += st.gpu_time_ns.value_or(0);
      total.n_calls += st.n_calls;
      total.total_flops += st.total_flops;
    }
    write_stats(stats, total);
  });
}

int ta_llama_decode_breakdown(ta_llama *model, uint32_t token, ta_llama_breakdown_row *rows, size_t cap,
                              size_t *n_rows, size_t *n_launches, uint32_t *next_token) {
  return guarded([&]() {
    if (!model) fail("ta_llama_decode_breakdown: model is null");
    if (!rows || !n_rows) fail("ta_llama_decode_breakdown: rows / n_rows is null");
    ta_llama &m = *model;
    if (m.pos + 1 > m.cfg.t_max) fail("ta_llama_decode_breakdown: KV cache overflow (%u + 1 > %u)", m.pos, m.cfg.t_max);
    m.ctx->make_current();
    *(volatile uint32_t *)m.token_cell.host = token;
    m.exec->embed_gather(m.token_cell, m.embd, m.x_a);
    *(volatile uint32_t *)m.pos_cell.host = m.pos;
    const std::vector<ExecOp> ops = decode_ops(m);
    const std::vector<const char *> cls = decode_op_classes(m);
    if (cls.size() != ops.size()) fail("internal: %zu op classes for %zu decode ops", cls.size(), ops.size());
    std::vector<std::pair<size_t, uint64_t>> per_launch;
    m.exec->run_exec_ops_timed(ops, &per_launch);
    m.pos += 1;
    m.pos_last_decode = true;
    if (next_token) *next_token = *(volatile uint32_t *)m.token_cell.host;
    if (n_launches) *n_launches = per_launch.size();
    // a launch that fuses several ops (q, k, v; up + gate) is booked under its first op's class
    std::vector<ta_llama_breakdown_row> acc;
    for (const auto &pl : per_launch) {
      const char *name = cls[pl.first];
      size_t i = 0;
      while (i < acc.size() && strcmp(acc[i].op_class, name)) ++i;
      if (i == acc.size()) acc.push_back(ta_llama_breakdown_row{name, 0, 0});
      acc[i].gpu_ns += pl.second;
      acc[i].calls += 1;
    }
    std::sort(acc.begin(), acc.end(), [](const ta_llama_breakdown_row &a, const ta_llama_breakdown_row &b) { return a.gpu_ns > b.gpu_ns; });
    *n_rows = acc.size();
    for (size_t i = 0; i < acc.size() && i < cap; ++i) rows[i] = acc[i];
  });
}

int ta_llama_logits(ta_llama *model, float *out, size_t len) {
  return guarded([&]() {
    if (!model) fail("ta_llama_logits: model is null");
    if (!out) fail("ta_llama_logits: out is null");
    ta_llama &m = *model;
    if (m.world > 1 && m.logits_stale && m.pos_last_decode) {
      // the sharded decode step keeps only this rank's slice: gather now (collective: every rank calls)
      ExecOp ag;
      ag.kind = ExecKind::AllGather;
      ag.in0 = &m.logits_l; ag.out = &m.logits; ag.comm = m.comm;
      m.exec->run_exec_ops({ag});
    }
    m.exec->download(m.logits, out, std::min(len, (size_t)m.cfg.vocab));
  });
}

uint32_t ta_llama_position(const ta_llama *model) { return model ? model->pos : 0; }

// benchmarks/THESES.md:46-50 formula: f16 bytes of every matrix read per token
uint64_t ta_llama_weight_bytes_per_token(const ta_llama *model) {
  if (!model) return 0;
  const ta_llama_config &c = model->cfg;
  const uint64_t per_layer = 2ull * c.embd * model->q_w + 2ull * c.embd * model->kv_w + 3ull * c.embd * model->ffn_l;
  return 2ull * (c.layers * per_layer + (uint64_t)c.embd * model->vocab_l);
}

}  // extern "C"
#pragma GCC visibility pop
