// Pure host logic: error helpers, f16 conversion, shape resolution, kernel
// registry, routing heuristics, packed-weight layout, tuned-winner store.
// Nothing here touches a device, so it is exercised on machines without one.
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <functional>
#include <sstream>
#include <tuple>

#include "ta_core.hpp"

namespace ta {

std::atomic<uint64_t> g_launches{0};

// ------------------------------------------------------------------ errors
static std::string vstrf(const char *fmt, va_list ap) {
  va_list ap2;
  va_copy(ap2, ap);
  int n = vsnprintf(nullptr, 0, fmt, ap2);
  va_end(ap2);
  std::string s((size_t)(n > 0 ? n : 0), '\0');
  if (n > 0) vsnprintf(s.data(), (size_t)n + 1, fmt, ap);
  return s;
}

std::string strf(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  std::string s = vstrf(fmt, ap);
  va_end(ap);
  return s;
}

void fail(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  std::string s = vstrf(fmt, ap);
  va_end(ap);
  throw Error(s);
}

// ------------------------------------------------------------------ experiment switches
Tunables parse_tunables(const char *spec) {
  Tunables t;
  if (!spec) return t;
  std::string all(spec);
  size_t pos = 0;
  while (pos < all.size()) {
    size_t end = all.find(',', pos);
    if (end == std::string::npos) end = all.size();
    std::string item = all.substr(pos, end - pos);
    pos = end + 1;
    while (!item.empty() && isspace((unsigned char)item.front())) item.erase(item.begin());
    while (!item.empty() && isspace((unsigned char)item.back())) item.pop_back();
    if (item.empty()) continue;
    const size_t eq = item.find('=');
    if (eq == std::string::npos) fail("TA_EXPERIMENT: '%s' is not name=value", item.c_str());
    const std::string name = item.substr(0, eq);
    const long v = strtol(item.c_str() + eq + 1, nullptr, 10);
    if (name == "tf32x3_chunk_kb") t.tf32x3_chunk_kb = v > 0 ? (uint32_t)v : 0;
    else if (name == "tf32x3_ksplit") t.tf32x3_ksplit = (int)v;
    else if (name == "gemv_ksplit") t.gemv_ksplit = (int)v;
    else if (name == "gemv_bulk") t.gemv_bulk = (int)v;
    else if (name == "gemv_umma") t.gemv_umma = (int)v;
    else if (name == "f16w_pre") t.f16w_pre = v != 0;
    else if (name == "f16w_apad") t.f16w_apad = (uint32_t)(v > 0 ? v : 0) & ~7u;
    else if (name == "pdl") t.pdl = v != 0;
    else if (name == "peer_allreduce") t.peer_allreduce = v != 0;
    else if (name == "peer_allreduce_big") t.peer_allreduce_big = v != 0;
    else if (name == "splitk2_tensor") t.splitk2_tensor = v != 0;
    else if (name == "f16w_splitk") t.f16w_splitk = (int)v;
    else if (name == "f16w_bn") t.f16w_bn = (uint32_t)v;
    else if (name == "f16w_tma_store") t.f16w_tma_store = v != 0;
    else if (name == "f16w_dual") t.f16w_dual = v != 0;
    else if (name == "pos_stage") t.pos_stage = v != 0;
    else if (name == "attn_pairs") t.attn_pairs = v != 0;
    else if (name == "attn_wide") t.attn_wide = v != 0;
    else if (name == "gemv_handoff") t.gemv_handoff = v != 0;
    else if (name == "gemv_peer_wide") t.gemv_peer_wide = v != 0;
    else if (name == "flash_groups") t.flash_groups = v == 1 ? 1u : 2u;
    else if (name == "attn_chunks") t.attn_chunks = (uint32_t)std::max(0l, std::min(32l, v));
    else
      fail("TA_EXPERIMENT: unknown switch '%s' (known: tf32x3_chunk_kb, tf32x3_ksplit, gemv_ksplit, gemv_bulk, gemv_umma, "
           "f16w_pre, f16w_apad, pdl, peer_allreduce, peer_allreduce_big, splitk2_tensor, f16w_splitk, f16w_bn, f16w_tma_store, f16w_dual, attn_chunks, pos_stage, flash_groups, attn_pairs, attn_wide, gemv_handoff, gemv_peer_wide)", name.c_str());
  }
  return t;
}

const Tunables &tunables() {
  static const Tunables t = parse_tunables(getenv("TA_EXPERIMENT"));
  return t;
}

// ------------------------------------------------------------------ f16 (src/dtype.rs:42-112)
static inline uint32_t bits_of(float v) {
  uint32_t b;
  memcpy(&b, &v, 4);
  return b;
}
static inline float float_of(uint32_t b) {
  float v;
  memcpy(&v, &b, 4);
  return v;
}

uint16_t f32_to_f16_bits(float value) {
  const uint32_t bits = bits_of(value);
  const uint32_t sign = (bits >> 16) & 0x8000u;
  const int32_t exp = (int32_t)((bits >> 23) & 0xffu);
  const uint32_t frac = bits & 0x007fffffu;
  if (exp == 0xff) return (uint16_t)(sign | 0x7c00u | (frac ? 0x0200u : 0u));
  const int32_t e = exp - 127;
  if (e >= 16) return (uint16_t)(sign | 0x7c00u);
  if (e >= -14) {
    // normal half: keep 10 fraction bits, round the 13 dropped ones to even
    uint32_t out = sign | ((uint32_t)(e + 15) << 10) | (frac >> 13);
    const uint32_t dropped = frac & 0x1fffu;
    if (dropped > 0x1000u || (dropped == 0x1000u && (out & 1u))) out += 1;  // carry is right
    return (uint16_t)out;
  }
  if (e >= -25) {
    // subnormal half: shift the 24-bit significand into place, round to even
    const uint32_t sig = frac | 0x00800000u;
    const uint32_t sh = (uint32_t)(-14 - e) + 13;
    uint32_t out = sign | (sig >> sh);
    const uint32_t dropped = sig & ((1u << sh) - 1u);
    const uint32_t half = 1u << (sh - 1);
    if (dropped > half || (dropped == half && (out & 1u))) out += 1;
    return (uint16_t)out;
  }
  return (uint16_t)sign;
}

float f16_bits_to_f32(uint16_t h) {
  const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1fu;
  const uint32_t frac = h & 0x03ffu;
  if (exp == 0) {
    if (frac == 0) return float_of(sign);
    const uint32_t lz = (uint32_t)__builtin_clz(frac) - 22;  // leading zeros within 10 bits
    return float_of(sign | ((127 - 15 - lz) << 23) | (((frac << (lz + 1)) & 0x03ffu) << 13));
  }
  if (exp == 0x1f) return float_of(sign | (frac ? 0x7fc00000u | (frac << 13) : 0x7f800000u));
  return float_of(sign | ((exp + 112) << 23) | (frac << 13));
}

// ------------------------------------------------------------------ tensor shape checks
uint64_t Tensor::numel_checked(const uint32_t *shape, size_t rank) {
  if (rank == 0) fail("tensor shape must have at least one dimension");
  uint64_t n = 1;
  for (size_t i = 0; i < rank; ++i) {
    if (shape[i] == 0) fail("tensor dimension %zu must be non-zero", i);
    if (__builtin_mul_overflow(n, (uint64_t)shape[i], &n)) fail("tensor element count overflows u64");
  }
  return n;
}

std::string Tensor::shape_str() const {
  std::string s = "[";
  for (size_t i = 0; i < shape.size(); ++i) s += (i ? ", " : "") + std::to_string(shape[i]);
  return s + "]";
}

static std::string shape_str(const std::vector<uint32_t> &shape) {
  std::string s = "[";
  for (size_t i = 0; i < shape.size(); ++i) s += (i ? ", " : "") + std::to_string(shape[i]);
  return s + "]";
}

// ------------------------------------------------------------------ resolution
// (src/matmul/resolution.rs:16-76, 123-212, 217-351, 421-476)
MatrixShape MatrixShape::from_shape(const uint32_t *shape, size_t rank) {
  MatrixShape s{};
  if (rank == 2) s = {1, shape[0], shape[1]};
  else if (rank == 3) s = {shape[0], shape[1], shape[2]};
  else fail("tensor rank %zu not supported by matmul (must be 2 or 3)", rank);
  if (s.batch == 0 || s.rows == 0 || s.cols == 0)
    fail("matmul dimensions must be non-zero, got B=%u rows=%u cols=%u", s.batch, s.rows, s.cols);
  return s;
}

uint32_t MatrixShape::batch_stride(const char *label) const {
  const uint64_t plane = (uint64_t)rows * cols;  // u32*u32 cannot overflow u64
  uint32_t stride = 0;
  if (batch != 1) {
    if (plane > 0xffffffffull) fail("%s batch stride overflows u32", label);
    stride = (uint32_t)plane;
  }
  // Kernel index arithmetic is 32-bit per plane set: a contiguous layout is
  // addressable while its element count is at most 2^32.
  uint64_t total;
  const bool ok = !__builtin_mul_overflow((uint64_t)batch, plane, &total) && total <= (1ull << 32);
  if (!ok)
    fail("%s layout exceeds shader u32 indexing: B=%u rows=%u cols=%u", label, batch, rows, cols);
  return stride;
}

static void ensure_dim_eq(const char *ll, uint32_t l, const char *rl, uint32_t r) {
  if (l != r) fail("matmul shape mismatch: %s=%u vs %s=%u", ll, l, rl, r);
}
static void ensure_broadcastable(const char *label, uint32_t in_b, uint32_t out_b) {
  if (in_b != 1 && in_b != out_b)
    fail("matmul incompatible batch dims: %s.B=%u cannot broadcast to C.B=%u", label, in_b, out_b);
}

ResolvedMatmul ResolvedMatmul::from_shapes(MatrixShape a, MatrixShape b, MatrixShape c) {
  ensure_dim_eq("A.K", a.cols, "B.K", b.rows);
  ensure_dim_eq("A.M", a.rows, "C.M", c.rows);
  ensure_dim_eq("B.N", b.cols, "C.N", c.cols);
  ensure_broadcastable("A", a.batch, c.batch);
  ensure_broadcastable("B", b.batch, c.batch);
  ResolvedMatmul r;
  r.m = a.rows;
  r.n = b.cols;
  r.k = a.cols;
  r.batch = c.batch;
  r.batch_stride_a = a.batch_stride("A");
  r.batch_stride_b = b.batch_stride("B");
  r.batch_stride_c = c.batch_stride("C");
  uint64_t f = 2;
  for (uint64_t v : {(uint64_t)c.batch, (uint64_t)a.rows, (uint64_t)b.cols, (uint64_t)a.cols})
    if (__builtin_mul_overflow(f, v, &f)) fail("matmul FLOP count overflows u64");
  r.total_flops = f;
  return r;
}

static MatrixShape shape_of(const Tensor &t) {
  return MatrixShape::from_shape(t.shape.data(), t.shape.size());
}

ResolvedMatmul ResolvedMatmul::from_call(const MatmulCall &call) {
  const bool a_f16 = call.a->dtype == DType::F16;
  if (a_f16) {
    if (call.b->dtype != DType::F16)
      fail("matmul with f16 A storage requires f16 B (got %s)", dtype_name(call.b->dtype));
    if (call.c->dtype != DType::F16)
      fail("matmul with f16 A storage requires f16 C (got %s)", dtype_name(call.c->dtype));
  } else if (call.c->dtype != DType::F32) {
    fail("matmul C must be f32 storage (got %s)", dtype_name(call.c->dtype));
  }
  ResolvedMatmul r = from_shapes(shape_of(*call.a), shape_of(*call.b), shape_of(*call.c));
  r.b_f16 = call.b->dtype == DType::F16;
  r.a_f16 = a_f16;
  if (a_f16 && (r.m % 64 || r.n % 64 || r.k % 32))
    fail("matmul with f16 A storage routes to the aligned coopmat kernels only: M/N/K must be "
         "multiples of (64, 64, 32), got (%u, %u, %u)", r.m, r.n, r.k);
  return r;
}

void ResolvedMatmul::validate_bias_shape(const std::vector<uint32_t> &shape) const {
  const bool shared = shape.size() == 1 && shape[0] == n;
  const bool batched = shape.size() == 2 && shape[0] == batch && shape[1] == n;
  if (!shared && !batched)
    fail("epilogue bias shape %s, expected [%u] or [%u, %u]", shape_str(shape).c_str(), n, batch, n);
}

ResolvedMatmul ResolvedMatmul::from_op(const MatmulOp &op) {
  ResolvedMatmul r = from_call(op.call);
  r.packed_b = op.packed_b;
  if (op.packed_b) {
    // The reference restricts packed B to M == 1 (resolution.rs:176-196); this
    // build's GEMV kernel walks up to 8 activation rows per weight pass, so the
    // limit is M <= 8.  Everything else is unchanged.
    if (r.m > 8 || r.batch != 1)
      fail("packed-B GEMV requires M <= 8 and batch == 1 (got M=%u, batch=%u)", r.m, r.batch);
    if (!r.b_f16) fail("packed-B GEMV requires f16 weights");
    if (r.a_f16) fail("packed-B GEMV does not support f16 activations");
    if (r.n % 32) fail("packed-B GEMV requires N to be a multiple of 32 (got %u)", r.n);
  }
  if (r.a_f16 && (!op.epilogue.is_none() || op.normed_weight || !op.store.is_none()))
    fail("matmul with f16 A storage cannot fuse epilogues, normed-A, or store ops (the coopmat "
         "route has no fused specializations)");
  // epilogue (resolution.rs:315-351)
  if (op.epilogue.bias) {
    r.validate_bias_shape(op.epilogue.bias->shape);
    if (op.epilogue.bias->dtype != DType::F32) fail("epilogue bias must be f32 storage");
  }
  if (op.epilogue.d) {
    if (op.epilogue.d->shape != op.call.c->shape)
      fail("epilogue D shape %s must equal C shape %s", op.epilogue.d->shape_str().c_str(),
           op.call.c->shape_str().c_str());
    if (op.epilogue.d->dtype != DType::F32) fail("epilogue D operand must be f32 storage");
  }
  // normed-A (resolution.rs:217-247)
  if (op.normed_weight) {
    if (op.normed_weight->dtype != DType::F32) fail("normed-A weight must be f32 storage");
    if (op.normed_weight->len() != r.k)
      fail("normed-A weight length %llu must equal K = %u",
           (unsigned long long)op.normed_weight->len(), r.k);
    if (op.epilogue.bias)
      fail("normed-A cannot combine with an epilogue bias (both use the bias slot)");
    if (op.epilogue.binary == BinaryKind::AddScaled)
      fail("normed-A cannot combine with the AddScaled epilogue (both use beta)");
  }
  // fused store (resolution.rs:249-313)
  if (!op.store.is_none()) {
    const MatmulStore &s = op.store;
    if (r.m != 1 || r.batch != 1)
      fail("fused store epilogue requires M == 1 and batch == 1 (got M=%u, batch=%u)", r.m, r.batch);
    if (!r.b_f16) fail("fused store epilogue requires f16 weights (f16w row-GEMV routes only)");
    if (op.call.accumulate) fail("fused store epilogue cannot combine with accumulate");
    if (!op.epilogue.is_none()) fail("fused store epilogue cannot combine with a fused epilogue");
    if (s.head_dim == 0 || s.head_dim % 2 || r.n % s.head_dim)
      fail("store head_dim %u must be even and divide N = %u", s.head_dim, r.n);
    const bool wants_table = s.kind == StoreKind::Rope || s.kind == StoreKind::RopeScatter;
    const bool wants_dst = s.kind == StoreKind::Scatter || s.kind == StoreKind::RopeScatter;
    if (wants_table) {
      if (!s.table) fail("store rope table is null");
      if (s.table->dtype != DType::F32) fail("store rope table must be f32 storage");
      const uint64_t needed = ((uint64_t)s.pos_base + 1) * s.head_dim;
      if (s.table->len() < needed)
        fail("store rope table len %llu does not cover pos_base %u (needs %llu)",
             (unsigned long long)s.table->len(), s.pos_base, (unsigned long long)needed);
    }
    if (wants_dst) {
      if (!s.dst) fail("store destination is null");
      const uint32_t heads = r.n / s.head_dim;
      const uint64_t last = (uint64_t)s.pos_base * s.pos_scale +
                            (uint64_t)(heads - 1) * s.stride_head +
                            (uint64_t)(s.head_dim - 1) * s.stride_dim;
      if (last >= s.dst->len())
        fail("store destination access %llu out of bounds for len %llu (pos_base %u, N %u, "
             "head_dim %u)", (unsigned long long)last, (unsigned long long)s.dst->len(),
             s.pos_base, r.n, s.head_dim);
    }
  }
  return r;
}

// ------------------------------------------------------------------ registry
// Order is stable: indices are persisted by name only, but tests and the tuner
// iterate in this order.  Aliases keep every ML_KERNEL spelling of the
// reference (src/pipeline/catalog.rs:205-376) resolving to the CUDA variant
// that supersedes that shader.

static const char *const A_TF32_256[] = {"tf32x3_m128n256", "tf32x3", "tensor", nullptr};
static const char *const A_TF32_128[] = {"tf32x3_m128n128", nullptr};
static const char *const A_FFMA_128[] = {
    "ffma_m128n128", "ffma", "large", "large_128", "128", "large_bda", "128x128_bda",
    "large_bda_v4", "large_bda_v4_aligned", "128x128_bda_v4_aligned", "bk16", "128x128bk16",
    "bk16_bda_v4", "128x128bk16_bda_v4", "v2", "128x128bk8", "sota", "v3", "128x128bk8static",
    "m128n128_t4", "128x128_t4", "m256n64", "256x64", "m128n64", "128x64", "tall", "m128n64_bda",
    "m128n64_bda_v4", "m128n64k64", "128x64k64", "m128n64k64_bda", "128x64k64_bda",
    "m128n64k64_bda_v4", "m128n64k64_bda_v4_tm8_tn8", "m128n64k64_bda_v4_tm16_tn4",
    "m128n64k64_bda_v4_aligned", "m64n128", "64x128", "wide", "m64n128_bda", "m64n128_bda_v4",
    "m64n128k64", "64x128k64", nullptr};
static const char *const A_TF32_PAIR[] = {"tf32x3_m256n256", "tf32x3_pair", "tf32x3_2cta", nullptr};
static const char *const A_FFMA_64[] = {
    "ffma_m64n64", "small", "small_64", "64", "small_bda", "64_bda", "small_bda_v4", "k64",
    "small_k64", "64k", "k64_bda", "k64_bda_v4", "k64_bda_v4_tm8_tn4", "k64_bda_v4_tm4_tn8",
    "k64_bda_v4_tm8_tn8", "m64n32", "64x32", "m64n32_bda", "64x32_bda", "col_bda", "col",
    "gemv_col_bda", "outer_bda", "outer", "k1", nullptr};
static const char *const A_F16W_FFMA_128[] = {
    "f16w_ffma_m128n128", "f16w_large_bda_v4", "f16w_large", "f16w_m128n64k64_bda_v4",
    "f16w_m128n64k64", nullptr};
static const char *const A_F16W_FFMA_64[] = {
    "f16w_ffma_m64n64", "f16w_small_bda_v4", "f16w_small", "f16w_k64_bda_v4", "f16w_k64", nullptr};
static const char *const A_F16W_UMMA[] = {
    "f16w_umma_m128n256", "f16w_umma", "f16w_coopmat_aligned", "f16w_coopmat", "coopmat",
    "f16w_cm2", "cm2", "cm2_gemm", nullptr};
static const char *const A_F16W_UMMA_128[] = {
    "f16w_umma_m128n128", "f16w_coopmat_m64n128", "coopmat_m64n128", nullptr};
static const char *const A_F16W_UMMA_64[] = {
    "f16w_umma_m128n64", "f16w_coopmat_m64n64", "coopmat_m64", "f16w_coopmat_m128n64",
    "coopmat_m128n64", nullptr};
static const char *const A_ROW[] = {"row_bda", "row", "gemv_bda", nullptr};
static const char *const A_F16W_ROW[] = {"f16w_row_bda", "f16w_row", nullptr};
static const char *const A_F16W_ROW_K16[] = {"f16w_row_bda_k16", "f16w_row_k16", nullptr};
static const char *const A_F16W_ROW_K16V2[] = {"f16w_row_bda_k16_v2", "f16w_row_k16_v2", nullptr};
static const char *const A_F16W_ROW_K16P[] = {"f16w_row_bda_k16_packed", "f16w_row_k16_packed",
                                              nullptr};
static const char *const A_F16W_ROW_K16V2P[] = {"f16w_row_bda_k16_v2_packed",
                                                "f16w_row_k16_v2_packed", nullptr};
static const char *const A_SK_128[] = {"split_k2_m128n128", nullptr};
static const char *const A_SK_64[] = {"split_k2_m64n64", nullptr};

const KernelSpec KERNEL_SPECS[] = {
    {"tf32x3_m256n256", 256, 256, 16, Family::Tf32x3, false, A_TF32_PAIR},
    {"tf32x3_m128n256", 128, 256, 16, Family::Tf32x3, false, A_TF32_256},
    {"tf32x3_m128n128", 128, 128, 16, Family::Tf32x3, false, A_TF32_128},
    {"ffma_m128n128", 128, 128, 16, Family::Ffma, false, A_FFMA_128},
    {"ffma_m64n64", 64, 64, 16, Family::Ffma, false, A_FFMA_64},
    {"f16w_ffma_m128n128", 128, 128, 16, Family::Ffma, true, A_F16W_FFMA_128},
    {"f16w_ffma_m64n64", 64, 64, 16, Family::Ffma, true, A_F16W_FFMA_64},
    {"f16w_umma_m128n256", 128, 256, 32, Family::F16wUmma, true, A_F16W_UMMA},
    {"f16w_umma_m128n128", 128, 128, 32, Family::F16wUmma, true, A_F16W_UMMA_128},
    {"f16w_umma_m128n64", 128, 64, 32, Family::F16wUmma, true, A_F16W_UMMA_64},
    {"row_bda", 1, 32, 1, Family::RowGemv, false, A_ROW},
    {"f16w_row_bda", 1, 32, 1, Family::RowGemv, true, A_F16W_ROW},
    {"f16w_row_bda_k16", 1, 32, 1, Family::RowGemv, true, A_F16W_ROW_K16},
    {"f16w_row_bda_k16_v2", 1, 64, 1, Family::RowGemv, true, A_F16W_ROW_K16V2},
    {"f16w_row_bda_k16_packed", 1, 32, 1, Family::RowGemv, true, A_F16W_ROW_K16P},
    {"f16w_row_bda_k16_v2_packed", 1, 64, 1, Family::RowGemv, true, A_F16W_ROW_K16V2P},
    {"split_k2_m128n128", 128, 128, 32, Family::SplitK2, false, A_SK_128},
    {"split_k2_m64n64", 64, 64, 32, Family::SplitK2, false, A_SK_64},
};
const size_t KERNEL_SPEC_COUNT = sizeof(KERNEL_SPECS) / sizeof(KERNEL_SPECS[0]);

int kernel_index_by_name(const char *name) {
  for (size_t i = 0; i < KERNEL_SPEC_COUNT; ++i)
    if (!strcmp(KERNEL_SPECS[i].name, name)) return (int)i;
  return -1;
}

int kernel_selection_parse(const std::string &value) {
  // trim + lowercase (catalog.rs:165)
  size_t b = 0, e = value.size();
  while (b < e && isspace((unsigned char)value[b])) ++b;
  while (e > b && isspace((unsigned char)value[e - 1])) --e;
  std::string v = value.substr(b, e - b);
  for (char &ch : v) ch = (char)tolower((unsigned char)ch);
  if (v.empty() || v == "auto") return -2;
  for (size_t i = 0; i < KERNEL_SPEC_COUNT; ++i)
    for (const char *const *al = KERNEL_SPECS[i].aliases; *al; ++al)
      if (v == *al) return (int)i;
  fail("invalid ML_KERNEL '%s', expected one of auto, tf32x3, ffma, large, small, m64n128, m128n64, "
       "m128n64k64, m64n32, k64, row_bda, col_bda, outer_bda, bk16, v2, m64n128k64, m128n128_t4, "
       "m256n64, v3, any *_bda / *_bda_v4 variant, or an f16w_* kernel (f16 weights)", v.c_str());
}

// ------------------------------------------------------------------ row GEMV routing
bool f16w_row_uses_k16(uint32_t k, uint32_t n) {
  return k >= 4096 || n <= 512 || (k >= 2048 && n <= 2048);
}
uint32_t f16w_row_tile_n(uint32_t k, uint32_t n) {
  return (f16w_row_uses_k16(k, n) || n % 64 != 0) ? 32 : 64;
}

// ------------------------------------------------------------------ split-K heuristics
static inline uint64_t ceil_div64(uint64_t a, uint64_t b) { return a / b + (a % b != 0); }
static inline uint64_t sat_mul64(uint64_t a, uint64_t b) {
  uint64_t r;
  return __builtin_mul_overflow(a, b, &r) ? UINT64_MAX : r;
}

void splitk2_stage1_tile(uint32_t m, uint32_t n, const char **name, uint32_t tile[3]) {
  if (m >= 128 && n >= 128) {
    *name = "split_k2_m128n128";
    tile[0] = 128; tile[1] = 128; tile[2] = 32;
  } else {
    *name = "split_k2_m64n64";
    tile[0] = 64; tile[1] = 64; tile[2] = 32;
  }
}

uint32_t default_num_k_splits(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, uint32_t tile_m,
                              uint32_t tile_n) {
  if (tile_m == 0 || tile_n == 0) return 1;
  const uint64_t tiles = sat_mul64(sat_mul64(ceil_div64(m, tile_m), ceil_div64(n, tile_n)),
                                  (uint64_t)(batch ? batch : 1));
  if (tiles == 0) return 1;
  const uint64_t want = std::max<uint64_t>(ceil_div64(64, tiles), 1);
  const uint64_t cap = std::max<uint64_t>((uint64_t)k / 32, 1);
  return (uint32_t)std::min(want, cap);
}

std::optional<uint32_t> heuristic_splits(uint32_t batch, uint32_t m, uint32_t n, uint32_t k) {
  if (batch == 0 || m <= 1 || n <= 1 || k < 1024) return std::nullopt;
  const bool big = m >= 128 && n >= 128;
  const uint32_t tile = big ? 128 : 64;
  const uint64_t tiles = sat_mul64(sat_mul64(batch, ceil_div64(m, tile)), ceil_div64(n, tile));
  uint64_t target;
  uint32_t min_k_per_split;
  if (big) {
    uint32_t min_k;
    if (tiles == 1) min_k = 1024;
    else if (tiles <= 4) min_k = 2048;
    else if (tiles <= 16) min_k = 4096;
    else return std::nullopt;
    if (k < min_k) return std::nullopt;
    target = (tiles >= 9 && k >= 8192) ? 128 : 64;
    min_k_per_split = 128;
  } else {
    if (tiles > 4) return std::nullopt;
    target = 128;
    min_k_per_split = 64;
  }
  const uint64_t wanted = ceil_div64(target, tiles);
  uint32_t max_splits = k / min_k_per_split;
  if (big && tiles == 1) max_splits = std::max(max_splits, 16u);
  for (uint32_t s : {64u, 32u, 16u, 8u, 4u})
    if (s <= wanted && s <= max_splits) return s;
  return std::nullopt;
}

// ------------------------------------------------------------------ packed weights
void pack_f16w_row_tiles(const float *src, float *dst, size_t k, size_t n, size_t tile_n) {
  if (tile_n == 0 || n % tile_n) fail("N=%zu is not a multiple of tile_n=%zu", n, tile_n);
  const size_t tiles = n / tile_n;
  for (size_t t = 0; t < tiles; ++t)
    for (size_t kk = 0; kk < k; ++kk)
      memcpy(dst + (t * k + kk) * tile_n, src + kk * n + t * tile_n, tile_n * sizeof(float));
}

// ------------------------------------------------------------------ tuner arithmetic
std::optional<uint64_t> tune_median(std::vector<uint64_t> v) {
  if (v.empty()) return std::nullopt;
  std::sort(v.begin(), v.end());
  const size_t mid = v.size() / 2;
  if (v.size() % 2 == 0) return (uint64_t)(((unsigned __int128)v[mid - 1] + v[mid]) / 2);
  return v[mid];
}

size_t tune_candidate_at(size_t len, uint32_t round, size_t offset) {
  if (round == 0) return offset;
  const size_t pair = (round - 1) / 2;
  const size_t start = pair * ((len + 1) / 2) % len;
  if (round % 2) return (start + offset) % len;
  return (start + len - 1 - offset) % len;
}

// ------------------------------------------------------------------ tuned-winner store
uint64_t registry_hash() {
  uint64_t h = 1469598103934665603ull;  // FNV-1a over names and tiles
  for (size_t i = 0; i < KERNEL_SPEC_COUNT; ++i) {
    for (const char *p = KERNEL_SPECS[i].name; *p; ++p) { h ^= (uint8_t)*p; h *= 1099511628211ull; }
    for (uint32_t t : {KERNEL_SPECS[i].tile_m, KERNEL_SPECS[i].tile_n, KERNEL_SPECS[i].tile_k}) {
      h ^= t; h *= 1099511628211ull;
    }
  }
  return h;
}

std::string tune_store_path(const std::string &device_name) {
  std::string base;
  if (const char *x = getenv("XDG_CACHE_HOME"); x && *x) base = x;
  else if (const char *home = getenv("HOME"); home && *home) base = std::string(home) + "/.cache";
  else return "";
  std::string dev;
  for (char ch : device_name) dev += isalnum((unsigned char)ch) ? (char)tolower((unsigned char)ch) : '_';
  return base + "/tensor-ash/tuned_kernels_cuda_" + dev + ".txt";
}

static std::string tune_header() {
  return strf("tensor-ash-tune-v3 backend=cuda-sm100a kernels=%016llx",
              (unsigned long long)registry_hash());
}

// One line per shape: `B M N K kernel [splitk2=S] [bf16]`; a file whose first line is not this
// build's header (another registry) is ignored as a whole, a malformed line alone
// (src/pipeline/tuning.rs:96-155).
std::unordered_map<TuneKey, TunedEntry, TuneKeyHash> load_tuned(const std::string &path) {
  std::unordered_map<TuneKey, TunedEntry, TuneKeyHash> out;
  if (path.empty()) return out;
  std::ifstream f(path);
  if (!f) return out;
  std::string line;
  if (!std::getline(f, line) || line != tune_header()) return out;  // stale registry: ignore
  while (std::getline(f, line)) {
    std::istringstream ss(line);
    TuneKey key{};
    std::string kernel, tok;
    if (!(ss >> key.batch >> key.m >> key.n >> key.k >> kernel)) continue;
    TunedEntry e;
    e.kernel = kernel_index_by_name(kernel.c_str());
    if (e.kernel < 0) continue;
    key.b_f16 = false;
    while (ss >> tok) {
      if (tok.rfind("splitk2=", 0) == 0) {
        char *end = nullptr;
        const unsigned long v = strtoul(tok.c_str() + 8, &end, 10);
        if (end != tok.c_str() + 8 && *end == 0 && v >= 2 && v <= 0xffff) e.splits = (uint32_t)v;
      } else if (tok == "bf16") {
        key.b_f16 = true;
      }
    }
    out[key] = e;
  }
  return out;
}

// Rewrites the whole store (it is small), sorted by shape, through a uniquely named temporary
// file and an atomic rename (src/pipeline/tuning.rs:158-199).
void save_tuned(const std::string &path,
                const std::unordered_map<TuneKey, TunedEntry, TuneKeyHash> &map) {
  if (path.empty()) return;
  const std::string dir = path.substr(0, path.find_last_of('/'));
  for (size_t i = 1; i <= dir.size(); ++i)
    if (i == dir.size() || dir[i] == '/') ::mkdir(dir.substr(0, i).c_str(), 0755);
  std::vector<std::pair<TuneKey, TunedEntry>> entries(map.begin(), map.end());
  std::sort(entries.begin(), entries.end(), [](const auto &x, const auto &y) {
    const TuneKey &a = x.first, &b = y.first;
    return std::make_tuple(a.batch, a.m, a.n, a.k, a.b_f16) < std::make_tuple(b.batch, b.m, b.n, b.k, b.b_f16);
  });
  static std::atomic<uint64_t> next_tmp{0};
  const std::string tmp = path + ".tmp." + std::to_string((long)getpid()) + "." + std::to_string(next_tmp.fetch_add(1));
  {
    std::ofstream f(tmp, std::ios::trunc);
    if (!f) return;
    f << tune_header() << "\n";
    for (const auto &kv : entries) {
      f << kv.first.batch << " " << kv.first.m << " " << kv.first.n << " " << kv.first.k << " "
        << KERNEL_SPECS[kv.second.kernel].name;
      if (kv.second.splits > 1) f << " splitk2=" << kv.second.splits;
      if (kv.first.b_f16) f << " bf16";
      f << "\n";
    }
  }
  ::rename(tmp.c_str(), path.c_str());  // atomic replace
}

}  // namespace ta
