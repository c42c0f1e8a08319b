// CUDA runtime layer: context (device ordinal), tensors (cudaMalloc), the
// executor (one stream + two events + grow-only scratch per slot), transfers,
// routing, submission and prepared replay (CUDA graphs).
//
// Reference call stack mirrored here (src/executor/dispatch.rs:87-188):
//   validate -> resolve shapes -> plan/route -> enqueue -> wait -> RunStats.
// There is no CPU path: when no CUDA device is present context creation fails.
#include <algorithm>
#include <cstring>
#include <functional>

#include "ta_core.hpp"

namespace ta {

void cuda_check(cudaError_t e, const char *what) {
  if (e != cudaSuccess) fail("CUDA error %s (%d) at %s", cudaGetErrorString(e), (int)e, what);
}

// ------------------------------------------------------------------ context
// DevicePreference strings (src/context/mod.rs:60-103): "auto", "discrete",
// "integrated", "virtual", "cpu", "index:N".  Only "index:N" selects among
// CUDA devices; the adapter-kind names all mean "the current CUDA device".
std::shared_ptr<Context> Context::create(bool validation, const std::string &preference) {
  std::string pref;
  for (char ch : preference) pref += (char)tolower((unsigned char)ch);
  int device = -1;
  if (pref.rfind("index:", 0) == 0) {
    char *end = nullptr;
    const long v = strtol(pref.c_str() + 6, &end, 10);
    if (end == pref.c_str() + 6 || *end || v < 0) fail("invalid ML_DEVICE '%s'", preference.c_str());
    device = (int)v;
  } else if (pref.empty() || pref == "auto" || pref == "discrete" || pref == "integrated" ||
             pref == "virtual" || pref == "cpu" || pref == "other") {
    device = -1;
  } else {
    fail("invalid ML_DEVICE '%s', expected auto, discrete, integrated, virtual, cpu, or index:N",
         preference.c_str());
  }
  int count = 0;
  const cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    fail("no CUDA device available (%s); this library has no CPU fallback",
         e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
  if (device < 0) {
    if (cudaGetDevice(&device) != cudaSuccess) device = 0;
  }
  if (device >= count) fail("ML_DEVICE index %d out of range (%d CUDA devices)", device, count);
  TA_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  TA_CUDA(cudaGetDeviceProperties(&prop, device));
  auto ctx = std::make_shared<Context>();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->cc_major = prop.major;
  ctx->cc_minor = prop.minor;
  ctx->smem_optin = prop.sharedMemPerBlockOptin;
  ctx->name = prop.name;
  ctx->validation = validation;
  if (prop.major != 10)
    fail("device %d (%s, sm_%d%d) is not a Blackwell sm_100 part; kernels are built for sm_100a only",
         device, prop.name, prop.major, prop.minor);
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    ctx->encode_tiled = fn;
  return ctx;
}

void Context::make_current() const { TA_CUDA(cudaSetDevice(device)); }

// ------------------------------------------------------------------ tensor
Buffer::~Buffer() {
  if (ptr) {
    cudaSetDevice(ctx->device);
    cudaFree(ptr);
  }
}

Tensor Tensor::uninit_device(const std::shared_ptr<Context> &ctx, const uint32_t *shape,
                             size_t rank, DType dtype) {
  const uint64_t n = numel_checked(shape, rank);
  uint64_t bytes;
  if (__builtin_mul_overflow(n, dtype_size(dtype), &bytes)) fail("tensor byte size overflows u64");
  // Round up to 16 bytes so 128-bit readers never leave the allocation
  // (src/tensor.rs:78-84).
  if (bytes > UINT64_MAX - 15) fail("tensor byte size overflows u64");
  bytes = (bytes + 15) & ~15ull;
  ctx->make_current();
  auto buf = std::make_shared<Buffer>();
  buf->ctx = ctx;
  buf->bytes = bytes;
  const cudaError_t e = cudaMalloc(&buf->ptr, bytes);
  if (e != cudaSuccess) {
    buf->ptr = nullptr;
    cudaGetLastError();
    fail("device allocation of %llu bytes failed: %s", (unsigned long long)bytes,
         cudaGetErrorString(e));
  }
  Tensor t;
  t.buf = std::move(buf);
  t.shape.assign(shape, shape + rank);
  t.dtype = dtype;
  return t;
}

Tensor Tensor::alias_with_shape(const uint32_t *new_shape, size_t rank) const {
  const uint64_t n = numel_checked(new_shape, rank);
  if (n != len()) {
    std::vector<uint32_t> s(new_shape, new_shape + rank);
    Tensor tmp;
    tmp.shape = s;
    fail("alias_with_shape: %llu elements for shape %s != %llu in %s", (unsigned long long)n,
         tmp.shape_str().c_str(), (unsigned long long)len(), shape_str().c_str());
  }
  Tensor t;
  t.buf = buf;
  t.shape.assign(new_shape, new_shape + rank);
  t.dtype = dtype;
  return t;
}

// ------------------------------------------------------------------ executor
Executor::Executor(std::shared_ptr<Context> ctx, int selection, ExecutorConfig cfg)
    : ctx_(std::move(ctx)), selection_(selection), cfg_(cfg) {
  if (cfg_.n_slots == 0) fail("Executor needs at least one slot");
  if (cfg_.max_calls_per_submit == 0) fail("Executor max_calls_per_submit must be > 0");
  ctx_->make_current();
  slots_.resize(cfg_.n_slots);
  for (Slot &s : slots_) {
    TA_CUDA(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
    TA_CUDA(cudaEventCreate(&s.ev_begin));
    TA_CUDA(cudaEventCreate(&s.ev_end));
    alloc_status_word(&s.status_host, &s.status);
    TA_CUDA(cudaMalloc((void **)&s.counters, SLOT_WORDS * sizeof(uint32_t)));
    TA_CUDA(cudaMemset(s.counters, 0, SLOT_WORDS * sizeof(uint32_t)));
  }
  tune_path_ = tune_store_path(ctx_->name);
  tuned_ = load_tuned(tune_path_);
  if (!cfg_.tune) {
    if (const char *t = getenv("ML_TUNE"); t && (!strcmp(t, "1") || !strcasecmp(t, "true")))
      cfg_.tune = true;
  }
}

Executor::~Executor() {
  cudaSetDevice(ctx_->device);
  for (Slot &s : slots_) {
    if (s.stream) cudaStreamSynchronize(s.stream);
    if (s.scratch) cudaFree(s.scratch);
    if (s.staging) cudaFreeHost(s.staging);
    free_status_word(s.status_host);
    if (s.counters) cudaFree(s.counters);
    if (s.ev_begin) cudaEventDestroy(s.ev_begin);
    if (s.ev_end) cudaEventDestroy(s.ev_end);
    if (s.stream) cudaStreamDestroy(s.stream);
  }
}

Slot &Executor::checkout_slot() {
  std::unique_lock<std::mutex> lk(mu_);
  for (;;) {
    for (Slot &s : slots_)
      if (!s.busy) {
        s.busy = true;
        return s;
      }
    cv_.wait(lk);
  }
}

void Executor::release_slot(Slot &s) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    s.busy = false;
  }
  cv_.notify_one();
}

namespace {

void ensure_staging(Slot &slot, size_t bytes) {
  if (slot.staging_bytes >= bytes) return;
  if (slot.staging) cudaFreeHost(slot.staging);
  slot.staging = nullptr;
  slot.staging_bytes = 0;
  TA_CUDA(cudaMallocHost(&slot.staging, bytes));
  slot.staging_bytes = bytes;
}
constexpr size_t STAGING_CHUNK = 32ull << 20;  // f16 conversion is pipelined in 32 MiB pieces
}  // namespace

void Executor::ensure_scratch(Slot &slot, size_t bytes) {
  if (slot.scratch_bytes >= bytes) return;
  TA_CUDA(cudaStreamSynchronize(slot.stream));
  if (slot.scratch) cudaFree(slot.scratch);
  slot.scratch = nullptr;
  slot.scratch_bytes = 0;
  TA_CUDA(cudaMalloc(&slot.scratch, bytes));
  slot.scratch_bytes = bytes;
}

void alloc_status_word(uint32_t **host, uint32_t **device) {
  TA_CUDA(cudaHostAlloc((void **)host, sizeof(uint32_t), cudaHostAllocMapped));
  **host = 0;
  TA_CUDA(cudaHostGetDevicePointer((void **)device, *host, 0));
}
void free_status_word(uint32_t *host) {
  if (host) cudaFreeHost(host);
}
void check_status_word(uint32_t *host, uint32_t *counters) {
  const uint32_t status = *(volatile uint32_t *)host;
  if (!status) return;
  *(volatile uint32_t *)host = 0;
  // a launch that gave up may have left tickets and partial flags behind: back to the state a new slot has
  if (counters) cudaMemset(counters, 0, SLOT_WORDS * sizeof(uint32_t));
  fail_device_status(status);
}

void Executor::validate_tensor(const Tensor &t, const char *what) const {
  if (t.ctx().get() != ctx_.get()) fail("%s belongs to a different context", what);
}

// ------------------------------------------------------------------ transfers
// (src/executor/transfer.rs:21-84, 184-197)
void Executor::upload(const float *src, size_t len, const Tensor &dst) {
  validate_tensor(dst, "upload destination");
  if (len == 0) return;
  const uint64_t bytes = (uint64_t)len * dtype_size(dst.dtype);
  if (bytes > dst.size_bytes())
    fail("upload: %llu bytes > tensor capacity %llu", (unsigned long long)bytes,
         (unsigned long long)dst.size_bytes());
  ctx_->make_current();
  Slot &slot = checkout_slot();
  SlotGuard g(*this, slot);
  if (dst.dtype == DType::F32) {
    TA_CUDA(cudaMemcpyAsync(dst.ptr(), src, bytes, cudaMemcpyHostToDevice, slot.stream));
    TA_CUDA(cudaStreamSynchronize(slot.stream));
    return;
  }
  // f16: software RNE on the host into pinned staging, chunk by chunk.
  const size_t chunk_elems = STAGING_CHUNK / 2;
  ensure_staging(slot, std::min(len, chunk_elems) * 2);
  uint16_t *stage = static_cast<uint16_t *>(slot.staging);
  for (size_t off = 0; off < len; off += chunk_elems) {
    const size_t n = std::min(chunk_elems, len - off);
    for (size_t i = 0; i < n; ++i) stage[i] = f32_to_f16_bits(src[off + i]);
    TA_CUDA(cudaMemcpyAsync(static_cast<uint16_t *>(dst.ptr()) + off, stage, n * 2,
                            cudaMemcpyHostToDevice, slot.stream));
    TA_CUDA(cudaStreamSynchronize(slot.stream));
  }
}

void Executor::upload_f16(const uint16_t *src, size_t len, const Tensor &dst) {
  validate_tensor(dst, "upload destination");
  if (len == 0) return;
  if (dst.dtype != DType::F16)
    fail("upload_f16 requires an f16 destination tensor, got %s", dtype_name(dst.dtype));
  const uint64_t bytes = (uint64_t)len * 2;
  if (bytes > dst.size_bytes())
    fail("upload: %llu bytes > tensor capacity %llu", (unsigned long long)bytes,
         (unsigned long long)dst.size_bytes());
  ctx_->make_current();
  Slot &slot = checkout_slot();
  SlotGuard g(*this, slot);
  TA_CUDA(cudaMemcpyAsync(dst.ptr(), src, bytes, cudaMemcpyHostToDevice, slot.stream));
  TA_CUDA(cudaStreamSynchronize(slot.stream));
}

void Executor::download(const Tensor &src, float *dst, size_t len) {
  validate_tensor(src, "download source");
  if (len == 0) return;
  const uint64_t bytes = (uint64_t)len * dtype_size(src.dtype);
  if (bytes > src.size_bytes())
    fail("download: %llu bytes > tensor capacity %llu", (unsigned long long)bytes,
         (unsigned long long)src.size_bytes());
  ctx_->make_current();
  Slot &slot = checkout_slot();
  SlotGuard g(*this, slot);
  if (src.dtype == DType::F32) {
    TA_CUDA(cudaMemcpyAsync(dst, src.ptr(), bytes, cudaMemcpyDeviceToHost, slot.stream));
    TA_CUDA(cudaStreamSynchronize(slot.stream));
    return;
  }
  const size_t chunk_elems = STAGING_CHUNK / 2;
  ensure_staging(slot, std::min(len, chunk_elems) * 2);
  uint16_t *stage = static_cast<uint16_t *>(slot.staging);
  for (size_t off = 0; off < len; off += chunk_elems) {
    const size_t n = std::min(chunk_elems, len - off);
    TA_CUDA(cudaMemcpyAsync(stage, static_cast<const uint16_t *>(src.ptr()) + off, n * 2,
                            cudaMemcpyDeviceToHost, slot.stream));
    TA_CUDA(cudaStreamSynchronize(slot.stream));
    for (size_t i = 0; i < n; ++i) dst[off + i] = f16_bits_to_f32(stage[i]);
  }
}

// ------------------------------------------------------------------ routing
namespace {

int idx_of(const char *name) {
  const int i = kernel_index_by_name(name);
  if (i < 0) fail("internal: kernel '%s' missing from registry", name);
  return i;
}

// Static shape heuristic for B200.  The tensor-core route wins whenever the
// problem fills at least a few 128-row tiles; tiny and very skinny problems stay
// on the SIMT tiles, which launch faster and waste no tile area.
int heuristic_kernel(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, bool b_f16, int sm_count) {
  if (b_f16) {
    // decode shapes: the bandwidth GEMV (src/pipeline/mod.rs:330-347, routing.rs:27-33)
    if (batch == 1 && m <= 8 && gemv_f16w_supported(m, n, k, false, 0))
      return idx_of(f16w_row_uses_k16(k, n) ? "f16w_row_bda_k16" : "f16w_row_bda_k16_v2");
    // prefill / training shapes: the tensor cores once a 128-row tile is at least a quarter full
    if (k % 4 == 0 && n % 8 == 0 && m >= 32 && n >= 64 && k >= 64) {
      const uint32_t bn = gemm_f16w_umma_tile_n(batch, m, n, sm_count);
      return idx_of(bn == 256 ? "f16w_umma_m128n256" : bn == 128 ? "f16w_umma_m128n128" : "f16w_umma_m128n64");
    }
    return idx_of((m >= 128 && n >= 128) ? "f16w_ffma_m128n128" : "f16w_ffma_m64n64");
  }
  const bool tma_ok = (k % 4 == 0) && (n % 4 == 0);
  // 33..63 rows over a large weight matrix also go to the tensor-core tile: half a tile of rows is
  // wasted, but 48 x 4096 x 4096 takes about 100 us there against 215 us on the 64 x 64 SIMT tile.
  const bool rows_ok = m >= 64 || (m > 32 && (uint64_t)n * k >= (1ull << 22));
  if (tma_ok && rows_ok && n >= 64 && k >= 64) {
    const uint64_t tiles256 = (uint64_t)batch * ((m + 127) / 128) * ((n + 255) / 256);
    const uint64_t tiles128 = (uint64_t)batch * ((m + 127) / 128) * ((n + 127) / 128);
    // Narrow problems, and problems whose 256-wide tiles leave more than half of the SMs idle, fill
    // the machine better with the 128-wide tile (measured: 1024^3 37 us against 48, 512^3 25 against
    // 32; 2048^3 and 4096 x 1024 x 1024, with 128 wide tiles each, are faster on the 256-wide tile).
    if (n <= 128 || (tiles256 < (uint64_t)sm_count && tiles128 >= tiles256 * 2 && n % 256 != 0) ||
        (tiles256 * 2 <= (uint64_t)sm_count && tiles128 > tiles256))
      return idx_of("tf32x3_m128n128");
    return idx_of("tf32x3_m128n256");
  }
  return idx_of((m >= 128 && n >= 128) ? "ffma_m128n128" : "ffma_m64n64");
}

bool family_matches_dtype(const KernelSpec &spec, bool b_f16) { return spec.weights_f16 == b_f16; }

}  // namespace

int heuristic_kernel_index(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, bool b_f16, int sm_count) {
  return heuristic_kernel(batch, m, n, k, b_f16, sm_count);
}

Route Executor::plan_shape(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, bool b_f16,
                           bool allow_split_k2) const {
  Route r;
  // explicit selection wins when it can run this dtype
  if (selection_ >= 0 && family_matches_dtype(KERNEL_SPECS[selection_], b_f16) &&
      KERNEL_SPECS[selection_].family != Family::SplitK2 &&
      KERNEL_SPECS[selection_].family != Family::RowGemv) {
    const KernelSpec &spec = KERNEL_SPECS[selection_];
    const bool tma_ok = (k % 4 == 0) && (n % 4 == 0);
    const bool umma_ok = (k % 4 == 0) && (n % 8 == 0);
    if (spec.family == Family::Ffma || (spec.family == Family::Tf32x3 && tma_ok) ||
        (spec.family == Family::F16wUmma && umma_ok)) {
      r.kernel = selection_;
      return r;
    }
  }
  {
    std::lock_guard<std::mutex> lk(tune_mu_);
    auto it = tuned_.find(TuneKey{batch, m, n, k, b_f16});
    if (it != tuned_.end()) {
      r.kernel = it->second.kernel;
      r.tuned = true;
      r.splits = allow_split_k2 ? it->second.splits : 0;
      if (KERNEL_SPECS[r.kernel].family != Family::SplitK2 || r.splits > 1) return r;
    }
  }
  if (allow_split_k2 && !b_f16) {
    if (auto s = heuristic_splits(batch, m, n, k)) {
      const uint64_t scratch = (uint64_t)batch * *s * m * n * 4;
      if (scratch <= (256ull << 20)) {  // src/executor/splitk2.rs:142
        r.kernel = idx_of((m >= 128 && n >= 128) ? "split_k2_m128n128" : "split_k2_m64n64");
        r.splits = *s;
        return r;
      }
    }
  }
  r.kernel = heuristic_kernel(batch, m, n, k, b_f16, ctx_->sm_count);
  return r;
}

// Capability demotion (src/executor/mod.rs:268-315): every CUDA family fuses
// the full epilogue, so only alignment can force a fallback to the SIMT tiles.
Route Executor::plan_op(const MatmulOp &op, const ResolvedMatmul &r, bool allow_split_k2) const {
  const bool plain = op.epilogue.is_none() && !op.call.accumulate && !op.normed_weight &&
                     op.store.is_none() && !op.packed_b;
  if (op.packed_b) {   // src/pipeline/routing.rs:35-41
    Route route;
    route.kernel = idx_of(f16w_row_tile_n(r.k, r.n) == 32 ? "f16w_row_bda_k16_packed"
                                                           : "f16w_row_bda_k16_v2_packed");
    return route;
  }
  Route route = plan_shape(r.batch, r.m, r.n, r.k, r.b_f16, allow_split_k2 && plain);
  if ((op.normed_weight || !op.store.is_none()) && KERNEL_SPECS[route.kernel].family != Family::RowGemv) {
    // only the row kernels implement normed-A and the fused stores (src/executor/mod.rs:268-315)
    if (!(r.b_f16 && r.batch == 1 && r.m <= 8 && gemv_f16w_supported(r.m, r.n, r.k, false, 0)))
      fail("normed-A / fused-store ops need the f16-weight row-GEMV route (f16 B, M <= 8, N %% 8 == 0); "
           "got M=%u N=%u f16_b=%d", r.m, r.n, (int)r.b_f16);
    route.kernel = idx_of(f16w_row_uses_k16(r.k, r.n) ? "f16w_row_bda_k16" : "f16w_row_bda_k16_v2");
    route.splits = 0;
  }
  return route;
}

// ------------------------------------------------------------------ enqueue
namespace {
GemmParams make_params(const MatmulOp &op, const ResolvedMatmul &r) {
  GemmParams p{};
  p.a = op.call.a->ptr();
  p.b = op.call.b->ptr();
  p.c = static_cast<float *>(op.call.c->ptr());
  p.bias = op.epilogue.bias ? static_cast<const float *>(op.epilogue.bias->ptr()) : nullptr;
  p.d = op.epilogue.d ? static_cast<const float *>(op.epilogue.d->ptr()) : nullptr;
  p.m = r.m; p.n = r.n; p.k = r.k; p.batch = r.batch;
  p.stride_a = r.batch_stride_a; p.stride_b = r.batch_stride_b; p.stride_c = r.batch_stride_c;
  p.bias_stride = (op.epilogue.bias && op.epilogue.bias->shape.size() == 2) ? r.n : 0;
  p.alpha = op.call.alpha;
  p.beta = op.epilogue.beta;
  p.accumulate = op.call.accumulate ? 1 : 0;
  p.act = (uint32_t)op.epilogue.activation;
  p.binary = (uint32_t)op.epilogue.binary;
  p.b_f16 = r.b_f16 ? 1 : 0;
  p.splits = 1;
  return p;
}
}  // namespace

// Stage 1 of the split-K2 route runs on the tensor cores where the partition allows; an executor
// whose kernel selection names a split_k2_* kernel explicitly keeps the SIMT stage 1, whose
// planes hold the reference shader's sequential fma chains.
SplitK2TensorPlan Executor::splitk2_plan_for(const GemmParams &p, uint32_t splits) const {
  if (selection_ >= 0 && KERNEL_SPECS[selection_].family == Family::SplitK2) return SplitK2TensorPlan{};
  return splitk2_tensor_plan(p, splits, ctx_->sm_count);
}

bool Executor::dual_f16w_params(const MatmulOp &up, const MatmulOp &gate, GemmParams *out) const {
  if (!up.call.a || !gate.call.a || up.call.a->ptr() != gate.call.a->ptr()) return false;
  const ResolvedMatmul ru = ResolvedMatmul::from_op(up), rg = ResolvedMatmul::from_op(gate);
  if (ru.a_f16 || rg.a_f16 || !ru.b_f16 || !rg.b_f16 || ru.batch != 1 || rg.batch != 1) return false;
  if (ru.m != rg.m || ru.n != rg.n || ru.k != rg.k) return false;
  const Route tu = plan_op(up, ru, false), tg = plan_op(gate, rg, false);
  if (tu.kernel < 0 || tg.kernel < 0 || tu.splits > 1 || tg.splits > 1) return false;
  if (KERNEL_SPECS[tu.kernel].family != Family::F16wUmma || KERNEL_SPECS[tg.kernel].family != Family::F16wUmma) return false;
  if (selection_ != -2 || tu.tuned || tg.tuned) return false;          // an explicit or tuned kernel choice is kept as given
  if (!op_scratch_bytes(ru, tu) || !op_scratch_bytes(rg, tg)) return false;
  // up: plain product; gate: silu, times the up output, nothing else
  const Epilogue &eu = up.epilogue, &eg = gate.epilogue;
  if (up.call.alpha != 1.0f || up.call.accumulate || eu.bias || eu.d || eu.activation != Activation::None ||
      eu.binary != BinaryKind::None)
    return false;
  if (gate.call.alpha != 1.0f || gate.call.accumulate || eg.bias || eg.activation != Activation::Silu ||
      eg.binary != BinaryKind::Mul || !eg.d || eg.d->ptr() != up.call.c->ptr())
    return false;
  if (up.call.c->ptr() == gate.call.c->ptr() || up.call.c->ptr() == up.call.a->ptr() || gate.call.c->ptr() == up.call.a->ptr())
    return false;
  GemmParams p = make_params(gate, rg);
  p.d = nullptr;
  p.act = 0;
  p.binary = 0;
  p.b2 = up.call.b->ptr();
  p.c2 = static_cast<float *>(up.call.c->ptr());
  if (!gemm_f16w_umma_dual_eligible(p)) return false;
  *out = p;
  return true;
}

// Bytes of plane scratch the split-K2 route of this problem needs in its slot.
size_t Executor::splitk2_scratch_bytes(const MatmulOp &op, const ResolvedMatmul &r, uint32_t splits) const {
  if (splits <= 1) return 0;
  const SplitK2TensorPlan tplan = splitk2_plan_for(make_params(op, r), splits);
  const uint64_t planes = tplan.eligible ? tplan.planes : splits;
  return (size_t)((uint64_t)r.batch * planes * r.m * r.n * 4);
}

// The f16w tensor-core GEMM rounds A to f16 once per launch when its slot has room for the copy
// (ops of one submission run in stream order, so they share the region); capped at 256 MiB.
size_t Executor::op_scratch_bytes(const ResolvedMatmul &r, const Route &route) const {
  if (route.kernel < 0 || route.splits > 1) return 0;
  if (KERNEL_SPECS[route.kernel].family == Family::RowGemv && r.b_f16 && !r.a_f16 && r.batch == 1 && r.m <= 8 &&
      r.k % 16 == 0 && (tunables().gemv_umma == 1 || (r.m >= 3 && tunables().gemv_umma != 0)))
    // records of the tensor-memory GEMV; sized for the SwiGLU pair too (twice the groups)
    return gemv_umma_scratch_bytes(r.n, r.k, true, ctx_->sm_count);
  if (KERNEL_SPECS[route.kernel].family == Family::Tf32x3 && KERNEL_SPECS[route.kernel].tile_m != 256 && !r.b_f16 && !r.a_f16) {
    // planes of the K split a few-tile op runs as
    const size_t need = gemm_tf32x3_ksplit_scratch_bytes(r.batch, r.m, r.n, r.k, ctx_->sm_count);
    return need <= (256ull << 20) ? need : 0;
  }
  if (KERNEL_SPECS[route.kernel].family != Family::F16wUmma) return 0;
  // the f16 copy of A, and behind it the partial tiles of an in-kernel K split
  const size_t need = gemm_f16w_umma_scratch_bytes_split(r.batch, r.batch_stride_a ? r.batch : 1, r.m, r.n, r.k, ctx_->sm_count);
  return need <= (256ull << 20) ? need : gemm_f16w_umma_scratch_bytes(r.batch_stride_a ? r.batch : 1, r.m, r.k);
}

// GEMV launch description of an op on the row-GEMV route; false when the route is another family.
bool Executor::gemv_params_for(const MatmulOp &op, const ResolvedMatmul &r, const Route &route,
                               GemvParams *out) const {
  const KernelSpec &spec = KERNEL_SPECS[route.kernel];
  if (!(spec.family == Family::RowGemv && r.b_f16) || r.a_f16) return false;
  const uint32_t tile_n = op.packed_b ? f16w_row_tile_n(r.k, r.n) : 32;
  if (!gemv_f16w_supported(r.m, r.n, r.k, op.packed_b, tile_n) || r.batch != 1)
    fail("row-GEMV route cannot run M=%u N=%u K=%u batch=%u packed=%d", r.m, r.n, r.k, r.batch,
         (int)op.packed_b);
  GemvParams g{};
  g.x = static_cast<const float *>(op.call.a->ptr());
  g.w = op.call.b->ptr();
  g.w2 = nullptr;
  g.c = static_cast<float *>(op.call.c->ptr());
  g.c2 = nullptr;
  g.bias = op.epilogue.bias ? static_cast<const float *>(op.epilogue.bias->ptr()) : nullptr;
  g.d = op.epilogue.d ? static_cast<const float *>(op.epilogue.d->ptr()) : nullptr;
  g.norm_w = op.normed_weight ? static_cast<const float *>(op.normed_weight->ptr()) : nullptr;
  g.norm_eps = op.normed_eps;
  g.m = r.m; g.n = r.n; g.k = r.k;
  g.alpha = op.call.alpha; g.beta = op.epilogue.beta;
  g.accumulate = op.call.accumulate; g.act = (uint32_t)op.epilogue.activation;
  g.binary = (uint32_t)op.epilogue.binary;
  g.packed = op.packed_b; g.tile_n = tile_n;
  g.store_kind = (uint32_t)op.store.kind;
  g.head_dim = op.store.head_dim; g.pos_base = op.store.pos_base; g.pos_scale = op.store.pos_scale;
  g.stride_head = op.store.stride_head; g.stride_dim = op.store.stride_dim;
  g.table = op.store.table ? static_cast<const float *>(op.store.table->ptr()) : nullptr;
  g.dst = op.store.dst ? op.store.dst->ptr() : nullptr;
  g.dst_f16 = op.store.dst && op.store.dst->dtype == DType::F16;
  g.pos_ptr = op.store.pos_cell ? op.store.pos_cell->device : nullptr;
  g.pos_stage_idx = -1;
  // the largest position count for which every table row and destination element the store touches exists
  uint64_t limit = 0xffffffffull;
  if (g.store_kind != 0 && g.head_dim) {
    if (op.store.table && g.store_kind != 2) limit = std::min<uint64_t>(limit, op.store.table->len() / g.head_dim);
    if (op.store.dst && g.store_kind >= 2) {
      const uint64_t heads = r.n / g.head_dim;
      const uint64_t rest = (heads ? heads - 1 : 0) * (uint64_t)g.stride_head + (uint64_t)(g.head_dim - 1) * g.stride_dim;
      const uint64_t len = op.store.dst->len();
      if (len <= rest) limit = 0;
      else if (g.pos_scale) limit = std::min<uint64_t>(limit, (len - 1 - rest) / g.pos_scale + 1);
    }
  }
  g.pos_limit = (uint32_t)limit;
  *out = g;
  return true;
}

void Executor::enqueue_op(const MatmulOp &op, const ResolvedMatmul &r, const Route &route,
                          Slot &slot, cudaStream_t stream) {
  if (r.a_f16) {
    // a16 route (src/matmul/resolution.rs:123-172): f16 A / B / C, aligned shapes, no fused stages;
    // always the tensor-core pipeline, whatever the selection says (it is the only f16-A kernel)
    GemmParams p = make_params(op, r);
    launch_gemm_a16_umma(*ctx_, p, gemm_f16w_umma_tile_n(r.batch, r.m, r.n, ctx_->sm_count), slot.status, stream);
    return;
  }
  const KernelSpec &spec = KERNEL_SPECS[route.kernel];
  {
    GemvParams g;
    if (gemv_params_for(op, r, route, &g)) {
      launch_gemv_f16w(*ctx_, g, gemv_workspace(slot), stream);
      return;
    }
  }
  if (op.packed_b || op.normed_weight || !op.store.is_none())
    fail("packed-B / normed-A / fused-store ops need the f16-weight row-GEMV route");
  GemmParams p = make_params(op, r);
  if (route.splits > 1) {
    p.splits = route.splits;
    float *scratch = static_cast<float *>(slot.scratch);
    const SplitK2TensorPlan tplan = splitk2_plan_for(p, route.splits);
    if (tplan.eligible) {
      launch_splitk2_tensor(*ctx_, p, tplan, scratch, slot.status, stream);
      return;
    }
    launch_splitk2_stage1(p, spec.tile_m, scratch, stream);
    launch_splitk2_reduce(scratch, p.c, (uint64_t)r.batch * r.m * r.n, (uint64_t)r.m * r.n,
                          route.splits, stream);
    return;
  }
  switch (spec.family) {
    case Family::Tf32x3:
      if (gemm_tf32x3_eligible(p)) {
        if (spec.tile_m != 256) {
          // few output tiles: split K over the idle SMs when the slot holds the planes
          const SplitK2TensorPlan kplan = gemm_tf32x3_ksplit_plan(r.batch, r.m, r.n, r.k, ctx_->sm_count);
          if (kplan.eligible && slot.scratch && slot.scratch_bytes >= (size_t)r.batch * kplan.planes * r.m * r.n * 4) {
            launch_gemm_tf32x3_ksplit(*ctx_, p, kplan, static_cast<float *>(slot.scratch), slot.status, stream);
            return;
          }
        }
        if (spec.tile_m == 256) launch_gemm_tf32x3_pair(*ctx_, p, slot.status, stream);
        else launch_gemm_tf32x3(*ctx_, p, spec.tile_n, slot.status, stream);
        return;
      }
      launch_gemm_ffma(p, 128, stream);  // alignment demotion
      return;
    case Family::F16wUmma:
      if (gemm_f16w_umma_eligible(p)) {
        // an executor on automatic selection lets the launcher pick tile width and K split together
        launch_gemm_f16w_umma(*ctx_, p, spec.tile_n, slot.status, slot.scratch, slot.scratch_bytes, op.a16_ready, stream,
                              slot.counters, selection_ == -2 && route.tuned == false);
        return;
      }
      launch_gemm_ffma(p, (r.m >= 128 && r.n >= 128) ? 128 : 64, stream);  // alignment demotion
      return;
    case Family::Ffma:
      launch_gemm_ffma(p, spec.tile_m, stream);
      return;
    default:
      launch_gemm_ffma(p, (r.m >= 128 && r.n >= 128) ? 128 : 64, stream);
      return;
  }
}

RunStats Executor::timed(Slot &slot, size_t n_calls, uint64_t flops,
                         const std::function<void(cudaStream_t)> &record) {
  TA_CUDA(cudaEventRecord(slot.ev_begin, slot.stream));
  record(slot.stream);
  TA_CUDA(cudaEventRecord(slot.ev_end, slot.stream));
  TA_CUDA(cudaStreamSynchronize(slot.stream));
  check_status_word(slot.status_host, slot.counters);
  float ms = 0.0f;
  TA_CUDA(cudaEventElapsedTime(&ms, slot.ev_begin, slot.ev_end));
  RunStats st;
  st.gpu_time_ns = (uint64_t)((double)ms * 1e6 + 0.5);
  st.n_calls = n_calls;
  st.total_flops = flops;
  return st;
}

// C must not alias A or B (src/executor/validation.rs:18-52).
void validate_op_tensors(const Executor &e, const MatmulOp &op) {
  e.validate_tensor(*op.call.a, "matmul A");
  e.validate_tensor(*op.call.b, "matmul B");
  e.validate_tensor(*op.call.c, "matmul C");
  if (op.call.c->ptr() == op.call.a->ptr() || op.call.c->ptr() == op.call.b->ptr())
    fail("matmul output C must not alias an input (A or B)");
  if (op.epilogue.bias) e.validate_tensor(*op.epilogue.bias, "epilogue bias");
  if (op.epilogue.d) e.validate_tensor(*op.epilogue.d, "epilogue D");
}

RunStats Executor::run_ops_impl(const std::vector<MatmulOp> &ops, bool graph) {
  (void)graph;  // one in-order stream: later ops already see earlier outputs
  if (ops.empty()) return RunStats{std::nullopt, 0, 0};
  if (ops.size() > cfg_.max_calls_per_submit)
    fail("batch of %zu calls exceeds max_calls_per_submit = %u", ops.size(),
         cfg_.max_calls_per_submit);
  std::vector<ResolvedMatmul> resolved;
  resolved.reserve(ops.size());
  uint64_t flops = 0;
  for (const MatmulOp &op : ops) {
    validate_op_tensors(*this, op);
    resolved.push_back(ResolvedMatmul::from_op(op));
    if (__builtin_add_overflow(flops, resolved.back().total_flops, &flops))
      fail("total FLOP count overflows u64");
  }
  ctx_->make_current();
  // First sight of a plain single op under ML_TUNE: measure candidates once
  // (src/executor/dispatch.rs:121-149).
  if (cfg_.tune && ops.size() == 1) {
    const ResolvedMatmul &r = resolved[0];
    const bool plain = ops[0].epilogue.is_none() && !ops[0].call.accumulate;
    bool known;
    {
      std::lock_guard<std::mutex> lk(tune_mu_);
      known = tuned_.count(TuneKey{r.batch, r.m, r.n, r.k, r.b_f16}) != 0;
    }
    // row-GEMV shapes (f16 B, M <= 8) are a route of their own and are not tuned
    if (plain && !known && selection_ == -2 && !r.a_f16 && !ops[0].packed_b && !(r.b_f16 && r.m <= 8))
      tune_shape(r.batch, r.m, r.n, r.k, r.b_f16);
  }
  std::vector<Route> routes;
  routes.reserve(ops.size());
  size_t scratch_bytes = 0;
  for (size_t i = 0; i < ops.size(); ++i) {
    // split-K2 auto route only for a lone plain op (dispatch.rs:171-176)
    routes.push_back(plan_op(ops[i], resolved[i], ops.size() == 1));
    scratch_bytes = std::max(scratch_bytes, splitk2_scratch_bytes(ops[i], resolved[i], routes.back().splits));
    scratch_bytes = std::max(scratch_bytes, op_scratch_bytes(resolved[i], routes.back()));
  }
  Slot &slot = checkout_slot();
  SlotGuard g(*this, slot);
  if (scratch_bytes) ensure_scratch(slot, scratch_bytes);
  return timed(slot, ops.size(), flops, [&](cudaStream_t st) {
    for (size_t i = 0; i < ops.size(); ++i) enqueue_op(ops[i], resolved[i], routes[i], slot, st);
  });
}

RunStats Executor::run_ops(const std::vector<MatmulOp> &ops) { return run_ops_impl(ops, false); }
RunStats Executor::run_op_graph(const std::vector<MatmulOp> &ops) { return run_ops_impl(ops, true); }

RunStats Executor::run_matmuls(const std::vector<MatmulCall> &calls) {
  std::vector<MatmulOp> ops(calls.size());
  for (size_t i = 0; i < calls.size(); ++i) ops[i].call = calls[i];
  return run_ops_impl(ops, false);
}

// (src/executor/reduction.rs:21-70, splitk2.rs:213-271)
RunStats Executor::run_matmuls_split_k2(const std::vector<MatmulCall> &calls, uint32_t splits_in) {
  if (calls.empty()) return RunStats{std::nullopt, 0, 0};
  if (calls.size() > cfg_.max_calls_per_submit)
    fail("batch of %zu calls exceeds max_calls_per_submit = %u", calls.size(),
         cfg_.max_calls_per_submit);
  std::vector<MatmulOp> ops(calls.size());
  std::vector<ResolvedMatmul> resolved;
  std::vector<Route> routes;
  uint64_t flops = 0;
  size_t scratch_bytes = 0;
  bool any_split = false;
  for (size_t i = 0; i < calls.size(); ++i) {
    ops[i].call = calls[i];
    validate_op_tensors(*this, ops[i]);
    if (calls[i].accumulate)
      fail("run_matmuls_split_k2 does not support accumulate (the reduce stage overwrites C)");
    ResolvedMatmul r = ResolvedMatmul::from_op(ops[i]);
    if (r.b_f16 || r.a_f16) fail("run_matmuls_split_k2 requires f32 operands");
    const char *name;
    uint32_t tile[3];
    splitk2_stage1_tile(r.m, r.n, &name, tile);
    uint32_t s = splits_in ? splits_in : default_num_k_splits(r.batch, r.m, r.n, r.k, tile[0], tile[1]);
    if (s > r.k) fail("num_k_splits %u exceeds K=%u", s, r.k);
    if (s > 65535) fail("num_k_splits %u exceeds the 65535 limit", s);
    if ((uint64_t)r.batch * s > 65535)
      fail("split-K2 grid z = batch %u * splits %u exceeds 65535", r.batch, s);
    Route route;
    if (s <= 1) route = plan_op(ops[i], r, false);
    else {
      route.kernel = kernel_index_by_name(name);
      route.splits = s;
      any_split = true;
      const uint64_t bytes = splitk2_scratch_bytes(ops[i], r, s);
      if (bytes > (4ull << 30)) fail("split-K2 scratch of %llu bytes exceeds the 4 GiB cap", (unsigned long long)bytes);
      scratch_bytes = std::max(scratch_bytes, (size_t)bytes);
    }
    flops += r.total_flops;
    resolved.push_back(r);
    routes.push_back(route);
  }
  (void)any_split;
  if (calls.size() > 1 && scratch_bytes) {
    // ops in one submission share the slot scratch: give each its own region
    size_t total = 0;
    for (size_t i = 0; i < calls.size(); ++i) total += splitk2_scratch_bytes(ops[i], resolved[i], routes[i].splits);
    scratch_bytes = total;
  }
  ctx_->make_current();
  Slot &slot = checkout_slot();
  SlotGuard g(*this, slot);
  if (scratch_bytes) ensure_scratch(slot, scratch_bytes);
  return timed(slot, calls.size(), flops, [&](cudaStream_t st) {
    // In-order stream: a later op's stage 1 cannot start before the previous
    // reduce finished, so one scratch region is reused safely.
    for (size_t i = 0; i < calls.size(); ++i) enqueue_op(ops[i], resolved[i], routes[i], slot, st);
  });
}

// Decode SwiGLU gate in one launch: out = silu(x' @ Wg) * (x' @ Wup), packed f16
// weights sharing x (the reference's up GEMV + gate GEMV with a Mul epilogue,
// tools/llama-ash/src/model/forward/mod.rs:194-206).
RunStats Executor::swiglu_gemv(const Tensor &x, const Tensor &wg, const Tensor &wup, const Tensor &out,
                               const Tensor *norm_w, float eps) {
  for (const Tensor *t : {&x, &wg, &wup, &out}) validate_tensor(*t, "swiglu_gemv operand");
  if (x.dtype != DType::F32 || out.dtype != DType::F32) fail("swiglu_gemv: x and out must be f32 storage");
  if (wg.dtype != DType::F16 || wup.dtype != DType::F16) fail("swiglu_gemv requires f16 weights");
  if (wg.shape != wup.shape) fail("swiglu_gemv: gate shape %s != up shape %s", wg.shape_str().c_str(),
                                  wup.shape_str().c_str());
  MatmulCall call{&x, &wg, &out, 1.0f, false};
  const ResolvedMatmul r = ResolvedMatmul::from_call(call);
  if (r.batch != 1 || r.m > 8) fail("swiglu_gemv requires batch == 1 and M <= 8 (got M=%u, batch=%u)", r.m, r.batch);
  if (r.n % 32) fail("packed-B GEMV requires N to be a multiple of 32 (got %u)", r.n);
  if (norm_w) {
    validate_tensor(*norm_w, "swiglu_gemv normed weight");
    if (norm_w->dtype != DType::F32) fail("normed-A weight must be f32 storage");
    if (norm_w->len() != r.k) fail("normed-A weight length %llu must equal K = %u", (unsigned long long)norm_w->len(), r.k);
  }
  GemvParams g{};
  g.x = static_cast<const float *>(x.ptr());
  g.w = wg.ptr();
  g.w2 = wup.ptr();
  g.c = static_cast<float *>(out.ptr());
  g.norm_w = norm_w ? static_cast<const float *>(norm_w->ptr()) : nullptr;
  g.norm_eps = eps;
  g.m = r.m; g.n = r.n; g.k = r.k;
  g.alpha = 1.0f;
  g.packed = 1; g.tile_n = f16w_row_tile_n(r.k, r.n);
  ctx_->make_current();
  Slot &slot = checkout_slot();
  SlotGuard guard(*this, slot);
  if (gemv_routes_to_umma(g)) ensure_scratch(slot, gemv_umma_scratch_bytes(g.n, g.k, true, ctx_->sm_count));
  return timed(slot, 1, 2 * r.total_flops, [&](cudaStream_t s) { launch_gemv_f16w(*ctx_, g, gemv_workspace(slot), s); });
}

// ------------------------------------------------------------------ measured tuner
// (src/executor/tuning.rs:18-313): one clock-warming launch, then round 0 (discarded) plus R
// measured rounds over all candidates, interleaved in the alternating order of `tune_candidate_at`
// so that clock drift biases no kernel; median per candidate; the heuristic's pick stays unless a
// challenger beats it by more than 2 %; then the split-K2 probe {4 .. 64} against the winner.
std::vector<int> Executor::tune_candidates(uint32_t m, uint32_t n, uint32_t k, bool b_f16) const {
  std::vector<int> out;
  const bool tma_ok = (k % 4 == 0) && (n % 4 == 0), umma_ok = (k % 4 == 0) && (n % 8 == 0);
  for (size_t i = 0; i < KERNEL_SPEC_COUNT; ++i) {
    const KernelSpec &spec = KERNEL_SPECS[i];
    if (spec.weights_f16 != b_f16) continue;
    // row kernels, packed layouts and the split-K stage-1 kernels are routes of their own
    // (src/pipeline/mod.rs:491-535 leaves the same families out)
    if (spec.family == Family::RowGemv || spec.family == Family::SplitK2) continue;
    if (spec.family == Family::Tf32x3 && (!tma_ok || m < 33)) continue;
    if (spec.family == Family::F16wUmma && (!umma_ok || m < 32)) continue;
    out.push_back((int)i);
  }
  return out;
}

void Executor::tune_shape(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, bool b_f16) {
  {
    std::lock_guard<std::mutex> lk(tune_mu_);
    if (tuned_.count(TuneKey{batch, m, n, k, b_f16})) return;
  }
  ctx_->make_current();
  const uint32_t sa[3] = {batch, m, k}, sb[2] = {k, n}, sc[3] = {batch, m, n};
  Tensor a = Tensor::uninit_device(ctx_, sa, 3, DType::F32);
  Tensor b = Tensor::uninit_device(ctx_, sb, 2, b_f16 ? DType::F16 : DType::F32);
  Tensor c = Tensor::uninit_device(ctx_, sc, 3, DType::F32);
  TA_CUDA(cudaMemset(a.ptr(), 0, a.size_bytes()));
  TA_CUDA(cudaMemset(b.ptr(), 0, b.size_bytes()));
  MatmulOp op;
  op.call = MatmulCall{&a, &b, &c, 1.0f, false};
  const ResolvedMatmul r = ResolvedMatmul::from_op(op);

  const std::vector<int> cands = tune_candidates(m, n, k, b_f16);
  if (cands.empty()) fail("no tunable kernel fits this shape");
  int heuristic = heuristic_kernel(batch, m, n, k, b_f16, ctx_->sm_count);
  // fewer rounds for expensive shapes (src/executor/tuning.rs:105-108, scaled to this device)
  const double est_ms = (double)r.total_flops / 200e12 * 1e3;
  const uint32_t rounds = est_ms > 8.0 ? 2 : 4;

  std::vector<std::vector<uint64_t>> samples(cands.size());
  uint64_t winner_ns = 0;
  int winner = -1;
  {
    Slot &slot = checkout_slot();
    SlotGuard g(*this, slot);
    size_t scratch = 0;
    for (int ci : cands) scratch = std::max(scratch, op_scratch_bytes(r, Route{ci, 0}));
    if (scratch) ensure_scratch(slot, scratch);
    auto run_forced = [&](int kernel) {
      const Route rt{kernel, 0, true};   // forced: the launcher must run exactly this tile
      return *timed(slot, 1, r.total_flops, [&](cudaStream_t st) { enqueue_op(op, r, rt, slot, st); }).gpu_time_ns;
    };
    const bool heur_in = std::find(cands.begin(), cands.end(), heuristic) != cands.end();
    run_forced(heur_in ? heuristic : cands[0]);   // spin the clocks up before anything is timed
    for (uint32_t round = 0; round <= rounds; ++round)
      for (size_t offset = 0; offset < cands.size(); ++offset) {
        const size_t ci = tune_candidate_at(cands.size(), round, offset);
        const uint64_t ns = run_forced(cands[ci]);
        if (round > 0) samples[ci].push_back(ns);   // round 0 is warm-up
      }
    std::optional<uint64_t> heur_ns;
    for (size_t ci = 0; ci < cands.size(); ++ci) {
      const auto med = tune_median(samples[ci]);
      if (!med) continue;
      if (cands[ci] == heuristic) heur_ns = med;
      if (winner < 0 || *med < winner_ns) {
        winner = cands[ci];
        winner_ns = *med;
      }
    }
    if (winner < 0) fail("no candidate produced a measurement");
    if (heur_ns && (double)winner_ns >= (double)*heur_ns * 0.98) {
      winner = heuristic;
      winner_ns = *heur_ns;
    }
  }   // the split-K2 probe checks out its own slot

  // Reduction-strategy pass on deep-K, few-tile shapes (src/executor/tuning.rs:214-262).
  uint32_t best_splits = 0;
  const uint64_t tiles = (uint64_t)((m + 127) / 128) * ((n + 127) / 128) * batch;
  if (!b_f16 && k >= 1024 && tiles <= 48) {
    uint64_t best_ns = 0;
    for (uint32_t sp : {4u, 8u, 16u, 32u, 64u}) {
      if (k / sp < 128 || (uint64_t)batch * sp > 65535 || (uint64_t)batch * sp * m * n * 4 > (256ull << 20)) continue;
      std::vector<uint64_t> v;
      for (uint32_t round = 0; round <= rounds; ++round) {
        const RunStats st = run_matmuls_split_k2({op.call}, sp);
        if (round > 0 && st.gpu_time_ns) v.push_back(*st.gpu_time_ns);
      }
      const auto med = tune_median(v);
      if (med && (!best_splits || *med < best_ns)) {
        best_ns = *med;
        best_splits = sp;
      }
    }
    if (best_splits && !((double)best_ns < (double)winner_ns * 0.98)) best_splits = 0;
  }
  {
    std::lock_guard<std::mutex> lk(tune_mu_);
    tuned_[TuneKey{batch, m, n, k, b_f16}] = TunedEntry{winner, best_splits};
    save_tuned(tune_path_, tuned_);
  }
}

// ------------------------------------------------------------------ prepared replay
// (src/executor/prepared.rs:78-155): data-parallel routes only; recorded once
// into a CUDA graph on a private stream; one submission in flight per handle.
std::unique_ptr<PreparedOps> prepare_ops(Executor &exec, const std::vector<MatmulOp> &ops,
                                         bool as_graph) {
  (void)as_graph;
  if (ops.empty()) fail("prepare_ops: empty op list");
  if (ops.size() > exec.max_calls())
    fail("batch of %zu calls exceeds max_calls_per_submit = %u", ops.size(), exec.max_calls());
  exec.context()->make_current();
  auto prep = std::make_unique<PreparedOps>();
  prep->exec = &exec;
  prep->ctx = exec.context();
  std::vector<ResolvedMatmul> resolved;
  std::vector<Route> routes;
  for (const MatmulOp &op : ops) {
    validate_op_tensors(exec, op);
    resolved.push_back(ResolvedMatmul::from_op(op));
    routes.push_back(exec.plan_op(op, resolved.back(), false));
    prep->total_flops += resolved.back().total_flops;
  }
  prep->n_calls = ops.size();
  TA_CUDA(cudaStreamCreateWithFlags(&prep->stream, cudaStreamNonBlocking));
  TA_CUDA(cudaEventCreate(&prep->ev_begin));
  TA_CUDA(cudaEventCreate(&prep->ev_end));
  size_t scratch_bytes = 0;
  for (size_t i = 0; i < ops.size(); ++i) scratch_bytes = std::max(scratch_bytes, exec.op_scratch_bytes(resolved[i], routes[i]));
  if (scratch_bytes) TA_CUDA(cudaMalloc(&prep->scratch, scratch_bytes));
  TA_CUDA(cudaMalloc((void **)&prep->counters, SLOT_WORDS * sizeof(uint32_t)));
  TA_CUDA(cudaMemset(prep->counters, 0, SLOT_WORDS * sizeof(uint32_t)));
  alloc_status_word(&prep->status_host, &prep->status);
  // Captured directly, nothing runs at create time: encoding tensor maps and setting function
  // attributes are host calls, which a stream capture allows.
  Slot &real_slot = exec.checkout_slot();
  {
    SlotGuard g(exec, real_slot);
    Slot slot = real_slot;            // captured launches must point at this object's own scratch and status word
    slot.scratch = prep->scratch;
    slot.scratch_bytes = scratch_bytes;
    slot.counters = prep->counters;
    slot.status = prep->status;
    slot.status_host = prep->status_host;
    TA_CUDA(cudaStreamBeginCapture(prep->stream, cudaStreamCaptureModeThreadLocal));
    try {
      for (size_t i = 0; i < ops.size(); ++i)
        exec.enqueue_op(ops[i], resolved[i], routes[i], slot, prep->stream);
    } catch (...) {
      cudaGraph_t dead = nullptr;
      cudaStreamEndCapture(prep->stream, &dead);
      if (dead) cudaGraphDestroy(dead);
      throw;
    }
    TA_CUDA(cudaStreamEndCapture(prep->stream, &prep->graph));
  }
  TA_CUDA(cudaGraphInstantiate(&prep->graph_exec, prep->graph, 0));
  return prep;
}

PreparedOps::~PreparedOps() {
  // the executor may already be gone (handles are destroyed in any order): only the context is touched here
  if (ctx) cudaSetDevice(ctx->device);
  if (stream) cudaStreamSynchronize(stream);  // wait for in-flight work
  if (graph_exec) cudaGraphExecDestroy(graph_exec);
  if (graph) cudaGraphDestroy(graph);
  if (ev_begin) cudaEventDestroy(ev_begin);
  if (ev_end) cudaEventDestroy(ev_end);
  if (stream) cudaStreamDestroy(stream);
  if (counters) cudaFree(counters);
  if (scratch) cudaFree(scratch);
  free_status_word(status_host);
}

void PreparedOps::submit() {
  if (in_flight) fail("PreparedOps::submit: a submission is already in flight; call wait() first");
  exec->context()->make_current();
  exchange.advance();   // the replay's fused exchanges wait for the arrival counts of this submission
  TA_CUDA(cudaEventRecord(ev_begin, stream));
  TA_CUDA(cudaGraphLaunch(graph_exec, stream));
  TA_CUDA(cudaEventRecord(ev_end, stream));
  in_flight = true;
}

RunStats PreparedOps::wait() {
  if (!in_flight) fail("PreparedOps::wait: nothing in flight; call submit() first");
  exec->context()->make_current();
  TA_CUDA(cudaStreamSynchronize(stream));
  in_flight = false;
  // a kernel of the replayed graph that gave up on a bounded wait reports here, as for an eager run
  if (status_host) check_status_word(status_host, counters);
  float ms = 0.0f;
  TA_CUDA(cudaEventElapsedTime(&ms, ev_begin, ev_end));
  RunStats st;
  st.gpu_time_ns = (uint64_t)((double)ms * 1e6 + 0.5);
  st.n_calls = n_calls;
  st.total_flops = total_flops;
  return st;
}

RunStats PreparedOps::run() {
  submit();
  return wait();
}

}  // namespace ta
