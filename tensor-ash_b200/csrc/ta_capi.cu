// extern "C" boundary: the symbols of include/tensor_ash.h.
//
// Conventions follow the reference's Rust cdylib (capi/src/error.rs:8-121,
// capi/src/handles.rs:6-60): the per-thread error string is cleared on entry,
// status functions return 0 / -1, creators return pointer / NULL, any C++
// exception is caught here (the analogue of the reference's panic barrier),
// destroying NULL is a no-op, and a tensor from another context is rejected
// with "<operation>: <operand> belongs to a different ... context".
#include <cmath>
#include <cstring>
#include <functional>
#include <string>

#pragma GCC visibility push(default)
#include "../../include/tensor_ash.h"
#pragma GCC visibility pop
#include "ta_core.hpp"

using namespace ta;

#include "ta_handles.hpp"

namespace {

thread_local std::string g_last_error;
}  // namespace

// shared with the other translation units that export C symbols
void ta_set_last_error(const char *msg) { g_last_error = msg ? msg : ""; }

namespace {

int status_call(const std::function<void()> &f) {
  g_last_error.clear();
  try {
    f();
    return 0;
  } catch (const std::exception &e) {
    g_last_error = e.what();
  } catch (...) {
    g_last_error = "panic crossed tensor-ash C ABI boundary";
  }
  return -1;
}

template <class T>
T *create_call(const std::function<T *()> &f) {
  g_last_error.clear();
  try {
    return f();
  } catch (const std::exception &e) {
    g_last_error = e.what();
  } catch (...) {
    g_last_error = "panic crossed tensor-ash C ABI boundary";
  }
  return nullptr;
}

template <class T>
const T &checked_ref(const T *p, const char *msg) {
  if (!p) fail("%s", msg);
  return *p;
}

const Tensor &checked_tensor(const ta_executor &exec, const ta_tensor *t, const char *operation,
                             const char *operand) {
  if (!t) fail("%s: %s is null", operation, operand);
  if (t->tensor.ctx().get() != exec.ctx.get())
    fail("%s: %s belongs to a different Vulkan context", operation, operand);
  return t->tensor;
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

MatmulCall checked_call(const ta_executor &exec, const ta_matmul_call &raw, const char *operation) {
  MatmulCall c;
  c.a = &checked_tensor(exec, raw.a, operation, "a");
  c.b = &checked_tensor(exec, raw.b, operation, "b");
  c.c = &checked_tensor(exec, raw.c, operation, "c");
  c.alpha = raw.alpha;
  c.accumulate = raw.accumulate != 0;
  return c;
}

// (capi/src/api/ops.rs:14-69)
MatmulOp checked_op(const ta_executor &exec, const ta_matmul_op &raw, const char *operation) {
  MatmulOp op;
  op.call = checked_call(exec, raw.call, operation);
  const ta_epilogue &ep = raw.epilogue;
  if (ep.bias) op.epilogue.bias = &checked_tensor(exec, ep.bias, operation, "epilogue.bias");
  if (ep.activation > 3)
    fail("%s: epilogue.activation %u is invalid (0=none 1=relu 2=silu 3=gelu)", operation,
         ep.activation);
  op.epilogue.activation = (Activation)ep.activation;
  switch (ep.binary_kind) {
    case 0:
      if (ep.d) fail("%s: epilogue.d is set but binary_kind is 0 (none)", operation);
      break;
    case 1:
      op.epilogue.binary = BinaryKind::AddScaled;
      op.epilogue.d = &checked_tensor(exec, ep.d, operation, "epilogue.d");
      op.epilogue.beta = ep.beta;
      break;
    case 2:
      op.epilogue.binary = BinaryKind::Mul;
      op.epilogue.d = &checked_tensor(exec, ep.d, operation, "epilogue.d");
      break;
    default:
      fail("%s: epilogue.binary_kind %u is invalid (0=none 1=add_scaled 2=mul)", operation,
           ep.binary_kind);
  }
  return op;
}

std::vector<MatmulOp> checked_ops(const ta_executor &exec, const ta_matmul_op *ops, size_t n,
                                  const char *operation) {
  if (n && !ops) fail("%s: ops is null", operation);
  std::vector<MatmulOp> out;
  out.reserve(n);
  for (size_t i = 0; i < n; ++i)
    out.push_back(checked_op(exec, ops[i], strf("%s: op %zu", operation, i).c_str()));
  return out;
}

ta_executor *executor_create(const ta_context *ctx, size_t n_slots, uint32_t max_calls,
                             const char *selection, bool tune, const char *operation) {
  const ta_context &c = checked_ref(ctx, strf("%s: ctx is null", operation).c_str());
  const int sel = kernel_selection_parse(selection ? selection : "auto");
  ExecutorConfig cfg;
  cfg.n_slots = n_slots;
  cfg.max_calls_per_submit = max_calls;
  cfg.tune = tune;
  auto *h = new ta_executor;
  h->ctx = c.ctx;
  try {
    h->exec = std::make_unique<Executor>(c.ctx, sel, cfg);
  } catch (...) {
    delete h;
    throw;
  }
  return h;
}

ta_tensor *tensor_create(const std::shared_ptr<Context> &ctx, const uint32_t *shape, size_t rank,
                         DType dtype, const char *operation) {
  if (rank && !shape) fail("%s: shape is null", operation);
  auto *h = new ta_tensor;
  try {
    h->tensor = Tensor::uninit_device(ctx, shape, rank, dtype);
  } catch (...) {
    delete h;
    throw;
  }
  return h;
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

const char *ta_version(void) { return "2.0.0"; }
const char *ta_last_error(void) { return g_last_error.c_str(); }

ta_context *ta_context_create(uint32_t enable_validation, const char *device_preference) {
  return create_call<ta_context>([&]() {
    std::string pref = device_preference ? device_preference : "";
    if (!device_preference) {
      if (const char *env = getenv("ML_DEVICE")) pref = env;  // src/context/mod.rs:95-103
    }
    auto *h = new ta_context;
    try {
      h->ctx = Context::create(enable_validation != 0, pref);
    } catch (...) {
      delete h;
      throw;
    }
    return h;
  });
}

void ta_context_destroy(ta_context *ctx) {
  g_last_error.clear();
  delete ctx;
}

uint32_t ta_context_supports_f16(const ta_context *ctx) { return ctx ? 1u : 0u; }
uint32_t ta_context_supports_bda(const ta_context *ctx) { return ctx ? 1u : 0u; }

ta_executor *ta_executor_create(const ta_context *ctx, size_t n_slots, uint32_t max_calls_per_submit,
                                const char *kernel_selection) {
  return create_call<ta_executor>([&]() {
    const char *sel = kernel_selection;
    if (!sel) sel = getenv("ML_KERNEL");
    return executor_create(ctx, n_slots, max_calls_per_submit, sel, false, "ta_executor_create");
  });
}

ta_executor *ta_executor_create_v2(const ta_context *ctx, size_t n_slots,
                                   uint32_t max_calls_per_submit, const char *kernel_selection,
                                   uint32_t tune) {
  return create_call<ta_executor>([&]() {
    const char *sel = kernel_selection;
    if (!sel) sel = getenv("ML_KERNEL");
    return executor_create(ctx, n_slots, max_calls_per_submit, sel, tune != 0,
                           "ta_executor_create_v2");
  });
}

void ta_executor_destroy(ta_executor *exec) {
  g_last_error.clear();
  delete exec;
}

ta_tensor *ta_tensor_create(const ta_context *ctx, const uint32_t *shape, size_t rank) {
  return create_call<ta_tensor>([&]() {
    const ta_context &c = checked_ref(ctx, "ta_tensor_create: ctx is null");
    return tensor_create(c.ctx, shape, rank, DType::F32, "ta_tensor_create");
  });
}
ta_tensor *ta_tensor_create_on_executor(const ta_executor *exec, const uint32_t *shape, size_t rank) {
  return create_call<ta_tensor>([&]() {
    const ta_executor &e = checked_ref(exec, "ta_tensor_create_on_executor: exec is null");
    return tensor_create(e.ctx, shape, rank, DType::F32, "ta_tensor_create_on_executor");
  });
}
ta_tensor *ta_tensor_create_f16(const ta_context *ctx, const uint32_t *shape, size_t rank) {
  return create_call<ta_tensor>([&]() {
    const ta_context &c = checked_ref(ctx, "ta_tensor_create_f16: ctx is null");
    return tensor_create(c.ctx, shape, rank, DType::F16, "ta_tensor_create_f16");
  });
}
ta_tensor *ta_tensor_create_f16_on_executor(const ta_executor *exec, const uint32_t *shape,
                                            size_t rank) {
  return create_call<ta_tensor>([&]() {
    const ta_executor &e = checked_ref(exec, "ta_tensor_create_f16_on_executor: exec is null");
    return tensor_create(e.ctx, shape, rank, DType::F16, "ta_tensor_create_f16_on_executor");
  });
}
void ta_tensor_destroy(ta_tensor *tensor) {
  g_last_error.clear();
  delete tensor;
}
uint64_t ta_tensor_len(const ta_tensor *tensor) { return tensor ? tensor->tensor.len() : 0; }
uint64_t ta_tensor_size_bytes(const ta_tensor *tensor) {
  return tensor ? tensor->tensor.size_bytes() : 0;
}
uint32_t ta_tensor_is_f16(const ta_tensor *tensor) {
  return tensor && tensor->tensor.dtype == DType::F16 ? 1u : 0u;
}

int ta_upload(const ta_executor *exec, const ta_tensor *dst, const float *src, size_t len) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_upload: exec is null");
    const Tensor &d = checked_tensor(e, dst, "ta_upload", "dst");
    if (len && !src) fail("ta_upload: src is null");
    e.exec->upload(src, len, d);
  });
}

int ta_download(const ta_executor *exec, const ta_tensor *src, float *dst, size_t len) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_download: exec is null");
    const Tensor &s = checked_tensor(e, src, "ta_download", "src");
    if (len && !dst) fail("ta_download: dst is null");
    e.exec->download(s, dst, len);
  });
}

int ta_matmul(const ta_executor *exec, const ta_tensor *a, const ta_tensor *b, const ta_tensor *c,
              float alpha, uint32_t accumulate, ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_matmul: exec is null");
    const ta_matmul_call raw{a, b, c, alpha, accumulate};
    write_stats(stats, e.exec->run_matmuls({checked_call(e, raw, "ta_matmul")}));
  });
}

int ta_matmul_batch(const ta_executor *exec, const ta_matmul_call *calls, size_t n_calls,
                    ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_matmul_batch: exec is null");
    if (n_calls && !calls) fail("ta_matmul_batch: calls is null");
    std::vector<MatmulCall> v;
    for (size_t i = 0; i < n_calls; ++i)
      v.push_back(checked_call(e, calls[i], strf("ta_matmul_batch: call %zu", i).c_str()));
    write_stats(stats, e.exec->run_matmuls(v));
  });
}

int ta_run_ops(const ta_executor *exec, const ta_matmul_op *ops, size_t n_ops, ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_run_ops: exec is null");
    write_stats(stats, e.exec->run_ops(checked_ops(e, ops, n_ops, "ta_run_ops")));
  });
}

int ta_run_matmul_host_batched(const ta_executor *exec, const ta_host_batched_matmul *desc,
                               ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_run_matmul_host_batched: exec is null");
    if (!desc) fail("ta_run_matmul_host_batched: desc is null");
    if (desc->activation > 3) fail("ta_run_matmul_host_batched: activation %u is invalid", desc->activation);
    if (desc->binary > 2) fail("ta_run_matmul_host_batched: binary %u is invalid", desc->binary);
    HostBatchedMatmul h;
    h.batch = desc->batch; h.m = desc->m; h.n = desc->n; h.k = desc->k;
    h.a = desc->a; h.b_host = desc->b_host; h.c = desc->c;
    h.b = desc->b ? &checked_tensor(e, desc->b, "ta_run_matmul_host_batched", "b") : nullptr;
    h.bias = desc->bias; h.bias_per_batch = desc->bias_per_batch != 0;
    h.d = desc->d;
    h.activation = (Activation)desc->activation;
    h.binary = (BinaryKind)desc->binary;
    h.alpha = desc->alpha; h.beta = desc->beta;
    h.chunk_batch = desc->chunk_batch;
    write_stats(stats, e.exec->run_matmul_host_batched(h));
  });
}

void *ta_pinned_alloc(size_t bytes) {
  void *p = nullptr;
  if (!bytes || cudaHostAlloc(&p, bytes, cudaHostAllocDefault) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return p;
}

void ta_pinned_free(void *ptr) {
  if (ptr) cudaFreeHost(ptr);
}

int ta_run_op_graph(const ta_executor *exec, const ta_matmul_op *ops, size_t n_ops,
                    ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_run_op_graph: exec is null");
    write_stats(stats, e.exec->run_op_graph(checked_ops(e, ops, n_ops, "ta_run_op_graph")));
  });
}

int ta_softmax_rows(const ta_executor *exec, const ta_tensor *input, const ta_tensor *output,
                    float scale, uint32_t mask_kind, uint32_t valid_or_prefix,
                    uint32_t rows_per_group, ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_softmax_rows: exec is null");
    const Tensor &in = checked_tensor(e, input, "ta_softmax_rows", "input");
    const Tensor &out = checked_tensor(e, output, "ta_softmax_rows", "output");
    if (mask_kind > 2)
      fail("ta_softmax_rows: mask_kind %u is invalid (0=full 1=prefix 2=causal)", mask_kind);
    write_stats(stats, e.exec->softmax_rows(in, out, scale, mask_kind, valid_or_prefix, rows_per_group));
  });
}

int ta_rms_norm(const ta_executor *exec, const ta_tensor *input, const ta_tensor *weight,
                const ta_tensor *output, float eps, ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_rms_norm: exec is null");
    const Tensor &in = checked_tensor(e, input, "ta_rms_norm", "input");
    const Tensor &w = checked_tensor(e, weight, "ta_rms_norm", "weight");
    const Tensor &out = checked_tensor(e, output, "ta_rms_norm", "output");
    write_stats(stats, e.exec->rms_norm(in, w, out, eps));
  });
}

int ta_layer_norm(const ta_executor *exec, const ta_tensor *input, const ta_tensor *weight,
                  const ta_tensor *bias, const ta_tensor *output, float eps, ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_layer_norm: exec is null");
    const Tensor &in = checked_tensor(e, input, "ta_layer_norm", "input");
    const Tensor &w = checked_tensor(e, weight, "ta_layer_norm", "weight");
    const Tensor &b = checked_tensor(e, bias, "ta_layer_norm", "bias");
    const Tensor &out = checked_tensor(e, output, "ta_layer_norm", "output");
    write_stats(stats, e.exec->layer_norm(in, w, b, out, eps));
  });
}

int ta_rope(const ta_executor *exec, const ta_tensor *input, const ta_tensor *table,
            const ta_tensor *output, const ta_rope_desc *desc, ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_rope: exec is null");
    const Tensor &in = checked_tensor(e, input, "ta_rope", "input");
    const Tensor &tab = checked_tensor(e, table, "ta_rope", "table");
    const Tensor &out = checked_tensor(e, output, "ta_rope", "output");
    const ta_rope_desc &d = checked_ref(desc, "ta_rope: desc is null");
    write_stats(stats, e.exec->rope(in, tab, out, d.heads, d.head_dim, d.rot_dim, d.pos_base));
  });
}

int ta_copy_strided(const ta_executor *exec, const ta_tensor *src, const ta_tensor *dst,
                    const ta_copy_desc *desc, ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_copy_strided: exec is null");
    const Tensor &s = checked_tensor(e, src, "ta_copy_strided", "src");
    const Tensor &d = checked_tensor(e, dst, "ta_copy_strided", "dst");
    const ta_copy_desc &cd = checked_ref(desc, "ta_copy_strided: desc is null");
    write_stats(stats, e.exec->copy_strided(s, d, cd.extent, cd.src_offset, cd.src_strides,
                                            cd.dst_offset, cd.dst_strides));
  });
}

ta_prepared *ta_prepared_create(const ta_executor *exec, const ta_matmul_op *ops, size_t n_ops,
                                uint32_t as_graph) {
  return create_call<ta_prepared>([&]() {
    const ta_executor &e = checked_ref(exec, "ta_prepared_create: exec is null");
    auto v = checked_ops(e, ops, n_ops, "ta_prepared_create");
    auto *h = new ta_prepared;
    h->ctx = e.ctx;
    try {
      h->prepared = prepare_ops(*e.exec, v, as_graph != 0);
    } catch (...) {
      delete h;
      throw;
    }
    return h;
  });
}

int ta_prepared_run(ta_prepared *prepared, ta_run_stats *stats) {
  return status_call([&]() {
    if (!prepared) fail("ta_prepared_run: prepared is null");
    write_stats(stats, prepared->prepared->run());
  });
}
int ta_prepared_submit(ta_prepared *prepared) {
  return status_call([&]() {
    if (!prepared) fail("ta_prepared_submit: prepared is null");
    prepared->prepared->submit();
  });
}
int ta_prepared_wait(ta_prepared *prepared, ta_run_stats *stats) {
  return status_call([&]() {
    if (!prepared) fail("ta_prepared_wait: prepared is null");
    write_stats(stats, prepared->prepared->wait());
  });
}
void ta_prepared_destroy(ta_prepared *prepared) {
  g_last_error.clear();
  delete prepared;
}

int ta_dispatch_info_for(const ta_executor *exec, uint32_t batch, uint32_t m, uint32_t n, uint32_t k,
                         uint32_t b_f16, ta_dispatch_info *out) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_dispatch_info_for: exec is null");
    if (!out) fail("ta_dispatch_info_for: out is null");
    if (!batch || !m || !n || !k)
      fail("matmul dimensions must be non-zero, got B=%u rows=%u cols=%u", batch, m, n);
    const Route r = e.exec->plan_shape(batch, m, n, k, b_f16 != 0, true);
    const KernelSpec &spec = KERNEL_SPECS[r.kernel];
    out->kernel = spec.name;
    out->tile[0] = spec.tile_m;
    out->tile[1] = spec.tile_n;
    out->tile[2] = spec.tile_k;
    out->has_split_k2 = r.splits > 1;
    out->split_k2_splits = r.splits > 1 ? r.splits : 0;
  });
}

int ta_tune_shape(const ta_executor *exec, uint32_t batch, uint32_t m, uint32_t n, uint32_t k) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_tune_shape: exec is null");
    if (!batch || !m || !n || !k)
      fail("matmul dimensions must be non-zero, got B=%u rows=%u cols=%u", batch, m, n);
    e.exec->tune_shape(batch, m, n, k);
  });
}

// ===================================================================== PART 2

int ta_tune_shape_f16w(const ta_executor *exec, uint32_t batch, uint32_t m, uint32_t n, uint32_t k) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_tune_shape_f16w: exec is null");
    if (!batch || !m || !n || !k)
      fail("matmul dimensions must be non-zero, got B=%u rows=%u cols=%u", batch, m, n);
    e.exec->tune_shape(batch, m, n, k, true);
  });
}

int ta_tune_median(const uint64_t *samples, size_t n, uint64_t *out) {
  g_last_error.clear();
  if ((n && !samples) || !out) {
    g_last_error = "ta_tune_median: null argument";
    return -1;
  }
  const auto med = tune_median(std::vector<uint64_t>(samples, samples + n));
  if (!med) return 1;
  *out = *med;
  return 0;
}

size_t ta_tune_candidate_at(size_t len, uint32_t round, size_t offset) {
  return len ? tune_candidate_at(len, round, offset) : 0;
}

static int copy_out(const std::string &v, char *buf, size_t cap, const char *who) {
  return status_call([&]() {
    if (!buf || v.size() + 1 > cap) fail("%s: buffer of %zu bytes cannot hold %zu", who, cap, v.size() + 1);
    memcpy(buf, v.c_str(), v.size() + 1);
  });
}

int ta_tune_store_path(const char *device_name, char *buf, size_t cap) {
  return copy_out(tune_store_path(device_name ? device_name : ""), buf, cap, "ta_tune_store_path");
}

int ta_tune_store_rewrite(const char *in_path, const char *out_path, size_t *n_entries) {
  return status_call([&]() {
    if (!in_path) fail("ta_tune_store_rewrite: in_path is null");
    const auto map = load_tuned(in_path);
    if (n_entries) *n_entries = map.size();
    if (out_path) save_tuned(out_path, map);
  });
}

int ta_experiment_check(const char *spec) {
  return status_call([&]() { (void)parse_tunables(spec); });
}

int ta_selftest_bounded_wait(const ta_executor *exec, uint32_t limit_ns) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_selftest_bounded_wait: exec is null");
    if (limit_ns == 0 || limit_ns > 1000000000u)
      fail("ta_selftest_bounded_wait: limit_ns %u out of range (1 .. 1e9)", limit_ns);
    e.exec->selftest_bounded_wait(limit_ns);
  });
}

int ta_matmul_split_k2(const ta_executor *exec, const ta_matmul_call *calls, size_t n_calls,
                       uint32_t splits, ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_matmul_split_k2: exec is null");
    if (n_calls && !calls) fail("ta_matmul_split_k2: calls is null");
    std::vector<MatmulCall> v;
    for (size_t i = 0; i < n_calls; ++i)
      v.push_back(checked_call(e, calls[i], strf("ta_matmul_split_k2: call %zu", i).c_str()));
    write_stats(stats, e.exec->run_matmuls_split_k2(v, splits));
  });
}

int ta_split_k2_noalloc(const float *a, const float *b, float *c, uint32_t m, uint32_t n, uint32_t k,
                        uint32_t splits, float alpha, void *stream) {
  return status_call([&]() {
    if (!a || !b || !c) fail("ta_split_k2_noalloc: a, b and c must be device pointers (got null)");
    if (!m || !n || !k) fail("ta_split_k2_noalloc: M, N, K must be non-zero (got %u, %u, %u)", m, n, k);
    if (c == a || c == b) fail("ta_split_k2_noalloc: C must not alias an input");
    if (splits < 2) fail("ta_split_k2_noalloc: splits must be at least 2 (got %u)", splits);
    if (splits > k) fail("ta_split_k2_noalloc: num_k_splits %u exceeds K=%u", splits, k);
    if (splits > 65535) fail("ta_split_k2_noalloc: num_k_splits %u exceeds the 65535 limit", splits);
    if ((uint64_t)m * k > (1ull << 32) || (uint64_t)k * n > (1ull << 32))
      fail("ta_split_k2_noalloc: operand exceeds 2^32 elements");
    GemmParams p{};
    p.a = a; p.b = b; p.c = c;
    p.m = m; p.n = n; p.k = k; p.batch = 1;
    p.alpha = alpha;
    p.splits = splits;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    launch_splitk2_static(p, st);
    TA_CUDA(cudaStreamSynchronize(st));
  });
}

static MatmulOp checked_op_ex(const ta_executor &e, const ta_matmul_op_ex &raw, const std::string &label) {
      MatmulOp op = checked_op(e, raw.op, label.c_str());
      op.packed_b = raw.packed_b != 0;
      if (raw.normed_weight) {
        op.normed_weight = &checked_tensor(e, raw.normed_weight, label.c_str(), "normed_weight");
        op.normed_eps = raw.normed_eps;
      }
      const ta_store_desc &s = raw.store;
      if (s.kind > 3) fail("%s: store.kind %u is invalid (0..3)", label.c_str(), s.kind);
      op.store.kind = (StoreKind)s.kind;
      op.store.head_dim = s.head_dim;
      op.store.pos_base = s.pos_base;
      op.store.pos_scale = s.pos_scale;
      op.store.stride_head = s.stride_head;
      op.store.stride_dim = s.stride_dim;
      if (s.table) op.store.table = &checked_tensor(e, s.table, label.c_str(), "store.table");
      if (s.dst) op.store.dst = &checked_tensor(e, s.dst, label.c_str(), "store.dst");
      if (s.pos_cell) {
        if (s.pos_cell->cell.ctx.get() != e.ctx.get())
          fail("%s: store.pos_cell belongs to a different Vulkan context", label.c_str());
        op.store.pos_cell = &s.pos_cell->cell;
      }
      return op;
}

int ta_run_ops_ex(const ta_executor *exec, const ta_matmul_op_ex *ops, size_t n_ops,
                  uint32_t as_graph, ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_run_ops_ex: exec is null");
    if (n_ops && !ops) fail("ta_run_ops_ex: ops is null");
    std::vector<MatmulOp> v;
    for (size_t i = 0; i < n_ops; ++i) v.push_back(checked_op_ex(e, ops[i], strf("ta_run_ops_ex: op %zu", i)));
    write_stats(stats, as_graph ? e.exec->run_op_graph(v) : e.exec->run_ops(v));
  });
}

static std::vector<ExecOp> checked_exec_ops(const ta_executor &e, const ta_exec_op *ops, size_t n, const char *operation) {
  if (n && !ops) fail("%s: ops is null", operation);
  std::vector<ExecOp> v(n);
  for (size_t i = 0; i < n; ++i) {
    const ta_exec_op &r = ops[i];
    const std::string label = strf("%s: op %zu", operation, i);
    ExecOp &o = v[i];
    if (r.kind > TA_EXEC_ARGMAX_SHARDED) fail("%s: kind %u is invalid", label.c_str(), r.kind);
    o.kind = (ExecKind)r.kind;
    if (r.kind == TA_EXEC_MATMUL) o.mm = checked_op_ex(e, r.mm, label);
    auto opt = [&](const ta_tensor *t, const char *name) -> const Tensor * {
      return t ? &checked_tensor(e, t, label.c_str(), name) : nullptr;
    };
    o.in0 = opt(r.in0, "in0"); o.in1 = opt(r.in1, "in1"); o.in2 = opt(r.in2, "in2"); o.in3 = opt(r.in3, "in3");
    o.out = opt(r.out, "out");
    o.f0 = r.f0; o.u0 = r.u0; o.u1 = r.u1; o.u2 = r.u2;
    if (r.kind == TA_EXEC_ATTN_DECODE) o.u0 = 0;   // planner-internal hint, not caller input
    o.heads = r.rope.heads; o.head_dim = r.rope.head_dim; o.rot_dim = r.rope.rot_dim; o.pos_base = r.rope.pos_base;
    if (r.kind == TA_EXEC_COPY_STRIDED) {
      o.src_offset = r.copy.src_offset; o.dst_offset = r.copy.dst_offset;
      for (int d = 0; d < 3; ++d) {
        o.extent[d] = r.copy.extent[d];
        o.src_strides[d] = r.copy.src_strides[d];
        o.strides[d] = r.copy.dst_strides[d];
      }
    } else {
      o.dst_offset = r.dst_offset;
      for (int d = 0; d < 3; ++d) o.strides[d] = r.dst_strides[d];
    }
    o.pos_scale = r.pos_scale;
    o.flash.kv_len = r.flash.kv_len; o.flash.pos_base = r.flash.pos_base; o.flash.scale = r.flash.scale;
    o.flash.token_major_heads = r.flash.token_major_heads;
    o.flash.out_token_major_heads = r.flash.out_token_major_heads;
    o.flash.simt = r.flash.simt;
    o.attn.kv_len = r.attn.kv_len; o.attn.scale = r.attn.scale;
    o.attn.pos_cell = r.attn.pos_cell ? &r.attn.pos_cell->cell : nullptr;
    o.cell = r.cell ? &r.cell->cell : nullptr;
    o.tokens = r.tokens ? &r.tokens->ids : nullptr;
    o.comm = r.comm ? r.comm->comm.get() : nullptr;
  }
  return v;
}

int ta_run_exec_ops(const ta_executor *exec, const ta_exec_op *ops, size_t n_ops, ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_run_exec_ops: exec is null");
    write_stats(stats, e.exec->run_exec_ops(checked_exec_ops(e, ops, n_ops, "ta_run_exec_ops")));
  });
}

ta_prepared *ta_prepared_create_exec(const ta_executor *exec, const ta_exec_op *ops, size_t n_ops) {
  return create_call<ta_prepared>([&]() {
    const ta_executor &e = checked_ref(exec, "ta_prepared_create_exec: exec is null");
    auto v = checked_exec_ops(e, ops, n_ops, "ta_prepared_create_exec");
    auto *h = new ta_prepared;
    h->ctx = e.ctx;
    try {
      h->prepared = prepare_exec_ops(*e.exec, v);
    } catch (...) {
      delete h;
      throw;
    }
    return h;
  });
}

int ta_comm_unique_id(uint8_t out[TA_COMM_ID_BYTES]) {
  return status_call([&]() {
    if (!out) fail("ta_comm_unique_id: out is null");
    comm_unique_id(out);
  });
}
ta_comm *ta_comm_create(const ta_context *ctx, uint32_t rank, uint32_t world, const uint8_t *id) {
  return create_call<ta_comm>([&]() {
    const ta_context &c = checked_ref(ctx, "ta_comm_create: ctx is null");
    if (world > 1 && !id) fail("ta_comm_create: id is null");
    uint8_t zero[TA_COMM_ID_BYTES] = {0};
    auto *h = new ta_comm;
    try {
      h->comm = Comm::create(c.ctx, rank, world, id ? id : zero);
    } catch (...) {
      delete h;
      throw;
    }
    return h;
  });
}
void ta_comm_destroy(ta_comm *comm) {
  g_last_error.clear();
  delete comm;
}
int ta_comm_set_wait_limit_ns(ta_comm *comm, uint64_t limit_ns) {
  return status_call([&]() {
    if (!comm) fail("ta_comm_set_wait_limit_ns: comm is null");
    if (limit_ns < 1000 || limit_ns > 600000000000ull)
      fail("ta_comm_set_wait_limit_ns: %llu ns is outside 1 us .. 600 s", (unsigned long long)limit_ns);
    comm->comm->peer_wait_limit_ns = limit_ns;
  });
}

int ta_comm_resync(ta_comm *comm) {
  return status_call([&]() {
    if (!comm) fail("ta_comm_resync: comm is null");
    comm->comm->resync();
  });
}

uint32_t ta_comm_rank(const ta_comm *comm) { return comm ? comm->comm->rank : 0; }
uint32_t ta_comm_world(const ta_comm *comm) { return comm ? comm->comm->world : 0; }

ta_token_ids *ta_token_ids_create(const ta_context *ctx, uint32_t capacity) {
  return create_call<ta_token_ids>([&]() {
    const ta_context &c = checked_ref(ctx, "ta_token_ids_create: ctx is null");
    if (capacity == 0) fail("ta_token_ids_create: capacity must be non-zero");
    c.ctx->make_current();
    auto *h = new ta_token_ids;
    h->ids.ctx = c.ctx;
    h->ids.capacity = capacity;
    cudaError_t err = cudaHostAlloc((void **)&h->ids.host, (size_t)capacity * 4, cudaHostAllocMapped);
    if (err == cudaSuccess) err = cudaHostGetDevicePointer((void **)&h->ids.device, h->ids.host, 0);
    if (err != cudaSuccess) {
      if (h->ids.host) cudaFreeHost(h->ids.host);
      delete h;
      fail("ta_token_ids_create: pinned allocation failed: %s", cudaGetErrorString(err));
    }
    return h;
  });
}
void ta_token_ids_destroy(ta_token_ids *ids) {
  g_last_error.clear();
  if (!ids) return;
  if (ids->ids.host) {
    cudaSetDevice(ids->ids.ctx->device);
    cudaFreeHost(ids->ids.host);
  }
  delete ids;
}
int ta_token_ids_set(ta_token_ids *ids, const uint32_t *tokens, uint32_t n) {
  return status_call([&]() {
    if (!ids) fail("ta_token_ids_set: ids is null");
    if (n && !tokens) fail("ta_token_ids_set: tokens is null");
    if (n > ids->ids.capacity) fail("ta_token_ids_set: %u tokens exceed capacity %u", n, ids->ids.capacity);
    memcpy(ids->ids.host, tokens, (size_t)n * 4);
    ids->ids.len = n;
  });
}

int ta_swiglu_gemv(const ta_executor *exec, const ta_tensor *x, const ta_tensor *wg, const ta_tensor *wup,
                   const ta_tensor *out, const ta_tensor *normed_weight, float normed_eps,
                   ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_swiglu_gemv: exec is null");
    const Tensor &tx = checked_tensor(e, x, "ta_swiglu_gemv", "x");
    const Tensor &tg = checked_tensor(e, wg, "ta_swiglu_gemv", "wg");
    const Tensor &tu = checked_tensor(e, wup, "ta_swiglu_gemv", "wup");
    const Tensor &to = checked_tensor(e, out, "ta_swiglu_gemv", "out");
    const Tensor *tn = normed_weight ? &checked_tensor(e, normed_weight, "ta_swiglu_gemv", "normed_weight") : nullptr;
    write_stats(stats, e.exec->swiglu_gemv(tx, tg, tu, to, tn, normed_eps));
  });
}

int ta_pack_f16w_row_tiles(const float *src, float *dst, size_t k, size_t n, size_t tile_n) {
  return status_call([&]() {
    if (!src || !dst) fail("ta_pack_f16w_row_tiles: src/dst is null");
    pack_f16w_row_tiles(src, dst, k, n, tile_n);
  });
}
uint32_t ta_f16w_row_tile_n(uint32_t k, uint32_t n) { return f16w_row_tile_n(k, n); }

int ta_upload_f16(const ta_executor *exec, const ta_tensor *dst, const uint16_t *src, size_t len) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_upload_f16: exec is null");
    const Tensor &d = checked_tensor(e, dst, "ta_upload_f16", "dst");
    if (len && !src) fail("ta_upload_f16: src is null");
    e.exec->upload_f16(src, len, d);
  });
}

ta_tensor *ta_tensor_alias_with_shape(const ta_tensor *tensor, const uint32_t *shape, size_t rank) {
  return create_call<ta_tensor>([&]() {
    if (!tensor) fail("ta_tensor_alias_with_shape: tensor is null");
    if (rank && !shape) fail("ta_tensor_alias_with_shape: shape is null");
    auto *h = new ta_tensor;
    try {
      h->tensor = tensor->tensor.alias_with_shape(shape, rank);
    } catch (...) {
      delete h;
      throw;
    }
    return h;
  });
}

int ta_flash_attention(const ta_executor *exec, const ta_tensor *q, const ta_tensor *kt, const ta_tensor *v,
                       const ta_tensor *out, const ta_flash_desc *desc, ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_flash_attention: exec is null");
    const Tensor &tq = checked_tensor(e, q, "ta_flash_attention", "q");
    const Tensor &tk = checked_tensor(e, kt, "ta_flash_attention", "kt");
    const Tensor &tv = checked_tensor(e, v, "ta_flash_attention", "v");
    const Tensor &to = checked_tensor(e, out, "ta_flash_attention", "out");
    const ta_flash_desc &d = checked_ref(desc, "ta_flash_attention: desc is null");
    FlashAttentionDesc fd;
    fd.kv_len = d.kv_len; fd.pos_base = d.pos_base; fd.scale = d.scale;
    fd.token_major_heads = d.token_major_heads; fd.out_token_major_heads = d.out_token_major_heads;
    fd.simt = d.simt;
    write_stats(stats, e.exec->flash_attention(tq, tk, tv, to, fd));
  });
}

uint32_t ta_attn_decode_num_chunks(uint32_t kv_len) { return attn_decode_num_chunks(kv_len); }

int ta_attn_decode(const ta_executor *exec, const ta_tensor *q, const ta_tensor *kt, const ta_tensor *v,
                   const ta_tensor *scratch, const ta_tensor *out, const ta_attn_decode_desc *desc,
                   ta_run_stats *stats) {
  return status_call([&]() {
    const ta_executor &e = checked_ref(exec, "ta_attn_decode: exec is null");
    const Tensor &tq = checked_tensor(e, q, "ta_attn_decode", "q");
    const Tensor &tk = checked_tensor(e, kt, "ta_attn_decode", "kt");
    const Tensor &tv = checked_tensor(e, v, "ta_attn_decode", "v");
    const Tensor &ts = checked_tensor(e, scratch, "ta_attn_decode", "scratch");
    const Tensor &to = checked_tensor(e, out, "ta_attn_decode", "out");
    const ta_attn_decode_desc &d = checked_ref(desc, "ta_attn_decode: desc is null");
    AttnDecodeDesc ad;
    ad.kv_len = d.kv_len; ad.scale = d.scale;
    ad.pos_cell = d.pos_cell ? &d.pos_cell->cell : nullptr;
    write_stats(stats, e.exec->attn_decode(tq, tk, tv, ts, to, ad));
  });
}

ta_pos_cell *ta_pos_cell_create(const ta_context *ctx) {
  return create_call<ta_pos_cell>([&]() {
    const ta_context &c = checked_ref(ctx, "ta_pos_cell_create: ctx is null");
    c.ctx->make_current();
    auto *h = new ta_pos_cell;
    h->cell.ctx = c.ctx;
    cudaError_t e = cudaHostAlloc((void **)&h->cell.host, sizeof(uint32_t), cudaHostAllocMapped);
    if (e == cudaSuccess) e = cudaHostGetDevicePointer((void **)&h->cell.device, h->cell.host, 0);
    if (e != cudaSuccess) {
      if (h->cell.host) cudaFreeHost(h->cell.host);
      delete h;
      fail("ta_pos_cell_create: pinned allocation failed: %s", cudaGetErrorString(e));
    }
    *h->cell.host = 0;
    return h;
  });
}
void ta_pos_cell_destroy(ta_pos_cell *cell) {
  g_last_error.clear();
  if (!cell) return;
  if (cell->cell.host) {
    cudaSetDevice(cell->cell.ctx->device);
    cudaFreeHost(cell->cell.host);
  }
  delete cell;
}
int ta_pos_cell_set(ta_pos_cell *cell, uint32_t value) {
  return status_call([&]() {
    if (!cell) fail("ta_pos_cell_set: cell is null");
    *(volatile uint32_t *)cell->cell.host = value;
  });
}
int ta_pos_cell_get(const ta_pos_cell *cell, uint32_t *value) {
  return status_call([&]() {
    if (!cell) fail("ta_pos_cell_get: cell is null");
    if (!value) fail("ta_pos_cell_get: value is null");
    *value = *(volatile uint32_t *)cell->cell.host;
  });
}

size_t ta_kernel_spec_count(void) { return KERNEL_SPEC_COUNT; }

int ta_kernel_spec_at(size_t index, ta_dispatch_info *out) {
  return status_call([&]() {
    if (!out) fail("ta_kernel_spec_at: out is null");
    if (index >= KERNEL_SPEC_COUNT)
      fail("ta_kernel_spec_at: index %zu out of range (%zu kernels)", index, KERNEL_SPEC_COUNT);
    const KernelSpec &s = KERNEL_SPECS[index];
    out->kernel = s.name;
    out->tile[0] = s.tile_m;
    out->tile[1] = s.tile_n;
    out->tile[2] = s.tile_k;
    out->has_split_k2 = s.family == Family::SplitK2;
    out->split_k2_splits = 0;
  });
}

int ta_kernel_selection_parse(const char *name) {
  g_last_error.clear();
  try {
    return kernel_selection_parse(name ? name : "");
  } catch (const std::exception &e) {
    g_last_error = e.what();
    return -1;
  }
}

int ta_resolve_shapes(const uint32_t *a, size_t a_rank, const uint32_t *b, size_t b_rank,
                      const uint32_t *c, size_t c_rank, uint32_t out[9]) {
  return status_call([&]() {
    if (!a || !b || !c || !out) fail("ta_resolve_shapes: null argument");
    const ResolvedMatmul r = ResolvedMatmul::from_shapes(MatrixShape::from_shape(a, a_rank),
                                                         MatrixShape::from_shape(b, b_rank),
                                                         MatrixShape::from_shape(c, c_rank));
    out[0] = r.m; out[1] = r.n; out[2] = r.k; out[3] = r.batch;
    out[4] = r.batch_stride_a; out[5] = r.batch_stride_b; out[6] = r.batch_stride_c;
    out[7] = (uint32_t)(r.total_flops & 0xffffffffu);
    out[8] = (uint32_t)(r.total_flops >> 32);
  });
}

uint32_t ta_default_num_k_splits(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, uint32_t tile_m,
                                 uint32_t tile_n) {
  return default_num_k_splits(batch, m, n, k, tile_m, tile_n);
}
uint32_t ta_heuristic_splits(uint32_t batch, uint32_t m, uint32_t n, uint32_t k) {
  return heuristic_splits(batch, m, n, k).value_or(0);
}

const char *ta_heuristic_kernel(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, int weights_f16, int sm_count) {
  const int idx = heuristic_kernel_index(batch, m, n, k, weights_f16 != 0, sm_count > 0 ? sm_count : 1);
  return KERNEL_SPECS[idx].name;
}

uint16_t ta_f32_to_f16_bits(float value) { return f32_to_f16_bits(value); }
float ta_f16_bits_to_f32(uint16_t bits) { return f16_bits_to_f32(bits); }

void *ta_tensor_device_ptr(const ta_tensor *tensor) { return tensor ? tensor->tensor.ptr() : nullptr; }
int ta_context_device_index(const ta_context *ctx) { return ctx ? ctx->ctx->device : -1; }
const char *ta_context_device_name(const ta_context *ctx) { return ctx ? ctx->ctx->name.c_str() : ""; }
uint64_t ta_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
#pragma GCC visibility pop
