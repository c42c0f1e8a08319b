// ml_bench: the GEMM benchmark tool of the reference (tools/ml-bench/src/bench/{mod,commands,
// cases,env,report}.rs) on this library's C ABI.  Same subcommands for the GEMM path, the same
// environment knobs, compact case specs, sample summaries (min / median / nearest-rank p95),
// table and CSV columns, and the same sampled validation after timing.
//
//   ml_bench self-check | correctness | sweep | single | cases label,b,m,n,k[,f16w] ... | concurrent | transfer |
//            prepared | all
//   ml_bench summary x1 x2 ...      (host only: prints the sample summary of the numbers)
//   ml_bench thesis [--all] [t1 t2 t4 t6 t7 ...] [--list] [-m model.gguf | --random]
//            the performance-thesis harness (tools/ml-bench/src/bench/thesis/*.rs, benchmarks/THESES.md):
//            prediction / measurement / verdict rows against the per-GPU section of
//            thesis-expectations.toml (beside the package; $ML_THESIS_EXPECT overrides); a FAIL row
//            makes the exit status non-zero.  `thesis parse <file> <device>` (host only) prints the
//            section a device name selects.
//
//   ML_ITERS (20) ML_WARMUP (3) ML_OUTPUT (table | csv) ML_SWEEP (smoke | standard | full)
//   ML_B ML_M ML_N ML_K   ML_SPLIT_K2 (0)   ML_SLOTS (2)   ML_THREADS   ML_KERNEL (auto)   ML_DEVICE   ML_VALIDATE
//   ML_PEAK_TFLOPS: the "%peak" denominator; default 232.5, the FP32-through-3xTF32 ceiling of a
//   B200 (measured sustained bf16 rate / 2 / 3); the reference's default is its own GPU's 20.3.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <strings.h>
#include <thread>
#include <vector>

#include <map>
#include <optional>
#include <unistd.h>

#include "../../include/tensor_ash.h"
#include "../../include/tensor_ash_llama.h"

namespace {

[[noreturn]] void die(const std::string &msg) {
  fprintf(stderr, "ml_bench: %s\n", msg.c_str());
  exit(1);
}
[[noreturn]] void die_lib(const std::string &what) { die(what + ": " + ta_last_error()); }

// ---- environment (env.rs)
uint32_t env_u32(const char *k, uint32_t d) {
  const char *v = getenv(k);
  if (!v || !*v) return d;
  char *end = nullptr;
  const unsigned long x = strtoul(v, &end, 10);
  return (*end || x > 0xfffffffful) ? d : (uint32_t)x;
}
bool env_bool(const char *k) {
  const char *v = getenv(k);
  return v && (!strcmp(v, "1") || !strcasecmp(v, "true"));
}
std::string env_string(const char *k, const char *d) {
  const char *v = getenv(k);
  return v ? v : d;
}
bool output_csv() { return !strcasecmp(env_string("ML_OUTPUT", "table").c_str(), "csv"); }

// ---- deterministic inputs and the reference's tolerance (tools/test-support/src/lib.rs:9-55, 157-162)
void fill_det(std::vector<float> &v, uint64_t seed) {
  uint64_t s = (seed * 0x9E3779B97F4A7C15ull) | 1ull;
  for (float &x : v) {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    x = (float)(uint32_t)(s >> 40) / (float)(1u << 24) * 2.0f - 1.0f;
  }
}
float tolerance(uint32_t k) { return 8.0f * (float)k * 1.1920929e-07f; }

// ---- cases (cases.rs)
struct Case {
  std::string label;
  uint32_t b = 1, m = 0, n = 0, k = 0;
  bool b_f16 = false;
};

Case parse_case(const std::string &spec) {
  std::vector<std::string> f;
  size_t start = 0;
  for (;;) {
    const size_t comma = spec.find(',', start);
    f.push_back(spec.substr(start, comma == std::string::npos ? std::string::npos : comma - start));
    if (comma == std::string::npos) break;
    start = comma + 1;
  }
  if (f[0].empty()) die("benchmark case must use label,b,m,n,k with a non-empty label");
  Case c;
  c.label = f[0];
  const char *names[4] = {"B", "M", "N", "K"};
  uint32_t *dst[4] = {&c.b, &c.m, &c.n, &c.k};
  for (int i = 0; i < 4; ++i) {
    if (f.size() <= (size_t)i + 1) die("benchmark case '" + c.label + "' is missing " + names[i]);
    const std::string &v = f[i + 1];
    char *end = nullptr;
    const unsigned long x = strtoul(v.c_str(), &end, 10);
    if (v.empty() || *end || x > 0xfffffffful || v[0] == '-' || v[0] == '+')
      die("benchmark case '" + c.label + "' has invalid " + names[i] + "='" + v + "'");
    if (x == 0) die("benchmark case '" + c.label + "' has zero " + names[i]);
    *dst[i] = (uint32_t)x;
  }
  if (f.size() > 5) {
    if (f[5] != "f16w")
      die("benchmark case '" + c.label + "' has unknown flag '" + f[5] + "'; expected label,b,m,n,k[,f16w]");
    c.b_f16 = true;
  }
  if (f.size() > 6) die("benchmark case '" + c.label + "' has extra fields; expected label,b,m,n,k[,f16w]");
  return c;
}

std::vector<Case> sweep_cases(const std::string &mode) {
  auto fx = [](const char *l, uint32_t b, uint32_t m, uint32_t n, uint32_t k) { return Case{l, b, m, n, k, false}; };
  if (mode == "smoke") return {fx("smoke 128^3 B=1", 1, 128, 128, 128), fx("smoke 256^3 B=1", 1, 256, 256, 256)};
  if (mode == "full")
    return {fx("square 512^3   B=1", 1, 512, 512, 512), fx("square 1024^3  B=1", 1, 1024, 1024, 1024),
            fx("square 2048^3  B=1", 1, 2048, 2048, 2048), fx("square 4096^3  B=1", 1, 4096, 4096, 4096),
            fx("batched 32x1024^2", 32, 1024, 1024, 1024), fx("batched 8x2048^2", 8, 2048, 2048, 2048),
            fx("tall   8192x1024x1024", 1, 8192, 1024, 1024), fx("wide   1024x8192x1024", 1, 1024, 8192, 1024),
            fx("thin K 4096x4096x512", 1, 4096, 4096, 512), fx("fat  K 1024x1024x8192", 1, 1024, 1024, 8192),
            fx("deep K 64x64x8192", 1, 64, 64, 8192), fx("row 1x4096x4096", 1, 1, 4096, 4096),
            fx("column 4096x1x4096", 1, 4096, 1, 4096), fx("edge 4095^3", 1, 4095, 4095, 4095),
            fx("odd   1023x1025x1027", 1, 1023, 1025, 1027)};
  return {fx("square 512^3   B=1", 1, 512, 512, 512), fx("square 1024^3  B=1", 1, 1024, 1024, 1024),
          fx("square 2048^3  B=1", 1, 2048, 2048, 2048), fx("batched 8x1024^2", 8, 1024, 1024, 1024),
          fx("tall   4096x1024x1024", 1, 4096, 1024, 1024), fx("wide   1024x4096x1024", 1, 1024, 4096, 1024),
          fx("odd   1023x1025x1027", 1, 1023, 1025, 1027)};
}

// ---- sample summary: finite non-negative samples, even median, nearest-rank p95 (cases.rs:95-123)
struct Summary {
  size_t count = 0;
  double min = NAN, median = NAN, p95 = NAN;
  bool ok() const { return count != 0; }
};
Summary summarize(std::vector<double> v) {
  v.erase(std::remove_if(v.begin(), v.end(), [](double x) { return !std::isfinite(x) || x < 0.0; }), v.end());
  Summary s;
  if (v.empty()) return s;
  std::sort(v.begin(), v.end());
  s.count = v.size();
  const size_t mid = s.count / 2;
  s.median = s.count % 2 == 0 ? (v[mid - 1] + v[mid]) / 2.0 : v[mid];
  const size_t idx = (s.count * 95 + 99) / 100;
  s.min = v[0];
  s.p95 = v[idx ? idx - 1 : 0];
  return s;
}
std::string triplet(const Summary &s) {
  if (!s.ok()) return "-";
  char buf[96];
  snprintf(buf, sizeof buf, "%.3f/%.3f/%.3f", s.min, s.median, s.p95);
  return buf;
}
std::string csv_escape(const std::string &v) {
  if (v.find_first_of(",\"\n") == std::string::npos) return v;
  std::string out = "\"";
  for (char c : v) out += c == '"' ? std::string("\"\"") : std::string(1, c);
  return out + "\"";
}

double now_ms() {
  return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct Session {
  ta_context *ctx = nullptr;
  ta_executor *exec = nullptr;
  ~Session() {
    ta_executor_destroy(exec);
    ta_context_destroy(ctx);
  }
};

struct Result {
  Case c;
  ta_dispatch_info dispatch{};
  double flops = 0, tflops = NAN, wall_tflops = NAN;
  Summary wall, gpu, host;
};

// ---- reporter (report.rs)
struct Reporter {
  bool csv;
  double peak;
  std::string device;
  void header() const {
    if (csv) {
      printf("device,kind,label,b,m,n,k,flops,wall_ms,gpu_ms,tflops,percent_peak,sample_count,gpu_sample_count,"
             "wall_min_ms,wall_median_ms,wall_p95_ms,gpu_min_ms,gpu_median_ms,gpu_p95_ms,host_overhead_min_ms,"
             "host_overhead_median_ms,host_overhead_p95_ms,wall_tflops,kernel,tile_m,tile_n,tile_k,strategy,"
             "split_k2_splits\n");
    } else {
      printf("\n%-28s %-28s %10s %9s %25s %25s %25s %8s %8s %8s\n", "shape", "kernel / route", "GFLOPs", "samples",
             "wall ms (min/med/p95)", "gpu ms (min/med/p95)", "host ms (min/med/p95)", "TF/s", "wall TF", "%peak");
      printf("%s\n", std::string(187, '-').c_str());
    }
  }
  void row(const Result &r) const {
    const double pct = r.tflops / peak * 100.0;
    const std::string splits = r.dispatch.has_split_k2 ? std::to_string(r.dispatch.split_k2_splits) : "";
    const char *strategy = splits.empty() ? "data_parallel" : "split_k2";
    if (csv) {
      printf("%s,%s,%s,%u,%u,%u,%u,%.0f,%.6f,%.6f,%.6f,%.3f,%zu,%zu,%.6f,%.6f,%.6f,%.6f,%.6f,%.6f,%.6f,%.6f,%.6f,%.6f,"
             "%s,%u,%u,%u,%s,%s\n",
             csv_escape(device).c_str(), "discrete", csv_escape(r.c.label).c_str(), r.c.b, r.c.m, r.c.n, r.c.k, r.flops,
             r.wall.median, r.gpu.median, r.tflops, pct, r.wall.count, r.gpu.count, r.wall.min, r.wall.median, r.wall.p95,
             r.gpu.min, r.gpu.median, r.gpu.p95, r.host.min, r.host.median, r.host.p95, r.wall_tflops, r.dispatch.kernel,
             r.dispatch.tile[0], r.dispatch.tile[1], r.dispatch.tile[2], strategy, splits.c_str());
    } else {
      const std::string route = std::string(r.dispatch.kernel) + " / " + strategy;
      printf("%-28s %-28s %10.3f %4zu/%-4zu %25s %25s %25s %8.2f %8.2f %7.1f%%\n", r.c.label.c_str(), route.c_str(),
             r.flops / 1e9, r.wall.count, r.gpu.count, triplet(r.wall).c_str(), triplet(r.gpu).c_str(),
             triplet(r.host).c_str(), r.tflops, r.wall_tflops, pct);
    }
    fflush(stdout);
  }
};

Reporter reporter_setup(const Session &s, uint32_t *iters, uint32_t *warmup) {
  *iters = std::max(1u, env_u32("ML_ITERS", 20));
  *warmup = env_u32("ML_WARMUP", 3);
  double peak = 232.5;
  if (const char *v = getenv("ML_PEAK_TFLOPS")) {
    char *end = nullptr;
    const double x = strtod(v, &end);
    if (end != v && !*end && x > 0) peak = x;
  }
  Reporter r{output_csv(), peak, ta_context_device_name(s.ctx)};
  r.header();
  return r;
}

struct Tensors {
  ta_tensor *a = nullptr, *b = nullptr, *c = nullptr;
  ~Tensors() {
    ta_tensor_destroy(a);
    ta_tensor_destroy(b);
    ta_tensor_destroy(c);
  }
};

size_t host_len(uint32_t b, uint32_t r, uint32_t c) {
  const unsigned __int128 n = (unsigned __int128)b * r * c;
  if (n == 0 || n > (((unsigned __int128)1) << 40)) die("tensor shape is empty or too large for a host buffer");
  return (size_t)n;
}

// 8 well-spaced outputs recomputed on the host after timing (commands.rs:225-273); f32 products summed in f32
void validate_samples(const Session &s, const ta_tensor *c, const std::vector<float> &a, const std::vector<float> &b,
                      uint32_t batch, uint32_t m, uint32_t n, uint32_t k) {
  std::vector<float> out(host_len(batch, m, n));
  if (ta_download(s.exec, c, out.data(), out.size()) != 0) die_lib("download");
  const size_t checks = std::min<size_t>(out.size(), 8), plane = (size_t)m * n;
  float max_error = 0.0f;
  size_t worst = 0;
  for (size_t i = 0; i < checks; ++i) {
    const size_t index = checks == 1 ? 0 : i * (out.size() - 1) / (checks - 1);
    const size_t bi = index / plane, row = (index % plane) / n, col = (index % plane) % n;
    float expected = 0.0f;
    for (uint32_t kk = 0; kk < k; ++kk) expected += a[(bi * m + row) * k + kk] * b[(bi * k + kk) * n + col];
    const float err = std::fabs(out[index] - expected);
    if (!std::isfinite(err) || err > max_error) {
      max_error = err;
      worst = index;
    }
  }
  const float budget = 2.0f * tolerance(k);
  if (!(max_error <= budget)) {
    char buf[160];
    snprintf(buf, sizeof buf, "sampled correctness failed at output %zu: error %.3e > %.3e", worst, max_error, budget);
    die(buf);
  }
}

// commands.rs:116-223
Result run_case(const Session &s, const Case &c, uint32_t iters, uint32_t warmup) {
  Tensors t;
  const uint32_t sa[3] = {c.b, c.m, c.k}, sb[3] = {c.b, c.k, c.n}, sc[3] = {c.b, c.m, c.n};
  t.a = ta_tensor_create(s.ctx, sa, 3);
  t.b = c.b_f16 ? ta_tensor_create_f16(s.ctx, sb, 3) : ta_tensor_create(s.ctx, sb, 3);
  t.c = ta_tensor_create(s.ctx, sc, 3);
  if (!t.a || !t.b || !t.c) die_lib("tensor");
  std::vector<float> ha(host_len(c.b, c.m, c.k)), hb(host_len(c.b, c.k, c.n));
  fill_det(ha, 7);
  fill_det(hb, 11);
  if (ta_upload(s.exec, t.a, ha.data(), ha.size()) != 0 || ta_upload(s.exec, t.b, hb.data(), hb.size()) != 0)
    die_lib("upload");
  ta_dispatch_info info{};
  if (ta_dispatch_info_for(s.exec, c.b, c.m, c.n, c.k, c.b_f16, &info) != 0) die_lib("dispatch_info_for");
  if (c.b_f16) {
    // validation compares against what the GPU stores; the tensor-core route also rounds A to f16
    for (float &v : hb) v = ta_f16_bits_to_f32(ta_f32_to_f16_bits(v));
    if (strstr(info.kernel, "umma")) {
      for (float &v : ha) v = ta_f16_bits_to_f32(ta_f32_to_f16_bits(v));
      if (ta_upload(s.exec, t.a, ha.data(), ha.size()) != 0) die_lib("upload");
    }
  }
  const double flops = 2.0 * c.b * (double)c.m * c.n * c.k;
  const uint32_t split_k2 = env_u32("ML_SPLIT_K2", 0);
  const ta_matmul_call call{t.a, t.b, t.c, 1.0f, 0};
  auto run_once = [&](ta_run_stats *st) {
    const int rc = split_k2 < 2 ? ta_matmul_batch(s.exec, &call, 1, st) : ta_matmul_split_k2(s.exec, &call, 1, split_k2, st);
    if (rc != 0) die_lib("matmul '" + c.label + "'");
  };
  ta_run_stats st{};
  for (uint32_t i = 0; i < warmup; ++i) run_once(&st);
  std::vector<double> wall, gpu, host;
  for (uint32_t i = 0; i < iters; ++i) {
    const double t0 = now_ms();
    run_once(&st);
    const double w = now_ms() - t0;
    wall.push_back(w);
    if (st.has_gpu_time) {
      gpu.push_back(st.gpu_time_ns / 1e6);
      host.push_back(std::max(0.0, w - st.gpu_time_ns / 1e6));
    }
  }
  validate_samples(s, t.c, ha, hb, c.b, c.m, c.n, c.k);
  Result r;
  r.c = c;
  r.flops = flops;
  r.wall = summarize(wall);
  r.gpu = summarize(gpu);
  r.host = summarize(host);
  if (r.gpu.ok() && r.gpu.median > 0) r.tflops = flops / r.gpu.median * 1e-9;
  if (r.wall.median > 0) r.wall_tflops = flops / r.wall.median * 1e-9;
  if (split_k2 < 2) {
    r.dispatch = info;
  } else {   // DispatchInfo::split_k2(m, n, splits): the stage-1 tile and the requested split count
    r.dispatch.kernel = "split_k2";
    r.dispatch.tile[0] = r.dispatch.tile[1] = (c.m <= 64 && c.n <= 256) ? 64 : 128;
    r.dispatch.tile[2] = 16;
    r.dispatch.has_split_k2 = 1;
    r.dispatch.split_k2_splits = split_k2;
  }
  return r;
}

// commands.rs:30-83: full compare against an f64-accumulating host GEMM, tolerance 8 K eps
void correctness(const Session &s) {
  const uint32_t B = env_u32("ML_B", 2), M = env_u32("ML_M", 64), N = env_u32("ML_N", 80), K = env_u32("ML_K", 48);
  Tensors t;
  const uint32_t sa[3] = {B, M, K}, sb[3] = {B, K, N}, sc[3] = {B, M, N};
  t.a = ta_tensor_create(s.ctx, sa, 3);
  t.b = ta_tensor_create(s.ctx, sb, 3);
  t.c = ta_tensor_create(s.ctx, sc, 3);
  if (!t.a || !t.b || !t.c) die_lib("tensor");
  std::vector<float> ha(host_len(B, M, K)), hb(host_len(B, K, N)), hc(host_len(B, M, N));
  fill_det(ha, 1);
  fill_det(hb, 2);
  if (ta_upload(s.exec, t.a, ha.data(), ha.size()) != 0 || ta_upload(s.exec, t.b, hb.data(), hb.size()) != 0)
    die_lib("upload");
  if (ta_matmul(s.exec, t.a, t.b, t.c, 1.0f, 0, nullptr) != 0) die_lib("matmul");
  if (ta_download(s.exec, t.c, hc.data(), hc.size()) != 0) die_lib("download");
  float e = 0.0f;
  size_t idx = 0;
  float cpu_at = 0.0f;
  for (uint32_t b = 0; b < B; ++b)
    for (uint32_t i = 0; i < M; ++i)
      for (uint32_t j = 0; j < N; ++j) {
        double acc = 0.0;
        for (uint32_t k = 0; k < K; ++k) acc += (double)ha[((size_t)b * M + i) * K + k] * (double)hb[((size_t)b * K + k) * N + j];
        const size_t o = ((size_t)b * M + i) * N + j;
        const float err = std::fabs(hc[o] - (float)acc);
        if (!(err <= e)) {
          e = err;
          idx = o;
          cpu_at = (float)acc;
        }
      }
  const float tol = tolerance(K);
  fprintf(stderr, "correctness: max|err|=%.3e  tol=%.3e  at idx %zu: gpu=%.6f  cpu=%.6f\n", e, tol, idx, hc[idx], cpu_at);
  if (!(e <= tol)) {
    char buf[128];
    snprintf(buf, sizeof buf, "correctness failed: err %.3e > tol %.3e", e, tol);
    die(buf);
  }
  printf("CORRECTNESS OK (err=%.3e, tol=%.3e)\n", e, tol);
}

void sweep(const Session &s) {
  std::string mode = env_string("ML_SWEEP", "");
  std::transform(mode.begin(), mode.end(), mode.begin(), ::tolower);
  if (mode != "smoke" && mode != "standard" && mode != "full") mode = "standard";
  uint32_t iters, warmup;
  const Reporter rep = reporter_setup(s, &iters, &warmup);
  for (const Case &c : sweep_cases(mode)) rep.row(run_case(s, c, iters, warmup));
}

void single(const Session &s) {
  Case c;
  c.b = env_u32("ML_B", 1); c.m = env_u32("ML_M", 4096); c.n = env_u32("ML_N", 4096); c.k = env_u32("ML_K", 4096);
  c.label = "B=" + std::to_string(c.b) + " M=" + std::to_string(c.m) + " N=" + std::to_string(c.n) + " K=" + std::to_string(c.k);
  uint32_t iters, warmup;
  const Reporter rep = reporter_setup(s, &iters, &warmup);
  rep.row(run_case(s, c, iters, warmup));
}

void cases(const Session &s, const std::vector<std::string> &specs) {
  std::vector<Case> cs;
  for (const std::string &spec : specs) cs.push_back(parse_case(spec));
  if (cs.empty()) die("cases requires at least one label,b,m,n,k argument");
  uint32_t iters, warmup;
  const Reporter rep = reporter_setup(s, &iters, &warmup);
  for (const Case &c : cs) rep.row(run_case(s, c, iters, warmup));
}

// commands.rs:357-427: one tensor of ML_TRANSFER_MB (16) MiB up and down, ML_ITERS (10) wall-clock samples each
void transfer(const Session &s) {
  const uint32_t mb = std::max(1u, env_u32("ML_TRANSFER_MB", 16));
  const uint32_t iters = std::max(1u, env_u32("ML_ITERS", 10));
  const size_t bytes = (size_t)mb << 20, elems = bytes / 4;
  const uint32_t shape[1] = {(uint32_t)elems};
  ta_tensor *t = ta_tensor_create(s.ctx, shape, 1);
  if (!t) die_lib("tensor");
  std::vector<float> src(elems), dst(elems);
  fill_det(src, 99);
  if (ta_upload(s.exec, t, src.data(), elems) != 0 || ta_download(s.exec, t, dst.data(), elems) != 0) die_lib("transfer");
  if (memcmp(src.data(), dst.data(), bytes) != 0) die("transfer round trip changed the data");
  std::vector<double> up, down;
  for (uint32_t i = 0; i < iters; ++i) {
    double t0 = now_ms();
    if (ta_upload(s.exec, t, src.data(), elems) != 0) die_lib("upload");
    up.push_back(now_ms() - t0);
    t0 = now_ms();
    if (ta_download(s.exec, t, dst.data(), elems) != 0) die_lib("download");
    down.push_back(now_ms() - t0);
  }
  ta_tensor_destroy(t);
  const Summary u = summarize(up), d = summarize(down);
  const double gib = bytes / 1024.0 / 1024.0 / 1024.0;
  const double ug = gib / (u.median / 1e3), dg = gib / (d.median / 1e3);
  if (!output_csv()) {
    printf("\ntransfer: %u MiB x %zu samples  upload=%.2f GiB/s  download=%.2f GiB/s\n", mb, u.count, ug, dg);
    printf("latency ms (min/median/p95): upload=%.3f/%.3f/%.3f  download=%.3f/%.3f/%.3f\n", u.min, u.median, u.p95, d.min,
           d.median, d.p95);
  } else {
    printf("device,kind,bytes,iters,upload_gibs,download_gibs,sample_count,upload_min_ms,upload_median_ms,upload_p95_ms,"
           "download_min_ms,download_median_ms,download_p95_ms\n");
    printf("%s,%s,%zu,%u,%.6f,%.6f,%zu,%.6f,%.6f,%.6f,%.6f,%.6f,%.6f\n", csv_escape(ta_context_device_name(s.ctx)).c_str(),
           "discrete", bytes, iters, ug, dg, u.count, u.min, u.median, u.p95, d.min, d.median, d.p95);
  }
}

// commands.rs:429-560: synchronous calls vs prepared replay vs two prepared objects ping-ponged
void prepared(const Session &s) {
  const uint32_t b = env_u32("ML_B", 1), m = env_u32("ML_M", 256), n = env_u32("ML_N", 256), k = env_u32("ML_K", 256);
  const size_t iters = std::max(1u, env_u32("ML_ITERS", 500)), warmup = env_u32("ML_WARMUP", 20);
  const uint32_t sa[3] = {b, m, k}, sb[3] = {b, k, n}, sc[3] = {b, m, n};
  ta_tensor *a = ta_tensor_create(s.ctx, sa, 3), *bt = ta_tensor_create(s.ctx, sb, 3);
  ta_tensor *c[4];
  for (auto &t : c) t = ta_tensor_create(s.ctx, sc, 3);
  if (!a || !bt || !c[0] || !c[1] || !c[2] || !c[3]) die_lib("tensor");
  std::vector<float> ha(host_len(b, m, k)), hb(host_len(b, k, n));
  fill_det(ha, 41);
  fill_det(hb, 42);
  if (ta_upload(s.exec, a, ha.data(), ha.size()) != 0 || ta_upload(s.exec, bt, hb.data(), hb.size()) != 0) die_lib("upload");
  auto op = [&](ta_tensor *out) {
    ta_matmul_op o{};
    o.call = ta_matmul_call{a, bt, out, 1.0f, 0};
    return o;
  };
  const ta_matmul_op o1 = op(c[1]), o2 = op(c[2]), o3 = op(c[3]);
  ta_prepared *prep = ta_prepared_create(s.exec, &o1, 1, 0), *ping = ta_prepared_create(s.exec, &o2, 1, 0),
              *pong = ta_prepared_create(s.exec, &o3, 1, 0);
  if (!prep || !ping || !pong) die_lib("prepare");
  auto sync_call = [&]() {
    if (ta_matmul(s.exec, a, bt, c[0], 1.0f, 0, nullptr) != 0) die_lib("matmul");
  };
  auto must = [&](int rc, const char *what) {
    if (rc != 0) die_lib(what);
  };
  const double burn = now_ms();
  while (now_ms() - burn < 300.0) sync_call();
  for (size_t i = 0; i < warmup; ++i) sync_call();
  double t0 = now_ms();
  for (size_t i = 0; i < iters; ++i) sync_call();
  const double sync_us = (now_ms() - t0) * 1e3 / iters;
  for (size_t i = 0; i < warmup; ++i) must(ta_prepared_run(prep, nullptr), "prepared run");
  t0 = now_ms();
  for (size_t i = 0; i < iters; ++i) must(ta_prepared_run(prep, nullptr), "prepared run");
  const double prepared_us = (now_ms() - t0) * 1e3 / iters;
  for (size_t i = 0; i < (warmup + 1) / 2; ++i) {
    must(ta_prepared_run(ping, nullptr), "ping");
    must(ta_prepared_run(pong, nullptr), "pong");
  }
  const size_t pairs = (iters + 1) / 2;
  t0 = now_ms();
  must(ta_prepared_submit(ping), "submit");
  must(ta_prepared_submit(pong), "submit");
  for (size_t i = 1; i < pairs; ++i) {
    must(ta_prepared_wait(ping, nullptr), "wait");
    must(ta_prepared_submit(ping), "submit");
    must(ta_prepared_wait(pong, nullptr), "wait");
    must(ta_prepared_submit(pong), "submit");
  }
  must(ta_prepared_wait(ping, nullptr), "wait");
  must(ta_prepared_wait(pong, nullptr), "wait");
  const double pipelined_us = (now_ms() - t0) * 1e3 / (pairs * 2);
  // every output against the f64-accumulating host product, 2 x tolerance(k)
  std::vector<float> expect(host_len(b, m, n)), got(expect.size());
  for (uint32_t bi = 0; bi < b; ++bi)
    for (uint32_t i = 0; i < m; ++i)
      for (uint32_t j = 0; j < n; ++j) {
        double acc = 0.0;
        for (uint32_t kk = 0; kk < k; ++kk) acc += (double)ha[((size_t)bi * m + i) * k + kk] * (double)hb[((size_t)bi * k + kk) * n + j];
        expect[((size_t)bi * m + i) * n + j] = (float)acc;
      }
  const char *labels[4] = {"sync", "prepared", "ping", "pong"};
  for (int t = 0; t < 4; ++t) {
    must(ta_download(s.exec, c[t], got.data(), got.size()), "download");
    float err = 0.0f;
    size_t at = 0;
    for (size_t i = 0; i < got.size(); ++i) {
      const float e = std::fabs(got[i] - expect[i]);
      if (!(e <= err)) { err = e; at = i; }
    }
    if (!(err <= 2.0f * tolerance(k))) {
      char buf[128];
      snprintf(buf, sizeof buf, "prepared bench '%s' output error %.3e at %zu", labels[t], err, at);
      die(buf);
    }
  }
  ta_dispatch_info info{};
  must(ta_dispatch_info_for(s.exec, b, m, n, k, 0, &info), "dispatch_info_for");
  printf("prepared: B=%u %ux%ux%u, %zu iters (all outputs validated)\n", b, m, n, k, iters);
  if (info.has_split_k2)
    printf("  note: sync auto-routes split-K2 x%u; prepared replays the DP kernel -- the ratios include that routing difference\n",
           info.split_k2_splits);
  else
    printf("  kernel: %s\n", info.kernel);
  printf("  sync run_matmuls : %8.2f us/call\n", sync_us);
  printf("  prepared replay  : %8.2f us/call  (%.2fx)\n", prepared_us, sync_us / prepared_us);
  printf("  pipelined x2     : %8.2f us/call  (%.2fx)\n", pipelined_us, sync_us / pipelined_us);
  ta_prepared_destroy(prep);
  ta_prepared_destroy(ping);
  ta_prepared_destroy(pong);
  ta_tensor_destroy(a);
  ta_tensor_destroy(bt);
  for (auto &t : c) ta_tensor_destroy(t);
}

// commands.rs:292-356: ML_THREADS host threads (default: the hardware concurrency) share one
// executor, each running ML_ITERS (50) products of 512^3 on its own tensors; every output is
// validated afterwards.
void concurrent(const Session &s) {
  const uint32_t hw = std::max(1u, std::thread::hardware_concurrency());
  const uint32_t n_threads = std::max(1u, env_u32("ML_THREADS", hw ? hw : 4));
  const uint32_t iters = std::max(1u, env_u32("ML_ITERS", 50));
  const uint32_t m = 512, n = 512, k = 512, shape_a[2] = {m, k}, shape_b[2] = {k, n}, shape_c[2] = {m, n};
  struct Triple {
    ta_tensor *a, *b, *c;
    std::vector<float> ha, hb;
  };
  std::vector<Triple> tr(n_threads);
  for (uint32_t t = 0; t < n_threads; ++t) {
    tr[t].a = ta_tensor_create(s.ctx, shape_a, 2);
    tr[t].b = ta_tensor_create(s.ctx, shape_b, 2);
    tr[t].c = ta_tensor_create(s.ctx, shape_c, 2);
    if (!tr[t].a || !tr[t].b || !tr[t].c) die_lib("tensor");
    tr[t].ha.resize((size_t)m * k);
    tr[t].hb.resize((size_t)k * n);
    fill_det(tr[t].ha, 100 + t);
    fill_det(tr[t].hb, 200 + t);
    if (ta_upload(s.exec, tr[t].a, tr[t].ha.data(), tr[t].ha.size()) != 0 ||
        ta_upload(s.exec, tr[t].b, tr[t].hb.data(), tr[t].hb.size()) != 0)
      die_lib("upload");
  }
  std::vector<std::string> errors(n_threads);
  const double t0 = now_ms();
  std::vector<std::thread> pool;
  for (uint32_t t = 0; t < n_threads; ++t)
    pool.emplace_back([&, t]() {
      for (uint32_t i = 0; i < iters; ++i)
        if (ta_matmul(s.exec, tr[t].a, tr[t].b, tr[t].c, 1.0f, 0, nullptr) != 0) {
          errors[t] = ta_last_error();   // the message is per thread
          return;
        }
    });
  for (auto &th : pool) th.join();
  const double dt = (now_ms() - t0) / 1e3;
  for (uint32_t t = 0; t < n_threads; ++t)
    if (!errors[t].empty()) die("run_matmuls (thread " + std::to_string(t) + "): " + errors[t]);
  for (uint32_t t = 0; t < n_threads; ++t) validate_samples(s, tr[t].c, tr[t].ha, tr[t].hb, 1, m, n, k);
  const double total = 2.0 * m * n * k * (double)iters * n_threads;
  printf("concurrent: %u threads x %u iters of 512^3   total %.1f GFLOPs  in %.3fs  ->  %.2f TFLOPS (aggregate)\n",
         n_threads, iters, total * 1e-9, dt, total / dt * 1e-12);
  for (auto &x : tr) {
    ta_tensor_destroy(x.a);
    ta_tensor_destroy(x.b);
    ta_tensor_destroy(x.c);
  }
}

// ===================================================================== thesis harness
// (tools/ml-bench/src/bench/thesis/{mod,expect,gemv,micro,model_theses}.rs, benchmarks/THESES.md)
using Section = std::map<std::string, double>;

std::string trim(const std::string &v) {
  const size_t b = v.find_first_not_of(" \t\r"), e = v.find_last_not_of(" \t\r");
  return b == std::string::npos ? "" : v.substr(b, e - b + 1);
}

// Strict TOML subset (expect.rs:66-112): ["quoted" or bare] section headers, key = <float>, # comments.
// Returns false with *err set on a malformed line.
bool parse_expectations(const std::string &text, std::map<std::string, Section> *out, std::string *err) {
  std::string current;
  bool have_section = false;
  size_t lineno = 0, pos = 0;
  while (pos <= text.size()) {
    size_t nl = text.find('\n', pos);
    if (nl == std::string::npos) nl = text.size();
    std::string line = text.substr(pos, nl - pos);
    pos = nl + 1;
    ++lineno;
    line = trim(line.substr(0, line.find('#')));
    if (line.empty()) continue;
    auto bad = [&](const char *what) {
      *err = "line " + std::to_string(lineno) + ": " + what;
      return false;
    };
    if (line[0] == '[') {
      if (line.back() != ']') return bad("unterminated section header");
      std::string name = trim(line.substr(1, line.size() - 2));
      if (name.size() >= 2 && name.front() == '"' && name.back() == '"') name = name.substr(1, name.size() - 2);
      if (name.empty()) return bad("empty section name");
      (*out)[name];
      current = name;
      have_section = true;
      continue;
    }
    const size_t eq = line.find('=');
    if (eq == std::string::npos) return bad("expected key = value");
    if (!have_section) return bad("key before any [section]");
    const std::string value = trim(line.substr(eq + 1));
    char *end = nullptr;
    const double v = strtod(value.c_str(), &end);
    if (value.empty() || *end) return bad("value is not a number");
    (*out)[current][trim(line.substr(0, eq))] = v;
  }
  return true;
}

std::string expectations_path() {
  if (const char *e = getenv("ML_THESIS_EXPECT")) return e;
  char exe[4096];
  const ssize_t n = readlink("/proc/self/exe", exe, sizeof exe - 1);
  if (n > 0) {
    std::string dir(exe, (size_t)n);
    dir = dir.substr(0, dir.find_last_of('/'));            // .../bin
    return dir.substr(0, dir.find_last_of('/')) + "/thesis-expectations.toml";
  }
  return "thesis-expectations.toml";
}

bool read_file(const std::string &path, std::string *out) {
  FILE *f = fopen(path.c_str(), "rb");
  if (!f) return false;
  char buf[4096];
  size_t n;
  while ((n = fread(buf, 1, sizeof buf, f)) > 0) out->append(buf, n);
  fclose(f);
  return true;
}

enum class Verdict { Pass, Fail, Info, Skip };
const char *verdict_str(Verdict v) {
  switch (v) {
    case Verdict::Pass: return "PASS";
    case Verdict::Fail: return "FAIL";
    case Verdict::Info: return "info";
    default: return "SKIP";
  }
}
struct Row {
  std::string thesis, item, prediction, measured;
  Verdict verdict;
};
std::optional<double> key(const Section *s, const char *name) {
  if (!s) return std::nullopt;
  auto it = s->find(name);
  return it == s->end() ? std::nullopt : std::optional<double>(it->second);
}
Verdict check_min(double value, std::optional<double> min) { return !min ? Verdict::Info : (value >= *min ? Verdict::Pass : Verdict::Fail); }
std::string fmt(const char *f, ...) __attribute__((format(printf, 1, 2)));
std::string fmt(const char *f, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, f);
  vsnprintf(buf, sizeof buf, f, ap);
  va_end(ap);
  return buf;
}

void print_thesis_table(const std::string &device, const std::vector<Row> &rows) {
  const char *headers[5] = {"thesis", "item", "prediction", "measured", "verdict"};
  size_t w[5];
  for (int i = 0; i < 5; ++i) w[i] = strlen(headers[i]);
  for (const Row &r : rows) {
    const std::string cells[5] = {r.thesis, r.item, r.prediction, r.measured, verdict_str(r.verdict)};
    for (int i = 0; i < 5; ++i) w[i] = std::max(w[i], cells[i].size());
  }
  auto line = [&](const std::string cells[5]) {
    std::string out = "|";
    for (int i = 0; i < 5; ++i) out += " " + cells[i] + std::string(w[i] - cells[i].size(), ' ') + " |";
    printf("%s\n", out.c_str());
  };
  printf("\nperformance-thesis results — %s\n", device.c_str());
  const std::string h[5] = {headers[0], headers[1], headers[2], headers[3], headers[4]};
  line(h);
  const std::string sep[5] = {std::string(w[0], '-'), std::string(w[1], '-'), std::string(w[2], '-'), std::string(w[3], '-'),
                              std::string(w[4], '-')};
  line(sep);
  for (const Row &r : rows) {
    const std::string cells[5] = {r.thesis, r.item, r.prediction, r.measured, verdict_str(r.verdict)};
    line(cells);
  }
  printf("\n");
}

// ~300 ms of 1024^3 GEMMs before anything is timed (mod.rs:209-230)
void thesis_burn_in(const Session &s) {
  Tensors t;
  const uint32_t sh[2] = {1024, 1024};
  t.a = ta_tensor_create(s.ctx, sh, 2);
  t.b = ta_tensor_create(s.ctx, sh, 2);
  t.c = ta_tensor_create(s.ctx, sh, 2);
  if (!t.a || !t.b || !t.c) die_lib("tensor");
  std::vector<float> host(1024 * 1024);
  fill_det(host, 3);
  if (ta_upload(s.exec, t.a, host.data(), host.size()) != 0 || ta_upload(s.exec, t.b, host.data(), host.size()) != 0)
    die_lib("upload");
  const double deadline = now_ms() + 300.0;
  while (now_ms() < deadline)
    if (ta_matmul(s.exec, t.a, t.b, t.c, 1.0f, 0, nullptr) != 0) die_lib("burn-in");
}

// T2 (gemv.rs:35-128): every decode GEMV class against its bandwidth floor.  Two adaptations to a
// GPU whose launches cost as much as these kernels run: the weights of one class fit the 126 MB L2,
// so the launches rotate over enough copies of the matrix to stream at least 384 MB before one
// repeats (what is measured is memory bandwidth, as on the reference's GPU); and a sample is one
// submission of 16 back-to-back launches divided by 16, so the time between two timestamps is the
// kernels' and not one launch's set-up (a decode step runs them back to back in the same way).
std::vector<Row> t2_gemv_efficiency(const Session &s, const Section *sec) {
  static const struct { const char *label; uint32_t k, n; } shapes[] = {
      {"q/o 2048x2048", 2048, 2048}, {"k/v 2048x256", 2048, 256}, {"gate/up 2048x5632", 2048, 5632},
      {"down 5632x2048", 5632, 2048}, {"lm_head 2048x32000", 2048, 32000}};
  const uint32_t iters = std::max(1u, env_u32("ML_ITERS", 50)), warmup = env_u32("ML_WARMUP", 5);
  const auto bw = key(sec, "mem_bw_gbps"), min_frac = key(sec, "t2_min_bw_frac");
  std::vector<Row> rows;
  for (const auto &sh : shapes) {
    const double wbytes = 2.0 * sh.k * sh.n;
    const size_t copies = (size_t)std::max(2.0, std::ceil(384e6 / wbytes));
    const uint32_t sa[2] = {1, sh.k}, sb[2] = {sh.k, sh.n}, sc[2] = {1, sh.n};
    ta_tensor *a = ta_tensor_create(s.ctx, sa, 2), *c = ta_tensor_create(s.ctx, sc, 2);
    std::vector<ta_tensor *> bs(copies);
    std::vector<float> ha(sh.k), hb((size_t)sh.k * sh.n);
    fill_det(ha, 7);
    fill_det(hb, 11);
    if (!a || !c || ta_upload(s.exec, a, ha.data(), ha.size()) != 0) die_lib("tensor");
    for (size_t i = 0; i < copies; ++i) {
      bs[i] = ta_tensor_create_f16(s.ctx, sb, 2);
      if (!bs[i] || ta_upload(s.exec, bs[i], hb.data(), hb.size()) != 0) die_lib("tensor");
    }
    ta_dispatch_info info{};
    if (ta_dispatch_info_for(s.exec, 1, 1, sh.n, sh.k, 1, &info) != 0) die_lib("dispatch_info_for");
    std::vector<double> gpu;
    ta_run_stats st{};
    constexpr int CHAIN = 16;
    std::vector<ta_exec_op> chain(CHAIN);
    for (uint32_t i = 0; i < warmup + iters; ++i) {
      for (int j = 0; j < CHAIN; ++j) {
        memset(&chain[j], 0, sizeof(ta_exec_op));
        chain[j].kind = TA_EXEC_MATMUL;
        chain[j].mm.op.call.a = a;
        chain[j].mm.op.call.b = bs[((size_t)i * CHAIN + j) % copies];
        chain[j].mm.op.call.c = c;
        chain[j].mm.op.call.alpha = 1.0f;
      }
      if (ta_run_exec_ops(s.exec, chain.data(), CHAIN, &st) != 0) die_lib("run_exec_ops");
      if (i >= warmup && st.has_gpu_time) gpu.push_back(st.gpu_time_ns / 1e6 / CHAIN);
    }
    for (float &v : hb) v = ta_f16_bits_to_f32(ta_f32_to_f16_bits(v));
    validate_samples(s, c, ha, hb, 1, 1, sh.n, sh.k);
    const Summary sm = summarize(gpu);
    const double bytes = wbytes + 4.0 * ((double)sh.k + sh.n);      // f16 weights + f32 row in + f32 row out
    const double gbps = bytes / (sm.median * 1e6);
    Row r{"T2", std::string("GEMV ") + sh.label + " f16w", "", "", Verdict::Info};
    if (bw) {
      const double frac = gbps / *bw;
      r.prediction = fmt(">= %.0f%% of BW floor (%.1f us at %.0f GB/s)", min_frac.value_or(NAN) * 100.0, bytes / (*bw * 1e3), *bw);
      r.measured = fmt("%.1f us = %.0f GB/s = %.0f%% [%s]", sm.median * 1e3, gbps, frac * 100.0, info.kernel);
      r.verdict = check_min(frac, min_frac);
    } else {
      r.prediction = "unrecorded (needs mem_bw_gbps)";
      r.measured = fmt("%.1f us = %.0f GB/s [%s]", sm.median * 1e3, gbps, info.kernel);
    }
    rows.push_back(r);
    ta_tensor_destroy(a);
    ta_tensor_destroy(c);
    for (ta_tensor *b : bs) ta_tensor_destroy(b);
  }
  return rows;
}

// T6 (gemv.rs:130-200): the f16-weight tensor-core GEMM on the real 512-row prefill shapes, with
// 4096^3 as the regression reference.  A shape that routes away from the tensor cores fails its row.
std::vector<Row> t6_tensor_core_ceiling(const Session &s, const Section *sec) {
  const uint32_t iters = std::max(1u, env_u32("ML_ITERS", 20)), warmup = env_u32("ML_WARMUP", 3);
  const auto min_tf = key(sec, "t6_min_tflops"), ref_tf = key(sec, "t6_ref_tflops");
  const double ref_tol = key(sec, "t6_ref_rel_tol").value_or(0.15);
  static const struct { const char *label; uint32_t m, n, k; } shapes[] = {
      {"prefill q/o 512x2048x2048", 512, 2048, 2048}, {"prefill gate/up 512x5632x2048", 512, 5632, 2048},
      {"prefill down 512x2048x5632", 512, 2048, 5632}};
  std::vector<Row> rows;
  auto measure = [&](const char *label, uint32_t m, uint32_t n, uint32_t k, double *tflops, std::string *kernel) {
    const Result r = run_case(s, Case{std::string("tensor ") + label, 1, m, n, k, true}, iters, warmup);
    *tflops = r.tflops;
    *kernel = r.dispatch.kernel;
    return fmt("%.2f TF/s (%.0f us) [%s]", r.tflops, r.gpu.median * 1e3, r.dispatch.kernel);
  };
  for (const auto &sh : shapes) {
    double tf;
    std::string kernel;
    const std::string measured = measure(sh.label, sh.m, sh.n, sh.k, &tf, &kernel);
    Verdict v = check_min(tf, min_tf);
    if (kernel.find("umma") == std::string::npos && min_tf) v = Verdict::Fail;
    rows.push_back(Row{"T6", std::string("tensor-core ") + sh.label + " f16w", min_tf ? fmt(">= %.0f TF/s", *min_tf) : "unrecorded",
                       measured, v});
  }
  double tf;
  std::string kernel;
  const std::string measured = measure("reference 4096^3", 4096, 4096, 4096, &tf, &kernel);
  rows.push_back(Row{"T6", "tensor-core reference 4096^3 f16w",
                     ref_tf ? fmt("~%.1f TF/s (-%.0f%% floor)", *ref_tf, ref_tol * 100.0) : "unrecorded", measured,
                     check_min(tf, ref_tf ? std::optional<double>(*ref_tf * (1.0 - ref_tol)) : std::nullopt)});
  return rows;
}

// T4 (micro.rs): one submission round trip.  N = 64 single-op submissions against one submission of
// the same 64 independent trivial ops, nine times; per-submit cost = (median_many - median_one) / (N - 1).
std::vector<Row> t4_submission_cost(const Session &s, const Section *sec) {
  constexpr int N = 64;
  const uint32_t sh[1] = {256};
  std::vector<ta_tensor *> a(N), b(N), o(N);
  std::vector<float> host(256, 1.0f);
  for (int i = 0; i < N; ++i) {
    a[i] = ta_tensor_create(s.ctx, sh, 1);
    b[i] = ta_tensor_create(s.ctx, sh, 1);
    o[i] = ta_tensor_create(s.ctx, sh, 1);
    if (!a[i] || !b[i] || !o[i] || ta_upload(s.exec, a[i], host.data(), 256) != 0 || ta_upload(s.exec, b[i], host.data(), 256) != 0)
      die_lib("tensor");
  }
  std::vector<ta_exec_op> ops(N);
  for (int i = 0; i < N; ++i) {
    memset(&ops[i], 0, sizeof(ta_exec_op));
    ops[i].kind = TA_EXEC_BINARY;
    ops[i].in0 = a[i]; ops[i].in1 = b[i]; ops[i].out = o[i];
    ops[i].u0 = 0; ops[i].f0 = 1.0f;
  }
  std::vector<double> many, one;
  for (int rep = 0; rep < 10; ++rep) {
    double t0 = now_ms();
    for (int i = 0; i < N; ++i)
      if (ta_run_exec_ops(s.exec, &ops[i], 1, nullptr) != 0) die_lib("run_exec_ops");
    const double tm = now_ms() - t0;
    t0 = now_ms();
    if (ta_run_exec_ops(s.exec, ops.data(), N, nullptr) != 0) die_lib("run_exec_ops");
    const double to = now_ms() - t0;
    if (rep) {   // the first repetition warms the path
      many.push_back(tm);
      one.push_back(to);
    }
  }
  const double per_submit_us = (summarize(many).median - summarize(one).median) / (N - 1) * 1e3;
  for (int i = 0; i < N; ++i) {
    ta_tensor_destroy(a[i]);
    ta_tensor_destroy(b[i]);
    ta_tensor_destroy(o[i]);
  }
  const auto lo = key(sec, "t4_submit_us_lo"), hi = key(sec, "t4_submit_us_hi");
  const double tol = key(sec, "t4_edge_tol").value_or(0.20);
  Row r{"T4", "submission round trip (launch + stream wait)", "", fmt("%.1f us per submission", per_submit_us), Verdict::Info};
  if (lo && hi) {
    r.prediction = fmt("%.0f-%.0f us (+-%.0f%% at the edges)", *lo, *hi, tol * 100.0);
    r.verdict = (per_submit_us >= *lo * (1.0 - tol) && per_submit_us <= *hi * (1.0 + tol)) ? Verdict::Pass : Verdict::Fail;
  } else {
    r.prediction = "unrecorded";
  }
  return {r};
}

struct ThesisModel {
  ta_llama *model = nullptr;
  ta_llama_config cfg{};
  ~ThesisModel() { ta_llama_destroy(model); }
};

void load_thesis_model(const Session &s, const std::string &path, bool random, ThesisModel *m) {
  if (random) {
    ta_llama_config c{};
    c.layers = 22; c.embd = 2048; c.heads = 32; c.kv_heads = 4; c.head_dim = 64; c.ffn = 5632; c.vocab = 32000;
    c.t_max = 1024; c.rms_eps = 1e-5f; c.rope_theta = 1e4f; c.weight_sigma = 0.02f; c.norm_jitter = 0.0f; c.seed = 1;
    m->model = ta_llama_create_random(s.exec, &c);
  } else {
    m->model = ta_llama_load_gguf(s.exec, path.c_str(), 1024, nullptr);
  }
  if (!m->model) die_lib("model");
  if (ta_llama_get_config(m->model, &m->cfg) != 0) die_lib("config");
}

std::vector<uint32_t> thesis_prompt(uint32_t n, uint32_t vocab) {   // BOS, then arbitrary in-vocabulary ids
  std::vector<uint32_t> p(n);
  p[0] = 1 % vocab;
  for (uint32_t i = 1; i < n; ++i) p[i] = (100 + (i % 1000)) % vocab;
  return p;
}

// T1 (model_theses.rs:60-170): decode GPU time per token priced by weight traffic.
std::vector<Row> t1_decode_bandwidth(const Section *sec, ThesisModel &m) {
  constexpr uint32_t PP = 512, TG = 128;
  if (m.cfg.t_max < PP + TG) return {Row{"T1", "decode weight bandwidth", "-", "context shorter than pp512 + tg128", Verdict::Skip}};
  const std::vector<uint32_t> prompt = thesis_prompt(PP, m.cfg.vocab);
  std::vector<uint32_t> out(TG);
  uint32_t next = 0;
  ta_run_stats st{};
  // warm-up: prefill + 16 decode steps, then reset
  if (ta_llama_prefill(m.model, prompt.data(), PP, &next, &st) != 0 || ta_llama_decode(m.model, next, 16, out.data(), &st) != 0 ||
      ta_llama_reset(m.model) != 0)
    die_lib("T1 warm-up");
  if (ta_llama_prefill(m.model, prompt.data(), PP, &next, &st) != 0) die_lib("T1 prefill");
  const uint64_t launches0 = ta_kernel_launch_count();
  const double t0 = now_ms();
  if (ta_llama_decode(m.model, next, TG, out.data(), &st) != 0) die_lib("T1 decode");
  const double wall_ms_tok = (now_ms() - t0) / TG;
  const double launches_tok = (double)(ta_kernel_launch_count() - launches0) / TG;
  ta_llama_reset(m.model);
  const double gpu_ms_tok = st.gpu_time_ns / 1e6 / TG;
  const double bytes = (double)ta_llama_weight_bytes_per_token(m.model);
  const double gbps = bytes / (st.gpu_time_ns / (double)TG);          // bytes per token / ns per token = GB/s
  const auto bw = key(sec, "mem_bw_gbps"), min_frac = key(sec, "t1_min_bw_frac");
  std::vector<Row> rows;
  Row r{"T1", "decode weight bandwidth (prepared graph, f16 KV, tg128 after pp512)", "", "", Verdict::Info};
  if (bw && min_frac) {
    r.prediction = fmt(">= %.0f GB/s (%.0f%% of %.0f)", *bw * *min_frac, *min_frac * 100.0, *bw);
    r.verdict = check_min(gbps / *bw, min_frac);
  } else {
    r.prediction = "unrecorded (needs mem_bw_gbps, t1_min_bw_frac)";
  }
  r.measured = fmt("%.3f ms/token GPU = %.0f GB/s of %.2f GB weights%s", gpu_ms_tok, gbps, bytes / 1e9,
                   bw ? fmt(" = %.0f%%", gbps / *bw * 100.0).c_str() : "");
  rows.push_back(r);
  rows.push_back(Row{"T1", "decode graph census", "-",
                     fmt("%.0f launches/token, %.3f ms/token wall (%.3f ms host)", launches_tok, wall_ms_tok, wall_ms_tok - gpu_ms_tok),
                     Verdict::Info});
  return rows;
}

// T7 (model_theses.rs:460-531): greedy generation is identical across execution strategies and
// prefill widths.  Strategies here: the replayed prepared graph, and the same op list submitted launch
// by launch with events in between (the per-op mode); the KV cache of this runner is always f16.
// Widths 1 / 64 / 300 / 512 take the single-token, small-row and tensor-core prefill branches.
std::vector<Row> t7_token_exactness(ThesisModel &m) {
  std::vector<Row> rows;
  for (uint32_t width : {1u, 64u, 300u, 512u}) {
    if (m.cfg.t_max < width + 17) continue;
    const std::vector<uint32_t> prompt = thesis_prompt(width, m.cfg.vocab);
    std::vector<uint32_t> a(17), b(17);
    ta_run_stats st{};
    if (ta_llama_reset(m.model) != 0 || ta_llama_prefill(m.model, prompt.data(), width, &a[0], &st) != 0 ||
        ta_llama_decode(m.model, a[0], 16, a.data() + 1, &st) != 0)
      die_lib("T7 prepared");
    if (ta_llama_reset(m.model) != 0 || ta_llama_prefill(m.model, prompt.data(), width, &b[0], &st) != 0) die_lib("T7 per-op");
    for (int i = 0; i < 16; ++i) {
      ta_llama_breakdown_row tmp[32];
      size_t n_rows = 0, n_launches = 0;
      if (ta_llama_decode_breakdown(m.model, b[i], tmp, 32, &n_rows, &n_launches, &b[i + 1]) != 0) die_lib("T7 per-op step");
    }
    size_t first = 17;
    for (size_t i = 0; i < 17; ++i)
      if (a[i] != b[i]) { first = i; break; }
    rows.push_back(Row{"T7", fmt("token exactness, prefill width %u + 16 greedy steps", width), "identical across strategies",
                       first == 17 ? "17 / 17 tokens identical (prepared graph vs per-launch)"
                                   : fmt("diverges at token %zu: %u vs %u", first, a[first], b[first]),
                       first == 17 ? Verdict::Pass : Verdict::Fail});
  }
  ta_llama_reset(m.model);
  return rows;
}

int thesis(int argc, char **argv) {
  static const char *USAGE = "usage: ml_bench thesis [--all] [t1 t2 t4 t6 t7 ...] [--list] [-m/--model <gguf> | --random]\n"
                             "  model path fallback: $ML_MODEL; --random runs the model theses on the random-init 22-layer\n"
                             "  configuration; expectations: thesis-expectations.toml beside the package ($ML_THESIS_EXPECT)";
  static const char *DESCRIPTIONS[][2] = {
      {"t1", "decode-bandwidth-bound: weight bytes/token over decode GPU ms against the device bandwidth"},
      {"t2", "GEMV efficiency: each decode GEMV class against its bandwidth floor"},
      {"t4", "submission cost: one launch + stream-wait round trip"},
      {"t6", "tensor-core ceiling: f16-weight GEMM TF/s on the real 512-row prefill shapes"},
      {"t7", "token exactness: prepared-graph and per-launch decoding emit identical tokens at every prefill width"}};
  std::vector<int> theses;
  std::string model;
  bool list = false, all = false, random = false;
  if (argc >= 1 && !strcmp(argv[0], "parse")) {   // host only: thesis parse <file> <device>
    if (argc < 3) die("thesis parse <file> <device name>");
    std::string text, err;
    if (!read_file(argv[1], &text)) die(std::string("cannot read ") + argv[1]);
    std::map<std::string, Section> secs;
    if (!parse_expectations(text, &secs, &err)) die("parsing " + std::string(argv[1]) + ": " + err);
    auto it = secs.find(argv[2]);
    if (it == secs.end()) {
      printf("no section for '%s'\n", argv[2]);
      return 0;
    }
    for (const auto &kv : it->second) printf("%s = %g\n", kv.first.c_str(), kv.second);
    return 0;
  }
  for (int i = 0; i < argc; ++i) {
    const std::string arg = argv[i];
    if (arg == "--all") all = true;
    else if (arg == "--list") list = true;
    else if (arg == "--random") random = true;
    else if (arg == "-m" || arg == "--model") {
      if (i + 1 >= argc) die(arg + " needs a value\n" + USAGE);
      model = argv[++i];
    } else {
      const bool t = (arg[0] == 't' || arg[0] == 'T') && arg.size() == 2 && arg[1] >= '1' && arg[1] <= '7';
      if (!t) die("unknown thesis '" + arg + "'\n" + USAGE);
      theses.push_back(arg[1] - '0');
    }
  }
  if (list) {
    printf("performance theses:\n");
    for (auto &d : DESCRIPTIONS) printf("  %s  %s\n", d[0], d[1]);
    printf("  t3, t5  not measured here: one in-order stream per submission has no barrier to price\n");
    return 0;
  }
  if (all || theses.empty()) theses = {1, 2, 4, 6, 7};
  std::sort(theses.begin(), theses.end());
  theses.erase(std::unique(theses.begin(), theses.end()), theses.end());
  auto wants = [&](int id) { return std::find(theses.begin(), theses.end(), id) != theses.end(); };
  if (model.empty())
    if (const char *e = getenv("ML_MODEL")) model = e;

  Session s;
  s.ctx = ta_context_create(0, getenv("ML_DEVICE"));
  if (!s.ctx) die_lib("context");
  s.exec = ta_executor_create_v2(s.ctx, 2, 1024, getenv("ML_KERNEL"), 0);
  if (!s.exec) die_lib("executor");
  const std::string device = ta_context_device_name(s.ctx);
  const std::string path = expectations_path();
  std::map<std::string, Section> secs;
  std::string text, err;
  const Section *sec = nullptr;
  if (!read_file(path, &text)) {
    fprintf(stderr, "expectations file %s not found; all verdicts will be informational\n", path.c_str());
  } else {
    if (!parse_expectations(text, &secs, &err)) die("parsing " + path + ": " + err);
    auto it = secs.find(device);
    if (it == secs.end())
      fprintf(stderr, "no recorded expectations for device '%s' in %s; all verdicts will be informational\n", device.c_str(), path.c_str());
    else {
      sec = &it->second;
      fprintf(stderr, "expectations: %s [%s]\n", path.c_str(), device.c_str());
    }
  }
  fprintf(stderr, "burn-in: ~300 ms of 1024^3 GEMMs before first measurement\n");
  thesis_burn_in(s);
  std::vector<Row> rows;
  auto add = [&](std::vector<Row> r) { rows.insert(rows.end(), r.begin(), r.end()); };
  if (wants(3) || wants(5))
    rows.push_back(Row{wants(3) ? "T3" : "T5", "barrier cost / prefill accounting", "-",
                       "not measured: a submission is one in-order stream, there is no barrier to price", Verdict::Skip});
  if (wants(4)) add(t4_submission_cost(s, sec));
  if (wants(2)) add(t2_gemv_efficiency(s, sec));
  if (wants(6)) add(t6_tensor_core_ceiling(s, sec));
  if (wants(1) || wants(7)) {
    if (model.empty() && !random) {
      for (int id : {1, 7})
        if (wants(id))
          rows.push_back(Row{id == 1 ? "T1" : "T7", "model-level thesis", "-", "no GGUF model (pass -m/--model, set ML_MODEL, or --random)",
                             Verdict::Skip});
    } else {
      ThesisModel m;
      load_thesis_model(s, model, random, &m);
      if (wants(1)) add(t1_decode_bandwidth(sec, m));
      if (wants(7)) add(t7_token_exactness(m));
    }
  }
  std::stable_sort(rows.begin(), rows.end(), [](const Row &a, const Row &b) { return a.thesis < b.thesis; });
  print_thesis_table(device, rows);
  size_t failures = 0;
  for (const Row &r : rows) failures += r.verdict == Verdict::Fail;
  if (failures) {
    fprintf(stderr, "ml_bench: %zu thesis measurement(s) FAILED against recorded expectations\n", failures);
    return 1;
  }
  return 0;
}

}  // namespace

int main(int argc, char **argv) {
  const std::string cmd = argc > 1 ? argv[1] : "all";
  if (cmd == "thesis") return thesis(argc - 2, argv + 2);
  static const char *known[] = {"self-check", "correctness", "sweep", "single", "cases", "concurrent", "transfer", "prepared", "all", "summary"};
  if (std::find_if(std::begin(known), std::end(known), [&](const char *k) { return cmd == k; }) == std::end(known))
    die("unknown subcommand '" + cmd + "'; expected self-check, correctness, sweep, single, cases, concurrent, transfer, prepared, thesis, or all");
  std::vector<std::string> rest;
  for (int i = 2; i < argc; ++i) rest.push_back(argv[i]);
  if (cmd == "summary") {   // host only: the sample summary of the given numbers (nan / inf / negatives are dropped)
    std::vector<double> v;
    for (const std::string &x : rest) v.push_back(strtod(x.c_str(), nullptr));
    const Summary sm = summarize(v);
    if (!sm.ok()) {
      printf("none\n");
    } else {
      printf("count=%zu min=%g median=%g p95=%g\n", sm.count, sm.min, sm.median, sm.p95);
    }
    return 0;
  }
  if (cmd == "cases") {   // specs are checked before any device work, as a wrong one is a usage error
    if (rest.empty()) die("cases requires at least one label,b,m,n,k argument");
    for (const std::string &spec : rest) parse_case(spec);
  }
  const uint32_t n_slots = std::max(1u, env_u32("ML_SLOTS", 2));
  Session s;
  s.ctx = ta_context_create(env_bool("ML_VALIDATE") ? 1 : 0, getenv("ML_DEVICE"));
  if (!s.ctx) die_lib("context");
  s.exec = ta_executor_create_v2(s.ctx, n_slots, 256, getenv("ML_KERNEL"), env_bool("ML_TUNE") ? 1 : 0);
  if (!s.exec) die_lib("executor");
  fprintf(stderr, "%s (cuda:%d) slots=%u kernel=%s\n", ta_context_device_name(s.ctx), ta_context_device_index(s.ctx), n_slots,
          env_string("ML_KERNEL", "auto").c_str());
  if (cmd == "self-check") {
    printf("tensor-ash self-check\nstatus: OK\nselected: %s (cuda:%d)\nexecutor_slots: %u\nversion: %s\n",
           ta_context_device_name(s.ctx), ta_context_device_index(s.ctx), n_slots, ta_version());
  } else if (cmd == "correctness") {
    correctness(s);
  } else if (cmd == "sweep") {
    sweep(s);
  } else if (cmd == "single") {
    single(s);
  } else if (cmd == "cases") {
    cases(s, rest);
  } else if (cmd == "concurrent") {
    concurrent(s);
  } else if (cmd == "transfer") {
    transfer(s);
  } else if (cmd == "prepared") {
    prepared(s);
  } else {
    correctness(s);
    sweep(s);
  }
  return 0;
}
