// ml_bench: the GEMM benchmark tool of the reference (tools/ml-bench/src/bench/{mod,commands,
// cases,env,report}.rs) on this library's C ABI.  Same subcommands for the GEMM path, the same
// environment knobs, compact case specs, sample summaries (min / median / nearest-rank p95),
// table and CSV columns, and the same sampled validation after timing.
//
//   ml_bench self-check | correctness | sweep | single | cases label,b,m,n,k[,f16w] ... | concurrent | transfer |
//            prepared | all
//   ml_bench summary x1 x2 ...      (host only: prints the sample summary of the numbers)
//
//   ML_ITERS (20) ML_WARMUP (3) ML_OUTPUT (table | csv) ML_SWEEP (smoke | standard | full)
//   ML_B ML_M ML_N ML_K   ML_SPLIT_K2 (0)   ML_SLOTS (2)   ML_THREADS   ML_KERNEL (auto)   ML_DEVICE   ML_VALIDATE
//   ML_PEAK_TFLOPS: the "%peak" denominator; default 232.5, the FP32-through-3xTF32 ceiling of a
//   B200 (measured sustained bf16 rate / 2 / 3); the reference's default is its own GPU's 20.3.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <strings.h>
#include <thread>
#include <vector>

#include "../../include/tensor_ash.h"

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

}  // namespace

int main(int argc, char **argv) {
  const std::string cmd = argc > 1 ? argv[1] : "all";
  static const char *known[] = {"self-check", "correctness", "sweep", "single", "cases", "concurrent", "transfer", "prepared", "all", "summary"};
  if (std::find_if(std::begin(known), std::end(known), [&](const char *k) { return cmd == k; }) == std::end(known))
    die("unknown subcommand '" + cmd + "'; expected self-check, correctness, sweep, single, cases, concurrent, transfer, prepared, or all");
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
