// llama_ash: run an F32 / F16 llama-family GGUF (or a random-initialised model of the benchmark
// geometry) end to end on the library and report prefill / decode throughput.  Same subcommands,
// flags, prompt and output table as the reference's tool (tools/llama-ash/src/main.rs:1-260);
// written against the C ABI only (tensor_ash.h + tensor_ash_llama.h).
//
//   llama_ash bench    (-m <gguf> | --random) [--pp 512] [--tg 128] [--ctx 2048]
//   llama_ash generate (-m <gguf> | --random) --ids "1,15043,3186" [-n 24] [--ctx 2048]
//
// ML_DEVICE picks the GPU (index:N), ML_KERNEL the GEMM kernel, as everywhere in the library.
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/tensor_ash_llama.h"

namespace {

const char *USAGE =
    "usage:\n"
    "  llama_ash bench (-m <gguf> | --random) [--pp 512] [--tg 128] [--ctx 2048]\n"
    "  llama_ash generate (-m <gguf> | --random) --ids \"1,15043,3186\" [-n 24] [--ctx 2048]\n";

struct Args {
  std::string model;
  bool random = false;
  uint32_t pp = 512, tg = 128, ctx = 2048, n = 24;
  std::vector<uint32_t> ids;
};

[[noreturn]] void die(const std::string &msg) {
  fprintf(stderr, "llama_ash: %s\n", msg.c_str());
  exit(1);
}

[[noreturn]] void die_lib(const char *what) { die(std::string(what) + ": " + ta_last_error()); }

uint32_t parse_u32(const std::string &flag, const std::string &v) {
  char *end = nullptr;
  const unsigned long x = strtoul(v.c_str(), &end, 10);
  if (v.empty() || *end || x > 0xfffffffful) die(flag + ": '" + v + "' is not an unsigned integer");
  return (uint32_t)x;
}

Args parse(int argc, char **argv, std::string *cmd) {
  if (argc < 2) die(USAGE);
  *cmd = argv[1];
  Args a;
  for (int i = 2; i < argc; ++i) {
    const std::string flag = argv[i];
    auto value = [&]() -> std::string {
      if (i + 1 >= argc) die("flag " + flag + " needs a value");
      return argv[++i];
    };
    if (flag == "-m" || flag == "--model") a.model = value();
    else if (flag == "--random") a.random = true;
    else if (flag == "--pp") a.pp = parse_u32(flag, value());
    else if (flag == "--tg") a.tg = parse_u32(flag, value());
    else if (flag == "--ctx") a.ctx = parse_u32(flag, value());
    else if (flag == "-n") a.n = parse_u32(flag, value());
    else if (flag == "--ids") {
      std::string v = value(), item;
      for (size_t p = 0; p <= v.size(); ++p) {
        if (p == v.size() || v[p] == ',') {
          size_t b = item.find_first_not_of(' '), e = item.find_last_not_of(' ');
          if (b == std::string::npos) die("--ids: empty item");
          a.ids.push_back(parse_u32("--ids", item.substr(b, e - b + 1)));
          item.clear();
        } else {
          item += v[p];
        }
      }
    } else {
      die("unknown flag " + flag + "\n" + USAGE);
    }
  }
  if (a.model.empty() && !a.random) die(std::string("missing -m <gguf> (or --random)\n") + USAGE);
  return a;
}

struct Session {
  ta_context *ctx = nullptr;
  ta_executor *exec = nullptr;
  ta_llama *model = nullptr;
  ta_llama_config cfg{};
  double load_s = 0.0;
  ~Session() {
    ta_llama_destroy(model);
    ta_executor_destroy(exec);
    ta_context_destroy(ctx);
  }
};

double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

void open_session(const Args &a, Session *s) {
  const double t0 = now_s();
  s->ctx = ta_context_create(0, getenv("ML_DEVICE"));
  if (!s->ctx) die_lib("context");
  s->exec = ta_executor_create(s->ctx, 2, 256, getenv("ML_KERNEL"));   // main.rs:78: 2 slots, 256 calls
  if (!s->exec) die_lib("executor");
  if (a.random) {
    ta_llama_config c{};
    c.layers = 22; c.embd = 2048; c.heads = 32; c.kv_heads = 4; c.head_dim = 64; c.ffn = 5632; c.vocab = 32000;
    c.t_max = a.ctx; c.rms_eps = 1e-5f; c.rope_theta = 1e4f; c.weight_sigma = 0.02f; c.norm_jitter = 0.0f; c.seed = 1;
    s->model = ta_llama_create_random(s->exec, &c);
  } else {
    s->model = ta_llama_load_gguf(s->exec, a.model.c_str(), a.ctx, nullptr);
  }
  if (!s->model) die_lib("model");
  if (ta_llama_get_config(s->model, &s->cfg) != 0) die_lib("config");
  s->load_s = now_s() - t0;
  fprintf(stderr, "config: layers=%u embd=%u heads=%u kv_heads=%u dh=%u ffn=%u vocab=%u eps=%g rope_base=%g t_max=%u\n",
          s->cfg.layers, s->cfg.embd, s->cfg.heads, s->cfg.kv_heads, s->cfg.head_dim, s->cfg.ffn, s->cfg.vocab,
          (double)s->cfg.rms_eps, (double)s->cfg.rope_theta, s->cfg.t_max);
}

void check_logits(Session &s, const char *when) {
  std::vector<float> logits(s.cfg.vocab);
  if (ta_llama_logits(s.model, logits.data(), logits.size()) != 0) die_lib("logits");
  for (float v : logits)
    if (!std::isfinite(v)) die(std::string(when) + " produced non-finite logits");
}

std::string join(const std::vector<uint32_t> &ids) {
  std::string out;
  for (size_t i = 0; i < ids.size(); ++i) out += (i ? "," : "") + std::to_string(ids[i]);
  return out;
}

int bench(const Args &a) {
  Session s;
  open_session(a, &s);
  if (a.pp == 0) die("--pp must be at least 1");
  if ((uint64_t)a.pp + a.tg > s.cfg.t_max)
    die("pp " + std::to_string(a.pp) + " + tg " + std::to_string(a.tg) + " exceeds context " + std::to_string(s.cfg.t_max));
  // Fixed synthetic prompt: BOS then arbitrary in-vocab ids (main.rs:92-95).
  std::vector<uint32_t> prompt(a.pp);
  prompt[0] = 1 % s.cfg.vocab;
  for (uint32_t i = 1; i < a.pp; ++i) prompt[i] = (100 + (i % 1000)) % s.cfg.vocab;

  // Warm-up: an untimed prefill plus decode steps, then reset (main.rs:97-106).
  uint32_t next = 0;
  ta_run_stats st{};
  std::vector<uint32_t> out(a.tg ? a.tg : 1);
  if (ta_llama_prefill(s.model, prompt.data(), a.pp, &next, &st) != 0) die_lib("warmup prefill");
  check_logits(s, "warmup prefill");
  if (a.tg && ta_llama_decode(s.model, next, a.tg, out.data(), &st) != 0) die_lib("warmup decode");
  if (ta_llama_reset(s.model) != 0) die_lib("reset");

  double t0 = now_s();
  if (ta_llama_prefill(s.model, prompt.data(), a.pp, &next, &st) != 0) die_lib("prefill");
  const double prefill_s = now_s() - t0;
  fprintf(stderr, "prefill timing: %.3f ms GPU vs %.3f ms wall (%.3f ms host)\n", st.gpu_time_ns / 1e6, prefill_s * 1e3,
          prefill_s * 1e3 - st.gpu_time_ns / 1e6);
  t0 = now_s();
  if (a.tg && ta_llama_decode(s.model, next, a.tg, out.data(), &st) != 0) die_lib("decode");
  const double decode_s = now_s() - t0;
  if (a.tg)
    fprintf(stderr, "decode timing: %.3f ms/token GPU vs %.3f ms/token wall (%.3f ms host)\n",
            st.gpu_time_ns / 1e6 / a.tg, decode_s * 1e3 / a.tg, decode_s * 1e3 / a.tg - st.gpu_time_ns / 1e6 / a.tg);

  // Per-op-class GPU-time breakdown of one more decode step (main.rs:161-193).
  if (const char *e = getenv("LLAMA_ASH_BREAKDOWN"); e && !strcmp(e, "1") && a.tg) {
    ta_llama_breakdown_row rows[32];
    size_t n_rows = 0, n_launches = 0;
    uint32_t tok = 0;
    if (ta_llama_decode_breakdown(s.model, out[a.tg - 1], rows, 32, &n_rows, &n_launches, &tok) != 0) die_lib("breakdown");
    uint64_t total = 0;
    for (size_t i = 0; i < n_rows && i < 32; ++i) total += rows[i].gpu_ns;
    printf("decode GPU breakdown (one token, %zu dispatches):\n", n_launches);
    for (size_t i = 0; i < n_rows && i < 32; ++i)
      printf("  %-16s %8.1f us  (%3u calls, %4.1f%%)\n", rows[i].op_class, rows[i].gpu_ns / 1e3, rows[i].calls,
             total ? rows[i].gpu_ns * 100.0 / total : 0.0);
    printf("  %-16s %8.1f us  (GPU-timestamped total)\n", "sum", total / 1e3);
  }

  printf("model    : %s\n", a.random ? "(random-init, llama 22L/2048/32q/4kv/5632/32000)" : a.model.c_str());
  printf("load     : %.2f s\n", s.load_s);
  printf("| test        | tokens | time (s) | tokens/s |\n");
  printf("|-------------|--------|----------|----------|\n");
  printf("| pp%-9u | %6u | %8.3f | %8.2f |\n", a.pp, a.pp, prefill_s, a.pp / prefill_s);
  if (a.tg) printf("| tg%-9u | %6u | %8.3f | %8.2f |\n", a.tg, a.tg, decode_s, a.tg / decode_s);
  return 0;
}

int generate(const Args &a) {
  if (a.ids.empty()) die(std::string("generate needs --ids \"1,...\"\n") + USAGE);
  Session s;
  open_session(a, &s);
  for (uint32_t id : a.ids)
    if (id >= s.cfg.vocab) die("--ids: token " + std::to_string(id) + " is outside the vocabulary of " + std::to_string(s.cfg.vocab));
  if (a.n == 0) die("-n must be at least 1");
  if ((uint64_t)a.ids.size() + a.n > s.cfg.t_max) die("prompt + -n exceeds context " + std::to_string(s.cfg.t_max));
  uint32_t first = 0;
  ta_run_stats st{};
  double t0 = now_s();
  if (ta_llama_prefill(s.model, a.ids.data(), (uint32_t)a.ids.size(), &first, &st) != 0) die_lib("prefill");
  const double prefill_s = now_s() - t0;
  check_logits(s, "prefill");
  std::vector<uint32_t> generated{first}, rest(a.n > 1 ? a.n - 1 : 1);
  t0 = now_s();
  if (a.n > 1) {
    if (ta_llama_decode(s.model, first, a.n - 1, rest.data(), &st) != 0) die_lib("decode");
    generated.insert(generated.end(), rest.begin(), rest.begin() + (a.n - 1));
  }
  const double decode_s = now_s() - t0;
  printf("prompt_ids   : %s\n", join(a.ids).c_str());
  printf("generated_ids: %s\n", join(generated).c_str());
  printf("timings      : load %.2f s | prefill %zu tok in %.3f s (%.2f t/s) | decode %zu tok in %.3f s (%.2f t/s)\n",
         s.load_s, a.ids.size(), prefill_s, a.ids.size() / prefill_s, generated.size() - 1, decode_s,
         (generated.size() - 1) / (decode_s > 1e-9 ? decode_s : 1e-9));
  return 0;
}

}  // namespace

int main(int argc, char **argv) {
  std::string cmd;
  const Args a = parse(argc, argv, &cmd);
  if (cmd == "bench") return bench(a);
  if (cmd == "generate") return generate(a);
  die("unknown subcommand " + cmd + "\n" + USAGE);
}
