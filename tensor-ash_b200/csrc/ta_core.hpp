// Host-side core of the B200-native tensor-ash GEMM path.
//
// The types mirror the reference crate's public API one for one so that code
// and tests written against it read the same here:
//   Context        <- VulkanContext            (src/context/mod.rs)
//   Tensor         <- Tensor                   (src/tensor.rs:20-201)
//   MatmulCall/Op, Epilogue, Activation, EpilogueBinary, MatmulStore, RunStats
//                  <- src/matmul/api.rs:3-353
//   ResolvedMatmul <- src/matmul/resolution.rs:78-441
//   Executor       <- src/executor/mod.rs:85-369, dispatch.rs, reduction.rs,
//                     prepared.rs, transfer.rs, elementwise/*.rs
//   PreparedOps    <- src/executor/prepared.rs:46-353 (a captured CUDA graph)
//   KernelSpec / KERNEL_SPECS / KernelSelection <- src/pipeline/catalog.rs
// What Vulkan did (instance, queues, descriptor sets, pipeline cache, fences)
// is a CUDA device ordinal, one stream per executor slot and two events.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <condition_variable>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <functional>
#include <memory>
#include <mutex>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace ta {

// ------------------------------------------------------------------ errors
struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

[[noreturn]] void fail(const char *fmt, ...) __attribute__((format(printf, 1, 2)));
std::string strf(const char *fmt, ...) __attribute__((format(printf, 1, 2)));
void cuda_check(cudaError_t e, const char *what);
#define TA_CUDA(expr) ::ta::cuda_check((expr), #expr)

// Launch counter behind ta_kernel_launch_count().
extern std::atomic<uint64_t> g_launches;

// ------------------------------------------------------------------ experiment switches
// Every A/B switch of the kernels lives here, read once per process from the ONE environment
// variable TA_EXPERIMENT, a comma-separated list of `name=value` pairs, e.g.
//   TA_EXPERIMENT="tf32x3_chunk_kb=32,peer_allreduce=0"
// Unknown names are an error at first use.  Defaults are the shipped configuration; nothing on
// the launch path calls getenv.
struct Tunables {
  uint32_t tf32x3_chunk_kb = 0;   // K blocks of 16 per tensor-memory accumulation (0 = kernel default)
  int tf32x3_ksplit = 1;          // few-tile 3xTF32 GEMM split along K over the idle SMs (0 = off, 1 = on, 128 / 256 = on with that tile width)
  int gemv_ksplit = 0;            // force the GEMV cluster split along K (1/2/4/8; 0 = chosen per shape)
  int gemv_bulk = -1;             // 1/0: force the bulk-copy ring of the 1-2 row GEMV on/off (-1 = per shape)
  int gemv_umma = -1;             // 1/0: force the tensor-memory GEMV (3..8 rows) on/off (-1 = per shape)
  bool f16w_pre = true;           // f16w tensor-core GEMM: convert A once per launch into scratch
  uint32_t f16w_apad = 0;         // extra halves of row pitch of that f16 copy (multiple of 8)
  bool pdl = true;                // programmatic dependent launch between decode kernels
  bool peer_allreduce = true;     // one-launch peer-write all-reduce for small tensor-parallel exchanges
  bool peer_allreduce_big = false; // all-reduce of prefill-sized tensors by the two-step peer kernel instead of NCCL (measured slower: 4.25 vs 3.85 ms per 512-token prefill on 4 GPUs)
  bool splitk2_tensor = true;     // split-K2 stage 1 on the tensor cores where the shape allows
  int f16w_splitk = -1;           // f16w tensor-core GEMM: K split for grids under one wave (-1 = per shape, 0/1 = off)
  uint32_t f16w_bn = 0;           // f16w tensor-core GEMM: tile width of the planned route (0 = per shape; 64 / 128 / 192 / 256)
  bool f16w_tma_store = true;     // f16w tensor-core GEMM: C leaves through TMA stores (0: the kernel stores it itself)
  bool f16w_dual = true;          // f16w tensor-core GEMM: up and gate of a SwiGLU pair as one dual-matrix launch
  uint32_t attn_chunks = 0;       // decode attention with a position cell: chunk grid (0 = one 64-position tile per chunk, 8..32)
  uint32_t flash_groups = 2;     // tensor-core prefill attention: warp groups per query block that split its K/V tiles (1 or 2)
  bool gemv_peer_wide = true;     // exchange GEMV launches that fit one wave at two CTAs per SM take the 128-register variant
  bool gemv_handoff = true;       // row GEMV: cluster ranks reach rank 0 with st.async counted on an mbarrier (0: stores + cluster barrier)
  bool attn_wide = true;          // decode attention on the flagged route runs the 256-thread kernel (a warp per query row)
  bool attn_pairs = true;         // decode attention hands its chunk partials over as flagged pairs (no fence, no ticket)
  bool pos_stage = true;          // position cells read by graph launches are staged to device memory per submission
};
const Tunables &tunables();
// parses `name=value,...` into a Tunables (throws on an unknown name); exposed for the host tests
Tunables parse_tunables(const char *spec);

// ------------------------------------------------------------------ dtype
enum class DType : uint8_t { F32 = 0, F16 = 1 };
inline uint64_t dtype_size(DType d) { return d == DType::F32 ? 4 : 2; }
inline const char *dtype_name(DType d) { return d == DType::F32 ? "f32" : "f16"; }

// Bit-exact RNE conversions (src/dtype.rs:42-112).
uint16_t f32_to_f16_bits(float v);
float f16_bits_to_f32(uint16_t h);

// ------------------------------------------------------------------ context
struct Context {
  int device = 0;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  size_t smem_optin = 0;
  std::string name;
  bool validation = false;
  // cuTensorMapEncodeTiled, fetched through the runtime so the library has no
  // link-time dependency on the driver library.
  void *encode_tiled = nullptr;

  static std::shared_ptr<Context> create(bool validation, const std::string &preference);
  void make_current() const;
};

// ------------------------------------------------------------------ tensor
struct Buffer {
  std::shared_ptr<Context> ctx;
  void *ptr = nullptr;
  uint64_t bytes = 0;
  ~Buffer();
};

struct Tensor {
  std::shared_ptr<Buffer> buf;
  std::vector<uint32_t> shape;
  DType dtype = DType::F32;

  static uint64_t numel_checked(const uint32_t *shape, size_t rank);
  static Tensor uninit_device(const std::shared_ptr<Context> &ctx, const uint32_t *shape,
                              size_t rank, DType dtype);
  Tensor alias_with_shape(const uint32_t *shape, size_t rank) const;

  uint64_t len() const {
    uint64_t n = 1;
    for (uint32_t d : shape) n *= d;
    return n;
  }
  uint64_t size_bytes() const { return buf->bytes; }
  void *ptr() const { return buf->ptr; }
  const std::shared_ptr<Context> &ctx() const { return buf->ctx; }
  std::string shape_str() const;
};

// ------------------------------------------------------------------ op description
enum class Activation : uint32_t { None = 0, Relu = 1, Silu = 2, Gelu = 3 };
enum class BinaryKind : uint32_t { None = 0, AddScaled = 1, Mul = 2 };
enum class StoreKind : uint32_t { None = 0, Rope = 1, Scatter = 2, RopeScatter = 3 };

struct MatmulCall {
  const Tensor *a = nullptr, *b = nullptr, *c = nullptr;
  float alpha = 1.0f;
  bool accumulate = false;
};

struct Epilogue {
  const Tensor *bias = nullptr;
  Activation activation = Activation::None;
  BinaryKind binary = BinaryKind::None;
  const Tensor *d = nullptr;
  float beta = 0.0f;
  bool is_none() const {
    return !bias && activation == Activation::None && binary == BinaryKind::None;
  }
};

// 4-byte pinned, device-mapped host cell (PosBuffer / HostU32Buffer of
// src/executor/cells.rs:51-201): kernels in replayed graphs read the token
// position from it or write a result word into it.
struct PosCell {
  std::shared_ptr<Context> ctx;
  uint32_t *host = nullptr;        // pinned host word
  uint32_t *device = nullptr;      // the same word as seen from the device
};

struct MatmulStore {
  StoreKind kind = StoreKind::None;
  uint32_t head_dim = 0, pos_base = 0, pos_scale = 0, stride_head = 0, stride_dim = 0;
  const Tensor *table = nullptr;
  const Tensor *dst = nullptr;
  const PosCell *pos_cell = nullptr;
  bool is_none() const { return kind == StoreKind::None; }
};

struct MatmulOp {
  MatmulCall call;
  Epilogue epilogue;
  const Tensor *normed_weight = nullptr;  // normed-A (weight[K], eps)
  float normed_eps = 0.0f;
  MatmulStore store;
  bool packed_b = false;
  bool a16_ready = false;   // planner-internal: the slot scratch already holds this A rounded to f16
};

struct RunStats {
  std::optional<uint64_t> gpu_time_ns;
  size_t n_calls = 0;
  uint64_t total_flops = 0;
  // flops / ns * 1e-3 (src/matmul/api.rs:346-353); nullopt when no/zero time.
  std::optional<double> tflops() const {
    if (!gpu_time_ns || *gpu_time_ns == 0) return std::nullopt;
    return (double)total_flops / (double)*gpu_time_ns * 1e-3;
  }
};

// ------------------------------------------------------------------ resolution
struct MatrixShape {
  uint32_t batch, rows, cols;
  static MatrixShape from_shape(const uint32_t *shape, size_t rank);
  uint32_t batch_stride(const char *label) const;
};

struct ResolvedMatmul {
  uint32_t m = 0, n = 0, k = 0, batch = 0;
  uint32_t batch_stride_a = 0, batch_stride_b = 0, batch_stride_c = 0;
  uint64_t total_flops = 0;
  bool b_f16 = false, a_f16 = false, packed_b = false;

  static ResolvedMatmul from_shapes(MatrixShape a, MatrixShape b, MatrixShape c);
  static ResolvedMatmul from_call(const MatmulCall &call);
  static ResolvedMatmul from_op(const MatmulOp &op);
  void validate_bias_shape(const std::vector<uint32_t> &shape) const;
};

// ------------------------------------------------------------------ registry
// One CUDA tile variant.  `family` drives eligibility checks and launch.
enum class Family : uint8_t {
  Tf32x3,     // tcgen05 kind::tf32, 3-pass split, TMEM accumulate (FP32 parity)
  Ffma,       // SIMT FFMA tiles, any shape / alignment, f32 or f16 B
  F16wUmma,   // tcgen05 kind::f16: A f32->f16 RNE at staging, B f16
  RowGemv,    // M-row GEMV over f16 (optionally packed) or f32 weights
  SplitK2     // stage-1 kernels of the two-stage split-K route
};

struct KernelSpec {
  const char *name;
  uint32_t tile_m, tile_n, tile_k;
  Family family;
  bool weights_f16;  // reads B as f16 storage
  const char *const *aliases;  // NULL-terminated; includes the reference names it supersedes
};

extern const KernelSpec KERNEL_SPECS[];
extern const size_t KERNEL_SPEC_COUNT;

// Returns -2 for "auto"/"", an index into KERNEL_SPECS, or throws.
int kernel_selection_parse(const std::string &value);
int kernel_index_by_name(const char *name);  // -1 when absent
// Heuristic stage of the routing order: index into KERNEL_SPECS for a plain shape.
int heuristic_kernel_index(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, bool b_f16, int sm_count);

// Row-GEMV routing (src/pipeline/routing.rs:10-41).
bool f16w_row_uses_k16(uint32_t k, uint32_t n);
uint32_t f16w_row_tile_n(uint32_t k, uint32_t n);

// Split-K heuristics (src/executor/splitk2.rs:36-122).
uint32_t default_num_k_splits(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, uint32_t tile_m,
                              uint32_t tile_n);
std::optional<uint32_t> heuristic_splits(uint32_t batch, uint32_t m, uint32_t n, uint32_t k);
void splitk2_stage1_tile(uint32_t m, uint32_t n, const char **name, uint32_t tile[3]);

void pack_f16w_row_tiles(const float *src, float *dst, size_t k, size_t n, size_t tile_n);

// Tuned-winner store (src/pipeline/tuning.rs:60-199): text file, one line per
// shape "B M N K kernel [splitk2=S]", header carries the registry hash.
struct TunedEntry {
  int kernel = -1;
  uint32_t splits = 0;
};
struct TuneKey {
  uint32_t batch, m, n, k;
  bool b_f16;
  bool operator==(const TuneKey &o) const {
    return batch == o.batch && m == o.m && n == o.n && k == o.k && b_f16 == o.b_f16;
  }
};
struct TuneKeyHash {
  size_t operator()(const TuneKey &t) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t v : {(uint64_t)t.batch, (uint64_t)t.m, (uint64_t)t.n, (uint64_t)t.k,
                       (uint64_t)t.b_f16}) {
      h ^= v;
      h *= 1099511628211ull;
    }
    return (size_t)h;
  }
};
// Tuner arithmetic (src/executor/tuning.rs:319-344): median of u64 samples (mean of the middle pair,
// rounded down, for an even count; nullopt when empty) and the candidate measured at `offset` of
// `round` (round 0 in index order; measured rounds come in pairs, forward then backward from a
// start that moves by half the list per pair, so every candidate sees every rank sum equally).
std::optional<uint64_t> tune_median(std::vector<uint64_t> samples);
size_t tune_candidate_at(size_t len, uint32_t round, size_t offset);
uint64_t registry_hash();
std::string tune_store_path(const std::string &device_name);
std::unordered_map<TuneKey, TunedEntry, TuneKeyHash> load_tuned(const std::string &path);
void save_tuned(const std::string &path,
                const std::unordered_map<TuneKey, TunedEntry, TuneKeyHash> &map);

// ------------------------------------------------------------------ device parameter blocks
// Everything a GEMM kernel needs, in elements (not bytes) for strides.
struct GemmParams {
  const void *a;
  const void *b;
  float *c;
  const float *bias;
  const float *d;
  uint32_t m, n, k, batch;
  uint32_t stride_a, stride_b, stride_c;  // batch strides, 0 = broadcast
  uint32_t bias_stride;                    // 0 = [N], n = [B, N]
  float alpha, beta;
  uint32_t accumulate, act, binary, b_f16;
  // split-K stage 1 only: K range partition count; plane = (batch*splits+s)
  uint32_t splits;
  // tf32x3 tensor-core kernel: K blocks of 16 accumulated in tensor memory between drains (set by its launcher)
  uint32_t chunk_kb;
  uint32_t b_grouped = 0;    // launcher-set: the B tensor map is the rank-4 grouped view (one TMA per stage)
  uint32_t c_f16 = 0;        // a16 route: C (and the old C when accumulating) is f16 storage
  // tensor-core split-K stage 1 (launcher-set): planes per batch = splits * sk_c, K blocks of 16 per
  // caller-visible split and per plane, destination of the planes
  uint32_t sk_subs = 0, sk_c = 0, sk_kb_per_split = 0, sk_kb_per_sub = 0;
  float *sk_planes = nullptr;
  // f16-weight tensor-core GEMM with an in-kernel K split (launcher-set): slices per tile, partial
  // tiles in scratch, two ticket words per tile
  uint32_t fw_splits = 0;
  float *fw_partials = nullptr;
  uint32_t *fw_counters = nullptr;
  uint32_t pdl_wait = 0;     // launcher-set: the kernel was launched to overlap its predecessor and waits for it on the device
  uint32_t c_tma = 0;        // launcher-set (f16w tensor-core GEMM): C leaves through TMA stores of the launch's C tensor map
  // f16w tensor-core GEMM, two weight matrices sharing A (the SwiGLU pair of a prefill MLP): a tile
  // holds BN/2 columns of b (gate) and the same BN/2 columns of b2 (up); C = silu(A b) * (A b2), and
  // c2, when set, receives A b2
  const void *b2 = nullptr;
  float *c2 = nullptr;
};

// Tile width / K split of the f16-weight tensor-core GEMM for a shape (see k_gemm_f16w.cu)
struct F16wPlan {
  uint32_t tile_n = 256, splits = 1;
  size_t partial_bytes = 0;
};
F16wPlan gemm_f16w_umma_plan(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, int sm_count, bool allow_split);
// C = silu(A @ b) * (A @ b2) (and c2 = A @ b2) in one launch; p.b2 / p.c2 set.  Eligibility: the
// checks of gemm_f16w_umma_dual_eligible; scratch as for the single GEMM (the f16 copy of A).
bool gemm_f16w_umma_dual_eligible(const GemmParams &p);
void launch_gemm_f16w_umma_dual(const Context &ctx, const GemmParams &p, uint32_t *status, void *scratch, size_t scratch_bytes,
                                bool a16_ready, cudaStream_t stream);
size_t gemm_f16w_umma_scratch_bytes_split(uint32_t batch, uint32_t batch_a, uint32_t m, uint32_t n, uint32_t k, int sm_count);

// How the tensor-core stage 1 of split-K2 cuts a problem (see k_gemm_tf32x3.cu).  `planes` per batch
// = splits * c; eligible = false keeps the problem on the SIMT stage 1.
struct SplitK2TensorPlan {
  bool eligible = false;
  uint32_t tile_n = 0, c = 0, kb_per_split = 0, kb_per_sub = 0, planes = 0;
};
SplitK2TensorPlan splitk2_tensor_plan(const GemmParams &p, uint32_t splits, int sm_count);
// K split of a lone 3xTF32 GEMM with few output tiles (stage 1 planes + reduce with the op's epilogue)
SplitK2TensorPlan gemm_tf32x3_ksplit_plan(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, int sm_count);
size_t gemm_tf32x3_ksplit_scratch_bytes(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, int sm_count);

// Parameters of the f16-weight GEMV kernel (M <= 8 activation rows).
struct GemvParams {
  const float *x;          // [M, K] f32
  const void *w;           // f16 weights, [K, N] or packed [N/tile][K][tile]
  const void *w2;          // optional second matrix sharing x: out = silu(x@w) * (x@w2)
  float *c;                // [M, N]
  float *c2;               // with w2: optional [M, N] destination of x@w2 itself
  const float *bias, *d;   // epilogue operands (bias [N]; D [M, N])
  const float *norm_w;     // fused RMSNorm weight [K] (nullptr = off)
  float norm_eps;
  uint32_t m, n, k;
  float alpha, beta;
  uint32_t accumulate, act, binary;
  uint32_t packed, tile_n;
  // fused store (StoreKind): rope table, scatter destination, position cell
  uint32_t store_kind, head_dim, pos_base, pos_scale, stride_head, stride_dim, dst_f16;
  const float *table;
  void *dst;
  const uint32_t *pos_ptr;
  int32_t pos_stage_idx;   // planner-internal: >= 0 when the launch reads the position from the slot's staged device word
  uint32_t pos_limit;   // positions the rope table and the scatter destination hold; pos_base + *pos_ptr beyond it
                        // raises status bit 3 and the kernel skips every access that uses the position
  // tensor-parallel exchange fused into the store: instead of C, the outputs go to slot `push_slot`
  // of every rank's exchange buffer as this rank's contribution to exchange point push_point1 - 1
  // (0 = off: an ordinary store)
  uint32_t push_point1, push_slot;
};

// Exchange buffers of a tensor-parallel group as one rank sees them, and what a GEMV launch pulls
// from them: its activation x is the sum over ranks (rank order) of what they pushed at
// `pull_point1 - 1` (0 = off).  A pushed element is an 8-byte (value, flag) pair written with one
// store; flag = use count of the point * 512 + point + 1, unique per point and submission, so a
// reader knows each element is this submission's by looking at it: no fence and no counter on the
// path, one NVLink crossing between a producer's store and its readers.
constexpr uint32_t PEER_MAX_WORLD = 8, PEER_MAX_FLOATS = 8192, PEER_MAX_POINTS = 256;
struct PeerLink {
  uint8_t *buf[PEER_MAX_WORLD];
  uint32_t rank, world;
  uint32_t pull_point1, pull_slot;
  float *x_out;                 // where the summed activation is also written (by the first column tile)
  // use counts of the exchange points (and, at PEER_MAX_POINTS, of the argmax pair exchange): advanced by
  // the host before every submission and staged to device memory by the submission's first operation
  const uint32_t *expect_base;
  const uint32_t *expect_ptr;   // the sharded argmax's word
  uint64_t limit_ns;            // bounded wait for the peers' data
};
__host__ __device__ inline uint32_t peer_flag_of(uint32_t use_count, uint32_t point1) { return use_count * 512u + point1; }

// Up to three GEMVs sharing x, M, K, norm and tile width in one launch.
constexpr int GEMV_MAX_SEGS = 3;
struct GemvGroup {
  GemvParams seg[GEMV_MAX_SEGS];
  uint32_t tile_end[GEMV_MAX_SEGS];   // running tile count after each segment
  uint32_t nseg;
  uint32_t ksplit, k_cta;             // cluster size along K and rows per rank
  uint32_t pdl;                       // 1: launched with programmatic stream serialization
  uint32_t handoff_async;             // 1: cluster ranks hand their partial tiles over with st.async + mbarrier
  uint32_t *status;                   // device word for bounded-wait timeouts (may be null)
  PeerLink peer;                      // world == 0: no tensor-parallel exchange in this launch
};

struct FlashParams {
  const float *q;
  const void *kt, *v;
  float *out;
  uint32_t heads, group, dh, t_q, t_max, kv_len, pos_base;
  float scale;
  uint32_t q_head_stride, q_row_stride, o_head_stride, o_row_stride;
  uint32_t kv_f16;
  uint32_t simt;   // 1: pin the f32-operand kernel (run_flash_attention_simt of the reference)
  uint32_t io_f16; // 1: q and out are f16 storage (the reference's kv16 io16 dh64 route); tensor-core kernel only
  // optional f16 mirror of a token-major f32 output ([T, heads * dh], row pitch out16_row_stride halves)
  void *out16;
  uint32_t out16_row_stride;
};

struct AttnDecodeParams {
  const float *q;
  const void *kt, *v;
  float *scratch, *out;
  uint32_t kv_heads, group, t_max, kv_len, num_chunks;
  float scale;
  uint32_t kv_f16;
  const uint32_t *pos_ptr;
  uint32_t *status;     // bit 3 is raised when kv_len + *pos_ptr exceeds t_max (the length is then clamped)
  uint32_t *counters;   // per-kv-head tickets (zero between launches), owned by the submitting slot
  uint32_t pdl;
  uint32_t prefetch_kv; // 1: the launch before this one wrote at most position kv_len - 1 of the cache
  uint32_t *pairs;      // flagged partials (attn_pairs_of the slot) when the launch fits them, else null: tickets
  uint32_t *pair_seq;   // with pairs: launch counts, one per kv head
};

struct FlashAttentionDesc {
  uint32_t kv_len = 0, pos_base = 0;
  float scale = 1.0f;
  uint32_t token_major_heads = 0, out_token_major_heads = 0;
  uint32_t simt = 0;
};

struct AttnDecodeDesc {
  uint32_t kv_len = 0;
  float scale = 1.0f;
  const PosCell *pos_cell = nullptr;
};

// Token-id list in pinned, device-mapped host memory (TokenIdBuffer of
// src/executor/cells.rs:140-201): prefill writes the prompt ids here and a
// gather kernel reads them on the device.
struct TokenIds {
  std::shared_ptr<Context> ctx;
  uint32_t *host = nullptr, *device = nullptr;
  uint32_t capacity = 0, len = 0;
};

// One op of a mixed graph (ExecOp of src/executor/graph_ops.rs:27-161).
// Operand slots by kind:
//   Matmul           mm
//   RmsNorm          in0 input, in1 weight, out; f0 eps
//   LayerNorm        in0 input, in1 weight, in2 bias, out; f0 eps
//   SoftmaxRows      in0 input, out; f0 scale; u0 mask kind, u1 valid/prefix, u2 rows per group
//   Rope             in0 input, in1 table, out; heads/head_dim/rot_dim/pos_base; cell = position (optional)
//   RopeScatter      in0 input, in1 table, out = dst; rope fields; dst_offset, strides[3], pos_scale; cell
//   CopyStrided      in0 src, out dst; extent, src_offset, src_strides, dst_offset, strides
//   Binary           in0 a, in1 b, out; u0 mode (0 a+beta*b, 1 silu(a)*b); f0 beta
//   AttnDecode       in0 q, in1 kt, in2 v, in3 scratch, out; attn
//   FlashAttn        in0 q, in1 kt, in2 v, out; flash
//   Argmax           in0 input; cell = result word
//   EmbedGather      cell = token word; in0 table, out
//   EmbedGatherRows  tokens; in0 table, out [n, embd]
//   ArgmaxSharded    in0 this rank's slice of the row, comm, cell = result word; u0 = global index of in0[0]
enum class ExecKind : uint32_t {
  Matmul = 0, RmsNorm, LayerNorm, SoftmaxRows, Rope, RopeScatter, CopyStrided, Binary, AttnDecode,
  FlashAttn, Argmax, EmbedGather, EmbedGatherRows, AllReduce, AllGather, PrefillQkvPack, ArgmaxSharded
};

// ------------------------------------------------------------------ communicator (tensor parallel)
constexpr size_t COMM_ID_BYTES = 128;
// Layout of one rank's exchange buffer (all ranks map all buffers):
//   [0, PEER_AR_BYTES)        the one-launch all-reduce kernel: data, flags, call counters
//   then the fused exchange:  data[2 slots][world][PEER_MAX_FLOATS] pairs of (f32 bits, flag),
//                             argmax pairs[2][world] (value bits, index; slot = use parity) and arrivals[world] u32
constexpr size_t PEER_AR_DATA_BYTES = 2ull * PEER_MAX_WORLD * PEER_MAX_FLOATS * sizeof(float);
constexpr size_t PEER_AR_FLAG_BYTES = 2ull * PEER_MAX_WORLD * 8 * sizeof(uint32_t);
constexpr size_t PEER_AR_BYTES = PEER_AR_DATA_BYTES + PEER_AR_FLAG_BYTES + 8 * sizeof(uint32_t) + 96;   // 16-byte multiple
constexpr size_t PEER_X_DATA_OFF = PEER_AR_BYTES;
constexpr size_t PEER_X_DATA_BYTES = 2ull * PEER_MAX_WORLD * PEER_MAX_FLOATS * 8;
constexpr size_t PEER_AMAX_PAIR_OFF = PEER_X_DATA_OFF + PEER_X_DATA_BYTES;
constexpr size_t PEER_AMAX_FLAG_OFF = PEER_AMAX_PAIR_OFF + 2 * PEER_MAX_WORLD * 8;   // pairs of two consecutive uses
constexpr size_t PEER_SMALL_TOTAL = PEER_AMAX_FLAG_OFF + PEER_MAX_WORLD * sizeof(uint32_t);
//   then the two-step all-reduce of larger tensors (up to PEER_BIG_MAX_FLOATS, a prefill activation):
//   in[world][slice] (partial slices pushed by the peers), out[world][slice] (reduced slices pushed
//   by their owners), flags of both steps [2][world][PEER_BIG_CTAS] and per-CTA call counters
constexpr uint32_t PEER_BIG_MAX_FLOATS = 1u << 20, PEER_BIG_CTAS = 64;
constexpr size_t PEER_BIG_IN_OFF = (PEER_SMALL_TOTAL + 255) & ~(size_t)255;
constexpr size_t PEER_BIG_OUT_OFF = PEER_BIG_IN_OFF + (size_t)PEER_BIG_MAX_FLOATS * sizeof(float) + 4096;
constexpr size_t PEER_BIG_FLAG_OFF = PEER_BIG_OUT_OFF + (size_t)PEER_BIG_MAX_FLOATS * sizeof(float) + 4096;
constexpr size_t PEER_BIG_EPOCH_OFF = PEER_BIG_FLAG_OFF + 2ull * PEER_MAX_WORLD * PEER_BIG_CTAS * sizeof(uint32_t);
constexpr size_t PEER_BUF_TOTAL = PEER_BIG_EPOCH_OFF + PEER_BIG_CTAS * sizeof(uint32_t);
void comm_unique_id(uint8_t out[COMM_ID_BYTES]);
struct Comm {
  std::shared_ptr<Context> ctx;
  uint32_t rank = 0, world = 1;
  void *handle = nullptr;   // ncclComm_t; null when world == 1
  void *peer_own = nullptr;            // this rank's exchange buffer (small all-reduces), null = NCCL only
  // how long a rank waits on the device for a peer's flag before it gives up and reports (status bit
  // 2): generous by default, because ranks of one job drift apart by whole milliseconds while one
  // of them still loads weights or instantiates a graph
  uint64_t peer_wait_limit_ns = 10000000000ull;
  std::vector<void *> peer_bufs;       // every rank's buffer as mapped here (index = rank)
  // Exchanges fused into kernels count arrivals: word p of this pinned, device-mapped array is the
  // number of arrivals per source rank that completes the current use of exchange point p (word
  // PEER_MAX_POINTS: of the argmax pair exchange).  The host advances the words of the points a
  // submission uses before it launches; kernels read them like the position cell.  Every rank
  // submits the same plans in the same order, so the words agree across ranks.
  // expected-arrival words: written by the host (pinned memory) right before a submission and copied
  // to device memory by the submission's first stream operation; kernels read only the device copy
  // (a word in host memory costs every reading warp a PCIe round trip)
  uint32_t *expect_host = nullptr, *expect_copy = nullptr;
  bool fused_exchange_ready() const { return peer_own != nullptr && expect_host != nullptr && expect_copy != nullptr; }
  PeerLink link() const;   // buffers, rank, world, wait limit; pull fields zero
  // one-launch greedy pick over column-sharded logits; false when the peer path is unavailable
  bool argmax_sharded(const float *in, uint32_t n, uint32_t index_offset, uint32_t *result, uint32_t *status,
                      cudaStream_t stream) const;
  void setup_peer_exchange();
  void resync();
  // one-launch peer-write all-reduce; false when the request does not fit it (caller uses NCCL)
  bool peer_all_reduce_sum(float *data, size_t count, uint32_t *status, bool pdl, cudaStream_t stream) const;
  // two-step (reduce-scatter by pushes, then the reduced slices pushed back) all-reduce over peer
  // memory for tensors of up to PEER_BIG_MAX_FLOATS floats; false when the request does not fit it
  bool peer_all_reduce_big(float *data, size_t count, uint32_t *status, cudaStream_t stream) const;
  static std::unique_ptr<Comm> create(const std::shared_ptr<Context> &ctx, uint32_t rank, uint32_t world,
                                      const uint8_t id[COMM_ID_BYTES]);
  ~Comm();
  void all_reduce_sum(float *data, size_t count, cudaStream_t stream) const;   // in place
  void all_gather(const float *src, float *dst, size_t count_per_rank, cudaStream_t stream) const;
};

// The fused exchange points one submission uses: (point, arrivals per source rank), point
// PEER_MAX_POINTS standing for the argmax pair exchange.  advance() is called on the host right
// before the submission is launched; stage() is the submission's first stream operation (recorded
// into a prepared graph like any launch) and brings the words to the device.  Submissions that use
// one communicator's exchange follow one another on the host: the next advance() comes after the
// previous submission has completed.
struct ExchangeUse {
  const Comm *comm = nullptr;
  std::vector<std::pair<uint32_t, uint32_t>> points;
  void advance() const {
    if (!comm || !comm->expect_host) return;
    for (const auto &pt : points) *(volatile uint32_t *)(comm->expect_host + pt.first) += pt.second;
  }
  // Position cells the submission's GEMV stores and decode attentions read (pinned host words):
  // copied to the slot's device words by the same first stream operation, so that the kernels read
  // device memory (a word in host memory costs every reading warp a PCIe round trip, and the
  // late-starting blocks of a launch cannot hide it behind their predecessor).  The host sets a cell
  // before it submits and leaves it alone until the submission has completed.
  std::vector<const uint32_t *> pos_cells_host;
  void stage(cudaStream_t stream, uint32_t *pos_stage = nullptr) const {
    if (pos_stage)
      for (size_t i = 0; i < pos_cells_host.size(); ++i)
        TA_CUDA(cudaMemcpyAsync(pos_stage + i, pos_cells_host[i], sizeof(uint32_t), cudaMemcpyHostToDevice, stream));
    if (!comm || !comm->expect_host || !comm->expect_copy || points.empty()) return;
    TA_CUDA(cudaMemcpyAsync(comm->expect_copy, comm->expect_host, (PEER_MAX_POINTS + 1) * sizeof(uint32_t),
                            cudaMemcpyHostToDevice, stream));
  }
};

struct ExecOp {
  ExecKind kind = ExecKind::Matmul;
  MatmulOp mm;
  const Tensor *in0 = nullptr, *in1 = nullptr, *in2 = nullptr, *in3 = nullptr, *out = nullptr;
  float f0 = 0.0f;
  uint32_t u0 = 0, u1 = 0, u2 = 0;
  // planner-internal (never set through the C ABI): the op also leaves its output rounded to f16, row
  // pitch a16_pitch halves, at the start of the slot scratch, where the f16-weight tensor-core GEMM
  // that reads the output next expects the f16 copy of its A (RmsNorm and token-major flash attention)
  uint32_t a16_pitch = 0;
  uint32_t heads = 0, head_dim = 0, rot_dim = 0, pos_base = 0;
  uint32_t extent[3] = {0, 0, 0}, src_offset = 0, src_strides[3] = {0, 0, 0};
  uint32_t dst_offset = 0, strides[3] = {0, 0, 0}, pos_scale = 0;
  FlashAttentionDesc flash;
  AttnDecodeDesc attn;
  const PosCell *cell = nullptr;
  const TokenIds *tokens = nullptr;
  const Comm *comm = nullptr;   // AllReduce (in place on `out`) / AllGather (in0 -> out)
};

struct Slot;
// A planned op: only launches.
using Launch = std::function<void(Slot &, cudaStream_t)>;

constexpr uint32_t ATTN_DECODE_MAX_CHUNKS = 32;
constexpr uint32_t ATTN_DECODE_MAX_KV_HEADS = 256;
// ticket words per slot / prepared object: [0, 256) decode attention (one per kv head), then GEMV column groups
constexpr uint32_t F16W_SPLIT_COUNTER0 = 256 + 4096;   // then two words per tile of a split f16-weight GEMM
constexpr uint32_t SLOT_COUNTERS = F16W_SPLIT_COUNTER0 + 512;
// behind the ticket words of a slot / prepared object: device copies of the position cells a submission reads
constexpr uint32_t POS_STAGE_WORDS = 8;
inline uint32_t *pos_stage_of(uint32_t *counters) { return counters + SLOT_COUNTERS; }
// behind those: one launch count per kv head and the (value, flag) pairs of the decode attention's chunk
// partials.  Only the attention kernel touches them: a launch tags its pairs with its kv head's count + 1,
// the combining CTA advances the count, so a pair of an earlier launch never looks current.
constexpr uint32_t ATTN_SEQ_OFFSET = SLOT_COUNTERS + POS_STAGE_WORDS;       // ATTN_DECODE_MAX_KV_HEADS words
constexpr uint32_t ATTN_PAIR_ROWS = 1024;                                   // kv heads x chunks x 8 query rows it holds
constexpr uint32_t ATTN_PAIR_ROW_WORDS = (64 + 2) * 2;                      // dh + (max, sum), two words each
constexpr uint32_t ATTN_PAIRS_OFFSET = (ATTN_SEQ_OFFSET + ATTN_DECODE_MAX_KV_HEADS + 3u) & ~3u;   // 16-byte aligned
constexpr uint32_t SLOT_WORDS = ATTN_PAIRS_OFFSET + ATTN_PAIR_ROWS * ATTN_PAIR_ROW_WORDS;   // whole allocation
inline uint32_t *attn_pairs_of(uint32_t *counters) { return counters + ATTN_PAIRS_OFFSET; }
inline uint32_t attn_decode_num_chunks(uint32_t kv_len) {
  const uint32_t c = (kv_len + 31) / 32;
  return c < 8 ? 8 : (c > ATTN_DECODE_MAX_CHUNKS ? ATTN_DECODE_MAX_CHUNKS : c);
}

struct Route {
  int kernel = -1;       // index into KERNEL_SPECS
  uint32_t splits = 0;   // >1: two-stage split-K route
  bool tuned = false;    // the kernel is a measured winner from the tuned store
};

// ------------------------------------------------------------------ executor
struct Slot {
  cudaStream_t stream = nullptr;
  cudaEvent_t ev_begin = nullptr, ev_end = nullptr;
  void *scratch = nullptr;       // grow-only device scratch (split-K planes)
  size_t scratch_bytes = 0;
  void *staging = nullptr;       // grow-only pinned host staging
  size_t staging_bytes = 0;
  uint32_t *status = nullptr;       // status word as kernels address it (raised only on a failure)
  uint32_t *status_host = nullptr;  // the same word in page-locked host memory: read after a sync, no copy
  uint32_t *counters = nullptr;  // SLOT_COUNTERS zeroed device words (tickets of the decode attention and the GEMV finishers)
  bool busy = false;
};
// Status word shared by host and device: page-locked, device-mapped host memory.  Kernels write it
// only when something went wrong (a bounded wait ran out), so it costs nothing per launch, and the
// host reads it after the stream synchronised without a device-to-host copy.
void alloc_status_word(uint32_t **host, uint32_t **device);
void free_status_word(uint32_t *host);
// reads and clears the word; raises the matching error when a bit is set
void check_status_word(uint32_t *host, uint32_t *counters = nullptr);

// What a GEMV launch may use of its slot (or prepared object): the status word, and for the
// tensor-memory kernel the plane scratch and the ticket words.
struct GemvWorkspace {
  uint32_t *status = nullptr;
  void *scratch = nullptr;
  size_t scratch_bytes = 0;
  uint32_t *counters = nullptr;
};
inline GemvWorkspace gemv_workspace(const Slot &s) { return GemvWorkspace{s.status, s.scratch, s.scratch_bytes, s.counters}; }

struct ExecutorConfig {
  size_t n_slots = 2;
  uint32_t max_calls_per_submit = 16;
  bool tune = false;
};

struct PreparedOps;

// One batched matmul whose per-plane operands live in HOST memory (page-locked for overlap):
// C[b] = epilogue(alpha * A[b] @ B).  The planes are cut into chunks and pipelined through a
// ring of device staging sets on three streams, so that the host->device copies of chunk i+1,
// the GEMM of chunk i and the device->host copy of chunk i-1 run at the same time.
struct HostBatchedMatmul {
  uint32_t batch = 0, m = 0, n = 0, k = 0;
  const float *a = nullptr;        // host [batch, M, K]
  const Tensor *b = nullptr;       // device [K, N] (f32 or f16), shared by every plane; or
  const float *b_host = nullptr;   // host [K, N] f32, uploaded once per call
  float *c = nullptr;              // host [batch, M, N]
  const float *bias = nullptr;     // host [N] or [batch, N]
  bool bias_per_batch = false;
  const float *d = nullptr;        // host [batch, M, N] epilogue operand
  Activation activation = Activation::None;
  BinaryKind binary = BinaryKind::None;
  float alpha = 1.0f, beta = 0.0f;
  uint32_t chunk_batch = 0;        // planes per pipeline stage; 0: chosen by the library
};
struct HostStreamState;

class Executor {
 public:
  Executor(std::shared_ptr<Context> ctx, int selection, ExecutorConfig cfg);
  ~Executor();

  const std::shared_ptr<Context> &context() const { return ctx_; }

  void upload(const float *src, size_t len, const Tensor &dst);
  void upload_f16(const uint16_t *src, size_t len, const Tensor &dst);
  void download(const Tensor &src, float *dst, size_t len);

  RunStats run_matmuls(const std::vector<MatmulCall> &calls);
  RunStats run_ops(const std::vector<MatmulOp> &ops);
  RunStats run_op_graph(const std::vector<MatmulOp> &ops);
  RunStats run_matmuls_split_k2(const std::vector<MatmulCall> &calls, uint32_t splits);

  // Route a plain shape: explicit selection > tuned winner > heuristic
  // (src/pipeline/mod.rs:259-360, src/executor/mod.rs:145-218).
  Route plan_shape(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, bool b_f16,
                   bool allow_split_k2) const;
  Route plan_op(const MatmulOp &op, const ResolvedMatmul &r, bool allow_split_k2) const;
  // Fused attention (src/executor/elementwise/flash.rs:26-253, attn.rs:27-185).
  FlashParams plan_flash_attention(const Tensor &q, const Tensor &kt, const Tensor &v, const Tensor &out,
                                   const FlashAttentionDesc &desc) const;
  RunStats flash_attention(const Tensor &q, const Tensor &kt, const Tensor &v, const Tensor &out,
                           const FlashAttentionDesc &desc);
  AttnDecodeParams plan_attn_decode(const Tensor &q, const Tensor &kt, const Tensor &v,
                                    const Tensor &scratch, const Tensor &out, const AttnDecodeDesc &desc) const;
  RunStats attn_decode(const Tensor &q, const Tensor &kt, const Tensor &v, const Tensor &scratch,
                       const Tensor &out, const AttnDecodeDesc &desc);
  // Mixed graphs (src/executor/graph_ops.rs:249-353).  n_launches returns how
  // many kernels the op enqueues.
  Launch plan_exec_op(const ExecOp &op, uint64_t *flops, size_t *n_calls) const;
  Launch plan_exec_op_tail(const ExecOp &op, size_t *n_calls) const;
  RunStats run_exec_ops(const std::vector<ExecOp> &ops);
  RunStats run_single(const ExecOp &op);
  RunStats binary(const Tensor &a, const Tensor &b, const Tensor &out, uint32_t mode, float beta);
  RunStats rope_scatter(const Tensor &in, const Tensor &table, const Tensor &dst, uint32_t heads,
                        uint32_t head_dim, uint32_t rot_dim, uint32_t pos_base, uint32_t dst_offset,
                        const uint32_t strides[3], uint32_t pos_scale, const PosCell *cell);
  RunStats argmax(const Tensor &in, const PosCell &result);
  // launches the bounded-wait self-test kernel; always ends in the bounded-wait error
  void selftest_bounded_wait(uint32_t limit_ns);
  RunStats embed_gather(const PosCell &token, const Tensor &table, const Tensor &out);
  RunStats embed_gather_rows(const TokenIds &tokens, const Tensor &table, const Tensor &out);
  // scratch an op wants in its slot beyond split-K planes (the f16 copy of A for the f16w tensor-core GEMM)
  size_t op_scratch_bytes(const ResolvedMatmul &r, const Route &route) const;
  SplitK2TensorPlan splitk2_plan_for(const GemmParams &p, uint32_t splits) const;
  // `up` (plain) followed by `gate` = silu(A Wg) * up on the same A, both on the f16-weight tensor-core
  // route: the parameters of the one dual-matrix launch that computes both, or false
  bool dual_f16w_params(const MatmulOp &up, const MatmulOp &gate, GemmParams *out) const;
  size_t splitk2_scratch_bytes(const MatmulOp &op, const ResolvedMatmul &r, uint32_t splits) const;
  bool gemv_params_for(const MatmulOp &op, const ResolvedMatmul &r, const Route &route, GemvParams *out) const;
  // first_op (optional): for every planned launch, the index of the first op of `ops` it executes
  // exchange (optional): receives the fused exchange points of the plan; the caller advances them
  // before every submission
  std::vector<Launch> plan_exec_ops(const std::vector<ExecOp> &ops, uint64_t *flops, size_t *n_calls,
                                    size_t *scratch_bytes = nullptr, std::vector<size_t> *first_op = nullptr,
                                    ExchangeUse *exchange = nullptr) const;
  RunStats run_exec_ops_timed(const std::vector<ExecOp> &ops, std::vector<std::pair<size_t, uint64_t>> *per_launch);
  RunStats swiglu_gemv(const Tensor &x, const Tensor &wg, const Tensor &wup, const Tensor &out,
                       const Tensor *norm_w, float eps);
  void tune_shape(uint32_t batch, uint32_t m, uint32_t n, uint32_t k, bool b_f16 = false);
  // candidate kernels the tuner measures for a shape (src/pipeline/mod.rs:491-535)
  std::vector<int> tune_candidates(uint32_t m, uint32_t n, uint32_t k, bool b_f16) const;

  // Model ops (src/executor/elementwise/ops.rs).
  RunStats softmax_rows(const Tensor &in, const Tensor &out, float scale, uint32_t mask_kind,
                        uint32_t valid_or_prefix, uint32_t rows_per_group);
  RunStats rms_norm(const Tensor &in, const Tensor &w, const Tensor &out, float eps);
  RunStats layer_norm(const Tensor &in, const Tensor &w, const Tensor &b, const Tensor &out,
                      float eps);
  RunStats rope(const Tensor &in, const Tensor &table, const Tensor &out, uint32_t heads,
                uint32_t head_dim, uint32_t rot_dim, uint32_t pos_base);
  RunStats copy_strided(const Tensor &src, const Tensor &dst, const uint32_t extent[3],
                        uint32_t src_off, const uint32_t src_strides[3], uint32_t dst_off,
                        const uint32_t dst_strides[3]);

  void validate_tensor(const Tensor &t, const char *what) const;

  // Host-resident batched matmul, copies overlapped with compute (see HostBatchedMatmul).
  // gpu_time_ns spans the first upload to the last download.
  RunStats run_matmul_host_batched(const HostBatchedMatmul &desc);

  // Slot checkout (src/executor/submission.rs:37-53): blocks while all busy.
  Slot &checkout_slot();
  void release_slot(Slot &s);

  // Enqueue one validated op on a stream (no sync).  Used by run_* and by
  // graph capture.
  void enqueue_op(const MatmulOp &op, const ResolvedMatmul &r, const Route &route, Slot &slot,
                  cudaStream_t stream);
  void ensure_scratch(Slot &slot, size_t bytes);

  uint32_t max_calls() const { return cfg_.max_calls_per_submit; }
  int selection() const { return selection_; }

 private:
  friend struct PreparedOps;
  RunStats run_ops_impl(const std::vector<MatmulOp> &ops, bool graph);
  RunStats timed(Slot &slot, size_t n_calls, uint64_t flops, const std::function<void(cudaStream_t)> &record);
  friend std::unique_ptr<PreparedOps> prepare_exec_ops(Executor &exec, const std::vector<ExecOp> &ops);

  std::shared_ptr<Context> ctx_;
  int selection_;  // -2 auto, else registry index
  ExecutorConfig cfg_;
  std::vector<Slot> slots_;
  std::mutex mu_;
  std::condition_variable cv_;
  mutable std::mutex tune_mu_;
  mutable std::unordered_map<TuneKey, TunedEntry, TuneKeyHash> tuned_;
  std::string tune_path_;
  std::mutex host_stream_mu_;                     // one host-streamed call at a time per executor
  std::shared_ptr<HostStreamState> host_stream_;  // copy streams, events and the staging ring
};

// Device status word of a slot: bit 0 = a bounded wait inside a kernel ran out (a barrier, a copy),
// bit 2 = the peer exchange of a tensor-parallel all-reduce waited for a rank that did not arrive.
[[noreturn]] inline void fail_device_status(uint32_t status) {
  if (status & 8u)
    fail("a position cell held a position outside the cache / rope table a kernel addresses with it "
         "(status 0x%x); the kernel skipped those accesses, results are invalid", status);
  if (status & 4u)
    fail("a kernel gave up on a bounded device-side wait for a peer rank of the tensor-parallel exchange "
         "(status 0x%x); results are invalid", status);
  fail("a kernel gave up on a bounded device-side wait (status 0x%x); results are invalid", status);
}

// Launch with programmatic stream serialization: the kernel may be scheduled while its predecessor
// in the stream still runs and must execute TA_CHAIN_ENTER() before it touches global memory (the
// wait returns when the predecessor has completed and its writes are visible; the trigger lets the
// next kernel of the stream be scheduled in turn).  What is saved is the launch latency between
// dependent kernels of a chain.  In a kernel launched without the attribute both instructions do nothing.
#ifdef __CUDACC__
#define TA_CHAIN_ENTER()                                             \
  do {                                                               \
    asm volatile("griddepcontrol.wait;" ::: "memory");               \
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); \
  } while (0)
template <typename... P, typename... A>
inline void launch_chained(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tunables().pdl ? 1 : 0;
  TA_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...));
}
#endif

struct SlotGuard {
  Executor &e;
  Slot &s;
  SlotGuard(Executor &e_, Slot &s_) : e(e_), s(s_) {}
  ~SlotGuard() { e.release_slot(s); }
};
void validate_op_tensors(const Executor &e, const MatmulOp &op);

// Record-once / replay-many op batch (src/executor/prepared.rs:46-353).
struct PreparedOps {
  Executor *exec = nullptr;            // must outlive submit()/wait(); not needed to destroy
  std::shared_ptr<Context> ctx;        // keeps the device alive for the destructor
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t graph_exec = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev_begin = nullptr, ev_end = nullptr;
  void *scratch = nullptr;
  uint32_t *counters = nullptr;   // this object's own ticket words
  uint32_t *status = nullptr, *status_host = nullptr;   // this object's own status word (see Slot)
  ExchangeUse exchange;              // fused exchange points every submission of this object uses
  size_t n_calls = 0;
  uint64_t total_flops = 0;
  bool in_flight = false;

  ~PreparedOps();
  void submit();
  RunStats wait();
  RunStats run();
};
std::unique_ptr<PreparedOps> prepare_ops(Executor &exec, const std::vector<MatmulOp> &ops,
                                         bool as_graph);
std::unique_ptr<PreparedOps> prepare_exec_ops(Executor &exec, const std::vector<ExecOp> &ops);

// ------------------------------------------------------------------ kernel launchers
// Implemented beside each kernel.  All are asynchronous on `stream`.
void launch_gemm_ffma(const GemmParams &p, uint32_t tile, cudaStream_t stream);
bool gemm_tf32x3_eligible(const GemmParams &p);
bool gemm_tf32x3_pair_supported(const GemmParams &p, int sm_count);
void launch_gemm_tf32x3_pair(const Context &ctx, const GemmParams &p, uint32_t *status, cudaStream_t stream);
bool gemm_f16w_umma_eligible(const GemmParams &p);
uint32_t gemm_f16w_umma_tile_n(uint32_t batch, uint32_t m, uint32_t n, int sm_count);
size_t gemm_f16w_umma_scratch_bytes(uint32_t batch_a, uint32_t m, uint32_t k);
// a16 route (f16 A, f16 B, f16 C; M, N multiples of 64, K of 32; no fused epilogue): the same
// TMA -> tcgen05 pipeline reading A as stored, C rounded to f16 (nearest even) at the store
void launch_gemm_a16_umma(const Context &ctx, const GemmParams &p, uint32_t tile_n, uint32_t *status, cudaStream_t stream);
// scratch (may be null): room for the f16 copy of A; without it A is converted inside the kernel
// a16_ready: the scratch already holds this A (same pointer, M, K) from the launch just before
// counters (may be null): the slot's ticket words, needed for the in-kernel K split; auto_plan: the
// tile width came from the routing heuristic, so width and split are chosen together for the shape
void launch_gemm_f16w_umma(const Context &ctx, const GemmParams &p, uint32_t tile_n, uint32_t *status,
                           void *scratch, size_t scratch_bytes, bool a16_ready, cudaStream_t stream,
                           uint32_t *counters = nullptr, bool auto_plan = false);
void launch_gemm_tf32x3(const Context &ctx, const GemmParams &p, uint32_t tile_n, uint32_t *status,
                        cudaStream_t stream);
void launch_splitk2_stage1(const GemmParams &p, uint32_t tile, float *scratch, cudaStream_t stream);
// stage 1 on the tensor cores (plan.eligible) followed by the fixed-order reduce of plan.planes planes
void launch_gemm_tf32x3_ksplit(const Context &ctx, const GemmParams &p, const SplitK2TensorPlan &plan, float *scratch,
                               uint32_t *status, cudaStream_t stream);
void launch_splitk2_tensor(const Context &ctx, const GemmParams &p, const SplitK2TensorPlan &plan, float *scratch,
                           uint32_t *status, cudaStream_t stream);
// sum of `planes` planes per batch in plane order inside fixed groups, groups in order; launched so
// that it may be scheduled while the producer of the planes still runs (it waits for it on the device)
void launch_splitk2_reduce_wide(const float *scratch, float *c, uint64_t total, uint64_t mn, uint32_t planes,
                                cudaStream_t stream);
void launch_splitk2_reduce(const float *scratch, float *c, uint64_t total, uint64_t mn,
                           uint32_t splits, cudaStream_t stream);
// Split-K2 on the module's fixed scratch array: no allocation of any kind.
constexpr uint64_t SPLITK2_STATIC_MAX_FLOATS = 1ull << 20;  // 4 MiB
void launch_splitk2_static(const GemmParams &p, cudaStream_t stream);

bool gemv_f16w_supported(uint32_t m, uint32_t n, uint32_t k, bool packed, uint32_t tile_n);
void launch_gemv_f16w(const Context &ctx, GemvParams p, const GemvWorkspace &ws, cudaStream_t stream);
// tensor-memory kernel for 3..8 rows (k_gemv_umma.cu)
bool gemv_umma_eligible(const GemvParams &p);
bool gemv_routes_to_umma(const GemvParams &p);
size_t gemv_umma_scratch_bytes(uint32_t n, uint32_t k, bool dual, int sm_count);
void launch_gemv_umma(const Context &ctx, const GemvParams &p, float *scratch, size_t scratch_bytes, uint32_t *counters,
                      uint32_t *status, bool pdl, cudaStream_t stream);
bool gemv_f16w_groupable(const GemvParams &a, const GemvParams &b);
// peer (optional): the launch takes part in a fused tensor-parallel exchange (single-row GEMVs)
void launch_gemv_f16w_group(const Context &ctx, const GemvParams *segs, int nseg, bool pdl, const GemvWorkspace &ws,
                            cudaStream_t stream, const PeerLink *peer = nullptr);
// number of column tiles (= pushing CTAs) of a GEMV launch over these segments
uint32_t gemv_f16w_tiles(const GemvParams *segs, int nseg);

bool flash_prefill_mma_eligible(const FlashParams &p);   // the tensor-core kernel takes this problem (it alone writes out16)
void launch_flash_prefill(const FlashParams &p, cudaStream_t stream);
void launch_attn_decode(const AttnDecodeParams &p, cudaStream_t stream);

void launch_softmax_rows(const float *in, float *out, uint32_t rows, uint32_t cols, float scale,
                         uint32_t mask_kind, uint32_t valid_or_prefix, uint32_t rows_per_group,
                         cudaStream_t stream);
uint32_t gemm_f16w_umma_a16_pitch(uint32_t k);   // row pitch (halves) of the f16 copy of A that GEMM family reads
// out16 / pitch16: optional f16 mirror of the output (row pitch in halves; columns cols..pitch16-1 are zeroed)
void launch_rms_norm(const float *in, const float *w, float *out, uint32_t rows, uint32_t cols,
                     float eps, cudaStream_t stream, void *out16 = nullptr, uint32_t pitch16 = 0);
void launch_layer_norm(const float *in, const float *w, const float *b, float *out, uint32_t rows,
                       uint32_t cols, float eps, cudaStream_t stream);
void launch_rope(const float *in, const float *table, float *out, uint32_t tokens, uint32_t heads,
                 uint32_t head_dim, uint32_t rot_dim, uint32_t pos_base, cudaStream_t stream);
void launch_copy_strided(const void *src, bool src_f16, void *dst, bool dst_f16, const uint32_t extent[3],
                         uint32_t src_off, const uint32_t src_strides[3], uint32_t dst_off,
                         const uint32_t dst_strides[3], cudaStream_t stream);
void launch_binary(const float *a, const float *b, float *out, uint32_t n, uint32_t mode, float beta,
                   cudaStream_t stream);
void launch_argmax(const float *in, uint32_t n, uint32_t *result, cudaStream_t stream);
void launch_embed_gather(const uint32_t *tokens, uint32_t n_tokens, const void *table, bool table_f16,
                         float *out, uint32_t embd, uint32_t vocab, cudaStream_t stream);
void launch_prefill_qkv_pack(const float *qkv, const float *table, float *q, void *kt, void *v, bool kv_f16,
                             uint32_t tokens, uint32_t heads, uint32_t kv_heads, uint32_t head_dim,
                             uint32_t rot_dim, uint32_t pos_base, uint32_t t_max, cudaStream_t stream);
void launch_bounded_wait_probe(uint32_t *status, uint32_t limit_ns, cudaStream_t stream);
void launch_rope_scatter(const float *in, const float *table, void *dst, bool dst_f16, uint32_t tokens,
                         uint32_t heads, uint32_t head_dim, uint32_t rot_dim, uint32_t pos_base,
                         uint32_t dst_off, const uint32_t strides[3], uint32_t pos_scale,
                         const uint32_t *pos_ptr, cudaStream_t stream);

}  // namespace ta
