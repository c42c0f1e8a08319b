// Collectives for the tensor-parallel decoder: a communicator over NCCL (NVLink /
// NVSwitch), one rank per process and GPU.  The reference is single-device; this
// is the exchange step the sharded llama graph needs after its row-parallel
// projections (sum all-reduce of [T, embd] f32) and for the sharded lm_head
// (all-gather of logit slices).
//
// NCCL is bound at run time with dlopen("libnccl.so.2"): the library keeps no
// link-time dependency on it and still loads on machines without NCCL or a GPU;
// creating a communicator there fails with a message.  In a process that already
// imported torch the loader hands back the NCCL torch ships, so both use one copy.
// Collectives are enqueued on the caller's stream and can be captured into CUDA
// graphs like any other node.
// Small all-reduces (a decode step's [1, embd] partial sums, 8 KB) do not go through
// NCCL: every rank owns an exchange buffer that all peers map (CUDA IPC over NVLink peer
// access), and one kernel per rank pushes its vector into every peer's buffer, raises a
// flag there, waits (bounded) for the peers' flags in its own buffer and adds the vectors
// in rank order.  One launch, one NVLink store latency; every rank computes the same sum
// in the same order, so the result is bit-identical across ranks.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "ta_core.hpp"

namespace ta {

namespace {

// Minimal restatement of the public NCCL C API used here (nccl.h).
struct NcclUniqueId { char internal[128]; };
using NcclComm = void *;
enum { NCCL_SUCCESS = 0 };
enum { NCCL_FLOAT32 = 7 };
enum { NCCL_SUM = 0 };

struct NcclApi {
  int (*GetUniqueId)(NcclUniqueId *) = nullptr;
  int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  std::string load_error;
  bool ok = false;
};

NcclApi &nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
      api.load_error = dlerror() ? dlerror() : "libnccl.so.2 not found";
      return;
    }
    auto sym = [&](const char *name) { return dlsym(h, name); };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.AllGather;
    if (!api.ok) api.load_error = "libnccl.so.2 lacks an expected symbol";
  });
  return api;
}

void nccl_check(int rc, const char *what) {
  if (rc == NCCL_SUCCESS) return;
  NcclApi &api = nccl();
  fail("%s failed: NCCL error %d (%s)", what, rc, api.GetErrorString ? api.GetErrorString(rc) : "?");
}

NcclApi &nccl_required() {
  NcclApi &api = nccl();
  if (!api.ok) fail("NCCL is unavailable: %s", api.load_error.c_str());
  return api;
}

}  // namespace

// ------------------------------------------------------------------ peer-write all-reduce
// Exchange buffer of one rank: data[2 parities][world][PEER_MAX_FLOATS] then
// flags[2][world][PEER_MAX_CTAS] then epoch[PEER_MAX_CTAS] (this rank's call counters).
constexpr uint32_t PEER_MAX_CTAS = 8, PEER_THREADS = 256;
constexpr size_t PEER_DATA_BYTES = PEER_AR_DATA_BYTES;
constexpr size_t PEER_FLAG_BYTES = PEER_AR_FLAG_BYTES;
static_assert(PEER_AR_FLAG_BYTES == 2ull * PEER_MAX_WORLD * PEER_MAX_CTAS * sizeof(uint32_t), "flag layout");
static_assert(PEER_AR_BYTES % 16 == 0 && PEER_AR_BYTES >= PEER_DATA_BYTES + PEER_FLAG_BYTES + PEER_MAX_CTAS * sizeof(uint32_t), "layout");
constexpr size_t PEER_BUF_BYTES = PEER_BUF_TOTAL;   // all-reduce kernel region + fused-exchange region

struct PeerTable {
  uint8_t *buf[PEER_MAX_WORLD];   // every rank's exchange buffer as mapped in this process
  uint32_t rank, world;
};

__device__ __forceinline__ float *peer_data(uint8_t *buf, uint32_t parity, uint32_t src) {
  return reinterpret_cast<float *>(buf) + ((size_t)parity * PEER_MAX_WORLD + src) * PEER_MAX_FLOATS;
}
__device__ __forceinline__ uint32_t *peer_flag(uint8_t *buf, uint32_t parity, uint32_t src, uint32_t cta) {
  return reinterpret_cast<uint32_t *>(buf + PEER_DATA_BYTES) + ((size_t)parity * PEER_MAX_WORLD + src) * PEER_MAX_CTAS + cta;
}

// CTA c of every rank handles floats [c * 1024, (c + 1) * 1024) and synchronises only with CTA c
// of the peers.  Call e of a CTA uses parity e & 1: a rank can be at most one call ahead of a
// peer (it needs the peer's flag of call e to finish call e), so the slot a peer still reads
// is never the one being written.
__global__ void __launch_bounds__(PEER_THREADS)
peer_all_reduce_kernel(float *data, uint32_t count, PeerTable t, uint32_t *status, uint32_t pdl, uint64_t limit_ns) {
  if (pdl) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }
  const uint32_t cta = blockIdx.x, me = t.rank;
  uint8_t *mine = t.buf[me];
  uint32_t *epoch_p = reinterpret_cast<uint32_t *>(mine + PEER_DATA_BYTES + PEER_FLAG_BYTES) + cta;
  const uint32_t e = *epoch_p, parity = e & 1u, ticket = e + 1u;
  const uint32_t idx = (cta * PEER_THREADS + threadIdx.x) * 4;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool live = idx < count;   // count % 4 == 0
  if (live) {
    v = *reinterpret_cast<const float4 *>(data + idx);
    for (uint32_t r = 0; r < t.world; ++r)
      if (r != me) *reinterpret_cast<float4 *>(peer_data(t.buf[r], parity, me) + idx) = v;
  }
  __threadfence_system();
  __syncthreads();
  __shared__ uint32_t ok_flag;
  if (threadIdx.x == 0) ok_flag = 1u;
  __syncthreads();
  if (threadIdx.x < t.world && threadIdx.x != me) {
    const uint32_t r = threadIdx.x;
    // raise my flag in peer r's buffer, then wait for peer r's flag in mine
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flag(t.buf[r], parity, me, cta)), "r"(ticket) : "memory");
    const uint32_t *f = peer_flag(mine, parity, r, cta);
    uint64_t t0, now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    uint32_t seen = 0, spins = 0;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
      if (seen == ticket) break;
      if ((++spins & 255u) == 0) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (now - t0 > limit_ns) {   // give up, report, carry on with what is there
          ok_flag = 0u;
          break;
        }
      }
    }
  }
  __syncthreads();
  if (live) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t r = 0; r < t.world; ++r) {   // rank order: the same sum on every rank
      float4 x = v;
      if (r != me) x = __ldcg(reinterpret_cast<const float4 *>(peer_data(mine, parity, r) + idx));
      acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    *reinterpret_cast<float4 *>(data + idx) = acc;
  }
  if (threadIdx.x == 0) {
    *epoch_p = ticket;
    if (!ok_flag && status) atomicOr(status, 4u);
  }
}

// ------------------------------------------------------------------ two-step all-reduce (prefill activations)
// A [T, embd] activation of a prefill step is a few MB: too large for the one-launch kernel above.
// This kernel is an experiment switch (peer_allreduce_big), off by default: with its two system-scope
// fences per call it measured slower than NCCL at this size (512-token prefill of the 1.1 B model on
// 4 GPUs: 4.25 ms against 3.85 ms), so NCCL carries these tensors.  The tensor is cut into
// `world` slices; rank r owns slice r.  CTA b of every rank handles part b of every slice and
// synchronises only with CTA b of the peers, through two flag words per (rank, CTA):
//   step 1  push my values of slice s into rank s's `in` region, for every s != me; raise flag 1 there;
//   step 2  wait for the peers' flag 1; add the `world` versions of my own slice in rank order (mine
//           from the tensor itself), write the sum into the tensor and into every peer's `out`
//           region; raise flag 2 there;
//   step 3  wait for the peers' flag 2; copy their reduced slices from my `out` region into the tensor.
// Every rank adds in the same order: results are bit-identical across ranks.  Flags carry a per-CTA
// call count kept in the rank's own buffer, so no host word is involved; waits are bounded.
// A rank enters call e + 1 only after it has read every peer's step-2 push of call e, i.e. after
// every peer finished reading its `in` region: one buffer per region is enough.
__global__ void __launch_bounds__(256)
peer_all_reduce_big_kernel(float *data, uint32_t count, uint32_t slice, uint32_t part, PeerTable t, uint32_t *status,
                           uint64_t limit_ns) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t b = blockIdx.x, me = t.rank, W = t.world;
  uint8_t *mine = t.buf[me];
  uint32_t *epoch_p = reinterpret_cast<uint32_t *>(mine + PEER_BIG_EPOCH_OFF) + b;
  const uint32_t ticket = *epoch_p + 1u;
  auto in_of = [&](uint32_t owner, uint32_t src) { return reinterpret_cast<float *>(t.buf[owner] + PEER_BIG_IN_OFF) + (size_t)src * slice; };
  auto out_of = [&](uint32_t owner, uint32_t s) { return reinterpret_cast<float *>(t.buf[owner] + PEER_BIG_OUT_OFF) + (size_t)s * slice; };
  auto flag_of = [&](uint32_t owner, uint32_t step, uint32_t src) {
    return reinterpret_cast<uint32_t *>(t.buf[owner] + PEER_BIG_FLAG_OFF) + ((size_t)step * PEER_MAX_WORLD + src) * PEER_BIG_CTAS + b;
  };
  __shared__ uint32_t ok_flag;
  if (threadIdx.x == 0) ok_flag = 1u;
  const uint32_t lo = b * part, hi = min(slice, lo + part);     // this CTA's range inside a slice (multiples of 4)
  auto wait_peers = [&](uint32_t step) {
    if (threadIdx.x < W && threadIdx.x != me) {
      const uint32_t *f = flag_of(me, step, threadIdx.x);
      uint64_t t0, now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
      uint32_t seen = 0, spins = 0;
      for (;;) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
        if (seen == ticket) break;
        if ((++spins & 255u) == 0) {
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
          if (now - t0 > limit_ns) { ok_flag = 0u; break; }
        }
      }
    }
    __syncthreads();
  };
  auto raise = [&](uint32_t step) {     // after this CTA's pushes: visible system-wide, then one flag per peer
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < W && threadIdx.x != me)
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag_of(threadIdx.x, step, me)), "r"(ticket) : "memory");
  };
  // ---- step 1
  for (uint32_t s = 0; s < W; ++s) {
    if (s == me) continue;
    float *dst = in_of(s, me);
    for (uint32_t i = lo + threadIdx.x * 4; i < hi; i += 256 * 4) {
      const size_t g = (size_t)s * slice + i;
      if (g < count) *reinterpret_cast<float4 *>(dst + i) = *reinterpret_cast<const float4 *>(data + g);
    }
  }
  raise(0);
  // ---- step 2
  wait_peers(0);
  for (uint32_t i = lo + threadIdx.x * 4; i < hi; i += 256 * 4) {
    const size_t g = (size_t)me * slice + i;
    if (g >= count) continue;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t r = 0; r < W; ++r) {
      const float4 x = r == me ? *reinterpret_cast<const float4 *>(data + g)
                               : __ldcg(reinterpret_cast<const float4 *>(in_of(me, r) + i));
      acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    *reinterpret_cast<float4 *>(data + g) = acc;
    for (uint32_t r = 0; r < W; ++r)
      if (r != me) *reinterpret_cast<float4 *>(out_of(r, me) + i) = acc;
  }
  raise(1);
  // ---- step 3
  wait_peers(1);
  for (uint32_t s = 0; s < W; ++s) {
    if (s == me) continue;
    const float *src = out_of(me, s);
    for (uint32_t i = lo + threadIdx.x * 4; i < hi; i += 256 * 4) {
      const size_t g = (size_t)s * slice + i;
      if (g < count) *reinterpret_cast<float4 *>(data + g) = __ldcg(reinterpret_cast<const float4 *>(src + i));
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *epoch_p = ticket;
    if (!ok_flag && status) atomicOr(status, 4u);
  }
}

bool Comm::peer_all_reduce_big(float *data, size_t count, uint32_t *status, cudaStream_t stream) const {
  if (!tunables().peer_allreduce_big || !peer_own || count == 0 || count > PEER_BIG_MAX_FLOATS || (count & 3u) ||
      (reinterpret_cast<uintptr_t>(data) & 15u))
    return false;
  PeerTable t{};
  for (uint32_t r = 0; r < world; ++r) t.buf[r] = static_cast<uint8_t *>(peer_bufs[r]);
  t.rank = rank;
  t.world = world;
  const uint32_t slice = (uint32_t)(((count + world - 1) / world + 3) & ~(size_t)3);        // floats per rank, a multiple of 4
  const uint32_t part = ((slice + PEER_BIG_CTAS - 1) / PEER_BIG_CTAS + 3) & ~3u;           // floats per CTA within a slice
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(PEER_BIG_CTAS, 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TA_CUDA(cudaLaunchKernelEx(&cfg, peer_all_reduce_big_kernel, data, (uint32_t)count, slice, part, t, status, peer_wait_limit_ns));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return true;
}

// ------------------------------------------------------------------ sharded argmax
// Greedy pick over a vocabulary whose logits are split by column over the ranks: every rank folds
// its own slice to one (value, global index) pair, pushes the pair into every rank's buffer, waits
// (bounded) for the others' pairs and folds the `world` pairs in rank order with the same rule as
// the single-device kernel -- the maximum, ties to the LARGEST index
// (shaders/op_argmax_f32.comp:44-75) -- so that all ranks write the same token.  One launch per
// rank; replaces gathering the whole vocabulary.  NaNs never win.
constexpr int AMAX_THREADS = 1024;
__device__ __forceinline__ void amax_fold(float &bv, uint32_t &bi, float v, uint32_t i) {
  if (v > bv || (v == bv && i > bi)) {
    bv = v;
    bi = i;
  }
}
__global__ void __launch_bounds__(AMAX_THREADS)
argmax_sharded_kernel(const float *__restrict__ in, uint32_t n, uint32_t index_offset, PeerLink l, uint32_t *result,
                      uint32_t *status, uint32_t pdl) {
  __shared__ float sval[AMAX_THREADS / 32];
  __shared__ uint32_t sidx[AMAX_THREADS / 32];
  const uint32_t tid = threadIdx.x;
  const uint32_t step = *l.expect_ptr;    // arrivals word of the pair exchange: host-advanced, staged to the device by the submission
  if (pdl) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }
  float bv = -INFINITY;
  uint32_t bi = 0;
  for (uint32_t i = tid; i < n; i += AMAX_THREADS) amax_fold(bv, bi, in[i], i);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
    amax_fold(bv, bi, ov, oi);
  }
  if ((tid & 31u) == 0) {
    sval[tid >> 5] = bv;
    sidx[tid >> 5] = bi;
  }
  __syncthreads();
  if (tid < 32) {
    bv = sval[tid];
    bi = sidx[tid];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
      amax_fold(bv, bi, ov, oi);
    }
    // lanes 0 .. world-1: lane r hands this rank's pair to rank r, then raises the arrival word there
    if (tid < l.world) {
      // pairs alternate between two slots by use parity: a rank can be one use ahead of a peer, never two
      uint2 *pair = reinterpret_cast<uint2 *>(l.buf[tid] + PEER_AMAX_PAIR_OFF) + (step & 1u) * PEER_MAX_WORLD + l.rank;
      uint32_t *flag = reinterpret_cast<uint32_t *>(l.buf[tid] + PEER_AMAX_FLAG_OFF) + l.rank;
      *pair = make_uint2(__float_as_uint(bv), bi + index_offset);
      __threadfence_system();
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(step) : "memory");
      // ... and waits for rank r's pair in this rank's own buffer
      const uint32_t *mine = reinterpret_cast<const uint32_t *>(l.buf[l.rank] + PEER_AMAX_FLAG_OFF) + tid;
      const uint64_t t0 = [] { uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }();
      uint32_t seen = 0, spins = 0;
      for (;;) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if ((int32_t)(seen - step) >= 0) break;
        if ((++spins & 255u) == 0) {
          uint64_t now;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
          if (now - t0 > l.limit_ns) {
            if (status) atomicOr(status, 4u);
            break;
          }
        }
      }
    }
    __syncwarp();
    if (tid == 0) {
      float fv = -INFINITY;
      uint32_t fi = 0;
      for (uint32_t r = 0; r < l.world; ++r) {   // rank order; the fold is order-independent anyway
        const uint2 pr = __ldcg(reinterpret_cast<const uint2 *>(l.buf[l.rank] + PEER_AMAX_PAIR_OFF) + (step & 1u) * PEER_MAX_WORLD + r);
        amax_fold(fv, fi, __uint_as_float(pr.x), pr.y);
      }
      *result = fi;
    }
  }
}

bool Comm::argmax_sharded(const float *in, uint32_t n, uint32_t index_offset, uint32_t *result, uint32_t *status,
                          cudaStream_t stream) const {
  if (!fused_exchange_ready() || world < 2 || world > PEER_MAX_WORLD) return false;
  PeerLink l = link();
  l.expect_ptr = expect_copy + PEER_MAX_POINTS;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, 1, 1);
  cfg.blockDim = dim3(AMAX_THREADS, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TA_CUDA(cudaLaunchKernelEx(&cfg, argmax_sharded_kernel, in, n, index_offset, l, result, status, 1u));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return true;
}

void comm_unique_id(uint8_t out[COMM_ID_BYTES]) {
  static_assert(COMM_ID_BYTES == sizeof(NcclUniqueId), "id size");
  NcclUniqueId id;
  nccl_check(nccl_required().GetUniqueId(&id), "ncclGetUniqueId");
  memcpy(out, &id, sizeof(id));
}

std::unique_ptr<Comm> Comm::create(const std::shared_ptr<Context> &ctx, uint32_t rank, uint32_t world,
                                   const uint8_t id_bytes[COMM_ID_BYTES]) {
  if (world == 0 || rank >= world) fail("ta_comm_create: rank %u is outside world %u", rank, world);
  auto c = std::make_unique<Comm>();
  c->ctx = ctx;
  c->rank = rank;
  c->world = world;
  if (world == 1) return c;   // no exchange needed: collectives are no-ops / copies
  NcclApi &api = nccl_required();
  ctx->make_current();
  NcclUniqueId id;
  memcpy(&id, id_bytes, sizeof(id));
  nccl_check(api.CommInitRank(&c->handle, (int)world, id, (int)rank), "ncclCommInitRank");
  c->setup_peer_exchange();
  return c;
}

// Maps every rank's exchange buffer into this process: IPC handles travel through an
// NCCL all-gather.  Any failure (no peer access, IPC unavailable) leaves the communicator
// on NCCL for all sizes.
void Comm::setup_peer_exchange() {
  // Every rank takes part in both collectives below whatever happened locally: a rank that cannot
  // (or is told not to) use the peer path carries a failure flag through them, so that no rank is
  // left waiting inside NCCL for one that returned early.
  bool ok = tunables().peer_allreduce && world <= PEER_MAX_WORLD;
  NcclApi &api = nccl();
  void *buf = nullptr;
  cudaIpcMemHandle_t mine;
  memset(&mine, 0, sizeof(mine));
  if (ok && cudaMalloc(&buf, PEER_BUF_BYTES) != cudaSuccess) { cudaGetLastError(); buf = nullptr; ok = false; }
  if (ok) cudaMemset(buf, 0, PEER_BUF_BYTES);
  if (ok && cudaIpcGetMemHandle(&mine, buf) != cudaSuccess) { cudaGetLastError(); ok = false; }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "ipc handle size");
  uint8_t *dev_handles = nullptr;   // [world + 1][64]: slot world holds this rank's handle and an ok byte
  TA_CUDA(cudaMalloc((void **)&dev_handles, (size_t)(world + 1) * 64));
  TA_CUDA(cudaMemcpy(dev_handles + (size_t)world * 64, &mine, 64, cudaMemcpyHostToDevice));
  cudaStream_t st;
  TA_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  nccl_check(api.AllGather(dev_handles + (size_t)world * 64, dev_handles, 16, NCCL_FLOAT32, handle, st),
             "ncclAllGather (ipc handles)");
  TA_CUDA(cudaStreamSynchronize(st));
  std::vector<cudaIpcMemHandle_t> all(world);
  TA_CUDA(cudaMemcpy(all.data(), dev_handles, (size_t)world * 64, cudaMemcpyDeviceToHost));
  cudaFree(dev_handles);
  std::vector<void *> mapped(world, nullptr);
  for (uint32_t r = 0; r < world && ok; ++r) {
    if (r == rank) { mapped[r] = buf; continue; }
    if (cudaIpcOpenMemHandle(&mapped[r], all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      cudaGetLastError();
      ok = false;
    }
  }
  // all ranks must agree: sum of failures over the group
  float *flag_dev = nullptr;
  TA_CUDA(cudaMalloc((void **)&flag_dev, sizeof(float)));
  const float bad = ok ? 0.0f : 1.0f;
  TA_CUDA(cudaMemcpy(flag_dev, &bad, sizeof(float), cudaMemcpyHostToDevice));
  nccl_check(api.AllReduce(flag_dev, flag_dev, 1, NCCL_FLOAT32, NCCL_SUM, handle, st), "ncclAllReduce (peer setup)");
  TA_CUDA(cudaStreamSynchronize(st));
  float total_bad = 0.0f;
  TA_CUDA(cudaMemcpy(&total_bad, flag_dev, sizeof(float), cudaMemcpyDeviceToHost));
  cudaFree(flag_dev);
  cudaStreamDestroy(st);
  if (total_bad != 0.0f) {
    for (uint32_t r = 0; r < world; ++r)
      if (r != rank && mapped[r]) cudaIpcCloseMemHandle(mapped[r]);
    if (buf) cudaFree(buf);
    return;
  }
  peer_own = buf;
  peer_bufs = mapped;
  if (cudaHostAlloc((void **)&expect_host, (PEER_MAX_POINTS + 1) * sizeof(uint32_t), cudaHostAllocDefault) == cudaSuccess) {
    memset(expect_host, 0, (PEER_MAX_POINTS + 1) * sizeof(uint32_t));
    if (cudaMalloc((void **)&expect_copy, (PEER_MAX_POINTS + 1) * sizeof(uint32_t)) != cudaSuccess) {
      cudaGetLastError();
      expect_copy = nullptr;
    } else {
      cudaMemset(expect_copy, 0, (PEER_MAX_POINTS + 1) * sizeof(uint32_t));
    }
  } else {
    cudaGetLastError();
    expect_host = nullptr;
  }
}

PeerLink Comm::link() const {
  PeerLink l{};
  for (uint32_t r = 0; r < world && r < PEER_MAX_WORLD; ++r) l.buf[r] = static_cast<uint8_t *>(peer_bufs[r]);
  l.rank = rank;
  l.world = world;
  l.expect_base = expect_copy;
  l.expect_ptr = nullptr;
  l.limit_ns = peer_wait_limit_ns;
  return l;
}

bool Comm::peer_all_reduce_sum(float *data, size_t count, uint32_t *status, bool pdl, cudaStream_t stream) const {
  if (!peer_own || count == 0 || count > PEER_MAX_FLOATS || (count & 3u) ||
      (reinterpret_cast<uintptr_t>(data) & 15u))
    return false;
  PeerTable t{};
  for (uint32_t r = 0; r < world; ++r) t.buf[r] = static_cast<uint8_t *>(peer_bufs[r]);
  t.rank = rank;
  t.world = world;
  const uint32_t ctas = (uint32_t)((count / 4 + PEER_THREADS - 1) / PEER_THREADS);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas, 1, 1);
  cfg.blockDim = dim3(PEER_THREADS, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  TA_CUDA(cudaLaunchKernelEx(&cfg, peer_all_reduce_kernel, data, (uint32_t)count, t, status, pdl ? 1u : 0u, peer_wait_limit_ns));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return true;
}

// Collective: every rank of the group calls it.  Brings the peer exchange back to a common state
// after a rank gave up on a wait (status bit 2): all ranks meet in NCCL, each zeroes its own
// flags and call counters, and they meet again before anyone pushes.
void Comm::resync() {
  if (world == 1 || !handle) return;
  ctx->make_current();
  TA_CUDA(cudaDeviceSynchronize());
  float *word = nullptr;
  TA_CUDA(cudaMalloc((void **)&word, sizeof(float)));
  TA_CUDA(cudaMemset(word, 0, sizeof(float)));
  cudaStream_t st;
  TA_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  for (int pass = 0; pass < 2; ++pass) {
    nccl_check(nccl().AllReduce(word, word, 1, NCCL_FLOAT32, NCCL_SUM, handle, st), "ncclAllReduce (resync)");
    TA_CUDA(cudaStreamSynchronize(st));
    if (pass == 0 && peer_own) {
      TA_CUDA(cudaMemset(static_cast<uint8_t *>(peer_own) + PEER_DATA_BYTES, 0, PEER_BUF_BYTES - PEER_DATA_BYTES));
      TA_CUDA(cudaDeviceSynchronize());
      if (expect_host) memset(expect_host, 0, (PEER_MAX_POINTS + 1) * sizeof(uint32_t));
      if (expect_copy) TA_CUDA(cudaMemset(expect_copy, 0, (PEER_MAX_POINTS + 1) * sizeof(uint32_t)));
    }
  }
  cudaStreamDestroy(st);
  cudaFree(word);
}

Comm::~Comm() {
  if (ctx) cudaSetDevice(ctx->device);
  if (peer_own) {
    cudaDeviceSynchronize();
    for (uint32_t r = 0; r < world; ++r)
      if (r != rank && r < peer_bufs.size() && peer_bufs[r]) cudaIpcCloseMemHandle(peer_bufs[r]);
    cudaFree(peer_own);
  }
  if (expect_host) cudaFreeHost(expect_host);
  if (expect_copy) cudaFree(expect_copy);
  if (handle) nccl().CommDestroy(handle);
}

void Comm::all_reduce_sum(float *data, size_t count, cudaStream_t stream) const {
  if (world == 1 || count == 0) return;
  nccl_check(nccl().AllReduce(data, data, count, NCCL_FLOAT32, NCCL_SUM, handle, stream), "ncclAllReduce");
}

void Comm::all_gather(const float *src, float *dst, size_t count_per_rank, cudaStream_t stream) const {
  if (count_per_rank == 0) return;
  if (world == 1) {
    if (src != dst)
      TA_CUDA(cudaMemcpyAsync(dst, src, count_per_rank * sizeof(float), cudaMemcpyDeviceToDevice, stream));
    return;
  }
  nccl_check(nccl().AllGather(src, dst, count_per_rank, NCCL_FLOAT32, handle, stream), "ncclAllGather");
}

}  // namespace ta
