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
#include <dlfcn.h>

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
  return c;
}

Comm::~Comm() {
  if (handle) {
    if (ctx) cudaSetDevice(ctx->device);
    nccl().CommDestroy(handle);
  }
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
