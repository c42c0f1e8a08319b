// Host-resident batched matmul: the end-to-end form of the batched GEMM path, for callers whose
// operands and results live in host memory (the reference's upload -> run -> download sequence,
// src/executor/transfer.rs:21-84 + src/executor/dispatch.rs, collapsed into one call).
//
// PCIe is full duplex and the copy engines run beside the SMs, so the three phases of a serial
// upload/run/download overlap almost completely once the batch is cut into chunks:
//
//   h2d stream   : A[i+1], D[i+1], bias[i+1]  ->  staging set (i+1) % RING
//   slot stream  : GEMM + fused epilogue of chunk i          (same kernels, same routing)
//   d2h stream   : C[i-1]                     ->  host
//
// Ordering is by events only; the host enqueues every chunk up front and waits once at the end.
// Each chunk is computed by exactly the kernel the device-resident path would pick for the chunk
// shape, so results are bit-identical to upload/run_ops/download applied chunk by chunk.
#include <algorithm>

#include "ta_core.hpp"

namespace ta {

constexpr int HOST_RING = 3;

struct HostStreamState {
  std::shared_ptr<Context> ctx;
  cudaStream_t h2d = nullptr, d2h = nullptr;
  cudaEvent_t ev_begin = nullptr, ev_end = nullptr, ev_b = nullptr;
  cudaEvent_t ev_up[HOST_RING] = {}, ev_comp[HOST_RING] = {}, ev_down[HOST_RING] = {};
  // staging ring, reallocated only when a call needs a different chunk geometry
  uint32_t cb = 0, m = 0, n = 0, k = 0;
  bool has_d = false, has_bias = false;
  Tensor a[HOST_RING], d[HOST_RING], c[HOST_RING], bias[HOST_RING];
  Tensor b_stage;   // [K, N] f32 when B comes from the host

  ~HostStreamState() {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (h2d) cudaStreamSynchronize(h2d);
    if (d2h) cudaStreamSynchronize(d2h);
    for (cudaEvent_t e : {ev_begin, ev_end, ev_b})
      if (e) cudaEventDestroy(e);
    for (int i = 0; i < HOST_RING; ++i)
      for (cudaEvent_t e : {ev_up[i], ev_comp[i], ev_down[i]})
        if (e) cudaEventDestroy(e);
    if (h2d) cudaStreamDestroy(h2d);
    if (d2h) cudaStreamDestroy(d2h);
  }
};

namespace {

Tensor device_f32(const std::shared_ptr<Context> &ctx, std::initializer_list<uint32_t> shape) {
  std::vector<uint32_t> s(shape);
  return Tensor::uninit_device(ctx, s.data(), s.size(), DType::F32);
}

// The first `planes` planes of a staging tensor whose leading dimension is the chunk size.
Tensor leading(const Tensor &t, uint32_t planes) {
  Tensor v = t;
  v.shape[0] = planes;
  return v;
}

}  // namespace

RunStats Executor::run_matmul_host_batched(const HostBatchedMatmul &h) {
  const char *nm = "run_matmul_host_batched";
  if (!h.batch || !h.m || !h.n || !h.k) fail("%s: batch, M, N and K must be non-zero", nm);
  if (!h.a || !h.c) fail("%s: host A and host C are required", nm);
  if (!h.b == !h.b_host) fail("%s: exactly one of a device B tensor and a host B pointer is required", nm);
  if (h.binary != BinaryKind::None && !h.d) fail("%s: a binary epilogue needs the host operand D", nm);
  if (h.binary == BinaryKind::None && h.d) fail("%s: host operand D given without a binary epilogue", nm);
  if ((uint64_t)h.m * h.k > 0xffffffffull || (uint64_t)h.m * h.n > 0xffffffffull)
    fail("%s: a plane of %u x %u x %u exceeds the u32 plane stride", nm, h.m, h.n, h.k);
  if (h.b) {
    validate_tensor(*h.b, "matmul B");
    if (h.b->shape != std::vector<uint32_t>{h.k, h.n})
      fail("%s: device B must be [K=%u, N=%u], got %s", nm, h.k, h.n, h.b->shape_str().c_str());
  }
  ctx_->make_current();
  std::lock_guard<std::mutex> call_lock(host_stream_mu_);
  if (!host_stream_) {
    auto st = std::make_shared<HostStreamState>();
    st->ctx = ctx_;
    TA_CUDA(cudaStreamCreateWithFlags(&st->h2d, cudaStreamNonBlocking));
    TA_CUDA(cudaStreamCreateWithFlags(&st->d2h, cudaStreamNonBlocking));
    TA_CUDA(cudaEventCreate(&st->ev_begin));
    TA_CUDA(cudaEventCreate(&st->ev_end));
    TA_CUDA(cudaEventCreateWithFlags(&st->ev_b, cudaEventDisableTiming));
    for (int i = 0; i < HOST_RING; ++i) {
      TA_CUDA(cudaEventCreateWithFlags(&st->ev_up[i], cudaEventDisableTiming));
      TA_CUDA(cudaEventCreateWithFlags(&st->ev_comp[i], cudaEventDisableTiming));
      TA_CUDA(cudaEventCreateWithFlags(&st->ev_down[i], cudaEventDisableTiming));
    }
    host_stream_ = st;
  }
  HostStreamState &st = *host_stream_;

  // Chunk size: enough chunks that pipeline fill and drain are a small part of the call, but not
  // so few planes that a chunk cannot fill the SMs.  An explicit request is honoured as is.
  uint32_t cb = h.chunk_batch;
  if (!cb) {
    cb = std::max(1u, h.batch / 16);
    const uint64_t plane_bytes = 4ull * ((uint64_t)h.m * h.k + 2ull * h.m * h.n);
    while (cb > 1 && (uint64_t)cb * plane_bytes > (512ull << 20)) cb /= 2;   // staging ring <= 1.5 GiB
  }
  cb = std::min(cb, h.batch);
  const bool has_d = h.d != nullptr, has_bias = h.bias != nullptr;
  if (st.cb != cb || st.m != h.m || st.n != h.n || st.k != h.k || (has_d && !st.has_d) ||
      (has_bias && !st.has_bias)) {
    TA_CUDA(cudaStreamSynchronize(st.h2d));
    TA_CUDA(cudaStreamSynchronize(st.d2h));
    for (int i = 0; i < HOST_RING; ++i) {
      st.a[i] = device_f32(ctx_, {cb, h.m, h.k});
      st.c[i] = device_f32(ctx_, {cb, h.m, h.n});
      st.d[i] = has_d ? device_f32(ctx_, {cb, h.m, h.n}) : Tensor{};
      st.bias[i] = has_bias ? device_f32(ctx_, {cb, h.n}) : Tensor{};
    }
    st.cb = cb; st.m = h.m; st.n = h.n; st.k = h.k; st.has_d = has_d; st.has_bias = has_bias;
  }
  const Tensor *b = h.b;
  if (h.b_host) {
    if (!st.b_stage.buf || st.b_stage.shape != std::vector<uint32_t>{h.k, h.n}) st.b_stage = device_f32(ctx_, {h.k, h.n});
    b = &st.b_stage;
  }

  // Plan both chunk shapes (full and ragged tail) before anything is enqueued.
  const uint32_t n_chunks = (h.batch + cb - 1) / cb, tail = h.batch - (n_chunks - 1) * cb;
  struct Planned {
    Tensor a, c, d, bias;
    MatmulOp op;
    ResolvedMatmul r;
    Route route;
  };
  std::vector<Planned> plan((size_t)HOST_RING * 2);   // [set][0 = full chunk, 1 = tail chunk]
  size_t scratch_bytes = 0;
  uint64_t flops = 0;
  for (int s = 0; s < HOST_RING; ++s)
    for (int t = 0; t < 2; ++t) {
      const uint32_t planes = t ? tail : cb;
      Planned &p = plan[(size_t)s * 2 + t];
      p.a = leading(st.a[s], planes);
      p.c = leading(st.c[s], planes);
      p.op.call.a = &p.a; p.op.call.b = b; p.op.call.c = &p.c;
      p.op.call.alpha = h.alpha;
      p.op.epilogue.activation = h.activation;
      p.op.epilogue.binary = h.binary;
      p.op.epilogue.beta = h.beta;
      if (has_d) {
        p.d = leading(st.d[s], planes);
        p.op.epilogue.d = &p.d;
      }
      if (has_bias) {
        if (h.bias_per_batch) {
          p.bias = leading(st.bias[s], planes);
        } else {
          p.bias = st.bias[s];
          p.bias.shape = {h.n};
        }
        p.op.epilogue.bias = &p.bias;
      }
      validate_op_tensors(*this, p.op);
      p.r = ResolvedMatmul::from_op(p.op);
      p.route = plan_op(p.op, p.r, false);
      if (p.route.splits > 1) fail("%s: internal error, split-K route chosen for a chunk", nm);
      scratch_bytes = std::max(scratch_bytes, op_scratch_bytes(p.r, p.route));
    }
  flops = 2ull * h.batch * h.m * h.n * h.k;

  Slot &slot = checkout_slot();
  SlotGuard guard(*this, slot);
  if (scratch_bytes) ensure_scratch(slot, scratch_bytes);
  cudaStream_t comp = slot.stream;

  const size_t a_plane = (size_t)h.m * h.k, c_plane = (size_t)h.m * h.n;
  TA_CUDA(cudaEventRecord(st.ev_begin, st.h2d));
  if (h.b_host) {
    TA_CUDA(cudaMemcpyAsync(st.b_stage.ptr(), h.b_host, (size_t)h.k * h.n * 4, cudaMemcpyHostToDevice, st.h2d));
    TA_CUDA(cudaEventRecord(st.ev_b, st.h2d));
    TA_CUDA(cudaStreamWaitEvent(comp, st.ev_b, 0));
  }
  if (has_bias && !h.bias_per_batch)
    for (int s = 0; s < HOST_RING; ++s)
      TA_CUDA(cudaMemcpyAsync(st.bias[s].ptr(), h.bias, (size_t)h.n * 4, cudaMemcpyHostToDevice, st.h2d));
  for (uint32_t i = 0; i < n_chunks; ++i) {
    const int s = (int)(i % HOST_RING);
    const uint32_t first = i * cb, planes = i + 1 == n_chunks ? tail : cb;
    Planned &p = plan[(size_t)s * 2 + (planes == cb ? 0 : 1)];
    // uploads of chunk i may overwrite set s once the GEMM of chunk i - RING has read it
    if (i >= HOST_RING) TA_CUDA(cudaStreamWaitEvent(st.h2d, st.ev_comp[s], 0));
    TA_CUDA(cudaMemcpyAsync(st.a[s].ptr(), h.a + (size_t)first * a_plane, (size_t)planes * a_plane * 4,
                            cudaMemcpyHostToDevice, st.h2d));
    if (has_d)
      TA_CUDA(cudaMemcpyAsync(st.d[s].ptr(), h.d + (size_t)first * c_plane, (size_t)planes * c_plane * 4,
                              cudaMemcpyHostToDevice, st.h2d));
    if (has_bias && h.bias_per_batch)
      TA_CUDA(cudaMemcpyAsync(st.bias[s].ptr(), h.bias + (size_t)first * h.n, (size_t)planes * h.n * 4,
                              cudaMemcpyHostToDevice, st.h2d));
    TA_CUDA(cudaEventRecord(st.ev_up[s], st.h2d));
    // the GEMM writes C of set s: the download of chunk i - RING must have drained it
    TA_CUDA(cudaStreamWaitEvent(comp, st.ev_up[s], 0));
    if (i >= HOST_RING) TA_CUDA(cudaStreamWaitEvent(comp, st.ev_down[s], 0));
    enqueue_op(p.op, p.r, p.route, slot, comp);
    TA_CUDA(cudaEventRecord(st.ev_comp[s], comp));
    TA_CUDA(cudaStreamWaitEvent(st.d2h, st.ev_comp[s], 0));
    TA_CUDA(cudaMemcpyAsync(h.c + (size_t)first * c_plane, st.c[s].ptr(), (size_t)planes * c_plane * 4,
                            cudaMemcpyDeviceToHost, st.d2h));
    TA_CUDA(cudaEventRecord(st.ev_down[s], st.d2h));
  }
  TA_CUDA(cudaEventRecord(st.ev_end, st.d2h));
  TA_CUDA(cudaStreamSynchronize(st.d2h));
  TA_CUDA(cudaStreamSynchronize(comp));
  TA_CUDA(cudaStreamSynchronize(st.h2d));
  check_status_word(slot.status_host, slot.counters);
  float ms = 0.0f;
  TA_CUDA(cudaEventElapsedTime(&ms, st.ev_begin, st.ev_end));
  RunStats out;
  out.gpu_time_ns = (uint64_t)((double)ms * 1e6 + 0.5);
  out.n_calls = n_chunks;
  out.total_flops = flops;
  return out;
}

}  // namespace ta
