// Mixed op graphs: matmuls and model ops in one submission or one captured
// replay (ExecOp, run_exec_ops, prepare_exec_ops of the reference,
// src/executor/graph_ops.rs:27-161, 249-353), and the single-op entry points
// built on the same planners.
//
// Every op is validated and planned before anything is enqueued (the
// reference's "validated and planned before anything is recorded",
// graph_ops.rs:246-248): planning returns a closure that only launches.  All
// closures of one submission run on one in-order CUDA stream, which is what
// resolves RAW / WAW / WAR hazards between ops here; the reference's explicit
// barrier bookkeeping (HazardCursor) has no CUDA counterpart to build.
#include <algorithm>
#include <functional>

#include "ta_core.hpp"

namespace ta {

namespace {
void ensure_f32(const Executor &e, const Tensor &t, const char *op, const char *operand) {
  e.validate_tensor(t, operand);
  if (t.dtype != DType::F32) fail("%s: %s must be f32 storage", op, operand);
}
void ensure_same_shape(const char *op, const Tensor &a, const Tensor &b) {
  if (a.shape != b.shape)
    fail("%s: input shape %s != output shape %s", op, a.shape_str().c_str(), b.shape_str().c_str());
}
void rows_cols(const Tensor &t, const char *label, uint32_t *rows, uint32_t *cols) {
  *cols = t.shape.back();
  const uint64_t r = t.len() / *cols;
  if (r > 0xffffffffull) fail("%s: row count %llu exceeds u32", label, (unsigned long long)r);
  *rows = (uint32_t)r;
}
}  // namespace

FlashParams Executor::plan_flash_attention(const Tensor &q, const Tensor &kt, const Tensor &v,
                                           const Tensor &out, const FlashAttentionDesc &desc) const {
  // q / out are both f32, or both f16 (f16 activations: src/executor/elementwise/flash.rs:76-78)
  validate_tensor(q, "input");
  validate_tensor(out, "output");
  if (q.dtype != out.dtype)
    fail("run_flash_attention: input (%s) and output (%s) must share a storage type", dtype_name(q.dtype),
         dtype_name(out.dtype));
  const bool io_f16 = q.dtype == DType::F16;
  validate_tensor(kt, "kt");
  validate_tensor(v, "v");
  if (kt.dtype != v.dtype)
    fail("run_flash_attention: kt (%s) and v (%s) must share a storage type", dtype_name(kt.dtype),
         dtype_name(v.dtype));
  if (kt.shape.size() != 3) fail("run_flash_attention: kt must be [H_kv, dh, T_max], got %s", kt.shape_str().c_str());
  if (v.shape.size() != 3) fail("run_flash_attention: v must be [H_kv, T_max, dh], got %s", v.shape_str().c_str());
  const uint32_t kv_heads = kt.shape[0], dh = kt.shape[1], t_max = kt.shape[2];
  if (v.shape[1] != t_max || v.shape[0] != kv_heads || v.shape[2] != dh)
    fail("run_flash_attention: inconsistent cache shapes kt %s, v %s", kt.shape_str().c_str(), v.shape_str().c_str());
  FlashParams p{};
  uint32_t heads, t_q;
  if (desc.token_major_heads) {
    heads = desc.token_major_heads;
    t_q = q.shape[0];
    if (q.len() != (uint64_t)t_q * heads * dh)
      fail("run_flash_attention: token-major q %s does not hold [T=%u, H=%u, dh=%u]", q.shape_str().c_str(), t_q, heads, dh);
    p.q_head_stride = dh;
    p.q_row_stride = heads * dh;
  } else {
    if (q.shape.size() != 3) fail("run_flash_attention: q must be [H, T_q, dh], got %s", q.shape_str().c_str());
    heads = q.shape[0];
    t_q = q.shape[1];
    if (q.shape[2] != dh)
      fail("run_flash_attention: q dh %u != cache dh %u (q %s, kt %s)", q.shape[2], dh, q.shape_str().c_str(),
           kt.shape_str().c_str());
    p.q_head_stride = t_q * dh;
    p.q_row_stride = dh;
  }
  if (desc.out_token_major_heads) {
    if (desc.out_token_major_heads != heads)
      fail("run_flash_attention: out_token_major_heads %u != q heads %u", desc.out_token_major_heads, heads);
    if (out.len() != (uint64_t)t_q * heads * dh)
      fail("run_flash_attention: token-major out %s does not hold [T=%u, H=%u, dh=%u]", out.shape_str().c_str(), t_q, heads, dh);
    p.o_head_stride = dh;
    p.o_row_stride = heads * dh;
  } else if (desc.token_major_heads) {
    if (out.len() != q.len())
      fail("run_flash_attention: out shape %s must match token-major q %s", out.shape_str().c_str(), q.shape_str().c_str());
    p.o_head_stride = p.q_head_stride;
    p.o_row_stride = p.q_row_stride;
  } else {
    if (out.shape != q.shape)
      fail("run_flash_attention: out shape %s must equal q shape %s", out.shape_str().c_str(), q.shape_str().c_str());
    p.o_head_stride = p.q_head_stride;
    p.o_row_stride = p.q_row_stride;
  }
  if (kv_heads == 0 || heads % kv_heads) fail("run_flash_attention: H=%u must be a multiple of H_kv=%u", heads, kv_heads);
  if (desc.kv_len > t_max) fail("run_flash_attention: kv_len %u exceeds cache T_max %u", desc.kv_len, t_max);
  if (dh != 64 && dh != 128) fail("run_flash_attention: head dimension %u unsupported (64 or 128)", dh);
  if (q.ptr() == out.ptr()) fail("run_flash_attention: q and out must be different tensors");
  p.q = static_cast<const float *>(q.ptr());
  p.kt = kt.ptr();
  p.v = v.ptr();
  p.out = static_cast<float *>(out.ptr());
  p.heads = heads; p.group = heads / kv_heads; p.dh = dh; p.t_q = t_q; p.t_max = t_max;
  p.kv_len = desc.kv_len; p.pos_base = desc.pos_base; p.scale = desc.scale;
  p.kv_f16 = kt.dtype == DType::F16;
  p.simt = desc.simt;
  p.io_f16 = io_f16 ? 1u : 0u;
  if (io_f16 && !(p.kv_f16 && dh == 64 && !desc.simt))   // flash.rs:193-212
    fail("run_flash_attention: f16 q/out are compiled for f16 KV caches with head dimension 64 on the "
         "tensor-core route only (kv %s, dh %u)", dtype_name(kt.dtype), dh);
  return p;
}

AttnDecodeParams Executor::plan_attn_decode(const Tensor &q, const Tensor &kt, const Tensor &v,
                                            const Tensor &scratch, const Tensor &out,
                                            const AttnDecodeDesc &desc) const {
  ensure_f32(*this, q, "run_attn_decode", "q");
  validate_tensor(kt, "kt");
  validate_tensor(v, "v");
  ensure_f32(*this, scratch, "run_attn_decode", "scratch");
  ensure_f32(*this, out, "run_attn_decode", "out");
  if (kt.dtype != v.dtype)
    fail("run_attn_decode: kt (%s) and v (%s) must share a storage type", dtype_name(kt.dtype), dtype_name(v.dtype));
  if (kt.shape.size() != 3) fail("run_attn_decode: kt must be [H_kv, dh, T_max], got %s", kt.shape_str().c_str());
  if (v.shape.size() != 3) fail("run_attn_decode: v must be [H_kv, T_max, dh], got %s", v.shape_str().c_str());
  const uint32_t kv_heads = kt.shape[0], dh = kt.shape[1], t_max = kt.shape[2];
  if (v.shape[2] != dh || v.shape[1] != t_max || v.shape[0] != kv_heads)
    fail("run_attn_decode: inconsistent caches kt %s, v %s", kt.shape_str().c_str(), v.shape_str().c_str());
  if (dh != 64) fail("run_attn_decode: head dimension %u unsupported (compiled variant: 64)", dh);
  const uint64_t heads_elems = (uint64_t)kv_heads * dh;
  if (q.len() % heads_elems)
    fail("run_attn_decode: q length %llu must be kv_heads*group*dh (kv_heads %u, dh %u)",
         (unsigned long long)q.len(), kv_heads, dh);
  const uint64_t group = q.len() / heads_elems;
  if (group == 0 || group > 8) fail("run_attn_decode: GQA group %llu unsupported (1..=8)", (unsigned long long)group);
  if (out.len() != q.len())
    fail("run_attn_decode: out length %llu must equal q length %llu", (unsigned long long)out.len(),
         (unsigned long long)q.len());
  if (desc.kv_len == 0 || desc.kv_len > t_max) fail("run_attn_decode: kv_len %u out of range 1..=%u", desc.kv_len, t_max);
  if (desc.pos_cell && desc.pos_cell->ctx.get() != ctx_.get())
    fail("run_attn_decode: pos cell belongs to a different context");
  // with a position cell the length is not known when the launch is recorded: the chunk grid is sized for
  // the whole cache, one 64-position tile per chunk where that fits the 8..32 chunk range (fewer chunks
  // = fewer partials for the last CTA to combine)
  uint32_t num_chunks = desc.pos_cell ? std::min(ATTN_DECODE_MAX_CHUNKS, std::max(8u, (t_max + 63u) / 64u))
                                      : attn_decode_num_chunks(desc.kv_len);
  if (desc.pos_cell && tunables().attn_chunks >= 1) num_chunks = tunables().attn_chunks;
  const uint64_t needed = (uint64_t)kv_heads * num_chunks * group * (dh + 2);
  if (scratch.len() < needed)
    fail("run_attn_decode: scratch length %llu < required %llu (kv_heads %u * chunks %u * group %llu * (dh+2))",
         (unsigned long long)scratch.len(), (unsigned long long)needed, kv_heads, num_chunks,
         (unsigned long long)group);
  AttnDecodeParams p{};
  p.q = static_cast<const float *>(q.ptr());
  p.kt = kt.ptr();
  p.v = v.ptr();
  p.scratch = static_cast<float *>(scratch.ptr());
  p.out = static_cast<float *>(out.ptr());
  p.kv_heads = kv_heads; p.group = (uint32_t)group; p.t_max = t_max; p.kv_len = desc.kv_len;
  p.num_chunks = num_chunks; p.scale = desc.scale; p.kv_f16 = kt.dtype == DType::F16;
  p.pos_ptr = desc.pos_cell ? desc.pos_cell->device : nullptr;
  return p;
}

// ------------------------------------------------------------------ planning
namespace {
const Tensor &need(const Tensor *t, const char *op, const char *operand) {
  if (!t) fail("%s: %s is null", op, operand);
  return *t;
}
const uint32_t *cell_ptr(const Executor &e, const PosCell *cell, const char *op) {
  if (!cell) return nullptr;
  if (cell->ctx.get() != e.context().get()) fail("%s: position/result cell belongs to a different context", op);
  return cell->device;
}
// Shared rope-geometry validation (src/executor/elementwise/ops.rs:176-207).
uint32_t rope_tokens(const char *op, const Tensor &in, const Tensor &table, const ExecOp &o) {
  if (o.rot_dim < 2 || o.rot_dim % 2 || o.rot_dim > o.head_dim)
    fail("%s: rot_dim %u must be even, >= 2, and <= head_dim %u", op, o.rot_dim, o.head_dim);
  const uint64_t vec = (uint64_t)o.heads * o.head_dim;
  if (vec == 0 || in.len() % vec)
    fail("%s: input length %llu is not a multiple of heads*head_dim %llu", op, (unsigned long long)in.len(),
         (unsigned long long)vec);
  const uint64_t tokens64 = in.len() / vec;
  if (tokens64 > 0xffffffffull) fail("%s: token count exceeds u32", op);
  const uint64_t needed = ((uint64_t)o.pos_base + tokens64) * o.rot_dim;
  if (table.len() < needed)
    fail("%s: table length %llu < required %llu (pos_base %u + %llu tokens, rot_dim %u)", op,
         (unsigned long long)table.len(), (unsigned long long)needed, o.pos_base,
         (unsigned long long)tokens64, o.rot_dim);
  return (uint32_t)tokens64;
}
}  // namespace

Launch Executor::plan_exec_op(const ExecOp &o, uint64_t *flops, size_t *n_calls) const {
  if (n_calls) *n_calls += 1;
  switch (o.kind) {
    case ExecKind::Matmul: {
      validate_op_tensors(*this, o.mm);
      const ResolvedMatmul r = ResolvedMatmul::from_op(o.mm);
      const Route route = plan_op(o.mm, r, false);   // data-parallel routes only inside graphs
      if (flops) *flops += r.total_flops;
      const MatmulOp mm = o.mm;
      Executor *self = const_cast<Executor *>(this);
      return [self, mm, r, route](Slot &slot, cudaStream_t st) { self->enqueue_op(mm, r, route, slot, st); };
    }
    case ExecKind::RmsNorm:
    case ExecKind::LayerNorm: {
      const bool ln = o.kind == ExecKind::LayerNorm;
      const char *name = ln ? "run_layer_norm" : "run_rms_norm";
      const Tensor &in = need(o.in0, name, "input"), &w = need(o.in1, name, "weight"), &out = need(o.out, name, "output");
      ensure_f32(*this, in, name, "input");
      ensure_f32(*this, w, name, "weight");
      ensure_f32(*this, out, name, "output");
      ensure_same_shape(name, in, out);
      uint32_t rows, cols;
      rows_cols(in, name, &rows, &cols);
      if (w.len() != cols) fail("%s: weight length %llu != row length %u", name, (unsigned long long)w.len(), cols);
      const float *bp = nullptr;
      if (ln) {
        const Tensor &b = need(o.in2, name, "bias");
        ensure_f32(*this, b, name, "bias");
        if (b.len() != cols) fail("%s: bias length %llu != row length %u", name, (unsigned long long)b.len(), cols);
        bp = (const float *)b.ptr();
      }
      const float *ip = (const float *)in.ptr(), *wp = (const float *)w.ptr();
      float *op = (float *)out.ptr();
      const float eps = o.f0;
      if (ln) return [=](Slot &, cudaStream_t st) { launch_layer_norm(ip, wp, bp, op, rows, cols, eps, st); };
      const uint32_t pitch16 = o.a16_pitch;
      return [=](Slot &slot, cudaStream_t st) {
        void *out16 = nullptr;
        if (pitch16) {   // planned only in front of a GEMM whose scratch demand covers this copy
          if (!slot.scratch || slot.scratch_bytes < (size_t)rows * pitch16 * 2) fail("internal: no scratch for the f16 copy of a norm output");
          out16 = slot.scratch;
        }
        launch_rms_norm(ip, wp, op, rows, cols, eps, st, out16, pitch16);
      };
    }
    case ExecKind::SoftmaxRows: {
      const Tensor &in = need(o.in0, "run_softmax_rows", "input"), &out = need(o.out, "run_softmax_rows", "output");
      ensure_f32(*this, in, "run_softmax_rows", "input");
      ensure_f32(*this, out, "run_softmax_rows", "output");
      ensure_same_shape("run_softmax_rows", in, out);
      uint32_t rows, cols;
      rows_cols(in, "run_softmax_rows", &rows, &cols);
      if (o.u0 > 2) fail("run_softmax_rows: mask kind %u is invalid (0=full 1=prefix 2=causal)", o.u0);
      if (o.u0 == 2 && (o.u2 == 0 || rows % o.u2))
        fail("run_softmax_rows: rows_per_group %u must divide rows %u", o.u2, rows);
      const float *ip = (const float *)in.ptr();
      float *op = (float *)out.ptr();
      const float scale = o.f0;
      const uint32_t mk = o.u0, vp = o.u1, rpg = o.u2;
      return [=](Slot &, cudaStream_t st) { launch_softmax_rows(ip, op, rows, cols, scale, mk, vp, rpg, st); };
    }
    case ExecKind::Rope: {
      const Tensor &in = need(o.in0, "run_rope", "input"), &tab = need(o.in1, "run_rope", "table"),
                   &out = need(o.out, "run_rope", "output");
      ensure_f32(*this, in, "run_rope", "input");
      ensure_f32(*this, out, "run_rope", "output");
      ensure_f32(*this, tab, "run_rope", "table");
      ensure_same_shape("run_rope", in, out);
      const uint32_t tokens = rope_tokens("run_rope", in, tab, o);
      const float *ip = (const float *)in.ptr(), *tp = (const float *)tab.ptr();
      float *op = (float *)out.ptr();
      const uint32_t heads = o.heads, hd = o.head_dim, rd = o.rot_dim, pb = o.pos_base;
      return [=](Slot &, cudaStream_t st) { launch_rope(ip, tp, op, tokens, heads, hd, rd, pb, st); };
    }
    case ExecKind::RopeScatter: {
      const Tensor &in = need(o.in0, "run_rope_scatter", "input"), &tab = need(o.in1, "run_rope_scatter", "table"),
                   &dst = need(o.out, "run_rope_scatter", "dst");
      ensure_f32(*this, in, "run_rope_scatter", "input");
      ensure_f32(*this, tab, "run_rope_scatter", "table");
      validate_tensor(dst, "dst");
      if (in.ptr() == dst.ptr()) fail("run_rope_scatter: input and dst must be different tensors");
      const uint32_t tokens = rope_tokens("run_rope_scatter", in, tab, o);
      const uint64_t max_index = (uint64_t)o.dst_offset + (uint64_t)(tokens - 1) * o.strides[0] +
                                 (uint64_t)(o.heads - 1) * o.strides[1] + (uint64_t)(o.head_dim - 1) * o.strides[2];
      if (max_index >= dst.len())
        fail("run_rope_scatter: destination access reaches element %llu but dst has %llu",
             (unsigned long long)max_index, (unsigned long long)dst.len());
      if (o.head_dim % 2) fail("run_rope_scatter: head_dim %u must be even", o.head_dim);
      const float *ip = (const float *)in.ptr(), *tp = (const float *)tab.ptr();
      void *dp = dst.ptr();
      const bool f16 = dst.dtype == DType::F16;
      const uint32_t *pp = cell_ptr(*this, o.cell, "run_rope_scatter");
      const ExecOp oc = o;
      return [=](Slot &, cudaStream_t st) {
        launch_rope_scatter(ip, tp, dp, f16, tokens, oc.heads, oc.head_dim, oc.rot_dim, oc.pos_base, oc.dst_offset,
                            oc.strides, oc.pos_scale, pp, st);
      };
    }
    case ExecKind::CopyStrided: {
      const Tensor &src = need(o.in0, "run_copy_strided", "src"), &dst = need(o.out, "run_copy_strided", "dst");
      validate_tensor(src, "src");
      validate_tensor(dst, "dst");
      if (src.ptr() == dst.ptr()) fail("run_copy_strided: src and dst must be different tensors");
      if (!o.extent[0] || !o.extent[1] || !o.extent[2])
        fail("run_copy_strided: extent [%u, %u, %u] has a zero axis", o.extent[0], o.extent[1], o.extent[2]);
      auto max_index = [&](uint32_t off, const uint32_t st[3]) {
        uint64_t v = off;
        for (int i = 0; i < 3; ++i) v += (uint64_t)(o.extent[i] - 1) * st[i];
        return v;
      };
      if (max_index(o.src_offset, o.src_strides) >= src.len())
        fail("run_copy_strided: source access reaches element %llu but src has %llu",
             (unsigned long long)max_index(o.src_offset, o.src_strides), (unsigned long long)src.len());
      if (max_index(o.dst_offset, o.strides) >= dst.len())
        fail("run_copy_strided: destination access reaches element %llu but dst has %llu",
             (unsigned long long)max_index(o.dst_offset, o.strides), (unsigned long long)dst.len());
      if ((uint64_t)o.extent[0] * o.extent[1] * o.extent[2] > 0xffffffffull)
        fail("run_copy_strided: extent product exceeds u32");
      const void *sp = src.ptr();
      void *dp = dst.ptr();
      const bool sf = src.dtype == DType::F16, df = dst.dtype == DType::F16;
      const ExecOp oc = o;
      return [=](Slot &, cudaStream_t st) {
        launch_copy_strided(sp, sf, dp, df, oc.extent, oc.src_offset, oc.src_strides, oc.dst_offset, oc.strides, st);
      };
    }
    case ExecKind::Binary: {
      const Tensor &a = need(o.in0, "run_binary", "a"), &b = need(o.in1, "run_binary", "b"), &out = need(o.out, "run_binary", "out");
      ensure_f32(*this, a, "run_binary", "a");
      ensure_f32(*this, out, "run_binary", "out");
      validate_tensor(b, "b");
      if (b.dtype != a.dtype) fail("run_binary: b (%s) must match a (%s) storage", dtype_name(b.dtype), dtype_name(a.dtype));
      if (a.len() != b.len() || a.len() != out.len())
        fail("run_binary: element counts differ (a %llu, b %llu, out %llu)", (unsigned long long)a.len(),
             (unsigned long long)b.len(), (unsigned long long)out.len());
      if (a.len() > 0xffffffffull) fail("run_binary: too large");
      if (o.u0 > 1) fail("run_binary: mode %u is invalid (0=add_scaled 1=silu_mul)", o.u0);
      const float *ap = (const float *)a.ptr(), *bp = (const float *)b.ptr();
      float *op = (float *)out.ptr();
      const uint32_t n = (uint32_t)a.len(), mode = o.u0;
      const float beta = o.f0;
      return [=](Slot &, cudaStream_t st) { launch_binary(ap, bp, op, n, mode, beta, st); };
    }
    default:
      break;
  }
  return plan_exec_op_tail(o, n_calls);
}

Launch Executor::plan_exec_op_tail(const ExecOp &o, size_t *n_calls) const {
  switch (o.kind) {
    case ExecKind::AttnDecode: {
      const AttnDecodeParams p = plan_attn_decode(need(o.in0, "run_attn_decode", "q"), need(o.in1, "run_attn_decode", "kt"),
                                                  need(o.in2, "run_attn_decode", "v"), need(o.in3, "run_attn_decode", "scratch"),
                                                  need(o.out, "run_attn_decode", "out"), o.attn);
      const uint32_t prefetch = o.u0;   // internal hint from plan_exec_ops (the C ABI clears it)
      const int pos_idx = (int)o.u1 - 1;   // internal: index of the position cell's staged device word (u1 = index + 1)
      return [p, prefetch, pos_idx](Slot &slot, cudaStream_t st) {
        AttnDecodeParams q = p;
        if (pos_idx >= 0 && q.pos_ptr) q.pos_ptr = pos_stage_of(slot.counters) + pos_idx;
        q.counters = slot.counters;
        q.status = slot.status;
        q.pdl = 1;
        q.prefetch_kv = prefetch;
        if (tunables().attn_pairs && q.kv_f16 && q.kv_heads * q.num_chunks * 8u <= ATTN_PAIR_ROWS) {
          q.pairs = attn_pairs_of(slot.counters);
          q.pair_seq = slot.counters + ATTN_SEQ_OFFSET;
        }
        launch_attn_decode(q, st);
      };
    }
    case ExecKind::FlashAttn: {
      const FlashParams p = plan_flash_attention(need(o.in0, "run_flash_attention", "q"), need(o.in1, "run_flash_attention", "kt"),
                                                 need(o.in2, "run_flash_attention", "v"), need(o.out, "run_flash_attention", "out"),
                                                 o.flash);
      const uint32_t pitch16 = o.a16_pitch;
      return [p, pitch16](Slot &slot, cudaStream_t st) {
        FlashParams q = p;
        if (pitch16) {
          if (!slot.scratch || slot.scratch_bytes < (size_t)q.t_q * pitch16 * 2) fail("internal: no scratch for the f16 copy of an attention output");
          q.out16 = slot.scratch;
          q.out16_row_stride = pitch16;
        }
        launch_flash_prefill(q, st);
      };
    }
    case ExecKind::Argmax: {
      const Tensor &in = need(o.in0, "run_argmax", "input");
      ensure_f32(*this, in, "run_argmax", "input");
      if (!o.cell) fail("run_argmax: result cell is null");
      if (o.cell->ctx.get() != ctx_.get()) fail("run_argmax: result buffer belongs to a different context");
      if (in.len() > 0xffffffffull) fail("run_argmax: input too large");
      const float *ip = (const float *)in.ptr();
      const uint32_t n = (uint32_t)in.len();
      uint32_t *rp = o.cell->device;
      return [=](Slot &, cudaStream_t st) { launch_argmax(ip, n, rp, st); };
    }
    case ExecKind::ArgmaxSharded: {
      const Tensor &in = need(o.in0, "run_argmax_sharded", "input");
      ensure_f32(*this, in, "run_argmax_sharded", "input");
      if (!o.cell) fail("run_argmax_sharded: result cell is null");
      if (o.cell->ctx.get() != ctx_.get()) fail("run_argmax_sharded: result buffer belongs to a different context");
      if (!o.comm) fail("run_argmax_sharded: communicator is null");
      if (o.comm->ctx.get() != ctx_.get()) fail("run_argmax_sharded: communicator belongs to a different context");
      if (in.len() > 0xffffffffull) fail("run_argmax_sharded: input too large");
      if (!o.comm->fused_exchange_ready())
        fail("run_argmax_sharded: the communicator has no peer exchange (one rank, or peer access unavailable); "
             "gather the slices and use the plain argmax");
      const Comm *comm = o.comm;
      const float *ip = (const float *)in.ptr();
      const uint32_t n = (uint32_t)in.len(), off = o.u0;
      uint32_t *rp = o.cell->device;
      return [=](Slot &slot, cudaStream_t st) {
        if (!comm->argmax_sharded(ip, n, off, rp, slot.status, st)) fail("run_argmax_sharded: peer exchange unavailable");
      };
    }
    case ExecKind::EmbedGather:
    case ExecKind::EmbedGatherRows: {
      const bool rows = o.kind == ExecKind::EmbedGatherRows;
      const Tensor &table = need(o.in0, "run_embed_gather", "table"), &out = need(o.out, "run_embed_gather", "out");
      validate_tensor(table, "table");
      ensure_f32(*this, out, "run_embed_gather", "out");
      if (table.shape.size() != 2)
        fail("run_embed_gather: table must be [vocab, embd], got %s", table.shape_str().c_str());
      const uint32_t vocab = table.shape[0], embd = table.shape[1];
      uint32_t n_tokens = 1;
      const uint32_t *tp;
      if (rows) {
        if (!o.tokens) fail("run_embed_gather: token buffer is null");
        if (o.tokens->ctx.get() != ctx_.get()) fail("run_embed_gather: token buffer belongs to a different context");
        n_tokens = o.tokens->len;
        if (n_tokens == 0) fail("run_embed_gather: token buffer is empty");
        tp = o.tokens->device;
      } else {
        if (!o.cell) fail("run_embed_gather: token cell is null");
        if (o.cell->ctx.get() != ctx_.get()) fail("run_embed_gather: token buffer belongs to a different context");
        tp = o.cell->device;
      }
      if (out.len() != (uint64_t)n_tokens * embd)
        fail("run_embed_gather: out length %llu != n_tokens %u * embd %u", (unsigned long long)out.len(), n_tokens, embd);
      const void *tab = table.ptr();
      const bool tf16 = table.dtype == DType::F16;
      float *op = (float *)out.ptr();
      return [=](Slot &, cudaStream_t st) { launch_embed_gather(tp, n_tokens, tab, tf16, op, embd, vocab, st); };
    }
    case ExecKind::PrefillQkvPack: {
      const char *nm = "run_prefill_qkv_pack";
      const Tensor &qkv = need(o.in0, nm, "qkv"), &tab = need(o.in1, nm, "table"), &q = need(o.out, nm, "q"),
                   &kt = need(o.in2, nm, "kt"), &v = need(o.in3, nm, "v");
      ensure_f32(*this, qkv, nm, "qkv");
      ensure_f32(*this, tab, nm, "table");
      ensure_f32(*this, q, nm, "q");
      validate_tensor(kt, "kt");
      validate_tensor(v, "v");
      if (kt.dtype != v.dtype) fail("%s: kt (%s) and v (%s) must share a storage type", nm, dtype_name(kt.dtype), dtype_name(v.dtype));
      const uint32_t heads = o.heads, kv_heads = o.u0, dh = o.head_dim, rot = o.rot_dim;
      if (!heads || !kv_heads || !dh || !rot || (rot & 1u) || rot > dh || (dh & 1u))
        fail("%s: invalid heads/kv_heads/dh/rot_dim (%u/%u/%u/%u)", nm, heads, kv_heads, dh, rot);
      if (qkv.shape.size() != 2) fail("%s: qkv must be [T, n_qkv], got %s", nm, qkv.shape_str().c_str());
      const uint32_t tokens = qkv.shape[0], want = heads * dh + 2 * kv_heads * dh;
      if (qkv.shape[1] != want) fail("%s: qkv N %u != H*dh + 2*H_kv*dh (%u)", nm, qkv.shape[1], want);
      if (q.shape != std::vector<uint32_t>{heads, tokens, dh})
        fail("%s: q must be head-major [H=%u, T=%u, dh=%u], got %s", nm, heads, tokens, dh, q.shape_str().c_str());
      if (kt.shape.size() != 3 || kt.shape[0] != kv_heads || kt.shape[1] != dh)
        fail("%s: kt must be [H_kv, dh, T_max], got %s", nm, kt.shape_str().c_str());
      const uint32_t t_max = kt.shape[2];
      if (v.shape != std::vector<uint32_t>{kv_heads, t_max, dh})
        fail("%s: v must be [H_kv=%u, T_max=%u, dh=%u], got %s", nm, kv_heads, t_max, dh, v.shape_str().c_str());
      if ((uint64_t)o.pos_base + tokens > t_max)
        fail("%s: pos_base %u + T %u exceeds cache T_max %u", nm, o.pos_base, tokens, t_max);
      if (tab.len() < (uint64_t)(o.pos_base + tokens) * rot)
        fail("%s: rope table holds %llu values, positions up to %u need %llu", nm, (unsigned long long)tab.len(),
             o.pos_base + tokens, (unsigned long long)(o.pos_base + tokens) * rot);
      if (q.ptr() == qkv.ptr()) fail("%s: q and qkv must be different tensors", nm);
      const float *sp = (const float *)qkv.ptr(), *tp = (const float *)tab.ptr();
      float *qp = (float *)q.ptr();
      void *kp = kt.ptr(), *vp = v.ptr();
      const bool f16 = kt.dtype == DType::F16;
      const uint32_t pb = o.pos_base;
      return [=](Slot &, cudaStream_t st) {
        launch_prefill_qkv_pack(sp, tp, qp, kp, vp, f16, tokens, heads, kv_heads, dh, rot, pb, t_max, st);
      };
    }
    case ExecKind::AllReduce: {
      const Tensor &t = need(o.out, "run_all_reduce", "tensor");
      ensure_f32(*this, t, "run_all_reduce", "tensor");
      if (!o.comm) fail("run_all_reduce: communicator is null");
      if (o.comm->ctx.get() != ctx_.get()) fail("run_all_reduce: communicator belongs to a different context");
      const Comm *comm = o.comm;
      float *ptr = (float *)t.ptr();
      const size_t count = (size_t)t.len();
      return [=](Slot &slot, cudaStream_t st) {
        // one-launch peer exchange for a row or two; NCCL beyond (or, as an experiment, the two-step peer kernel)
        if (!comm->peer_all_reduce_sum(ptr, count, slot.status, true, st) && !comm->peer_all_reduce_big(ptr, count, slot.status, st))
          comm->all_reduce_sum(ptr, count, st);
      };
    }
    case ExecKind::AllGather: {
      const Tensor &src = need(o.in0, "run_all_gather", "src"), &dst = need(o.out, "run_all_gather", "dst");
      ensure_f32(*this, src, "run_all_gather", "src");
      ensure_f32(*this, dst, "run_all_gather", "dst");
      if (!o.comm) fail("run_all_gather: communicator is null");
      if (o.comm->ctx.get() != ctx_.get()) fail("run_all_gather: communicator belongs to a different context");
      if (dst.len() != src.len() * o.comm->world)
        fail("run_all_gather: dst length %llu != src length %llu * world %u", (unsigned long long)dst.len(),
             (unsigned long long)src.len(), o.comm->world);
      const Comm *comm = o.comm;
      const float *sp = (const float *)src.ptr();
      float *dp = (float *)dst.ptr();
      const size_t count = (size_t)src.len();
      return [=](Slot &, cudaStream_t st) { comm->all_gather(sp, dp, count, st); };
    }
    default:
      fail("exec op kind %u is not recognised", (unsigned)o.kind);
  }
}

// ------------------------------------------------------------------ submission
// Plans a whole op list.  Besides planning op by op it fuses launches where the
// result is the same as running the ops one after another:
//   * consecutive row-GEMVs that read the same x (same fused norm, M, K, tile
//     width) and neither read nor overwrite one another's outputs become
//     segments of one launch (the q / k / v projections of a decode layer);
//   * `up = x@Wup` directly followed by `gate = silu(x@Wg) * up` becomes the
//     dual-matrix launch, which still writes `up`.
// The reference gets the same effect from eliding barriers between independent
// dispatches (HazardCursor, src/executor/graph_ops.rs:587-624); here a launch
// boundary is the barrier, so independent ops share a launch instead.
std::vector<Launch> Executor::plan_exec_ops(const std::vector<ExecOp> &ops, uint64_t *flops,
                                            size_t *n_calls, size_t *scratch_bytes,
                                            std::vector<size_t> *first_op, ExchangeUse *exchange) const {
  struct Cand {
    bool gemv = false;
    GemvParams g{};
    uint64_t flops = 0;
  };
  auto candidate = [&](const ExecOp &o) {
    Cand c;
    if (o.kind != ExecKind::Matmul) return c;
    validate_op_tensors(*this, o.mm);
    const ResolvedMatmul r = ResolvedMatmul::from_op(o.mm);
    const Route route = plan_op(o.mm, r, false);
    c.gemv = gemv_params_for(o.mm, r, route, &c.g);
    c.flops = r.total_flops;
    if (scratch_bytes) *scratch_bytes = std::max(*scratch_bytes, op_scratch_bytes(r, route));
    return c;
  };
  auto writes = [](const GemvParams &g) -> const void * { return g.store_kind >= 2 ? g.dst : (const void *)g.c; };
  auto reads_ptr = [](const GemvParams &g, const void *ptr) {
    return ptr == g.x || ptr == g.d || ptr == g.bias || ptr == g.norm_w || ptr == g.table ||
           (g.accumulate && ptr == g.c);
  };
  const Context *cx = ctx_.get();
  std::vector<Launch> plan;
  plan.reserve(ops.size());
  std::vector<GemvParams> prev_gemv;   // segments of the launch planned last, when it was a GEMV
  // Tensor-parallel exchange fused into its neighbours.  `row-parallel GEMV -> all-reduce of its
  // one-row output -> GEMV reading that row` becomes two launches: the first pushes its partial
  // row into every rank's exchange buffer, the second waits for all ranks' rows, adds them in rank
  // order while it stages x, and leaves the sum in the tensor for later readers.  The same values
  // in the same order on every rank, as the separate all-reduce gives.  Every pushed element carries
  // its own flag (see PeerLink), so nothing but the data crosses NVLink.
  struct Pending {
    const void *tensor = nullptr;
    uint32_t point = 0, tiles = 0, slot = 0;
    const Comm *comm = nullptr;
  } pending;
  uint32_t next_point = 0;
  auto fusable_push = [&](size_t at, const Cand &c) -> const Comm * {
    if (!tunables().peer_allreduce || !c.gemv || at + 2 >= ops.size() || next_point >= PEER_MAX_POINTS) return nullptr;
    const ExecOp &ar = ops[at + 1];
    if (ar.kind != ExecKind::AllReduce || !ar.comm || !ar.out || !ar.comm->fused_exchange_ready()) return nullptr;
    const GemvParams &gp = c.g;
    if (gp.m != 1 || gp.store_kind != 0 || gp.w2 || (uint64_t)gp.m * gp.n > PEER_MAX_FLOATS) return nullptr;
    if (ar.out->ptr() != (const void *)gp.c || ar.out->len() != (uint64_t)gp.m * gp.n) return nullptr;
    const Cand nxt = candidate(ops[at + 2]);
    if (!nxt.gemv || nxt.g.m != 1 || (const void *)nxt.g.x != (const void *)gp.c || nxt.g.k != gp.n) return nullptr;
    return ar.comm;
  };
  // exchange link of a GEMV launch: pulls `pending` when the launch reads that tensor as x
  auto link_for = [&](const GemvParams &first_seg, const Comm *push_comm, bool *has_link) {
    PeerLink link{};
    *has_link = false;
    const Comm *comm = push_comm;
    if (pending.tensor && (const void *)first_seg.x == pending.tensor) {
      comm = pending.comm;
      link = comm->link();
      link.pull_point1 = pending.point + 1;
      link.pull_slot = pending.slot;
      link.x_out = const_cast<float *>(first_seg.x);
      if (exchange) {
        exchange->comm = comm;
        exchange->points.emplace_back(pending.point, 1u);   // one use of the point per submission
      }
      pending = Pending{};
      *has_link = true;
    } else if (comm) {
      link = comm->link();
      *has_link = true;
    }
    return link;
  };
  // position cells read by GEMV stores and decode attentions get a device word of the slot, filled by
  // the submission's first stream operation; the launch closures swap the pointer in
  auto stage_index = [&](const PosCell *cell) -> int {
    if (!cell || !exchange || !tunables().pos_stage) return -1;
    for (size_t k = 0; k < exchange->pos_cells_host.size(); ++k)
      if (exchange->pos_cells_host[k] == cell->host) return (int)k;
    if (exchange->pos_cells_host.size() >= POS_STAGE_WORDS) return -1;
    exchange->pos_cells_host.push_back(cell->host);
    return (int)exchange->pos_cells_host.size() - 1;
  };
  auto stage_gemv = [&](GemvParams &g, const ExecOp &op) {
    if (g.pos_ptr && op.kind == ExecKind::Matmul) g.pos_stage_idx = stage_index(op.mm.store.pos_cell);
  };
  size_t i = 0, a16_ready_for = (size_t)-1;
  while (i < ops.size()) {
    Cand c0 = candidate(ops[i]);
    if (pending.tensor && !(c0.gemv && (const void *)c0.g.x == pending.tensor))
      fail("internal: a fused tensor-parallel push is not followed by the launch that pulls it");
    if (!c0.gemv) {
      ExecOp op = ops[i];
      // A norm or a token-major flash attention whose output is the A of the f16-weight tensor-core
      // GEMM right behind it also writes that A rounded to f16 where the GEMM expects its copy: the
      // separate conversion launch disappears (same values: the GEMM's own conversion rounds the same
      // f32 numbers to nearest even).
      if ((op.kind == ExecKind::RmsNorm || op.kind == ExecKind::FlashAttn) && op.out && i + 1 < ops.size() &&
          ops[i + 1].kind == ExecKind::Matmul && ops[i + 1].mm.call.a && ops[i + 1].mm.call.a->ptr() == op.out->ptr() &&
          !candidate(ops[i + 1]).gemv) {
        const MatmulOp &nx = ops[i + 1].mm;
        const ResolvedMatmul rn = ResolvedMatmul::from_op(nx);
        const Route rt = plan_op(nx, rn, false);
        const uint32_t pitch = gemm_f16w_umma_a16_pitch(rn.k);
        bool ok = KERNEL_SPECS[rt.kernel].family == Family::F16wUmma && op_scratch_bytes(rn, rt) > 0 && rn.batch == 1 &&
                  !rn.a_f16 && pitch == rn.k && op.out->dtype == DType::F32 && op.out->len() == (uint64_t)rn.m * rn.k;
        if (ok && op.kind == ExecKind::FlashAttn) {   // token-major f32 output of the tensor-core kernel only
          ok = op.flash.out_token_major_heads != 0 && op.in0 && op.in1 && op.in2;
          if (ok) {
            const FlashParams fp = plan_flash_attention(*op.in0, *op.in1, *op.in2, *op.out, op.flash);
            ok = flash_prefill_mma_eligible(fp) && !fp.io_f16 && fp.o_head_stride == fp.dh &&
                 fp.o_row_stride == fp.heads * fp.dh && fp.t_q == rn.m;
          }
        }
        if (ok) {
          op.a16_pitch = pitch;
          a16_ready_for = i + 1;
        }
      }
      if (op.kind == ExecKind::Matmul && a16_ready_for == i) op.mm.a16_ready = true;
      // up, then gate = silu(A Wg) * up, both on the f16-weight tensor-core route: one dual-matrix
      // launch computes both (the same MMA sequence per output element and the same epilogue
      // formulas as the two launches: bit-identical), A is staged once and `up` is not re-read
      if (op.kind == ExecKind::Matmul && i + 1 < ops.size() && ops[i + 1].kind == ExecKind::Matmul) {
        GemmParams dp;
        if (dual_f16w_params(op.mm, ops[i + 1].mm, &dp)) {
          validate_op_tensors(*this, op.mm);
          validate_op_tensors(*this, ops[i + 1].mm);
          const bool ready = op.mm.a16_ready;
          if (flops) *flops += 2ull * 2ull * dp.m * dp.n * dp.k;
          if (n_calls) *n_calls += 2;
          plan.push_back([dp, cx, ready](Slot &slot, cudaStream_t st) {
            launch_gemm_f16w_umma_dual(*cx, dp, slot.status, slot.scratch, slot.scratch_bytes, ready, st);
          });
          if (first_op) first_op->push_back(i);
          prev_gemv.clear();
          i += 2;
          continue;
        }
      }
      // two f16w tensor-core GEMMs in a row on the same A (up and gate of a prefill MLP): the f16
      // copy of A made for the first is still in the slot scratch when the second runs
      if (op.kind == ExecKind::Matmul && i > 0 && ops[i - 1].kind == ExecKind::Matmul) {
        const MatmulOp &prev = ops[i - 1].mm;
        const ResolvedMatmul rp = ResolvedMatmul::from_op(prev), rc = ResolvedMatmul::from_op(op.mm);
        const Route routep = plan_op(prev, rp, false), routec = plan_op(op.mm, rc, false);
        if (op_scratch_bytes(rp, routep) && op_scratch_bytes(rc, routec) && prev.call.a->ptr() == op.mm.call.a->ptr() &&
            rp.m == rc.m && rp.k == rc.k && rp.batch == rc.batch && rp.batch_stride_a == rc.batch_stride_a &&
            prev.call.c->ptr() != op.mm.call.a->ptr())
          op.mm.a16_ready = true;
      }
      if (op.kind == ExecKind::AttnDecode) {
        // Decode attention may read the cache ahead of its dependency wait when the launch
        // before it (the only one that can still be running then) appends nothing but
        // position kv_len - 1: a GEMV whose scatter stores use the same position cell.
        bool ok = !prev_gemv.empty() && op.in1 && op.in2;
        for (const GemvParams &e : prev_gemv) {
          const void *kt = op.in1 ? op.in1->ptr() : nullptr, *v = op.in2 ? op.in2->ptr() : nullptr;
          if (e.store_kind >= 2) {
            const uint32_t *cell = op.attn.pos_cell ? op.attn.pos_cell->device : nullptr;
            if (e.pos_ptr != cell || e.pos_base + 1 != op.attn.kv_len) ok = false;
          } else if ((const void *)e.c == kt || (const void *)e.c == v) {
            ok = false;
          }
          if ((const void *)e.c2 == kt || (const void *)e.c2 == v) ok = false;
        }
        op.u0 = ok ? 1u : 0u;
        op.u1 = (uint32_t)(stage_index(op.attn.pos_cell) + 1);
      }
      if (op.kind == ExecKind::ArgmaxSharded && exchange && op.comm) {
        exchange->comm = op.comm;
        exchange->points.emplace_back(PEER_MAX_POINTS, 1u);
      }
      plan.push_back(plan_exec_op(op, flops, n_calls));
      if (first_op) first_op->push_back(i);
      prev_gemv.clear();
      ++i;
      continue;
    }
    // SwiGLU pair
    if (i + 1 < ops.size()) {
      Cand c1 = candidate(ops[i + 1]);
      const GemvParams &u = c0.g, &gt = c1.g;
      const bool up_plain = u.alpha == 1.0f && !u.accumulate && !u.bias && u.act == 0 && u.binary == 0 &&
                            u.store_kind == 0;
      if (c1.gemv && up_plain && gemv_f16w_groupable(u, gt) && u.n == gt.n && gt.alpha == 1.0f &&
          !gt.accumulate && !gt.bias && gt.act == (uint32_t)Activation::Silu &&
          gt.binary == (uint32_t)BinaryKind::Mul && gt.d == u.c && gt.store_kind == 0 && gt.c != u.c &&
          gt.x != u.c) {
        GemvParams f = gt;
        stage_gemv(f, ops[i + 1]);
        f.w2 = u.w;
        f.c2 = u.c;
        f.act = 0; f.binary = 0; f.d = nullptr;
        if (flops) *flops += c0.flops + c1.flops;
        if (n_calls) *n_calls += 2;
        bool has_link = false;
        const PeerLink link = link_for(f, nullptr, &has_link);
        plan.push_back([f, cx, link, has_link](Slot &slot, cudaStream_t st) {
          GemvParams fs = f;
          if (fs.pos_stage_idx >= 0) fs.pos_ptr = pos_stage_of(slot.counters) + fs.pos_stage_idx;
          launch_gemv_f16w_group(*cx, &fs, 1, true, gemv_workspace(slot), st, has_link ? &link : nullptr);
        });
        if (first_op) first_op->push_back(i);
        prev_gemv.assign(1, f);
        i += 2;
        continue;
      }
    }
    // a row-parallel projection whose one-row output is all-reduced next and read by a GEMV after that
    if (const Comm *push_comm = fusable_push(i, c0)) {
      GemvParams f = c0.g;
      stage_gemv(f, ops[i]);
      f.push_point1 = next_point + 1;
      f.push_slot = next_point & 1u;
      bool has_link = false;
      const PeerLink link = link_for(f, push_comm, &has_link);
      pending.tensor = f.c;
      pending.point = next_point;
      pending.slot = f.push_slot;
      pending.tiles = gemv_f16w_tiles(&f, 1);
      pending.comm = push_comm;
      ++next_point;
      if (flops) *flops += c0.flops;
      if (n_calls) *n_calls += 2;   // the projection and the all-reduce it carries
      plan.push_back([f, cx, link](Slot &slot, cudaStream_t st) {
        GemvParams fs = f;
        if (fs.pos_stage_idx >= 0) fs.pos_ptr = pos_stage_of(slot.counters) + fs.pos_stage_idx;
        launch_gemv_f16w_group(*cx, &fs, 1, true, gemv_workspace(slot), st, &link);
      });
      if (first_op) first_op->push_back(i);
      prev_gemv.assign(1, f);
      i += 2;
      continue;
    }
    // group of independent GEMVs on the same x
    std::vector<GemvParams> segs{c0.g};
    stage_gemv(segs[0], ops[i]);
    uint64_t fl = c0.flops;
    size_t j = i + 1;
    while (j < ops.size() && segs.size() < (size_t)GEMV_MAX_SEGS) {
      Cand cj = candidate(ops[j]);
      if (!cj.gemv || cj.g.w2 || !gemv_f16w_groupable(segs[0], cj.g)) break;
      bool independent = true;
      for (const GemvParams &e : segs) {
        if (reads_ptr(cj.g, writes(e)) || reads_ptr(e, writes(cj.g)) || writes(e) == writes(cj.g))
          independent = false;
        // a scatter segment may also leave its plain C untouched; keep C buffers apart as well
        if (e.c == cj.g.c && (e.store_kind < 2 || cj.g.store_kind < 2)) independent = false;
      }
      if (!independent) break;
      segs.push_back(cj.g);
      stage_gemv(segs.back(), ops[j]);
      fl += cj.flops;
      ++j;
    }
    if (flops) *flops += fl;
    if (n_calls) *n_calls += segs.size();
    bool has_link = false;
    const PeerLink link = link_for(segs[0], nullptr, &has_link);
    plan.push_back([segs, cx, link, has_link](Slot &slot, cudaStream_t st) {
      std::vector<GemvParams> ss = segs;
      for (GemvParams &e : ss)
        if (e.pos_stage_idx >= 0) e.pos_ptr = pos_stage_of(slot.counters) + e.pos_stage_idx;
      launch_gemv_f16w_group(*cx, ss.data(), (int)ss.size(), true, gemv_workspace(slot), st, has_link ? &link : nullptr);
    });
    if (first_op) first_op->push_back(i);
    prev_gemv = segs;
    i = j;
  }
  if (pending.tensor) fail("internal: a fused tensor-parallel push is not followed by the launch that pulls it");
  return plan;
}

RunStats Executor::run_exec_ops(const std::vector<ExecOp> &ops) {
  if (ops.empty()) return RunStats{std::nullopt, 0, 0};
  uint64_t flops = 0;
  size_t n_calls = 0;
  size_t scratch_bytes = 0;
  ExchangeUse exchange;
  std::vector<Launch> plan = plan_exec_ops(ops, &flops, &n_calls, &scratch_bytes, nullptr, &exchange);
  ctx_->make_current();
  Slot &slot = checkout_slot();
  SlotGuard g(*this, slot);
  if (scratch_bytes) ensure_scratch(slot, scratch_bytes);
  exchange.advance();   // kernels with fused exchanges wait for the arrival counts of this submission
  return timed(slot, n_calls, flops, [&](cudaStream_t st) {
    exchange.stage(st, pos_stage_of(slot.counters));
    for (const Launch &l : plan) l(slot, st);
  });
}

// One submission with a pair of events around every planned launch: per_launch receives
// (index of the launch's first source op, device nanoseconds).  Diagnostics only: the events
// between launches remove the overlap programmatic dependent launch gives the plain path.
RunStats Executor::run_exec_ops_timed(const std::vector<ExecOp> &ops, std::vector<std::pair<size_t, uint64_t>> *per_launch) {
  uint64_t flops = 0;
  size_t n_calls = 0, scratch_bytes = 0;
  std::vector<size_t> first_op;
  ExchangeUse exchange;
  std::vector<Launch> plan = plan_exec_ops(ops, &flops, &n_calls, &scratch_bytes, &first_op, &exchange);
  ctx_->make_current();
  Slot &slot = checkout_slot();
  SlotGuard g(*this, slot);
  if (scratch_bytes) ensure_scratch(slot, scratch_bytes);
  exchange.advance();
  std::vector<cudaEvent_t> ev(plan.size() + 1);
  for (cudaEvent_t &e : ev) TA_CUDA(cudaEventCreate(&e));
  RunStats st;
  try {
    st = timed(slot, n_calls, flops, [&](cudaStream_t s) {
      exchange.stage(s, pos_stage_of(slot.counters));
      for (size_t i = 0; i < plan.size(); ++i) {
        TA_CUDA(cudaEventRecord(ev[i], s));
        plan[i](slot, s);
      }
      TA_CUDA(cudaEventRecord(ev[plan.size()], s));
    });
    if (per_launch) {
      per_launch->clear();
      for (size_t i = 0; i < plan.size(); ++i) {
        float ms = 0.0f;
        TA_CUDA(cudaEventElapsedTime(&ms, ev[i], ev[i + 1]));
        per_launch->emplace_back(first_op[i], (uint64_t)((double)ms * 1e6 + 0.5));
      }
    }
  } catch (...) {
    for (cudaEvent_t e : ev) cudaEventDestroy(e);
    throw;
  }
  for (cudaEvent_t e : ev) cudaEventDestroy(e);
  return st;
}

RunStats Executor::run_single(const ExecOp &op) { return run_exec_ops({op}); }

void Executor::selftest_bounded_wait(uint32_t limit_ns) {
  ctx_->make_current();
  Slot &slot = checkout_slot();
  SlotGuard g(*this, slot);
  timed(slot, 1, 0, [&](cudaStream_t st) { launch_bounded_wait_probe(slot.status, limit_ns, st); });
}

std::unique_ptr<PreparedOps> prepare_exec_ops(Executor &exec, const std::vector<ExecOp> &ops) {
  if (ops.empty()) fail("prepare_exec_ops: empty op list");
  exec.context()->make_current();
  auto prep = std::make_unique<PreparedOps>();
  prep->exec = &exec;
  prep->ctx = exec.context();
  size_t scratch_bytes = 0;
  std::vector<Launch> plan = exec.plan_exec_ops(ops, &prep->total_flops, &prep->n_calls, &scratch_bytes, nullptr,
                                                &prep->exchange);
  if (scratch_bytes) TA_CUDA(cudaMalloc(&prep->scratch, scratch_bytes));
  TA_CUDA(cudaStreamCreateWithFlags(&prep->stream, cudaStreamNonBlocking));
  TA_CUDA(cudaEventCreate(&prep->ev_begin));
  TA_CUDA(cudaEventCreate(&prep->ev_end));
  TA_CUDA(cudaMalloc((void **)&prep->counters, SLOT_WORDS * sizeof(uint32_t)));
  TA_CUDA(cudaMemset(prep->counters, 0, SLOT_WORDS * sizeof(uint32_t)));
  alloc_status_word(&prep->status_host, &prep->status);
  Slot &real_slot = exec.checkout_slot();
  {
    SlotGuard g(exec, real_slot);
    // the captured launches must not point at state another submission may use later
    Slot slot = real_slot;
    slot.counters = prep->counters;
    slot.scratch = prep->scratch;
    slot.scratch_bytes = scratch_bytes;
    slot.status = prep->status;
    slot.status_host = prep->status_host;
    // Recorded only, as the reference's prepare_exec_ops does (src/executor/graph_ops.rs:249-353):
    // nothing executes until the first run, so accumulating ops, in-place residuals, cache appends
    // and the argmax cell are untouched by creating the object.  First-use set-up (function
    // attributes, tensor maps) consists of host calls, which a capture allows.
    TA_CUDA(cudaStreamBeginCapture(prep->stream, cudaStreamCaptureModeThreadLocal));
    try {
      prep->exchange.stage(prep->stream, pos_stage_of(slot.counters));
      for (const Launch &l : plan) l(slot, prep->stream);
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

// ------------------------------------------------------------------ single-op entry points
RunStats Executor::softmax_rows(const Tensor &in, const Tensor &out, float scale, uint32_t mask_kind,
                                uint32_t valid_or_prefix, uint32_t rows_per_group) {
  ExecOp o;
  o.kind = ExecKind::SoftmaxRows;
  o.in0 = &in; o.out = &out; o.f0 = scale; o.u0 = mask_kind; o.u1 = valid_or_prefix; o.u2 = rows_per_group;
  return run_single(o);
}
RunStats Executor::rms_norm(const Tensor &in, const Tensor &w, const Tensor &out, float eps) {
  ExecOp o;
  o.kind = ExecKind::RmsNorm;
  o.in0 = &in; o.in1 = &w; o.out = &out; o.f0 = eps;
  return run_single(o);
}
RunStats Executor::layer_norm(const Tensor &in, const Tensor &w, const Tensor &b, const Tensor &out, float eps) {
  ExecOp o;
  o.kind = ExecKind::LayerNorm;
  o.in0 = &in; o.in1 = &w; o.in2 = &b; o.out = &out; o.f0 = eps;
  return run_single(o);
}
RunStats Executor::rope(const Tensor &in, const Tensor &table, const Tensor &out, uint32_t heads,
                        uint32_t head_dim, uint32_t rot_dim, uint32_t pos_base) {
  ExecOp o;
  o.kind = ExecKind::Rope;
  o.in0 = &in; o.in1 = &table; o.out = &out;
  o.heads = heads; o.head_dim = head_dim; o.rot_dim = rot_dim; o.pos_base = pos_base;
  return run_single(o);
}
RunStats Executor::rope_scatter(const Tensor &in, const Tensor &table, const Tensor &dst, uint32_t heads,
                                uint32_t head_dim, uint32_t rot_dim, uint32_t pos_base, uint32_t dst_offset,
                                const uint32_t strides[3], uint32_t pos_scale, const PosCell *cell) {
  ExecOp o;
  o.kind = ExecKind::RopeScatter;
  o.in0 = &in; o.in1 = &table; o.out = &dst;
  o.heads = heads; o.head_dim = head_dim; o.rot_dim = rot_dim; o.pos_base = pos_base;
  o.dst_offset = dst_offset; o.pos_scale = pos_scale; o.cell = cell;
  for (int i = 0; i < 3; ++i) o.strides[i] = strides[i];
  return run_single(o);
}
RunStats Executor::copy_strided(const Tensor &src, const Tensor &dst, const uint32_t extent[3],
                                uint32_t src_off, const uint32_t src_strides[3], uint32_t dst_off,
                                const uint32_t dst_strides[3]) {
  ExecOp o;
  o.kind = ExecKind::CopyStrided;
  o.in0 = &src; o.out = &dst; o.src_offset = src_off; o.dst_offset = dst_off;
  for (int i = 0; i < 3; ++i) {
    o.extent[i] = extent[i];
    o.src_strides[i] = src_strides[i];
    o.strides[i] = dst_strides[i];
  }
  return run_single(o);
}
RunStats Executor::binary(const Tensor &a, const Tensor &b, const Tensor &out, uint32_t mode, float beta) {
  ExecOp o;
  o.kind = ExecKind::Binary;
  o.in0 = &a; o.in1 = &b; o.out = &out; o.u0 = mode; o.f0 = beta;
  return run_single(o);
}
RunStats Executor::argmax(const Tensor &in, const PosCell &result) {
  ExecOp o;
  o.kind = ExecKind::Argmax;
  o.in0 = &in; o.cell = &result;
  return run_single(o);
}
RunStats Executor::embed_gather(const PosCell &token, const Tensor &table, const Tensor &out) {
  ExecOp o;
  o.kind = ExecKind::EmbedGather;
  o.cell = &token; o.in0 = &table; o.out = &out;
  return run_single(o);
}
RunStats Executor::embed_gather_rows(const TokenIds &tokens, const Tensor &table, const Tensor &out) {
  ExecOp o;
  o.kind = ExecKind::EmbedGatherRows;
  o.tokens = &tokens; o.in0 = &table; o.out = &out;
  return run_single(o);
}
RunStats Executor::flash_attention(const Tensor &q, const Tensor &kt, const Tensor &v, const Tensor &out,
                                   const FlashAttentionDesc &desc) {
  ExecOp o;
  o.kind = ExecKind::FlashAttn;
  o.in0 = &q; o.in1 = &kt; o.in2 = &v; o.out = &out; o.flash = desc;
  return run_single(o);
}
RunStats Executor::attn_decode(const Tensor &q, const Tensor &kt, const Tensor &v, const Tensor &scratch,
                               const Tensor &out, const AttnDecodeDesc &desc) {
  ExecOp o;
  o.kind = ExecKind::AttnDecode;
  o.in0 = &q; o.in1 = &kt; o.in2 = &v; o.in3 = &scratch; o.out = &out; o.attn = desc;
  return run_single(o);
}

}  // namespace ta
