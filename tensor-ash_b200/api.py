"""Host-side mirror of the reference crate's public API, over the C ABI.

Reference types mirrored (paths in the reference project):
  Executor / ExecutorConfig      src/executor/mod.rs:85-369
  Tensor                         src/tensor.rs:20-201
  MatmulCall / MatmulOp / Epilogue / Activation / EpilogueBinary / RunStats
                                 src/matmul/api.rs:3-353
  PreparedOps                    src/executor/prepared.rs:46-353
  DispatchInfo                   src/executor/mod.rs:61-81
Errors surface as :class:`TensorAshError` carrying ``ta_last_error()``, the
analogue of the crate's ``anyhow::Result`` failures.
"""
from __future__ import annotations

import ctypes as C
import enum
import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

from . import capi
from .capi import lib


class TensorAshError(RuntimeError):
    pass


def _err() -> str:
    return (lib().ta_last_error() or b"").decode("utf-8", "replace")


def _check(rc: int) -> None:
    if rc != 0:
        raise TensorAshError(_err())


def version() -> str:
    return lib().ta_version().decode()


class Activation(enum.IntEnum):
    NONE = 0
    RELU = 1
    SILU = 2
    GELU = 3


class Binary(enum.IntEnum):
    NONE = 0
    ADD_SCALED = 1
    MUL = 2


@dataclass
class RunStats:
    gpu_time_ns: Optional[int]
    n_calls: int
    total_flops: int

    def tflops(self) -> Optional[float]:
        if not self.gpu_time_ns:
            return None
        return self.total_flops / self.gpu_time_ns * 1e-3

    @staticmethod
    def _from(c: capi.RunStatsC) -> "RunStats":
        return RunStats(int(c.gpu_time_ns) if c.has_gpu_time else None, int(c.n_calls),
                        int(c.total_flops))


@dataclass
class DispatchInfo:
    kernel: str
    tile: tuple
    split_k2: Optional[int]


class Context:
    """A CUDA device (``VulkanContext`` in the reference)."""

    def __init__(self, validation: bool = False, device: Optional[str] = "auto"):
        h = lib().ta_context_create(int(validation), device.encode() if device is not None else None)
        if not h:
            raise TensorAshError(_err())
        self._h = h

    @property
    def supports_f16(self) -> bool:
        return bool(lib().ta_context_supports_f16(self._h))

    @property
    def supports_bda(self) -> bool:
        return bool(lib().ta_context_supports_bda(self._h))

    @property
    def device_index(self) -> int:
        return int(lib().ta_context_device_index(self._h))

    @property
    def device_name(self) -> str:
        return (lib().ta_context_device_name(self._h) or b"").decode()

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().ta_context_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _shape_arr(shape: Sequence[int]):
    return (C.c_uint32 * len(shape))(*[int(d) for d in shape]), len(shape)


class Tensor:
    """Row-major contiguous device tensor, f32 or f16 storage."""

    def __init__(self, handle, ctx: Context, shape, keepalive=None):
        self._h = handle
        self.ctx = ctx
        self.shape = tuple(int(d) for d in shape)
        self._keepalive = keepalive

    @staticmethod
    def uninit_device(ctx: Context, shape) -> "Tensor":
        arr, rank = _shape_arr(shape)
        h = lib().ta_tensor_create(ctx._h, arr, rank)
        if not h:
            raise TensorAshError(_err())
        return Tensor(h, ctx, shape)

    @staticmethod
    def uninit_device_f16(ctx: Context, shape) -> "Tensor":
        arr, rank = _shape_arr(shape)
        h = lib().ta_tensor_create_f16(ctx._h, arr, rank)
        if not h:
            raise TensorAshError(_err())
        return Tensor(h, ctx, shape)

    def alias_with_shape(self, shape) -> "Tensor":
        arr, rank = _shape_arr(shape)
        h = lib().ta_tensor_alias_with_shape(self._h, arr, rank)
        if not h:
            raise TensorAshError(_err())
        return Tensor(h, self.ctx, shape, keepalive=self)

    def len(self) -> int:
        return int(lib().ta_tensor_len(self._h))

    def size_bytes(self) -> int:
        return int(lib().ta_tensor_size_bytes(self._h))

    @property
    def is_f16(self) -> bool:
        return bool(lib().ta_tensor_is_f16(self._h))

    @property
    def device_ptr(self) -> int:
        return int(lib().ta_tensor_device_ptr(self._h) or 0)

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().ta_tensor_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


@dataclass
class MatmulCall:
    a: Tensor
    b: Tensor
    c: Tensor
    alpha: float = 1.0
    accumulate: bool = False

    def _c(self) -> capi.MatmulCallC:
        return capi.MatmulCallC(self.a._h, self.b._h, self.c._h, self.alpha, int(self.accumulate))


@dataclass
class Epilogue:
    bias: Optional[Tensor] = None
    activation: Activation = Activation.NONE
    binary: Binary = Binary.NONE
    d: Optional[Tensor] = None
    beta: float = 0.0

    def _c(self) -> capi.EpilogueC:
        return capi.EpilogueC(self.bias._h if self.bias is not None else None, int(self.activation),
                              int(self.binary), self.d._h if self.d is not None else None, self.beta)


@dataclass
class MatmulOp:
    call: MatmulCall
    epilogue: Epilogue = field(default_factory=Epilogue)

    def _c(self) -> capi.MatmulOpC:
        return capi.MatmulOpC(self.call._c(), self.epilogue._c())


class StoreKind(enum.IntEnum):
    NONE = 0
    ROPE = 1
    SCATTER = 2
    ROPE_SCATTER = 3


class PosCell:
    """4-byte host-visible cell read by kernels at run time (PosBuffer in the reference)."""

    def __init__(self, ctx: Context):
        h = lib().ta_pos_cell_create(ctx._h)
        if not h:
            raise TensorAshError(_err())
        self._h = h
        self.ctx = ctx

    def set(self, value: int) -> None:
        _check(lib().ta_pos_cell_set(self._h, value))

    def get(self) -> int:
        v = C.c_uint32(0)
        _check(lib().ta_pos_cell_get(self._h, C.byref(v)))
        return int(v.value)

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().ta_pos_cell_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


@dataclass
class MatmulStore:
    """Fused store of an M == 1 f16-weight GEMV (MatmulStore / MatmulStoreDesc in the reference)."""
    kind: StoreKind = StoreKind.NONE
    head_dim: int = 0
    pos_base: int = 0
    pos_scale: int = 0
    stride_head: int = 0
    stride_dim: int = 0
    table: Optional[Tensor] = None
    dst: Optional[Tensor] = None
    pos_cell: Optional[PosCell] = None

    def _c(self) -> capi.StoreDescC:
        return capi.StoreDescC(int(self.kind), self.head_dim, self.pos_base, self.pos_scale, self.stride_head,
                               self.stride_dim, self.table._h if self.table is not None else None,
                               self.dst._h if self.dst is not None else None,
                               self.pos_cell._h if self.pos_cell is not None else None)


@dataclass
class MatmulOpEx:
    """MatmulOp plus packed-B, normed-A and fused-store fields (with_packed_b /
    with_normed_a / with_store_* in the reference, src/matmul/api.rs:120-306)."""
    call: MatmulCall
    epilogue: Epilogue = field(default_factory=Epilogue)
    packed_b: bool = False
    normed_a: Optional[tuple] = None      # (weight tensor, eps)
    store: MatmulStore = field(default_factory=MatmulStore)

    def _c(self) -> capi.MatmulOpExC:
        w, eps = self.normed_a if self.normed_a is not None else (None, 0.0)
        return capi.MatmulOpExC(capi.MatmulOpC(self.call._c(), self.epilogue._c()), int(self.packed_b),
                                w._h if w is not None else None, eps, self.store._c())


class TokenIdBuffer:
    """Token-id list in host-visible memory (TokenIdBuffer in the reference)."""

    def __init__(self, ctx: Context, capacity: int):
        h = lib().ta_token_ids_create(ctx._h, capacity)
        if not h:
            raise TensorAshError(_err())
        self._h = h
        self.ctx = ctx

    def set(self, tokens) -> None:
        arr = np.ascontiguousarray(tokens, dtype=np.uint32)
        _check(lib().ta_token_ids_set(self._h, arr.ctypes.data, arr.size))

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().ta_token_ids_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Comm:
    """Communicator of a tensor-parallel group: one rank per process and GPU, NCCL underneath.

    ``Comm.unique_id()`` on rank 0 makes the 128-byte id; every rank receives it out of band
    (``from_torch_distributed`` broadcasts it over an initialised ``torch.distributed``
    group) and constructs its ``Comm`` collectively.  ``world == 1`` needs neither id nor NCCL.
    """

    ID_BYTES = 128

    def __init__(self, ctx: Context, rank: int, world: int, unique_id: Optional[bytes] = None):
        buf = None
        if world > 1:
            if unique_id is None or len(unique_id) != self.ID_BYTES:
                raise TensorAshError("Comm: a 128-byte unique id is required when world > 1")
            buf = (C.c_uint8 * self.ID_BYTES).from_buffer_copy(unique_id)
        h = lib().ta_comm_create(ctx._h, rank, world, buf)
        if not h:
            raise TensorAshError(_err())
        self._h, self.ctx, self.rank, self.world = h, ctx, rank, world

    @staticmethod
    def unique_id() -> bytes:
        buf = (C.c_uint8 * Comm.ID_BYTES)()
        _check(lib().ta_comm_unique_id(buf))
        return bytes(buf)

    @classmethod
    def from_torch_distributed(cls, ctx: Context) -> "Comm":
        """Collective over the default torch.distributed group (any backend)."""
        import torch
        import torch.distributed as dist

        rank, world = dist.get_rank(), dist.get_world_size()
        if world == 1:
            return cls(ctx, 0, 1)
        on_gpu = dist.get_backend() == "nccl"
        t = torch.zeros(cls.ID_BYTES, dtype=torch.uint8, device="cuda" if on_gpu else "cpu")
        if rank == 0:
            t.copy_(torch.frombuffer(bytearray(cls.unique_id()), dtype=torch.uint8))
        dist.broadcast(t, src=0)
        return cls(ctx, rank, world, bytes(t.cpu().numpy().tobytes()))

    def set_wait_limit_ns(self, limit_ns: int) -> None:
        """How long a rank waits on the device for a peer's flag before the call fails."""
        _check(lib().ta_comm_set_wait_limit_ns(self._h, limit_ns))

    def resync(self) -> None:
        """Collective: brings the peer exchange back to a common state after a failed wait."""
        _check(lib().ta_comm_resync(self._h))

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().ta_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ExecKind(enum.IntEnum):
    MATMUL = 0
    RMS_NORM = 1
    LAYER_NORM = 2
    SOFTMAX_ROWS = 3
    ROPE = 4
    ROPE_SCATTER = 5
    COPY_STRIDED = 6
    BINARY = 7
    ATTN_DECODE = 8
    FLASH_ATTN = 9
    ARGMAX = 10
    EMBED_GATHER = 11
    EMBED_GATHER_ROWS = 12
    ALL_REDUCE = 13
    ALL_GATHER = 14
    PREFILL_QKV_PACK = 15
    ARGMAX_SHARDED = 16


class ExecOp:
    """One op of a mixed graph (ExecOp in the reference, src/executor/graph_ops.rs:27-161).
    Build with the class methods; keeps its operands alive."""

    def __init__(self, kind: ExecKind, **kw):
        self.c = capi.ExecOpC()
        self.c.kind = int(kind)
        self._keep = []
        for name in ("in0", "in1", "in2", "in3", "out"):
            t = kw.get(name)
            if t is not None:
                setattr(self.c, name, t._h)
                self._keep.append(t)
        self.c.f0 = kw.get("f0", 0.0)
        for name in ("u0", "u1", "u2", "dst_offset", "pos_scale"):
            setattr(self.c, name, int(kw.get(name, 0)))
        if "dst_strides" in kw:
            self.c.dst_strides = (C.c_uint32 * 3)(*kw["dst_strides"])
        if "rope" in kw:
            self.c.rope = capi.RopeDescC(*kw["rope"])
        if "copy" in kw:
            ext, so, ss, do, ds = kw["copy"]
            self.c.copy = capi.CopyDescC((C.c_uint32 * 3)(*ext), so, (C.c_uint32 * 3)(*ss), do, (C.c_uint32 * 3)(*ds))
        if "flash" in kw:
            self.c.flash = capi.FlashDescC(*kw["flash"])
        if "attn" in kw:
            kv_len, scale, cell = kw["attn"]
            self.c.attn = capi.AttnDecodeDescC(kv_len, scale, cell._h if cell is not None else None)
            self._keep.append(cell)
        for name in ("cell", "tokens", "comm"):
            obj = kw.get(name)
            if obj is not None:
                setattr(self.c, name, obj._h)
                self._keep.append(obj)
        if "mm" in kw:
            op = kw["mm"]
            self.c.mm = op._c() if isinstance(op, MatmulOpEx) else MatmulOpEx(op.call, op.epilogue)._c()
            self._keep.append(op)

    @classmethod
    def matmul(cls, op):
        return cls(ExecKind.MATMUL, mm=op)

    @classmethod
    def rms_norm(cls, inp, weight, out, eps):
        return cls(ExecKind.RMS_NORM, in0=inp, in1=weight, out=out, f0=eps)

    @classmethod
    def layer_norm(cls, inp, weight, bias, out, eps):
        return cls(ExecKind.LAYER_NORM, in0=inp, in1=weight, in2=bias, out=out, f0=eps)

    @classmethod
    def softmax_rows(cls, inp, out, scale=1.0, mask_kind=0, valid_or_prefix=0, rows_per_group=0):
        return cls(ExecKind.SOFTMAX_ROWS, in0=inp, out=out, f0=scale, u0=mask_kind, u1=valid_or_prefix, u2=rows_per_group)

    @classmethod
    def rope(cls, inp, table, out, heads, head_dim, rot_dim, pos_base=0):
        return cls(ExecKind.ROPE, in0=inp, in1=table, out=out, rope=(heads, head_dim, rot_dim, pos_base))

    @classmethod
    def rope_scatter(cls, inp, table, dst, heads, head_dim, rot_dim, pos_base, dst_offset, dst_strides,
                     pos_scale=0, cell=None):
        return cls(ExecKind.ROPE_SCATTER, in0=inp, in1=table, out=dst, rope=(heads, head_dim, rot_dim, pos_base),
                   dst_offset=dst_offset, dst_strides=dst_strides, pos_scale=pos_scale, cell=cell)

    @classmethod
    def copy_strided(cls, src, dst, extent, src_offset, src_strides, dst_offset, dst_strides):
        return cls(ExecKind.COPY_STRIDED, in0=src, out=dst, copy=(extent, src_offset, src_strides, dst_offset, dst_strides))

    @classmethod
    def binary_add_scaled(cls, a, b, out, beta):
        return cls(ExecKind.BINARY, in0=a, in1=b, out=out, u0=0, f0=beta)

    @classmethod
    def binary_silu_mul(cls, a, b, out):
        return cls(ExecKind.BINARY, in0=a, in1=b, out=out, u0=1)

    @classmethod
    def attn_decode(cls, q, kt, v, scratch, out, kv_len, scale, pos_cell=None):
        return cls(ExecKind.ATTN_DECODE, in0=q, in1=kt, in2=v, in3=scratch, out=out, attn=(kv_len, scale, pos_cell))

    @classmethod
    def flash_attn(cls, q, kt, v, out, kv_len, pos_base, scale, token_major_heads=0, out_token_major_heads=0,
                   simt=False):
        return cls(ExecKind.FLASH_ATTN, in0=q, in1=kt, in2=v, out=out,
                   flash=(kv_len, pos_base, scale, token_major_heads, out_token_major_heads, int(simt)))

    @classmethod
    def argmax(cls, inp, result_cell):
        return cls(ExecKind.ARGMAX, in0=inp, cell=result_cell)

    @classmethod
    def embed_gather(cls, token_cell, table, out):
        return cls(ExecKind.EMBED_GATHER, cell=token_cell, in0=table, out=out)

    @classmethod
    def embed_gather_rows(cls, tokens, table, out):
        return cls(ExecKind.EMBED_GATHER_ROWS, tokens=tokens, in0=table, out=out)

    @classmethod
    def prefill_qkv_pack(cls, qkv, table, q, kt, v, heads, kv_heads, head_dim, rot_dim, pos_base=0):
        """RoPE(q) head-major, RoPE(k) into the Kt cache, v into the V cache, from one [T, n_qkv] row."""
        return cls(ExecKind.PREFILL_QKV_PACK, in0=qkv, in1=table, in2=kt, in3=v, out=q,
                   rope=(heads, head_dim, rot_dim, pos_base), u0=kv_heads)

    @classmethod
    def argmax_sharded(cls, inp, index_offset, result_cell, comm):
        return cls(ExecKind.ARGMAX_SHARDED, in0=inp, u0=index_offset, cell=result_cell, comm=comm)

    @classmethod
    def all_reduce(cls, tensor, comm):
        """Sum `tensor` (f32) in place over the ranks of `comm`."""
        return cls(ExecKind.ALL_REDUCE, out=tensor, comm=comm)

    @classmethod
    def all_gather(cls, src, dst, comm):
        """dst [world * n] = every rank's src [n], in rank order."""
        return cls(ExecKind.ALL_GATHER, in0=src, out=dst, comm=comm)


def _exec_array(ops):
    arr = (capi.ExecOpC * max(len(ops), 1))()
    for i, op in enumerate(ops):
        arr[i] = op.c
    return arr


def _ops_array(ops: Sequence[MatmulOp]):
    arr = (capi.MatmulOpC * max(len(ops), 1))()
    for i, op in enumerate(ops):
        arr[i] = op._c()
    return arr


class PreparedOps:
    """Record-once / replay-many op batch (a captured CUDA graph)."""

    def __init__(self, handle, keepalive):
        self._h = handle
        self._keepalive = keepalive

    def run(self) -> RunStats:
        st = capi.RunStatsC()
        _check(lib().ta_prepared_run(self._h, C.byref(st)))
        return RunStats._from(st)

    def submit(self) -> None:
        _check(lib().ta_prepared_submit(self._h))

    def wait(self) -> RunStats:
        st = capi.RunStatsC()
        _check(lib().ta_prepared_wait(self._h, C.byref(st)))
        return RunStats._from(st)

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().ta_prepared_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Executor:
    """Validates, routes and submits ops on one device."""

    def __init__(self, ctx: Context, n_slots: int = 2, max_calls_per_submit: int = 16,
                 kernel: Optional[str] = "auto", tune: bool = False):
        sel = kernel.encode() if kernel is not None else None
        h = lib().ta_executor_create_v2(ctx._h, n_slots, max_calls_per_submit, sel, int(tune))
        if not h:
            raise TensorAshError(_err())
        self._h = h
        self.ctx = ctx

    # ---- transfers (host side is always f32)
    def upload(self, src: np.ndarray, dst: Tensor) -> None:
        src = np.ascontiguousarray(src, dtype=np.float32)
        _check(lib().ta_upload(self._h, dst._h, src.ctypes.data, src.size))

    def upload_f16(self, src: np.ndarray, dst: Tensor) -> None:
        src = np.ascontiguousarray(src, dtype=np.uint16)
        _check(lib().ta_upload_f16(self._h, dst._h, src.ctypes.data, src.size))

    def download(self, src: Tensor, n: Optional[int] = None) -> np.ndarray:
        n = src.len() if n is None else n
        out = np.empty(n, dtype=np.float32)
        _check(lib().ta_download(self._h, src._h, out.ctypes.data, n))
        return out.reshape(src.shape) if n == src.len() else out

    def download_into(self, src: Tensor, out: np.ndarray) -> None:
        assert out.dtype == np.float32 and out.flags.c_contiguous
        _check(lib().ta_download(self._h, src._h, out.ctypes.data, out.size))

    # ---- GEMM
    def run_matmuls(self, calls: Sequence[MatmulCall]) -> RunStats:
        arr = (capi.MatmulCallC * max(len(calls), 1))()
        for i, c in enumerate(calls):
            arr[i] = c._c()
        st = capi.RunStatsC()
        _check(lib().ta_matmul_batch(self._h, arr, len(calls), C.byref(st)))
        return RunStats._from(st)

    def matmul(self, a: Tensor, b: Tensor, c: Tensor, alpha: float = 1.0,
               accumulate: bool = False) -> RunStats:
        st = capi.RunStatsC()
        _check(lib().ta_matmul(self._h, a._h, b._h, c._h, alpha, int(accumulate), C.byref(st)))
        return RunStats._from(st)

    def run_ops(self, ops: Sequence[MatmulOp]) -> RunStats:
        st = capi.RunStatsC()
        _check(lib().ta_run_ops(self._h, _ops_array(ops), len(ops), C.byref(st)))
        return RunStats._from(st)

    def run_matmul_host_batched(self, a: np.ndarray, b, c: np.ndarray, *, bias: Optional[np.ndarray] = None,
                                d: Optional[np.ndarray] = None, activation: int = 0, binary: int = 0,
                                alpha: float = 1.0, beta: float = 0.0, chunk_batch: int = 0) -> RunStats:
        """``c[i] = epilogue(alpha * a[i] @ b)`` with ``a`` [batch, M, K], ``d`` and ``c`` [batch, M, N]
        and ``bias`` ([N] or [batch, N]) in host memory; ``b`` is a device :class:`Tensor` [K, N] or a
        host array.  Copies in, compute and copies out are pipelined over chunks of the batch (pin
        the arrays, e.g. with :func:`pinned_empty`, for them to overlap).  Bit-identical to
        upload + run_ops + download applied chunk by chunk."""
        def host(x, name, shape=None):
            if x.dtype != np.float32 or not x.flags.c_contiguous:
                raise TypeError(f"{name} must be a C-contiguous float32 array")
            if shape is not None and tuple(x.shape) != tuple(shape):
                raise ValueError(f"{name} has shape {tuple(x.shape)}, expected {tuple(shape)}")
            return x.ctypes.data
        if a.ndim != 3:
            raise ValueError("a must be [batch, M, K]")
        batch, m, k = (int(v) for v in a.shape)
        n = int(c.shape[-1])
        desc = capi.HostBatchedMatmulC()
        desc.batch, desc.m, desc.n, desc.k = batch, m, n, k
        desc.a = host(a, "a")
        if isinstance(b, Tensor):
            desc.b, desc.b_host = b._h, None
        else:
            desc.b, desc.b_host = None, host(b, "b", (k, n))
        if not c.flags.writeable:
            raise TypeError("c must be writeable")
        desc.c = host(c, "c", (batch, m, n))
        if bias is not None:
            if bias.ndim == 2:
                desc.bias, desc.bias_per_batch = host(bias, "bias", (batch, n)), 1
            else:
                desc.bias, desc.bias_per_batch = host(bias, "bias", (n,)), 0
        if d is not None:
            desc.d = host(d, "d", (batch, m, n))
        desc.activation, desc.binary = int(activation), int(binary)
        desc.alpha, desc.beta, desc.chunk_batch = float(alpha), float(beta), int(chunk_batch)
        st = capi.RunStatsC()
        _check(lib().ta_run_matmul_host_batched(self._h, C.byref(desc), C.byref(st)))
        return RunStats._from(st)

    def run_op_graph(self, ops: Sequence[MatmulOp]) -> RunStats:
        st = capi.RunStatsC()
        _check(lib().ta_run_op_graph(self._h, _ops_array(ops), len(ops), C.byref(st)))
        return RunStats._from(st)

    def run_ops_ex(self, ops: Sequence["MatmulOpEx"], as_graph: bool = False) -> RunStats:
        arr = (capi.MatmulOpExC * max(len(ops), 1))()
        for i, op in enumerate(ops):
            arr[i] = op._c()
        st = capi.RunStatsC()
        _check(lib().ta_run_ops_ex(self._h, arr, len(ops), int(as_graph), C.byref(st)))
        return RunStats._from(st)

    def swiglu_gemv(self, x: Tensor, wg: Tensor, wup: Tensor, out: Tensor, normed_weight: Optional[Tensor] = None,
                    eps: float = 0.0) -> RunStats:
        st = capi.RunStatsC()
        _check(lib().ta_swiglu_gemv(self._h, x._h, wg._h, wup._h, out._h,
                                    normed_weight._h if normed_weight is not None else None, eps, C.byref(st)))
        return RunStats._from(st)

    def run_exec_ops(self, ops) -> RunStats:
        st = capi.RunStatsC()
        _check(lib().ta_run_exec_ops(self._h, _exec_array(ops), len(ops), C.byref(st)))
        return RunStats._from(st)

    def prepare_exec_ops(self, ops) -> PreparedOps:
        h = lib().ta_prepared_create_exec(self._h, _exec_array(ops), len(ops))
        if not h:
            raise TensorAshError(_err())
        return PreparedOps(h, (self, list(ops)))

    def run_flash_attention(self, q: Tensor, kt: Tensor, v: Tensor, out: Tensor, kv_len: int, pos_base: int,
                            scale: float, token_major_heads: int = 0, out_token_major_heads: int = 0,
                            simt: bool = False) -> RunStats:
        st = capi.RunStatsC()
        desc = capi.FlashDescC(kv_len, pos_base, scale, token_major_heads, out_token_major_heads, int(simt))
        _check(lib().ta_flash_attention(self._h, q._h, kt._h, v._h, out._h, C.byref(desc), C.byref(st)))
        return RunStats._from(st)

    def run_attn_decode(self, q: Tensor, kt: Tensor, v: Tensor, scratch: Tensor, out: Tensor, kv_len: int,
                        scale: float, pos_cell: Optional["PosCell"] = None) -> RunStats:
        st = capi.RunStatsC()
        desc = capi.AttnDecodeDescC(kv_len, scale, pos_cell._h if pos_cell is not None else None)
        _check(lib().ta_attn_decode(self._h, q._h, kt._h, v._h, scratch._h, out._h, C.byref(desc), C.byref(st)))
        return RunStats._from(st)

    def run_matmuls_split_k2(self, calls: Sequence[MatmulCall], splits: int = 0) -> RunStats:
        arr = (capi.MatmulCallC * max(len(calls), 1))()
        for i, c in enumerate(calls):
            arr[i] = c._c()
        st = capi.RunStatsC()
        _check(lib().ta_matmul_split_k2(self._h, arr, len(calls), splits, C.byref(st)))
        return RunStats._from(st)

    def prepare_ops(self, ops: Sequence[MatmulOp], as_graph: bool = False) -> PreparedOps:
        h = lib().ta_prepared_create(self._h, _ops_array(ops), len(ops), int(as_graph))
        if not h:
            raise TensorAshError(_err())
        return PreparedOps(h, (self, list(ops)))

    # ---- routing
    def dispatch_info_for(self, batch: int, m: int, n: int, k: int, b_f16: bool = False) -> DispatchInfo:
        out = capi.DispatchInfoC()
        _check(lib().ta_dispatch_info_for(self._h, batch, m, n, k, int(b_f16), C.byref(out)))
        return DispatchInfo(out.kernel.decode(), tuple(out.tile),
                            int(out.split_k2_splits) if out.has_split_k2 else None)

    def tune_shape(self, batch: int, m: int, n: int, k: int, b_f16: bool = False) -> None:
        fn = lib().ta_tune_shape_f16w if b_f16 else lib().ta_tune_shape
        _check(fn(self._h, batch, m, n, k))

    def selftest_bounded_wait(self, limit_ns: int) -> None:
        """Launches the bounded-wait self-test kernel; always raises the bounded-wait error."""
        _check(lib().ta_selftest_bounded_wait(self._h, limit_ns))

    # ---- model ops
    def softmax_rows(self, inp: Tensor, out: Tensor, scale: float = 1.0, mask_kind: int = 0,
                     valid_or_prefix: int = 0, rows_per_group: int = 0) -> RunStats:
        st = capi.RunStatsC()
        _check(lib().ta_softmax_rows(self._h, inp._h, out._h, scale, mask_kind, valid_or_prefix,
                                     rows_per_group, C.byref(st)))
        return RunStats._from(st)

    def rms_norm(self, inp: Tensor, weight: Tensor, out: Tensor, eps: float) -> RunStats:
        st = capi.RunStatsC()
        _check(lib().ta_rms_norm(self._h, inp._h, weight._h, out._h, eps, C.byref(st)))
        return RunStats._from(st)

    def layer_norm(self, inp: Tensor, weight: Tensor, bias: Tensor, out: Tensor, eps: float) -> RunStats:
        st = capi.RunStatsC()
        _check(lib().ta_layer_norm(self._h, inp._h, weight._h, bias._h, out._h, eps, C.byref(st)))
        return RunStats._from(st)

    def rope(self, inp: Tensor, table: Tensor, out: Tensor, heads: int, head_dim: int, rot_dim: int,
             pos_base: int = 0) -> RunStats:
        st = capi.RunStatsC()
        desc = capi.RopeDescC(heads, head_dim, rot_dim, pos_base)
        _check(lib().ta_rope(self._h, inp._h, table._h, out._h, C.byref(desc), C.byref(st)))
        return RunStats._from(st)

    def copy_strided(self, src: Tensor, dst: Tensor, extent, src_offset, src_strides, dst_offset,
                     dst_strides) -> RunStats:
        st = capi.RunStatsC()
        desc = capi.CopyDescC((C.c_uint32 * 3)(*extent), src_offset, (C.c_uint32 * 3)(*src_strides),
                              dst_offset, (C.c_uint32 * 3)(*dst_strides))
        _check(lib().ta_copy_strided(self._h, src._h, dst._h, C.byref(desc), C.byref(st)))
        return RunStats._from(st)

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().ta_executor_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------- host-only helpers
def pack_f16w_row_tiles(src: np.ndarray, k: int, n: int, tile_n: int) -> np.ndarray:
    src = np.ascontiguousarray(src, dtype=np.float32).reshape(-1)
    if src.size != k * n:
        raise TensorAshError("pack_f16w_row_tiles: src len")
    out = np.empty_like(src)
    _check(lib().ta_pack_f16w_row_tiles(src.ctypes.data, out.ctypes.data, k, n, tile_n))
    return out


def f16w_row_tile_n(k: int, n: int) -> int:
    return int(lib().ta_f16w_row_tile_n(k, n))


class _PinnedBlock:
    """Owner of one page-locked allocation; freed when the last array viewing it is collected."""

    def __init__(self, nbytes: int):
        self.ptr = lib().ta_pinned_alloc(nbytes)
        if not self.ptr:
            raise TensorAshError(f"ta_pinned_alloc({nbytes}) failed")

    def __del__(self):
        ptr, self.ptr = getattr(self, "ptr", None), None
        if ptr:
            try:
                lib().ta_pinned_free(ptr)
            except Exception:
                pass


def pinned_empty(shape, dtype=np.float32) -> np.ndarray:
    """A page-locked NumPy array (for :meth:`Executor.run_matmul_host_batched` and fast transfers).
    The memory is released when the array and every view of it are gone."""
    dtype = np.dtype(dtype)
    count = int(np.prod(shape, dtype=np.int64))
    nbytes = max(count * dtype.itemsize, 1)
    block = _PinnedBlock(nbytes)
    buf = (C.c_char * nbytes).from_address(block.ptr)
    buf._owner = block            # every array made from buf keeps buf, and so the block, alive
    return np.frombuffer(buf, dtype=dtype, count=count).reshape(shape)


def f32_to_f16_bits(v: float) -> int:
    return int(lib().ta_f32_to_f16_bits(v))


def f16_bits_to_f32(bits: int) -> float:
    return float(lib().ta_f16_bits_to_f32(bits))


def default_num_k_splits(batch, m, n, k, tile_m, tile_n) -> int:
    return int(lib().ta_default_num_k_splits(batch, m, n, k, tile_m, tile_n))


def heuristic_splits(batch, m, n, k) -> Optional[int]:
    return int(lib().ta_heuristic_splits(batch, m, n, k)) or None


def heuristic_kernel(batch, m, n, k, weights_f16: bool = False, sm_count: int = 148) -> str:
    """Registry name the routing heuristic picks for a plain shape (no explicit selection, no tuned entry)."""
    return lib().ta_heuristic_kernel(batch, m, n, k, int(weights_f16), sm_count).decode()


def tune_median(samples) -> Optional[int]:
    """Median as the tuner takes it (src/executor/tuning.rs:319-331); None for no samples."""
    arr = (C.c_uint64 * max(1, len(samples)))(*samples)
    out = C.c_uint64()
    rc = lib().ta_tune_median(arr, len(samples), C.byref(out))
    if rc < 0:
        raise TensorAshError(_err())
    return None if rc == 1 else int(out.value)


def tune_candidate_at(length: int, round_: int, offset: int) -> int:
    return int(lib().ta_tune_candidate_at(length, round_, offset))


def tune_store_path(device_name: str) -> str:
    buf = C.create_string_buffer(4096)
    _check(lib().ta_tune_store_path(device_name.encode(), buf, 4096))
    return buf.value.decode()


def tune_store_rewrite(in_path: str, out_path: Optional[str] = None) -> int:
    """Loads a tuned-winner store as the executor does and (optionally) writes it back; returns the entries kept."""
    n = C.c_size_t()
    _check(lib().ta_tune_store_rewrite(in_path.encode(), out_path.encode() if out_path else None, C.byref(n)))
    return int(n.value)


def experiment_check(spec: str) -> None:
    _check(lib().ta_experiment_check(spec.encode()))


def kernel_specs():
    out = []
    for i in range(lib().ta_kernel_spec_count()):
        d = capi.DispatchInfoC()
        _check(lib().ta_kernel_spec_at(i, C.byref(d)))
        out.append((d.kernel.decode(), tuple(d.tile)))
    return out


def kernel_selection_parse(name: str):
    """Registry index for an ML_KERNEL-style name, or None for auto."""
    rc = lib().ta_kernel_selection_parse(name.encode())
    if rc == -1:
        raise TensorAshError(_err())
    return None if rc == -2 else rc


def resolve_shapes(a, b, c) -> dict:
    aa, ar = _shape_arr(a)
    ba, br = _shape_arr(b)
    ca, cr = _shape_arr(c)
    out = (C.c_uint32 * 9)()
    _check(lib().ta_resolve_shapes(aa, ar, ba, br, ca, cr, out))
    return dict(m=out[0], n=out[1], k=out[2], batch=out[3], batch_stride_a=out[4],
                batch_stride_b=out[5], batch_stride_c=out[6], total_flops=out[7] | (out[8] << 32))


def kernel_launch_count() -> int:
    return int(lib().ta_kernel_launch_count())


def is_nan(x: float) -> bool:
    return math.isnan(x)
