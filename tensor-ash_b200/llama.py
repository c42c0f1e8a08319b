"""Llama-architecture runner (``tensor_ash_llama.h``) over the library's op graphs.

Mirrors the reference's ``tools/llama-ash`` model object (``model/mod.rs:59-190``):
``prefill`` submits one mixed graph, ``decode`` replays one prepared graph per
token.  Weights are random-initialised from a seed (``weight_stream`` documents
the generator so a checker can rebuild any tensor on the host) or loaded from an
F32 / F16 GGUF file (``Llama.load_gguf``; ``GgufFile`` / ``write_gguf`` read and
write the container on the host).
"""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import List, Tuple

import numpy as np

from . import capi
from .api import Executor, RunStats, TensorAshError, _check, _err


@dataclasses.dataclass
class LlamaConfig:
    layers: int = 22
    embd: int = 2048
    heads: int = 32
    kv_heads: int = 4
    head_dim: int = 64
    ffn: int = 5632
    vocab: int = 32000
    t_max: int = 2048
    rms_eps: float = 1e-5
    rope_theta: float = 1e4
    weight_sigma: float = 0.02
    norm_jitter: float = 0.0
    seed: int = 1

    def _c(self) -> capi.LlamaConfigC:
        return capi.LlamaConfigC(self.layers, self.embd, self.heads, self.kv_heads, self.head_dim, self.ffn,
                                 self.vocab, self.t_max, self.rms_eps, self.rope_theta, self.weight_sigma,
                                 self.norm_jitter, self.seed)


WEIGHT_CHUNK = 1 << 20
TENSOR_EMBD, TENSOR_OUTPUT_NORM, TENSOR_LM_HEAD = 0, 1, 2
LAYER_TENSORS = {"attn_norm": 0, "wq": 1, "wk": 2, "wv": 3, "wo": 4, "ffn_norm": 5, "w_gate": 6, "w_up": 7,
                 "w_down": 8}


def layer_tensor_id(layer: int, name: str) -> int:
    return 16 + 16 * layer + LAYER_TENSORS[name]


def chunk_seed(seed: int, tensor_id: int, chunk: int) -> int:
    """Seed of chunk ``chunk`` of tensor ``tensor_id`` (64-bit wrap-around)."""
    return ((seed * 1000003 + tensor_id) * 4096 + chunk) & 0xFFFFFFFFFFFFFFFF


def shard_plan(cfg: LlamaConfig, rank: int, world: int) -> dict:
    """The tensor-parallel shard of `rank` (the rule ``ta_llama_create_random_tp`` applies):
    query heads and MLP columns split evenly, kv heads split or shared by neighbouring ranks,
    lm_head split by vocabulary column.  Offsets are in elements of the unsharded axis."""
    if cfg.heads % world or cfg.ffn % world or cfg.vocab % world:
        raise ValueError("heads, ffn and vocab must divide by the world size")
    if cfg.kv_heads % world and world % cfg.kv_heads:
        raise ValueError("kv heads must divide by, or divide, the world size")
    heads_l = cfg.heads // world
    kv_l = cfg.kv_heads // world if cfg.kv_heads >= world else 1
    kv_first = rank * cfg.kv_heads // world
    return dict(heads_l=heads_l, kv_l=kv_l, kv_first=kv_first, group_l=heads_l // kv_l,
                q0=rank * heads_l * cfg.head_dim, q_w=heads_l * cfg.head_dim,
                kv0=kv_first * cfg.head_dim, kv_w=kv_l * cfg.head_dim,
                f0=rank * (cfg.ffn // world), ffn_l=cfg.ffn // world,
                v0=rank * (cfg.vocab // world), vocab_l=cfg.vocab // world,
                adds_residual=rank == 0)


class Llama:
    def __init__(self, exec_: Executor, cfg: LlamaConfig, comm=None):
        c = cfg._c()
        h = capi.lib().ta_llama_create_random_tp(exec_._h, C.byref(c), comm._h if comm is not None else None)
        if not h:
            raise TensorAshError(_err())
        self._h, self._exec, self.cfg, self._comm = h, exec_, cfg, comm

    @classmethod
    def load_gguf(cls, exec_: Executor, path: str, t_max: int = 2048, comm=None) -> "Llama":
        """Load an F32 / F16 llama GGUF (``tools/llama-ash/src/model/load.rs``); the geometry comes
        from the file's metadata and ``t_max`` is clamped to its context length."""
        h = capi.lib().ta_llama_load_gguf(exec_._h, str(path).encode(), t_max, comm._h if comm is not None else None)
        if not h:
            raise TensorAshError(_err())
        c = capi.LlamaConfigC()
        _check(capi.lib().ta_llama_get_config(h, C.byref(c)))
        self = cls.__new__(cls)
        cfg = LlamaConfig(*(getattr(c, name) for name, _ in capi.LlamaConfigC._fields_))
        self._h, self._exec, self.cfg, self._comm = h, exec_, cfg, comm
        return self

    def reset(self) -> None:
        _check(capi.lib().ta_llama_reset(self._h))

    def prefill(self, tokens) -> Tuple[int, RunStats]:
        arr = np.ascontiguousarray(tokens, dtype=np.uint32)
        nxt, st = C.c_uint32(0), capi.RunStatsC()
        _check(capi.lib().ta_llama_prefill(self._h, arr.ctypes.data_as(C.POINTER(C.c_uint32)), arr.size,
                                           C.byref(nxt), C.byref(st)))
        return int(nxt.value), RunStats._from(st)

    def decode(self, first_token: int, n: int) -> Tuple[List[int], RunStats]:
        out = (C.c_uint32 * max(n, 1))()
        st = capi.RunStatsC()
        _check(capi.lib().ta_llama_decode(self._h, first_token, n, out, C.byref(st)))
        return [int(out[i]) for i in range(n)], RunStats._from(st)

    def decode_breakdown(self, token: int):
        """One decode step with every launch timed separately: (next token, launches, rows) where rows
        is a list of (op class, device ns, calls), largest first (the LLAMA_ASH_BREAKDOWN table)."""
        rows = (capi.LlamaBreakdownRowC * 32)()
        n_rows, n_launches, nxt = C.c_size_t(), C.c_size_t(), C.c_uint32()
        _check(capi.lib().ta_llama_decode_breakdown(self._h, token, rows, 32, C.byref(n_rows), C.byref(n_launches),
                                                    C.byref(nxt)))
        out = [(rows[i].op_class.decode(), int(rows[i].gpu_ns), int(rows[i].calls)) for i in range(min(32, n_rows.value))]
        return int(nxt.value), int(n_launches.value), out

    def logits(self) -> np.ndarray:
        out = np.empty(self.cfg.vocab, dtype=np.float32)
        _check(capi.lib().ta_llama_logits(self._h, out.ctypes.data, out.size))
        return out

    @property
    def position(self) -> int:
        return int(capi.lib().ta_llama_position(self._h))

    @property
    def weight_bytes_per_token(self) -> int:
        return int(capi.lib().ta_llama_weight_bytes_per_token(self._h))

    def close(self) -> None:
        if self._h:
            capi.lib().ta_llama_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------------------- GGUF on the host
GGML_TYPE_F32, GGML_TYPE_F16 = 0, 1
_GGUF_KINDS = {0: "u64", 1: "i64", 2: "f64", 3: "bool", 4: "str", 5: "skipped"}


class GgufFile:
    """Read-only view of a GGUF v2 / v3 file (``tools/llama-ash/src/gguf.rs``): scalar and string
    metadata, tensor infos, F32 / F16 payloads as float32.  Needs no GPU."""

    def __init__(self, path: str):
        self._h = capi.lib().ta_gguf_open(str(path).encode())
        if not self._h:
            raise TensorAshError(_err())

    def kind(self, key: str):
        """'u64' | 'i64' | 'f64' | 'bool' | 'str' | 'skipped' (an array, not kept) | None (absent)."""
        return _GGUF_KINDS.get(capi.lib().ta_gguf_meta_kind(self._h, key.encode()))

    def require_u64(self, key: str) -> int:
        v = C.c_uint64(0)
        _check(capi.lib().ta_gguf_meta_u64(self._h, key.encode(), C.byref(v)))
        return int(v.value)

    def f64_or(self, key: str, fallback: float) -> float:
        v = C.c_double(0.0)
        _check(capi.lib().ta_gguf_meta_f64(self._h, key.encode(), fallback, C.byref(v)))
        return float(v.value)

    def string(self, key: str) -> str:
        buf = C.create_string_buffer(1 << 16)
        _check(capi.lib().ta_gguf_meta_str(self._h, key.encode(), buf, len(buf)))
        return buf.value.decode()

    def info(self, name: str) -> Tuple[List[int], int, int]:
        """(ne in file order, ggml type, offset within the data section)."""
        ne, nd, ty, off = (C.c_uint64 * 4)(), C.c_uint32(0), C.c_uint32(0), C.c_uint64(0)
        _check(capi.lib().ta_gguf_tensor_info(self._h, name.encode(), ne, C.byref(nd), C.byref(ty), C.byref(off)))
        return [int(ne[i]) for i in range(nd.value)], int(ty.value), int(off.value)

    def read_f32(self, name: str) -> np.ndarray:
        ne, _, _ = self.info(name)
        out = np.empty(int(np.prod(ne, dtype=np.int64)), dtype=np.float32)
        _check(capi.lib().ta_gguf_read_f32(self._h, name.encode(), out.ctypes.data, out.size))
        return out

    @property
    def data_start(self) -> int:
        return int(capi.lib().ta_gguf_data_start(self._h))

    def close(self) -> None:
        if self._h:
            capi.lib().ta_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def write_gguf(path: str, metadata: dict, tensors: dict, alignment: int = 32, version: int = 3) -> None:
    """Write a GGUF file.  ``metadata`` values: ``str``, ``bool``, ``int`` (u32 when it fits, else
    u64; negative: i32 / i64), ``float`` (f32), ``("f64", x)``, ``("u64", x)``, or a list of ``str`` /
    ``float`` (written as an array).  ``tensors``: name -> ndarray of float32 (F32) or float16 (F16);
    the array's C-order shape is [..., n1, n0], stored as ne = [n0, n1, ...]."""
    import struct

    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    def value(v) -> bytes:
        if isinstance(v, tuple):
            tag, x = v
            return {"f64": lambda: struct.pack("<Id", 12, x), "u64": lambda: struct.pack("<IQ", 10, x),
                    "i64": lambda: struct.pack("<Iq", 11, x), "u8": lambda: struct.pack("<IB", 0, x),
                    "i16": lambda: struct.pack("<Ih", 3, x)}[tag]()
        if isinstance(v, bool):
            return struct.pack("<IB", 7, int(v))
        if isinstance(v, str):
            return struct.pack("<I", 8) + s(v)
        if isinstance(v, int):
            if v < 0:
                return struct.pack("<Ii", 5, v) if v >= -2 ** 31 else struct.pack("<Iq", 11, v)
            return struct.pack("<II", 4, v) if v < 2 ** 32 else struct.pack("<IQ", 10, v)
        if isinstance(v, float):
            return struct.pack("<If", 6, v)
        if isinstance(v, (list, tuple)):
            if all(isinstance(e, str) for e in v):
                return struct.pack("<IIQ", 9, 8, len(v)) + b"".join(s(e) for e in v)
            return struct.pack("<IIQ", 9, 6, len(v)) + b"".join(struct.pack("<f", float(e)) for e in v)
        raise TypeError(f"unsupported GGUF metadata value {v!r}")

    if alignment != 32 and "general.alignment" not in metadata:
        metadata = {**metadata, "general.alignment": alignment}
    head = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(metadata))
    for k, v in metadata.items():
        head += s(k) + value(v)
    blobs, offset = [], 0
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr)
        if arr.dtype == np.float32:
            ty = GGML_TYPE_F32
        elif arr.dtype == np.float16:
            ty = GGML_TYPE_F16
        else:
            raise TypeError(f"tensor {name}: dtype {arr.dtype} is not float32 / float16")
        ne = list(reversed(arr.shape))
        head += s(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne)
        head += struct.pack("<IQ", ty, offset)
        raw = arr.tobytes()
        pad = (-len(raw)) % alignment
        blobs.append(raw + b"\0" * pad)
        offset += len(raw) + pad
    head += b"\0" * ((-len(head)) % alignment)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)
