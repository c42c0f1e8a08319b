"""Llama-architecture runner (``tensor_ash_llama.h``) over the library's op graphs.

Mirrors the reference's ``tools/llama-ash`` model object (``model/mod.rs:59-190``):
``prefill`` submits one mixed graph, ``decode`` replays one prepared graph per
token.  Weights are random-initialised from a seed; ``weight_stream`` documents
the generator so a checker can rebuild any tensor on the host.
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
