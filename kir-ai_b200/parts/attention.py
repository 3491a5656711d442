"""Causal grouped-query attention over the paged cache.

Order of operations as in the reference
(crates/llm-backend/src/core/qwen/ops/attention_full.rs:197-309): project q, k, v;
optional per-head RMSNorm of q and k with one weight [d] shared by the heads,
before the position encoding (:252-287); rotate q and k at the absolute
position; append k, v to the cache before attending, so a token sees itself
(crates/llm-backend/src/core/native_attention.rs:307-309); scores q.k * scale over the
visible rows, softmax, weighted sum of v (:731-764); output projection.  Query
head h reads kv head h // (q_heads / kv_heads) (:732).  A window W makes row i
see rows [i - W + 1, i].

Every size and constant is a constructor argument; the position encoding is a
part of its own.  A layer built with ``reads_only`` has no k and v projections:
it projects q alone and reads a cache that another layer filled.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import KVCacheNeed, Mixer, PositionEncoding, Runtime, WeightSpec
from .linear import Linear
from .rope import RotaryEmbedding


class GQAttention(Mixer):
    def __init__(self, prefix: str, hidden_size: int, q_heads: int, kv_heads: int, head_dim: int,
                 position: Optional[PositionEncoding], *, window: Optional[int] = None,
                 qk_norm_eps: Optional[float] = None, scale: Optional[float] = None, reads_only: bool = False,
                 names: Optional[Dict[str, str]] = None):
        if q_heads % kv_heads:
            raise ValueError(f"{q_heads} query heads are not a multiple of {kv_heads} kv heads")
        n = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight"}
        n.update(names or {})
        self.prefix = prefix
        self.hidden_size, self.q_heads, self.kv_heads, self.head_dim = hidden_size, q_heads, kv_heads, head_dim
        self.window = window
        self.qk_norm_eps = qk_norm_eps
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.position = position
        self.reads_only = reads_only
        sources = [(prefix + n["q"], q_heads * head_dim)]
        if not reads_only:
            sources += [(prefix + n["k"], kv_heads * head_dim), (prefix + n["v"], kv_heads * head_dim)]
        self.qkv = Linear(sources, hidden_size)
        self.out = Linear([(prefix + n["o"], hidden_size)], q_heads * head_dim)
        self.q_norm_name, self.k_norm_name = prefix + n["q_norm"], prefix + n["k_norm"]
        self.q_norm_weight = self.k_norm_weight = None

    def cache_need(self):
        return KVCacheNeed(self.kv_heads, self.head_dim, self.window)

    @property
    def capture_safe(self) -> bool:
        """The kernels read positions, lengths and block tables on the device; the position encoding is a part of
        its own and answers for itself."""
        return self.position is None or bool(self.position.capture_safe)

    @property
    def kernels_only(self) -> bool:
        return self.position is None or bool(self.position.kernels_only)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {**self.qkv.weight_specs(), **self.out.weight_specs()}
        if self.qk_norm_eps is not None:
            specs[self.q_norm_name] = WeightSpec((self.head_dim,), "norm")
            if not self.reads_only:
                specs[self.k_norm_name] = WeightSpec((self.head_dim,), "norm")
        if self.position is not None:
            specs.update(self.position.weight_specs())
        return specs

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.qkv.load(weights, rt)
        self.out.load(weights, rt)
        if self.qk_norm_eps is not None:
            self.q_norm_weight = weights.on_device(self.q_norm_name, torch.float32)
            if not self.reads_only:
                self.k_norm_weight = weights.on_device(self.k_norm_name, torch.float32)
        if self.position is not None:
            self.position.load(weights, rt)

    def takes_unscaled(self, rows: int) -> bool:
        return self.qkv.fuses_norms(rows)

    def fuses_into_norm(self, rows: int) -> bool:
        return self.out.fuses_norms(rows)

    def forward(self, x, batch, cache, write_cache: bool = True) -> torch.Tensor:
        return self.out.forward(self._mix(x, batch, cache, write_cache))

    def forward_into_norm(self, x, batch, cache, write_cache, resid, spec):
        return self.out.forward_into_norm(self._mix(x, batch, cache, write_cache), resid, spec)

    def _mix(self, x, batch, cache, write_cache: bool) -> torch.Tensor:
        """Everything before the output projection: [T, q_heads * head_dim]."""
        ops = self.rt.ops
        nq, d = self.q_heads, self.head_dim
        nkv = 0 if self.reads_only else self.kv_heads  # kv heads that this layer projects
        if write_cache and self.reads_only:
            raise ValueError("a reads_only attention layer cannot fill a cache")
        table = batch.block_tables[cache.group]
        qkv = self.qkv.forward(x)  # [T, (nq + 2 nkv) d]
        fused_table = self.position.fused_table() if isinstance(self.position, RotaryEmbedding) else None
        q = qkv[:, : nq * d].unflatten(1, (nq, d))
        if ((self.position is None or fused_table is not None) and write_cache and nkv == self.kv_heads
                and getattr(ops, "decode_prepares_qk", None) is not None
                and ops.decode_prepares_qk(qkv, cache.kv, batch, nq, nkv, d)):
            # every request brings one token: norm, rotation and the cache write happen inside the attention kernel
            return ops.attention_decode_qk(qkv, nq, nkv, d, self.q_norm_weight, self.k_norm_weight, fused_table,
                                           self.qk_norm_eps or 0.0, cache.kv, table, batch, self.window, self.scale)
        if self.position is None or fused_table is not None:
            ops.qk_norm_rope_kv_write_(qkv, nq, nkv, d, self.q_norm_weight, self.k_norm_weight, fused_table,
                                       self.qk_norm_eps or 0.0, cache.kv if write_cache else None, table,
                                       batch.request_of_token, batch.positions, write_cache)
        else:
            k = qkv[:, nq * d : (nq + nkv) * d].unflatten(1, (nkv, d))
            v = qkv[:, (nq + nkv) * d :].unflatten(1, (nkv, d))
            if self.qk_norm_eps is not None:
                ops.head_rmsnorm_(q, self.q_norm_weight, self.qk_norm_eps)
                if nkv:
                    ops.head_rmsnorm_(k, self.k_norm_weight, self.qk_norm_eps)
            self.position.apply(q, k, batch.positions)
            if write_cache:
                ops.kv_write(k, v, cache.kv, table, batch.request_of_token, batch.positions)
        return ops.paged_attention(q, cache.kv, table, batch, self.window, self.scale)
