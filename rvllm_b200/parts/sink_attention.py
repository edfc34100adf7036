"""Grouped-query attention with whole-row query/key norms, keys reused as values, a capped score,
a sink in the softmax and a gate per head, over the paged cache.

    q = Wq h, k = Wk h;  v = k as projected (no value matrix)
    q <- q / rms(q) * wq,  k <- k / rms(k) * wk          rms over the WHOLE row, all heads together
    the leading `rotary_dim` elements of every head of q and k are rotated (position part)
    s = cap * tanh(scale * (q . k) / cap), causal
    p_j = exp(s_j) / (sum_i exp(s_i) + exp(sink_h))        the sink has no value
    o_h <- o_h * sigmoid(Wg h)_h;  y = Wo o

One stacked product gives [q | k | gate logits]; one kernel normalises, rotates, writes the cache
(key = normalised and rotated k, value = k as it left the product) and applies the sigmoid; the
attention kernels take the cap, the sinks and the gate as options.  The constants (scale, cap, eps)
and every size are parameters; tensor names default to q, k, g, o, q.norm, k.norm, sink.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import MIXERS, KvCacheNeed, Part, TensorSpec
from .linear import Linear


class GatedSinkAttention(Part):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float, eps: float,
                 softcap: Optional[float] = None, sink: bool = True, gate: bool = True, window: Optional[int] = None,
                 position=None, suffix: str = ""):
        from ..errors import ConfigError
        if num_heads % num_kv_heads:
            raise ConfigError(f"{num_heads} query heads cannot share {num_kv_heads} key/value heads")
        if head_dim > 256:
            raise ConfigError(f"head_dim must be at most 256, got {head_dim}")
        if softcap is not None and not softcap > 0:
            raise ConfigError(f"the score cap must be positive, got {softcap}")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.scale, self.eps, self.softcap, self.window = scale, eps, softcap, window
        self.has_sink, self.has_gate = sink, gate
        self.position = position
        self.q_dim, self.kv_dim = num_heads * head_dim, num_kv_heads * head_dim
        outs, names = [self.q_dim, self.kv_dim], ["q", "k"]
        if gate:
            outs.append(num_heads)
            names.append("g")
        self.qkg = Linear(hidden_size, outs, names, suffix=suffix)
        self.out = Linear(self.q_dim, [hidden_size], ["o"], suffix=suffix)
        self.q_norm = self.k_norm = self.sink = None

    def tensor_specs(self):
        specs = {**self.qkg.tensor_specs(), **self.out.tensor_specs(),
                 "q.norm": TensorSpec((self.q_dim,), "norm"), "k.norm": TensorSpec((self.kv_dim,), "norm")}
        if self.has_sink:
            specs["sink"] = TensorSpec((self.num_heads,), "bias")
        return specs

    def bind(self, get):
        self.qkg.bind(get)
        self.out.bind(get)
        self.q_norm, self.k_norm = get("q.norm"), get("k.norm")
        self.sink = get("sink").float().contiguous() if self.has_sink else None     # the softmax is float32

    def cache_need(self):
        return KvCacheNeed(self.num_kv_heads, self.head_dim, self.window)

    def __call__(self, x, ctx, cache, residual=None, write_cache=True, out_dtype=None):
        k = ctx.kernels
        meta = ctx.attention[cache.group]
        tables = self.position.rotation_tables() if self.position is not None else None
        cos, sin = tables if tables is not None else (None, None)
        # the product leaves its kernel in float and is rounded once, after the norm and the rotation; a layer that
        # reads another layer's cache (`write_cache` False) takes the same path and leaves the cache alone
        proj = self.qkg(x, ctx, out_dtype=torch.float32)
        q, gate = k.qk_norm_rope_cache_write(proj, self.q_norm, self.k_norm, self.eps, ctx.positions, cos, sin,
                                             meta.slot_mapping, cache.kv, self.num_heads, self.num_kv_heads,
                                             self.head_dim, x.dtype, with_gate=self.has_gate, write_kv=write_cache)
        o = k.paged_attention(q, cache.kv, meta, self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.window,
                              softcap=self.softcap, sinks=self.sink, gate=gate)
        return self.out(o, ctx, residual=residual, out_dtype=out_dtype)


MIXERS.register("gated_sink_attention", GatedSinkAttention)
