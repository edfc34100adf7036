"""Selective state-space mixer in the state-space-duality form ("mamba2").

    [z | x | B | C | dt] = W_in h                 z, x: heads * head_dim;  B, C: groups * state;  dt: heads
    x, B, C <- silu(causal convolution per channel (taps, bias))
    dt <- softplus(dt + dt_bias)
    per head (its group's B and C):  S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T ;  y_t = S_t^T C_t + D x_t
    y <- RMSNorm in `norm_groups` equal parts of (y * silu(z)), times a weight;  out = W_o y

A request keeps, in one row of a float32 state tensor, S ([heads][state][head_dim]) and behind it the
convolution's last taps - 1 inputs; the cache manager zeroes the row when the slot is handed out.
Decays, step sizes, the state and the gated norm are float32; the products and the convolution's
result have the activations' type.  Nothing is read on the host, so a decode step can be captured.
"""
from __future__ import annotations

import torch

from .base import MIXERS, Part, StateNeed, TensorSpec
from .linear import Linear


class Mamba2Mixer(Part):
    def __init__(self, hidden_size: int, heads: int, head_dim: int, state: int, groups: int, conv: int, norm_groups: int,
                 eps: float, suffix: str = ""):
        from ..errors import ConfigError
        problems = []
        if heads % groups:
            problems.append(f"{heads} heads cannot share {groups} groups of B and C")
        if (heads * head_dim) % norm_groups:
            problems.append(f"{heads * head_dim} inner channels do not split into {norm_groups} norm groups")
        if not 1 <= conv <= 16:
            problems.append(f"the convolution has 1 to 16 taps, got {conv}")
        if state > 256:
            problems.append(f"the state dimension is at most 256, got {state}")
        if problems:
            raise ConfigError(problems, "mamba2 mixer")
        self.hidden_size, self.heads, self.head_dim, self.state, self.groups = hidden_size, heads, head_dim, state, groups
        self.taps, self.norm_groups, self.eps = conv, norm_groups, eps
        self.inner = heads * head_dim
        self.channels = self.inner + 2 * groups * state          # what passes the convolution: x | B | C
        self.in_proj = Linear(hidden_size, [2 * self.inner + 2 * groups * state + heads], ["in"], suffix=suffix)
        self.out = Linear(self.inner, [hidden_size], ["o"], suffix=suffix)
        self.ssm_floats = heads * state * head_dim
        self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.norm = None

    def tensor_specs(self):
        return {**self.in_proj.tensor_specs(), **self.out.tensor_specs(),
                "conv": TensorSpec((self.channels, self.taps), "conv_taps"), "conv.b": TensorSpec((self.channels,), "bias"),
                "dt_bias": TensorSpec((self.heads,), "bias"), "A_log": TensorSpec((self.heads,), "bias"),
                "D": TensorSpec((self.heads,), "norm"), "norm": TensorSpec((self.inner,), "norm")}

    def bind(self, get):
        self.in_proj.bind(get)
        self.out.bind(get)
        self.conv_w, self.conv_b = get("conv"), get("conv.b")
        # what enters the recurrence is float32
        self.dt_bias, self.a_log, self.d_skip = (get(n).float().contiguous() for n in ("dt_bias", "A_log", "D"))
        self.norm = get("norm")

    def cache_need(self):
        return StateNeed((self.ssm_floats + (self.taps - 1) * self.channels,), "float32")

    def __call__(self, x, ctx, cache, residual=None, write_cache=True, out_dtype=None):
        k = ctx.kernels
        proj = self.in_proj(x, ctx, out_dtype=torch.float32)
        xbc = k.causal_conv_silu(proj, self.inner, self.channels, self.conv_w, self.conv_b, ctx.token_seq, ctx.cu_seqlens,
                                 ctx.state_slots, cache.state, self.ssm_floats, x.dtype)
        y = k.ssm_scan(xbc, proj, self.inner + self.channels, self.dt_bias, self.a_log, self.d_skip, ctx.cu_seqlens,
                       ctx.state_slots, cache.state, self.heads, self.head_dim, self.state, self.groups, max_q_len=max(ctx.q_lens))
        y = k.gated_group_rmsnorm(y, proj, self.norm, self.eps, self.norm_groups, x.dtype)
        return self.out(y, ctx, residual=residual, out_dtype=out_dtype)


MIXERS.register("mamba2", Mamba2Mixer)
