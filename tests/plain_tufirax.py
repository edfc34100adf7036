"""Plain, slow implementation of the Tufirax decoder, used as the oracle of its tests.

Whole sequences only: no cache, no state carried between calls, no batching; one function per
mechanism (`store`, where a function has it, is applied to what an engine keeps between two kernels in
the activations' type - the identity, or a rounding to bfloat16 that measures what that storage costs), torch used purely as an array library (float64 on the CPU).  It shares no code with
the engine under ``rvllm_b200``: the configuration is a plain dictionary and the weights a plain
dictionary name -> tensor.

The design, layer by layer (h is a sublayer's input, the residual stream itself; W x means a
matrix stored [out, in] applied to a column):

* a layer:   x <- x + rms(mixer(x)) * w1 ;  x <- x + rms(ff(x)) * w2   (norm on the OUTPUT of the
  sublayer; a layer without feed-forward stops after the first line);
* attention: q = Wq h, k = Wk h, v = k (as projected).  q and k are each divided by the root mean
  square of their WHOLE row (all heads together) and multiplied by a weight of that size; then the
  leading `dims` elements of every head are rotated, element i with element i + dims/2, by the
  angle p * base^(-2i/dims).  s = cap * tanh(scale * q.k / cap), causal.  The softmax denominator
  also holds exp(sink_h), which has no value.  The head's output is multiplied by
  sigmoid(Wg h)_h, then Wo;
* mamba2:    [z | x | B | C | dt] = W_in h; x, B, C pass a causal convolution per channel (taps
  oldest first, the last one on the current token, zeros before the sequence) with bias, then
  silu; dt = softplus(dt + dt_bias); per head S <- exp(-exp(A_log) dt) S + dt B x^T,
  y = S^T C + D x; y * silu(z) is normalised in `norm_groups` equal parts, times a weight, then Wo;
* feed-forward: Wd (gelu_tanh(Wg h) * (Wu h)).
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence

import torch

F64 = torch.float64


def _keep(t: torch.Tensor) -> torch.Tensor:
    return t


def round_to_bfloat16(t: torch.Tensor) -> torch.Tensor:
    """What storing a tensor in bfloat16 between two kernels does to it (the arithmetic stays float64)."""
    return t.to(torch.bfloat16).to(t.dtype)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_leading(x: torch.Tensor, positions: Sequence[int], dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: elements i and i + dims/2 (i < dims/2) of every head turn by p * base^(-2i/dims)."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    ang = torch.tensor(list(positions), dtype=x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def sink_softmax_attention(q, k, v, scale: float, softcap: float, sink: torch.Tensor) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv], sink [H] -> [T, H, dv].  Query head h reads key/value
    head h // (H / G).  One loop per (token, head), written for clarity."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, h]) * scale
            s = softcap * torch.tanh(s / softcap)
            m = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            out[t, h] = (e[:, None] * v[:t + 1, g]).sum(0) / (e.sum() + torch.exp(sink[h] - m))
    return out


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, start: int = 0,
                    store=_keep) -> torch.Tensor:
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = h @ w[p + "q"].t()
    k = h @ w[p + "k"].t()
    v = store(k.view(T, G, d))
    qn = (rms(q, eps) * w[p + "q.norm"]).view(T, H, d)
    kn = (rms(k, eps) * w[p + "k.norm"]).view(T, G, d)
    pos = range(start, start + T)
    qn = rotate_leading(qn, pos, m["rot"]["dims"], m["rot"]["base"])
    kn = rotate_leading(kn, pos, m["rot"]["dims"], m["rot"]["base"])
    o = sink_softmax_attention(store(qn), store(kn), v, m["scale"], m["softcap"], w[p + "sink"])
    gate = torch.sigmoid(h @ w[p + "g"].t())                       # [T, H]
    o = store(o * gate[:, :, None])
    return o.reshape(T, -1) @ w[p + "o"].t()


def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, K] (column K-1 multiplies the current token), zeros before the sequence."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros((K - 1, C), dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j][None, :]
    return out + bias[None, :]


def selective_scan(x, B, C, dt, a_log, D, groups: int) -> torch.Tensor:
    """x [T, heads, P], B and C [T, groups, N], dt [T, heads] (already positive) -> y [T, heads, P]."""
    T, heads, P = x.shape
    N = B.shape[2]
    y = torch.zeros_like(x)
    for hd in range(heads):
        g = hd // (heads // groups)
        S = torch.zeros((N, P), dtype=x.dtype)
        a = -torch.exp(a_log[hd])
        for t in range(T):
            S = torch.exp(a * dt[t, hd]) * S + dt[t, hd] * B[t, g][:, None] * x[t, hd][None, :]
            y[t, hd] = S.t() @ C[t, g] + D[hd] * x[t, hd]
    return y


def grouped_rms(y: torch.Tensor, parts: int, eps: float) -> torch.Tensor:
    T, W = y.shape
    return rms(y.view(T, parts, W // parts), eps).reshape(T, W)


def mamba2_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, store=_keep) -> torch.Tensor:
    T = h.shape[0]
    heads, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * P
    proj = h @ w[p + "in"].t()
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = store(silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"])))
    x = xbc[:, :inner].reshape(T, heads, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"][None, :])
    y = selective_scan(x, B, C, dt, w[p + "A_log"], w[p + "D"], G).reshape(T, inner)
    y = store(grouped_rms(y * silu(z), m["norm_groups"], eps) * w[p + "norm"])
    return y @ w[p + "o"].t()


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, store=_keep) -> torch.Tensor:
    return store(gelu_tanh(h @ w[p + "gate"].t()) * (h @ w[p + "up"].t())) @ w[p + "down"].t()


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], residuals: List[torch.Tensor] = None,
            store=_keep) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  `residuals`, if a list, receives x after every layer run.
    The stream x itself is never passed through `store` (it is float32 in every engine type); the copy of it
    that a sublayer's products read is."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        p = f"l{src}."
        if layer["type"] == "attention":
            y = attention_mixer(store(x), w, p + "mix.", layer["mixer"], eps, store=store)
        elif layer["type"] == "mamba2":
            y = mamba2_mixer(store(x), w, p + "mix.", layer["mixer"], eps, store=store)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = x + rms(y, eps) * w[p + "norm1"]
        if layer.get("mlp") is not None:
            x = x + rms(dense_ff(store(x), w, p + "mlp.", store=store), eps) * w[p + "norm2"]
        if residuals is not None:
            residuals.append(x.clone())
    return store(rms(x, eps) * w["final.norm"]) @ w["head"].t()


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        logits = forward(cfg, w, toks)[-1]
        toks.append(int(torch.argmax(logits)))
    return toks[len(prompt):]
