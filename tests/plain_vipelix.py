"""The Vipelix design written out plainly: float64, whole sequences, no cache, one function per mechanism.

It shares nothing with the package: the tests compare the engine (its step function, cache, kernels) with this.
Notation: h a sublayer's input [T, width]; n(v) = v / sqrt(mean(v^2) + eps) over the last dimension.

`store` is applied to every tensor that an engine keeps between two kernels (identity by default;
`round_to_bfloat16` measures what bfloat16 storage costs by itself, all arithmetic staying float64).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def _keep(t):
    return t


def round_to_bfloat16(t):
    return t.to(torch.bfloat16).to(torch.float64)


def unit_rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def rms_norm(v: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(v, eps) * weight


def turn_pairs(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """v [T, ..., D]: elements (2i, 2i+1), i < dims/2, are turned by the angle position * base^(-2i/dims); the rest stays."""
    out = v.clone()
    for i in range(dims // 2):
        ang = positions.to(torch.float64) * (float(base) ** (-2.0 * i / dims))
        shape = [v.shape[0]] + [1] * (v.dim() - 2)
        c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
        a, b = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def latent_attention(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, positions, store=_keep) -> torch.Tensor:
    """Keys and values of every head from one latent per token; written head by head, key by key side: nothing is absorbed."""
    T = h.shape[0]
    H, D, Rd, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[p + "q"].T).reshape(T, H, D + Rd)
    down = h @ w[p + "dkv"].T
    c = store(rms_norm(down[:, :R], w[p + "dkv.norm"], eps))
    shared_key = store(turn_pairs(down[:, R:], positions, m["rot"]["dims"], m["rot"]["base"]))
    gate = torch.sigmoid(h @ w[p + "g"].T)
    heads = []
    for i in range(H):
        k_plain = c @ w[p + "uk"][i * D:(i + 1) * D].T                    # [T, D]
        value = c @ w[p + "uv"][i * V:(i + 1) * V].T                      # [T, V]
        q_plain = store(q[:, i, :D])
        q_turned = store(turn_pairs(q[:, i, D:], positions, m["rot"]["dims"], m["rot"]["base"]))
        score = (q_plain @ k_plain.T + q_turned @ shared_key.T) * m["scale"]
        score = score.masked_fill(positions[None, :] > positions[:, None], float("-inf"))
        heads.append(store(torch.softmax(score, -1) @ value * gate[:, i:i + 1]))
    return torch.cat(heads, dim=1) @ w[p + "o"].T


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    a, b, c, e = (float(x) for x in coef)
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_ff(h, w, p: str, eps: float, store=_keep) -> torch.Tensor:
    return store(polynorm(h @ w[p + "up"].T, w[p + "act"], eps)) @ w[p + "down"].T


def gated_expert(h, w, p: str, store=_keep) -> torch.Tensor:
    g = h @ w[p + "gate"].T
    return store(g * torch.sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def table_moe(h, tokens: torch.Tensor, w, p: str, mlp: dict, store=_keep) -> torch.Tensor:
    top = mlp["router"]["top"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in w[p + "table"][int(tokens[t])].tolist():
            out[t] += gated_expert(h[t:t + 1], w, f"{p}e{int(e)}.", store)[0] / top
    if mlp.get("shared"):
        out = out + gated_expert(h, w, p + "shared.", store)
    return out


def run_plan(cfg: dict):
    """(layer, number of the pass it opens or None) in execution order."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    plan = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        plan += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return plan + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], store=_keep, streams: Optional[list] = None) -> torch.Tensor:
    """float64 logits [T, vocab]; `streams` collects the residual stream after every layer run."""
    w = {k: (v.to(torch.float64) if v.is_floating_point() else v.long()) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    pos = torch.arange(len(tok))
    x = w["embed"][tok]
    embedded = x.clone()
    for i, opens in run_plan(cfg):
        if opens is not None:
            if opens > 0:
                x = x + embedded
            x = x + w["loop.step"][opens]
        layer, p = cfg["layers"][i], f"l{i}."
        y = latent_attention(store(rms_norm(x, w[p + "norm1"], eps)), w, p + "mix.", layer["mixer"], eps, pos, store)
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp"):
            hh = store(rms_norm(x, w[p + "norm2"], eps))
            if layer["mlp"]["kind"] == "dense":
                y = dense_ff(hh, w, p + "mlp.", eps, store)
            else:
                y = table_moe(hh, tok, w, p + "mlp.", layer["mlp"], store)
            x = x + rms_norm(y, w[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    logits = store(rms_norm(x, w["final.norm"], eps)) @ w["embed"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy(cfg: dict, weights, prompt: List[int], n: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(torch.argmax(forward(cfg, weights, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
