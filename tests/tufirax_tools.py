"""Small Tufirax configurations, model folders for them and plain logits, for the tests of that design.

The sizes differ from layer to layer and between the configurations, and avoid values that hide a
fault: groups of heads larger than one, a rotation of part of a head, a state size and a head size that
are no multiples of a warp, several norm groups, three and five taps, shared layers in both orders."""
from __future__ import annotations

import copy
import json
import os
import tempfile
from typing import Dict, List

import torch

import plain_tufirax as P

_keep = []


def attention(heads=6, kv_heads=2, dim=32, rot_dims=16, base=10000.0, scale=0.21, softcap=7.0, ff=88):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "softcap": softcap,
                      "rot": {"dims": rot_dims, "base": base}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mamba2(heads=6, vdim=20, state=24, groups=3, conv=3, norm_groups=4, ff=None):
    return {"type": "mamba2",
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def shared(layer: dict, source: int) -> dict:
    out = copy.deepcopy(layer)
    out["weights_of"] = source
    return out


def config(layers: List[dict], width=72, vocab=211, eps=1e-5) -> dict:
    return {"architecture": "Tufirax", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}


def small_a() -> dict:
    """Mixer first, attention with a rotation of half of each head, a shared layer of each kind."""
    m, a = mamba2(), attention()
    return config([m, a, shared(a, 1), mamba2(heads=4, vdim=33, state=40, groups=1, conv=5, norm_groups=1, ff=60), shared(m, 0)])


def small_b() -> dict:
    """Head size 64 (the sizes the tensor-core attention kernels are built for), a whole-head rotation,
    groups of four heads, an attention layer without feed-forward."""
    a = attention(heads=8, kv_heads=2, dim=64, rot_dims=64, base=500.0, scale=0.11, softcap=12.0, ff=None)
    return config([a, mamba2(heads=8, vdim=16, state=64, groups=2, conv=4, norm_groups=2, ff=96),
                   attention(heads=4, kv_heads=4, dim=64, rot_dims=32, base=100000.0, scale=0.3, softcap=30.0, ff=64),
                   shared(a, 0)], width=96, vocab=300, eps=1e-6)


def odd_shapes() -> dict:
    """Sizes that no kernel's fast path is made for: a width and a vocabulary that are no multiples of 8, head sizes
    40 (no tensor-core attention kernel) and 96, a state of 13 and one of 256, two and eight taps, as many groups as
    heads, a norm group per head, a feed-forward narrower than the model."""
    return config([mamba2(heads=3, vdim=24, state=13, groups=3, conv=2, norm_groups=3, ff=36),
                   attention(heads=4, kv_heads=4, dim=40, rot_dims=40, base=77.0, scale=0.2, softcap=4.0, ff=None),
                   mamba2(heads=2, vdim=8, state=256, groups=1, conv=8, norm_groups=2, ff=None),
                   attention(heads=6, kv_heads=3, dim=96, rot_dims=32, base=1e6, scale=0.09, softcap=50.0, ff=52)],
                  width=76, vocab=173, eps=1e-5)


def write_folder(cfg: dict, seed: int = 0, dtype: str = "bfloat16", edit=None) -> str:
    """A model folder written by the framework's random-weights mode; `edit(tensors)` may change the
    tensors (a dictionary name -> tensor) before they are written."""
    import rvllm_b200
    from rvllm_b200.models.decoder import expected_tensors
    from rvllm_b200.weights.random_init import random_tensors
    from rvllm_b200.weights.safetensors_io import write_safetensors
    conf = rvllm_b200.config_from_dict(cfg)
    d = tempfile.TemporaryDirectory(prefix="rvllm_tfx_")
    _keep.append(d)
    tensors = random_tensors(expected_tensors(conf.to_spec()), seed, {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype])
    if edit is not None:
        edit(tensors)
    with open(os.path.join(d.name, "config.json"), "w") as f:
        json.dump(conf.to_dict(), f)
    write_safetensors(os.path.join(d.name, "model.safetensors"), tensors, metadata={"format": "pt"})
    return d.name


def lively(tensors: Dict[str, torch.Tensor], seed: int = 1) -> None:
    """Make the random weights show more: sinks of order one, decays spread from fast to slow, step biases and
    skips of both signs, larger matrices inside the mixers so that scores reach the cap."""
    g = torch.Generator().manual_seed(seed)
    for name, t in tensors.items():
        def fill(lo, hi):
            t.copy_((torch.rand(t.shape, generator=g) * (hi - lo) + lo).to(t.dtype))
        if name.endswith(".mix.sink"):
            fill(-2.0, 3.0)
        elif name.endswith(".mix.A_log"):
            fill(-4.0, 1.0)
        elif name.endswith(".mix.dt_bias"):
            fill(-3.0, 1.0)
        elif name.endswith(".mix.D"):
            fill(-1.0, 1.0)
        elif name.endswith((".mix.q.norm", ".mix.k.norm")):
            fill(0.5, 2.5)
        elif name.endswith(".mix.g") or name.endswith(".mix.in"):
            t.mul_(8.0)


def read_folder(folder: str):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(folder, "model.safetensors"))


def plain_logits(folder: str, requests: Dict[str, List[int]], rounded: bool = False) -> Dict[str, torch.Tensor]:
    """float64 logits of the plain implementation; `rounded`: with everything an engine stores between two kernels
    rounded to bfloat16, which measures what that storage costs by itself on these requests."""
    cfg, w = read_folder(folder)
    store = P.round_to_bfloat16 if rounded else P._keep
    return {rid: P.forward(cfg, w, toks, store=store) for rid, toks in requests.items()}
