"""Small Vipelix configurations, model folders for them and plain logits, for the tests of that design.

The sizes differ from layer to layer and between the configurations and avoid values that hide a fault: a value
size unlike the key size, a rotation of part of the rotated block, a span of repeated layers in the middle of the
stack (layers before and after it), one pass and three passes, one expert per token and three, a layer without a
feed-forward, experts without a shared one."""
from __future__ import annotations

import copy
from typing import Dict, List

import torch

import plain_vipelix as P
from tufirax_tools import read_folder, write_folder      # (folders are written by the framework's random-weights mode)


def latent(heads=3, dim=24, rot_dim=16, rot_dims=None, vdim=20, kv_rank=40, base=10000.0, scale=0.17, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"dims": rot_dims or rot_dim, "base": base}},
            "mlp": copy.deepcopy(mlp)}


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def moe(ff=24, experts=5, top=2, shared=16):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top},
            "shared": None if shared is None else {"ff": shared}}


def config(layers: List[dict], width=48, vocab=131, eps=1e-5, loop=None, cap=20.0) -> dict:
    c = {"architecture": "Vipelix", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if cap is not None:
        c["logit_softcap"] = cap
    return c


def small_a() -> dict:
    """A repeated span in the middle (one layer before it, one behind), three passes; dense, experts with and without
    a shared one, a layer with no feed-forward; part of the rotated block turns."""
    return config([latent(mlp=dense()),
                   latent(heads=2, dim=16, rot_dim=8, vdim=32, kv_rank=24, base=500.0, scale=0.3, mlp=moe()),
                   latent(heads=4, dim=8, rot_dim=12, rot_dims=8, vdim=8, kv_rank=20, mlp=None),
                   latent(mlp=moe(ff=40, experts=3, top=1, shared=None))], loop=(1, 3, 3))


def small_b() -> dict:
    """Sizes the tensor-core kernels are built for (rows of 48 + 16 = 64 and 96 + 32 = 128 elements, multiples of 16
    everywhere), every layer repeated twice, three experts per token, no cap on the logits."""
    return config([latent(heads=4, dim=32, rot_dim=16, vdim=48, kv_rank=48, scale=0.11, mlp=moe(ff=32, experts=6, top=3, shared=48)),
                   latent(heads=2, dim=64, rot_dim=32, vdim=32, kv_rank=96, base=1e6, scale=0.08, mlp=dense(80))],
                  width=64, vocab=203, eps=1e-6, loop=(0, 2, 2), cap=None)


def odd_shapes() -> dict:
    """Sizes that no fast path is made for: a width and a vocabulary that are no multiples of 8, odd head and value
    sizes, a latent of 35, one head, and no repeated span at all."""
    return config([latent(heads=1, dim=9, rot_dim=6, vdim=7, kv_rank=35, scale=0.4, mlp=dense(30)),
                   latent(heads=5, dim=10, rot_dim=2, vdim=11, kv_rank=13, base=3.0, scale=0.25, mlp=moe(ff=9, experts=4, top=4, shared=5))],
                  width=44, vocab=77, loop=None, cap=3.0)


def lively(tensors: Dict[str, torch.Tensor], seed: int = 1) -> None:
    """Make the random weights show more: larger matrices inside the mixers (scores of order one, gates away from a
    half), pass vectors and activation coefficients of order one, norm weights that differ."""
    g = torch.Generator().manual_seed(seed)
    for name, t in tensors.items():
        def fill(lo, hi):
            t.copy_((torch.rand(t.shape, generator=g) * (hi - lo) + lo).to(t.dtype))
        if name.endswith((".mix.q", ".mix.dkv", ".mix.g")):
            t.mul_(10.0)
        elif name.endswith((".mix.uk", ".mix.uv")):
            t.mul_(6.0)
        elif name == "loop.step":
            fill(-1.0, 1.0)
        elif name.endswith(".mlp.act"):
            fill(-1.0, 1.5)
        elif name.endswith((".mix.dkv.norm", "norm1b", "norm2b")):
            fill(0.5, 2.0)


def plain_logits(folder: str, requests: Dict[str, List[int]], rounded: bool = False) -> Dict[str, torch.Tensor]:
    cfg, w = read_folder(folder)
    store = P.round_to_bfloat16 if rounded else P._keep
    return {rid: P.forward(cfg, w, toks, store=store) for rid, toks in requests.items()}
