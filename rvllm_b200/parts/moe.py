"""Feed-forwards beyond the gated MLP: a dense one with a PolyNorm activation, and a mixture of gated experts whose
choice is a table lookup by token id.

`polynorm_mlp`   down( P(up(x)) ),  P(z) = a n(z) + b n(z^2) + c n(z^3) + e  with powers taken element by element and
                 n(v) = v / sqrt(mean(v^2) + eps) over the token's whole vector; the four numbers are a tensor.
`table_moe`      every token runs `top` of `experts` gated MLPs  down_e( silu(gate_e x) * up_e x ), each weighted 1 / top;
                 which ones is read from an integer table [vocab, top] at the token's id (no router product, no
                 softmax); optionally a shared expert of the same form runs for every token and is added.
                 The experts' matrices are kept stacked ([experts, 2 ff, width] gate rows then up rows, and
                 [experts, width, ff]) so that one kernel serves all of them.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import FEED_FORWARDS, Part, TensorSpec
from .linear import Linear
from .mlp import GatedMLP


class PolyNormMLP(Part):
    def __init__(self, hidden_size: int, intermediate_size: int, eps: float, names=("up", "down", "act"), suffix: str = ""):
        self.hidden_size, self.intermediate_size, self.eps = hidden_size, intermediate_size, eps
        self.up = Linear(hidden_size, [intermediate_size], [names[0]], suffix=suffix)
        self.down = Linear(intermediate_size, [hidden_size], [names[1]], suffix=suffix)
        self.coef_name = names[2]
        self.coef = None

    def tensor_specs(self):
        return {**self.up.tensor_specs(), **self.down.tensor_specs(), self.coef_name: TensorSpec((4,), "coef")}

    def bind(self, get):
        self.up.bind(get)
        self.down.bind(get)
        self.coef = get(self.coef_name).float().contiguous()        # norms are float32

    def __call__(self, x, ctx, residual=None, out_dtype=None):
        z = self.up(x, ctx, out_dtype=torch.float32)
        h = ctx.kernels.polynorm(z, self.coef, self.eps, x.dtype)
        return self.down(h, ctx, residual=residual, out_dtype=out_dtype)


class TableMoE(Part):
    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int, vocab_size: int,
                 shared_intermediate_size: Optional[int] = None, names=("gate", "up", "down"), table: str = "table",
                 expert_prefix: str = "e", shared_prefix: str = "shared.", suffix: str = ""):
        from ..errors import ConfigError
        if not 1 <= top <= experts:
            raise ConfigError(f"a token uses {top} of {experts} experts")
        self.hidden_size, self.intermediate_size, self.experts, self.top = hidden_size, intermediate_size, experts, top
        self.vocab_size, self.names, self.table_name, self.expert_prefix = vocab_size, tuple(names), table, expert_prefix
        self.suffix = suffix
        self.shared_prefix = shared_prefix
        self.shared = None
        if shared_intermediate_size is not None:
            self.shared = GatedMLP(hidden_size, shared_intermediate_size, "silu", names=names, suffix=suffix)
        self.table = self.gate_up = self.down = None

    def tensor_specs(self):
        g, u, d = self.names
        specs = {self.table_name: TensorSpec((self.vocab_size, self.top), f"choice:{self.experts}")}
        for e in range(self.experts):
            p = f"{self.expert_prefix}{e}."
            specs[f"{p}{g}{self.suffix}"] = TensorSpec((self.intermediate_size, self.hidden_size), "matrix")
            specs[f"{p}{u}{self.suffix}"] = TensorSpec((self.intermediate_size, self.hidden_size), "matrix")
            specs[f"{p}{d}{self.suffix}"] = TensorSpec((self.hidden_size, self.intermediate_size), "matrix")
        if self.shared is not None:
            specs.update({self.shared_prefix + n: ts for n, ts in self.shared.tensor_specs().items()})
        return specs

    def bind(self, get):
        g, u, d = self.names
        self.table = get(self.table_name).to(torch.int32).contiguous()
        rows = []
        for e in range(self.experts):
            p = f"{self.expert_prefix}{e}."
            rows.append(torch.cat([get(f"{p}{g}{self.suffix}"), get(f"{p}{u}{self.suffix}")], dim=0))
        self.gate_up = torch.stack(rows).contiguous()                                   # [E, 2 ff, width]
        self.down = torch.stack([get(f"{self.expert_prefix}{e}.{d}{self.suffix}") for e in range(self.experts)]).contiguous()
        if self.shared is not None:
            self.shared.bind(lambda name: get(self.shared_prefix + name))

    def __call__(self, x, ctx, residual=None, out_dtype=None):
        k = ctx.kernels
        y = self.shared(x, ctx, residual=residual, out_dtype=torch.float32) if self.shared is not None else residual
        chosen = k.gather_rows(self.table, ctx.token_ids)                 # [tokens, top] expert numbers
        return k.moe_experts(x, chosen, self.gate_up, self.down, 1.0 / self.top, add=y, out_dtype=out_dtype or x.dtype)


FEED_FORWARDS.register("polynorm_mlp", PolyNormMLP)
FEED_FORWARDS.register("table_moe", TableMoE)
