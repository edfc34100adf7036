"""Gated feed-forward: down( act(gate(x)) * up(x) ), act = SiLU or the tanh form of GELU, the
residual added in the last product's epilogue.  gate and up are one stacked product whose rows are [gate | up]
(kernels/fused_silu_fp8_quant.cu:52-56 and v3/crates/rvllm-runtime/src/layer_exec.rs:476-522
of the reference)."""
from __future__ import annotations

from .base import FEED_FORWARDS, Part
from .linear import Linear


class GatedMLP(Part):
    takes_input_norm = True           # the gate/up product can apply the layer's RMSNorm itself

    ACTIVATIONS = ("silu", "gelu_tanh")

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 names=("gate_proj", "up_proj", "down_proj"), suffix: str = ".weight"):
        from ..errors import ConfigError
        if activation not in self.ACTIVATIONS:
            raise ConfigError(f"gated MLP activation {activation!r} is not supported (known: {', '.join(self.ACTIVATIONS)})")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.gate_up = Linear(hidden_size, [intermediate_size, intermediate_size], list(names[:2]), suffix=suffix)
        self.down = Linear(intermediate_size, [hidden_size], [names[2]], suffix=suffix)

    def tensor_specs(self):
        return {**self.gate_up.tensor_specs(), **self.down.tensor_specs()}

    def bind(self, get):
        self.gate_up.bind(get)
        self.down.bind(get)

    def __call__(self, x, ctx, residual=None, input_norm=None, out_dtype=None):
        if self.activation == "silu":
            h = ctx.kernels.gate_up_silu(x, self.gate_up.weight, norm=input_norm)
        else:
            h = ctx.kernels.gate_up_act(x, self.gate_up.weight, self.activation, norm=input_norm)
        return self.down(h, ctx, residual=residual, out_dtype=out_dtype)


FEED_FORWARDS.register("gated_mlp", GatedMLP)
