"""Configuration of the Tufirax decoder: a stack of layers that each hold one mixer - attention
with whole-row q/k norms, a score cap, a sink and a head gate, or a mamba2 state-space mixer - and
optionally a GELU-gated feed-forward, with an RMSNorm on the OUTPUT of each sublayer and a float32
residual stream.  A layer may reuse another layer's tensors while keeping a cache of its own.

config.json keys (all sizes and every constant that may differ between models are read, none is
assumed):

    architecture            "Tufirax"
    width, vocab            model width and vocabulary size
    norm.eps                eps of every RMSNorm (layer norms, q/k norms, the mixer's gated norm, the final norm)
    layers[i].type          "attention" | "mamba2"
    layers[i].mixer         attention: heads, kv_heads, dim, vdim (= dim: the values are the keys), scale, softcap,
                                       rot.dims, rot.base
                            mamba2:    heads, vdim, state, groups, conv, norm_groups
    layers[i].mlp           null | {"kind": "dense", "ff": n}
    layers[i].weights_of    j: the layer has no tensors of its own and runs with layer j's
    max_positions           optional: the longest sequence the rotation tables are ever built for

Tensor names: embed, head, final.norm, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.{gate,up,down}.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

DEFAULT_MAX_POSITIONS = 1 << 17       # the design sets no limit; the engine's tables are built for max_model_len

_ATTENTION_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale", "softcap", "rot")
_MAMBA2_KEYS = ("heads", "vdim", "state", "groups", "conv", "norm_groups")


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@dataclass(frozen=True)
class TufiraxLayer:
    type: str                              # "attention" | "mamba2"
    mixer: Dict[str, Any]
    ff: Optional[int]                      # width of the feed-forward, None for a layer without one
    weights_of: Optional[int] = None


@dataclass(frozen=True)
class TufiraxConfig:
    width: int
    vocab: int
    eps: float
    layers: Tuple[TufiraxLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    ARCHITECTURE = "Tufirax"

    @property
    def architecture(self) -> str:
        return self.ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    # ---- reading -------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, obj: Dict[str, Any], where: str = "config.json") -> "TufiraxConfig":
        p: List[str] = []

        def integer(d, key, what, minimum=1):
            v = d.get(key) if isinstance(d, dict) else None
            if not _is_int(v) or v < minimum:
                p.append(f"{what}`{key}` must be an integer >= {minimum}, got {v!r}")
                return minimum
            return v

        def number(d, key, what):
            v = d.get(key) if isinstance(d, dict) else None
            if not _is_num(v) or not v > 0:
                p.append(f"{what}`{key}` must be a number > 0, got {v!r}")
                return 1.0
            return float(v)

        width = integer(obj, "width", "")
        vocab = integer(obj, "vocab", "")
        eps = number(obj.get("norm"), "eps", "norm: ")
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(p + ["`layers` must be a non-empty list"], where)
        layers: List[TufiraxLayer] = []
        for i, e in enumerate(raw_layers):
            at = f"layers[{i}]: "
            if not isinstance(e, dict):
                p.append(at + "must be an object")
                continue
            kind, m = e.get("type"), e.get("mixer")
            if not isinstance(m, dict):
                p.append(at + "`mixer` must be an object")
                m = {}
            mixer: Dict[str, Any] = {}
            if kind == "attention":
                for key in ("heads", "kv_heads", "dim"):
                    mixer[key] = integer(m, key, at)
                mixer["vdim"] = m.get("vdim", mixer["dim"])
                if mixer["vdim"] != mixer["dim"]:
                    p.append(at + f"`vdim` {mixer['vdim']!r} differs from `dim` {mixer['dim']}: the values of this attention are its keys")
                mixer["scale"] = number(m, "scale", at)
                mixer["softcap"] = number(m, "softcap", at)
                rot = m.get("rot")
                mixer["rot_dims"] = integer(rot, "dims", at + "rot: ", minimum=2)
                mixer["rot_base"] = number(rot, "base", at + "rot: ")
                if mixer["heads"] % mixer["kv_heads"]:
                    p.append(at + f"`heads` {mixer['heads']} is not a multiple of `kv_heads` {mixer['kv_heads']}")
                if mixer["rot_dims"] % 2 or mixer["rot_dims"] > mixer["dim"]:
                    p.append(at + f"`rot.dims` must be even and at most `dim` {mixer['dim']}, got {mixer['rot_dims']}")
            elif kind == "mamba2":
                for key in _MAMBA2_KEYS:
                    mixer[key] = integer(m, key, at)
                if mixer["heads"] % mixer["groups"]:
                    p.append(at + f"`heads` {mixer['heads']} is not a multiple of `groups` {mixer['groups']}")
                if (mixer["heads"] * mixer["vdim"]) % mixer["norm_groups"]:
                    p.append(at + f"heads x vdim = {mixer['heads'] * mixer['vdim']} does not split into `norm_groups` {mixer['norm_groups']}")
            else:
                p.append(at + f"`type` = {kind!r} is not known (attention, mamba2)")
            mlp, ff = e.get("mlp"), None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    p.append(at + f"`mlp` must be null or an object of kind \"dense\", got {mlp!r}")
                else:
                    ff = integer(mlp, "ff", at + "mlp: ")
            src = e.get("weights_of")
            if src is not None and (not _is_int(src) or not 0 <= src < len(raw_layers) or src == i):
                p.append(at + f"`weights_of` must name another layer, got {src!r}")
                src = None
            layers.append(TufiraxLayer(kind if kind in ("attention", "mamba2") else "attention", mixer, ff, src))
        # a layer that borrows tensors runs as its source describes itself (its own description repeats the source's)
        for i, layer in enumerate(layers):
            seen = {i}
            j = layer.weights_of
            while j is not None and j < len(layers):
                if j in seen:
                    p.append(f"layers[{i}]: `weights_of` runs in a circle")
                    break
                seen.add(j)
                j = layers[j].weights_of
            else:
                continue
        max_pos = obj.get("max_positions", DEFAULT_MAX_POSITIONS)
        if not _is_int(max_pos) or max_pos < 1:
            p.append(f"`max_positions` must be a positive integer, got {max_pos!r}")
            max_pos = DEFAULT_MAX_POSITIONS
        eos = obj.get("eos_token_id")
        eos_ids: Tuple[int, ...] = ()
        if _is_int(eos):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(_is_int(t) for t in eos):
            eos_ids = tuple(eos)
        elif eos is not None:
            p.append(f"`eos_token_id` must be an integer or a list of integers, got {eos!r}")
        if p:
            raise ConfigError(p, where)
        return cls(width=width, vocab=vocab, eps=eps, layers=tuple(layers), max_positions=max_pos, eos_token_ids=eos_ids,
                   raw=dict(obj))

    # ---- writing -------------------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        out_layers = []
        for layer in self.layers:
            m = dict(layer.mixer)
            if layer.type == "attention":
                m["rot"] = {"dims": m.pop("rot_dims"), "base": m.pop("rot_base")}
            e: Dict[str, Any] = {"type": layer.type, "mixer": m,
                                 "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}}
            if layer.weights_of is not None:
                e["weights_of"] = layer.weights_of
            out_layers.append(e)
        d: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "width": self.width, "vocab": self.vocab,
                             "norm": {"eps": self.eps}, "layers": out_layers}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- the model this configuration describes ----------------------------------------------------
    def source_of(self, i: int) -> int:
        """The layer whose tensors layer i runs with (itself unless it names another)."""
        while self.layers[i].weights_of is not None:
            i = self.layers[i].weights_of
        return i

    def to_spec(self) -> ModelSpec:
        owners = sorted({self.source_of(i) for i in range(len(self.layers))})
        index = {layer: n for n, layer in enumerate(owners)}
        rotations: Dict[Tuple[int, int, float], str] = {}
        specs = []
        for i in owners:
            layer = self.layers[i]
            m = layer.mixer
            if layer.type == "attention":
                rkey = (m["dim"], m["rot_dims"], m["rot_base"])
                rotations.setdefault(rkey, f"rot{len(rotations)}")
                mixer = PartSpec("gated_sink_attention", {
                    "hidden_size": self.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                    "scale": m["scale"], "eps": self.eps, "softcap": m["softcap"], "sink": True, "gate": True,
                    "position": rotations[rkey], "suffix": ""}, "mixer")
            else:
                mixer = PartSpec("mamba2", {
                    "hidden_size": self.width, "heads": m["heads"], "head_dim": m["vdim"], "state": m["state"],
                    "groups": m["groups"], "conv": m["conv"], "norm_groups": m["norm_groups"], "eps": self.eps,
                    "suffix": ""}, "mixer")
            norm = PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "tensor": ""}, "norm")
            parts = {"mixer": mixer, "mixer_norm": norm}
            names = {"mixer": "mix.", "mixer_norm": "norm1"}
            if layer.ff is not None:
                parts["feed_forward"] = PartSpec("gated_mlp", {
                    "hidden_size": self.width, "intermediate_size": layer.ff, "activation": "gelu_tanh",
                    "names": ("gate", "up", "down"), "suffix": ""}, "feed_forward")
                parts["feed_forward_norm"] = norm
                names.update({"feed_forward": "mlp.", "feed_forward_norm": "norm2"})
            specs.append(LayerSpec(f"l{i}.", PartSpec("output_norm_residual"), parts, names))
        run_order = tuple(RunEntry(layer=index[self.source_of(i)], cache=i) for i in range(len(self.layers)))
        return ModelSpec(
            architecture=self.ARCHITECTURE, hidden_size=self.width, vocab_size=self.vocab,
            max_position_embeddings=self.max_positions, embedding_name="embed", layers=tuple(specs), run_order=run_order,
            final_norm=PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "tensor": ""}), final_norm_prefix="final.norm",
            lm_head_name="head",
            position_encodings={key: PartSpec("rotary", {"head_dim": hd, "theta": base, "rotary_dim": dims})
                                for (hd, dims, base), key in rotations.items()},
            residual_dtype="float32", eos_token_ids=self.eos_token_ids)
