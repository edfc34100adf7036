"""Configuration of the Vipelix decoder: layers of latent attention (one cached low-rank row per token, a rotated
key part shared by all heads, a sigmoid gate per head) with an RMSNorm in front of and behind every sublayer, a
float32 residual stream, feed-forwards that are dense with a PolyNorm activation or a mixture of gated experts
chosen by a table lookup on the token id (plus an optional shared expert), a span of layers that runs several times
with the same tensors, tied input and output embeddings and capped logits.

config.json keys (all sizes and every constant that may differ between models are read, none is assumed):

    architecture            "Vipelix"
    width, vocab            model width and vocabulary size
    norm.eps                eps of every RMSNorm (layer norms, the latent's norm, PolyNorm, the final norm)
    logit_softcap           c: logits <- c tanh(logits / c); absent or null: none
    loop                    {start, stop, times}: layers start .. stop-1 run `times` times in a row, every pass with a
                            cache of its own; before each pass but the first the embedded tokens are added to the
                            stream, and before every pass row `pass` of the tensor `loop.step`; absent: every layer once
    layers[i].type          "latent_attention"
    layers[i].mixer         heads, dim (unrotated query/key size per head), rot_dim (rotated size), vdim, kv_rank, scale,
                            rot.dims (leading elements of the rotated part that turn; pairs 2i, 2i+1), rot.base
    layers[i].mlp           null | {"kind": "dense", "ff": n}
                                 | {"kind": "moe", "expert": {"ff": n}, "router": {"experts": E, "top": k}, "shared": {"ff": m} | null}
    max_positions           optional: the longest sequence the rotation tables are ever built for

Tensor names: embed, final.norm, loop.step, l<i>.norm1, norm1b, norm2, norm2b, l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o},
l<i>.mlp.{up,down,act} or l<i>.mlp.{table, e<j>.gate, e<j>.up, e<j>.down, shared.gate, shared.up, shared.down}.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

DEFAULT_MAX_POSITIONS = 1 << 17       # the design sets no limit; the engine's tables are built for max_model_len


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@dataclass(frozen=True)
class VipelixLayer:
    type: str                              # "latent_attention"
    mixer: Dict[str, Any]                  # heads, dim, rot_dim, vdim, kv_rank, scale, rot_dims, rot_base
    mlp: Optional[Dict[str, Any]]          # None | {kind: dense, ff} | {kind: moe, ff, experts, top, shared_ff | None}


@dataclass(frozen=True)
class VipelixConfig:
    width: int
    vocab: int
    eps: float
    layers: Tuple[VipelixLayer, ...]
    loop: Optional[Tuple[int, int, int]] = None        # (start, stop, times)
    logit_softcap: Optional[float] = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    ARCHITECTURE = "Vipelix"

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
    def from_dict(cls, obj: Dict[str, Any], where: str = "config.json") -> "VipelixConfig":
        p: List[str] = []

        def integer(d, key, what, minimum=1):
            v = d.get(key) if isinstance(d, dict) else None
            if not _is_int(v) or v < minimum:
                p.append(f"{what}`{key}` must be an integer >= {minimum}, got {v!r}")
                return max(minimum, 1)
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
        layers: List[VipelixLayer] = []
        for i, e in enumerate(raw_layers):
            at = f"layers[{i}]: "
            if not isinstance(e, dict):
                p.append(at + "must be an object")
                continue
            kind, m = e.get("type"), e.get("mixer")
            if kind != "latent_attention":
                p.append(at + f"`type` = {kind!r} is not known (latent_attention)")
            if not isinstance(m, dict):
                p.append(at + "`mixer` must be an object")
                m = {}
            mixer: Dict[str, Any] = {key: integer(m, key, at) for key in ("heads", "dim", "vdim", "kv_rank")}
            mixer["rot_dim"] = integer(m, "rot_dim", at, minimum=2)
            mixer["scale"] = number(m, "scale", at)
            rot = m.get("rot")
            mixer["rot_dims"] = integer(rot, "dims", at + "rot: ", minimum=2)
            mixer["rot_base"] = number(rot, "base", at + "rot: ")
            if mixer["rot_dim"] % 2 or mixer["rot_dims"] % 2 or mixer["rot_dims"] > mixer["rot_dim"]:
                p.append(at + f"`rot_dim` and `rot.dims` must be even with rot.dims <= rot_dim, got {mixer['rot_dim']} and {mixer['rot_dims']}")
            raw_mlp, mlp = e.get("mlp"), None
            if raw_mlp is not None:
                mk = raw_mlp.get("kind") if isinstance(raw_mlp, dict) else None
                if mk == "dense":
                    mlp = {"kind": "dense", "ff": integer(raw_mlp, "ff", at + "mlp: ")}
                elif mk == "moe":
                    router = raw_mlp.get("router")
                    mlp = {"kind": "moe", "ff": integer(raw_mlp.get("expert"), "ff", at + "mlp.expert: "),
                           "experts": integer(router, "experts", at + "mlp.router: "),
                           "top": integer(router, "top", at + "mlp.router: "), "shared_ff": None}
                    if mlp["top"] > mlp["experts"]:
                        p.append(at + f"mlp.router: `top` {mlp['top']} exceeds `experts` {mlp['experts']}")
                    if raw_mlp.get("shared") is not None:
                        mlp["shared_ff"] = integer(raw_mlp.get("shared"), "ff", at + "mlp.shared: ")
                else:
                    p.append(at + f"`mlp` must be null or an object of kind \"dense\" or \"moe\", got {raw_mlp!r}")
            layers.append(VipelixLayer("latent_attention", mixer, mlp))
        loop = None
        raw_loop = obj.get("loop")
        if raw_loop is not None:
            start = integer(raw_loop, "start", "loop: ", minimum=0)
            stop = integer(raw_loop, "stop", "loop: ", minimum=0)
            times = integer(raw_loop, "times", "loop: ")
            if not (0 <= start <= stop <= len(raw_layers)):
                p.append(f"loop: start {start} and stop {stop} must name a span of the {len(raw_layers)} layers")
            loop = (start, stop, times)
        cap = obj.get("logit_softcap")
        if cap is not None and (not _is_num(cap) or not cap > 0):
            p.append(f"`logit_softcap` must be null or a number > 0, got {cap!r}")
            cap = None
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
        return cls(width=width, vocab=vocab, eps=eps, layers=tuple(layers), loop=loop,
                   logit_softcap=float(cap) if cap is not None else None, max_positions=max_pos, eos_token_ids=eos_ids,
                   raw=dict(obj))

    # ---- writing -------------------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        out_layers = []
        for layer in self.layers:
            m = dict(layer.mixer)
            m["rot"] = {"dims": m.pop("rot_dims"), "base": m.pop("rot_base")}
            mlp = None
            if layer.mlp is not None and layer.mlp["kind"] == "dense":
                mlp = {"kind": "dense", "ff": layer.mlp["ff"]}
            elif layer.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": layer.mlp["ff"]},
                       "router": {"experts": layer.mlp["experts"], "top": layer.mlp["top"]},
                       "shared": None if layer.mlp["shared_ff"] is None else {"ff": layer.mlp["shared_ff"]}}
            out_layers.append({"type": layer.type, "mixer": m, "mlp": mlp})
        d: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "width": self.width, "vocab": self.vocab,
                             "norm": {"eps": self.eps}, "layers": out_layers}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- the model this configuration describes ----------------------------------------------------
    def run_plan(self) -> List[Tuple[int, Optional[int]]]:
        """(layer, pass) in execution order; pass is the number of the pass that the entry opens, else None."""
        n = len(self.layers)
        if self.loop is None or self.loop[0] == self.loop[1]:       # no span, or an empty one: every layer once, nothing between
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        plan: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(start)]
        for t in range(times):
            plan.extend((i, t if i == start else None) for i in range(start, stop))
        plan.extend((i, None) for i in range(stop, n))
        return plan

    def to_spec(self) -> ModelSpec:
        rotations: Dict[Tuple[int, int, float], str] = {}
        norm = PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "tensor": ""}, "norm")
        specs = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            rkey = (m["rot_dim"], m["rot_dims"], m["rot_base"])
            rotations.setdefault(rkey, f"rot{len(rotations)}")
            parts = {"mixer": PartSpec("latent_attention", {
                "hidden_size": self.width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                "value_dim": m["vdim"], "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": self.eps, "gate": True,
                "position": rotations[rkey], "suffix": ""}, "mixer"),
                "mixer_norm": norm, "mixer_out_norm": norm}
            names = {"mixer": "mix.", "mixer_norm": "norm1", "mixer_out_norm": "norm1b"}
            if layer.mlp is not None:
                if layer.mlp["kind"] == "dense":
                    ff = PartSpec("polynorm_mlp", {"hidden_size": self.width, "intermediate_size": layer.mlp["ff"], "eps": self.eps,
                                                   "names": ("up", "down", "act"), "suffix": ""}, "feed_forward")
                else:
                    ff = PartSpec("table_moe", {"hidden_size": self.width, "intermediate_size": layer.mlp["ff"],
                                                "experts": layer.mlp["experts"], "top": layer.mlp["top"], "vocab_size": self.vocab,
                                                "shared_intermediate_size": layer.mlp["shared_ff"], "names": ("gate", "up", "down"),
                                                "table": "table", "expert_prefix": "e", "shared_prefix": "shared.", "suffix": ""},
                                  "feed_forward")
                parts.update({"feed_forward": ff, "feed_forward_norm": norm, "feed_forward_out_norm": norm})
                names.update({"feed_forward": "mlp.", "feed_forward_norm": "norm2", "feed_forward_out_norm": "norm2b"})
            specs.append(LayerSpec(f"l{i}.", PartSpec("sandwich_norm_residual"), parts, names))
        run_order = []
        for n, (i, opens) in enumerate(self.run_plan()):
            before = ()
            if opens is not None:
                before = (PartSpec("stream_offset", {"width": self.width, "rows": self.loop[2], "index": opens,
                                                     "add_embedding": opens > 0, "tensor": "loop.step"}),)
            run_order.append(RunEntry(layer=i, cache=n, before=before))
        hooks = () if self.logit_softcap is None else (PartSpec("logit_softcap", {"cap": self.logit_softcap}),)
        return ModelSpec(
            architecture=self.ARCHITECTURE, hidden_size=self.width, vocab_size=self.vocab,
            max_position_embeddings=self.max_positions, embedding_name="embed", layers=tuple(specs), run_order=tuple(run_order),
            final_norm=PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "tensor": ""}), final_norm_prefix="final.norm",
            lm_head_name=None,
            position_encodings={key: PartSpec("rotary", {"head_dim": rd, "theta": base, "rotary_dim": dims})
                                for (rd, dims, base), key in rotations.items()},
            logit_hooks=hooks, residual_dtype="float32", eos_token_ids=self.eos_token_ids,
            # (an empty span opens no pass: its table of pass vectors, if the checkpoint has one, is never read)
            ignored_tensors=("loop.step",) if self.loop is not None and self.loop[0] == self.loop[1] else ())
