"""The Vipelix design on the engine's host side, without a GPU: configuration, tensor names, the plain mechanisms
themselves, and the real step function, cache manager, scheduler, trace replay and entry point driven with the torch
stand-ins for the kernels (emulated_kernels.py) against the plain implementation (plain_vipelix.py).  What is checked
here is the bookkeeping - one cache per pass of a repeated span, pages freed and used again, portions cut anywhere,
the embedded tokens kept for the later passes; the kernels themselves are checked by the GPU tests."""
import io
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_vipelix as P
import trace_tools as TT
import vipelix_tools as X
from emulated_kernels import EmulatedKernels
from model_tools import random_requests

from rvllm_b200 import ConfigError, LLM, SamplingParams, config_from_dict, kernels as kernel_pkg, load_config
from rvllm_b200.engine import trace as trace_mod
from rvllm_b200.engine.step import StepEntry
from rvllm_b200.models.decoder import DecoderModel, expected_tensors
from rvllm_b200.parts.base import KvCacheNeed


@pytest.fixture
def emulated():
    kernel_pkg.set_library(EmulatedKernels())
    yield
    kernel_pkg.set_library(None)


# ---------------------------------------------------------------------------------------- configuration
def test_config_round_trip_and_spec():
    cfg = config_from_dict(X.small_a())
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.to_spec()
    assert spec.residual_dtype == "float32" and spec.lm_head_name is None and not spec.validate()
    # layer 0 once, layers 1-2 three times with a cache each, layer 3 once; a pass opens with an addition to the stream
    assert [(e.layer, e.cache, len(e.before)) for e in spec.run_order] == \
        [(0, 0, 0), (1, 1, 1), (2, 2, 0), (1, 3, 1), (2, 4, 0), (1, 5, 1), (2, 6, 0), (3, 7, 0)]
    opens = [e.before[0].params for e in spec.run_order if e.before]
    assert [(o["index"], o["add_embedding"]) for o in opens] == [(0, False), (1, True), (2, True)]
    shapes = {n: ts.shape for n, ts in expected_tensors(spec).items()}
    assert shapes["loop.step"] == (3, 48) and "head" not in shapes
    assert shapes["l0.mix.q"] == (3 * (24 + 16), 48) and shapes["l0.mix.dkv"] == (40 + 16, 48) and shapes["l0.mix.dkv.norm"] == (40,)
    assert shapes["l1.mix.uk"] == (2 * 16, 24) and shapes["l1.mix.uv"] == (2 * 32, 24) and shapes["l1.mix.g"] == (2, 48)
    assert shapes["l1.mix.o"] == (48, 2 * 32) and shapes["l0.mlp.act"] == (4,) and shapes["l0.mlp.up"] == (56, 48)
    assert shapes["l1.mlp.table"] == (131, 2) and shapes["l1.mlp.e4.down"] == (48, 24) and shapes["l1.mlp.shared.gate"] == (16, 48)
    assert "l3.mlp.shared.up" not in shapes and "l3.mlp.e2.up" in shapes and "l3.mlp.e3.up" not in shapes
    assert "l2.norm2" not in shapes and "l2.norm1b" in shapes                     # no feed-forward, no norms around one
    needs = DecoderModel(spec).cache_needs()
    assert needs[1] == KvCacheNeed(1, 24 + 8, None, planes=1) and needs[0] == KvCacheNeed(1, 40 + 16, None, planes=1)
    assert len(needs) == 8
    # without a repeated span every layer runs once and nothing is added between layers
    plain = config_from_dict(X.odd_shapes()).to_spec()
    assert [(e.layer, len(e.before)) for e in plain.run_order] == [(0, 0), (1, 0)] and "loop.step" not in expected_tensors(plain)
    assert [h.kind for h in plain.logit_hooks] == ["logit_softcap"] and not config_from_dict(X.small_b()).to_spec().logit_hooks
    # an empty span is no span: no pass is opened, and a table of pass vectors in the checkpoint is left alone
    empty = X.small_a()
    empty["loop"] = {"start": 2, "stop": 2, "times": 5}
    spec = config_from_dict(empty).to_spec()
    assert [(e.layer, len(e.before)) for e in spec.run_order] == [(0, 0), (1, 0), (2, 0), (3, 0)] and spec.ignored_tensors == ("loop.step",)


def test_config_problems_are_collected():
    bad = X.small_a()
    bad["layers"][0]["mixer"]["rot"]["dims"] = 18          # beyond the rotated block
    bad["layers"][1]["mixer"]["kv_rank"] = 0
    bad["layers"][1]["mlp"]["router"]["top"] = 9           # of 5 experts
    bad["layers"][2]["type"] = "attention"
    bad["layers"][3]["mlp"] = {"kind": "wide"}
    bad["loop"] = {"start": 3, "stop": 2, "times": 0}          # a span that ends before it starts
    bad["logit_softcap"] = -1
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    text = str(e.value)
    for piece in ("rot.dims", "kv_rank", "`top` 9", "'attention'", "wide", "loop", "`times`", "logit_softcap"):
        assert piece in text, (piece, text)


# ---------------------------------------------------------------------------------------- the plain mechanisms
def test_plain_rotation_turns_neighbouring_pairs():
    v = torch.zeros(3, 6, dtype=torch.float64)
    v[:, 0], v[:, 2], v[:, 4] = 1.0, 1.0, 1.0
    out = P.turn_pairs(v, torch.tensor([0, 1, 5]), 4, 100.0)
    assert torch.allclose(out[0], v[0])                                          # position 0: nothing turns
    for t, p in ((1, 1.0), (2, 5.0)):
        assert torch.allclose(out[t, :2], torch.tensor([torch.cos(torch.tensor(p)), torch.sin(torch.tensor(p))], dtype=torch.float64))
        a = p * 100.0 ** -0.5                                                    # pair 1 of 2: base^(-2/4)
        assert torch.allclose(out[t, 2:4], torch.tensor([torch.cos(torch.tensor(a)), torch.sin(torch.tensor(a))], dtype=torch.float64))
        assert float(out[t, 4]) == 1.0 and float(out[t, 5]) == 0.0               # beyond `dims`: untouched
    # a relative angle: the product of two turned vectors depends on the difference of their positions only
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(1, 8, generator=g, dtype=torch.float64), torch.randn(1, 8, generator=g, dtype=torch.float64)
    d1 = P.turn_pairs(a, torch.tensor([7]), 8, 50.0) @ P.turn_pairs(b, torch.tensor([3]), 8, 50.0).T
    d2 = P.turn_pairs(a, torch.tensor([104]), 8, 50.0) @ P.turn_pairs(b, torch.tensor([100]), 8, 50.0).T
    assert torch.allclose(d1, d2, atol=1e-12)


def test_plain_latent_attention_against_its_absorbed_form():
    """The same attention with the up-projections moved out of the sum over the keys (what an engine that caches the
    latent computes) gives the same numbers."""
    g = torch.Generator().manual_seed(3)
    T, width, m = 11, 20, {"heads": 3, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 7, "scale": 0.4, "rot": {"dims": 4, "base": 30.0}}
    H, D, Rd, V, R = 3, 6, 4, 5, 7
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    w = {"q": rnd(H * (D + Rd), width), "dkv": rnd(R + Rd, width), "dkv.norm": rnd(R), "uk": rnd(H * D, R), "uv": rnd(H * V, R),
         "g": rnd(H, width), "o": rnd(width, H * V)}
    h, pos = rnd(T, width), torch.arange(T)
    want = P.latent_attention(h, w, "", m, 1e-5, pos)
    q = (h @ w["q"].T).view(T, H, D + Rd)
    down = h @ w["dkv"].T
    row = torch.cat([P.rms_norm(down[:, :R], w["dkv.norm"], 1e-5), P.turn_pairs(down[:, R:], pos, 4, 30.0)], dim=1)   # what is cached
    outs = []
    for i in range(H):
        qi = torch.cat([q[:, i, :D] @ w["uk"][i * D:(i + 1) * D], P.turn_pairs(q[:, i, D:], pos, 4, 30.0)], dim=1)
        s = (qi @ row.T * 0.4).masked_fill(pos[None, :] > pos[:, None], float("-inf"))
        outs.append((torch.softmax(s, -1) @ row[:, :R]) @ w["uv"][i * V:(i + 1) * V].T * torch.sigmoid(h @ w["g"].T)[:, i:i + 1])
    assert torch.allclose(torch.cat(outs, 1) @ w["o"].T, want, atol=1e-10)
    # causal: the first token sees itself only, so its output is its own value under its gate
    first = torch.cat([(row[0, :R] @ w["uv"][i * V:(i + 1) * V].T) * torch.sigmoid(h[0] @ w["g"][i]) for i in range(H)]) @ w["o"].T
    assert torch.allclose(want[0], first, atol=1e-10)


def test_plain_polynorm_and_experts():
    z = torch.tensor([[1.0, -2.0, 3.0, 0.5]], dtype=torch.float64)
    coef = torch.tensor([2.0, -1.0, 0.5, 0.25], dtype=torch.float64)
    n = lambda v: v / torch.sqrt((v * v).mean() + 1e-5)
    assert torch.allclose(P.polynorm(z, coef, 1e-5)[0], 2 * n(z[0]) - n(z[0] ** 2) + 0.5 * n(z[0] ** 3) + 0.25)
    assert torch.allclose(P.polynorm(3 * z, torch.tensor([1.0, 0, 0, 0]), 0.0), P.polynorm(z, torch.tensor([1.0, 0, 0, 0]), 0.0))  # scale-free
    g = torch.Generator().manual_seed(2)
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    w = {"table": torch.tensor([[2, 0], [1, 2], [0, 1]])}
    for e in ("e0.", "e1.", "e2.", "shared."):
        w.update({e + "gate": rnd(4, 6), e + "up": rnd(4, 6), e + "down": rnd(6, 4)})
    h, tok = rnd(3, 6), torch.tensor([1, 1, 2])
    mlp = {"router": {"experts": 3, "top": 2}, "shared": {"ff": 4}}
    out = P.table_moe(h, tok, w, "", mlp)
    want1 = 0.5 * (P.gated_expert(h[1:2], w, "e1.") + P.gated_expert(h[1:2], w, "e2.")) + P.gated_expert(h[1:2], w, "shared.")
    assert torch.allclose(out[1:2], want1, atol=1e-12)
    assert torch.allclose(out[0] - P.gated_expert(h[0:1], w, "shared.")[0], 0.5 * (P.gated_expert(h[0:1], w, "e1.") + P.gated_expert(h[0:1], w, "e2."))[0])
    assert not torch.allclose(out[2], out[1])                                    # another token id, other experts


# ---------------------------------------------------------------------------------------- replay through the engine
LENGTHS = (41, 70, 23, 88, 1, 37)
SCHEDULES = {"whole": TT.schedule_whole, "bulk_tail": TT.schedule_bulk_tail, "portions": TT.schedule_portions,
             "mixed": TT.schedule_mixed}
_cache = {}


def _reference(which):
    if which not in _cache:
        folder = X.write_folder({"a": X.small_a, "b": X.small_b, "odd": X.odd_shapes}[which](), seed=5, edit=X.lively)
        vocab = load_config(folder).vocab_size
        reqs = random_requests(vocab, LENGTHS, seed=4)
        _cache[which] = (folder, vocab, reqs, X.plain_logits(folder, reqs))
    return _cache[which]


@pytest.mark.parametrize("which", ["a", "b"])
@pytest.mark.parametrize("schedule", list(SCHEDULES))
def test_replay_matches_plain_under_every_cut(emulated, tmp_path, which, schedule):
    folder, vocab, reqs, ref = _reference(which)
    trace = SCHEDULES[schedule](reqs)
    if schedule == "portions":
        assert min(len(e["tokens"]) for s in trace.steps for e in s["entries"]) <= 2
    if schedule == "mixed":
        assert max(len(s["entries"]) for s in trace.steps) == 4 and trace.preemptions == 1     # pages are freed and used again
    engine = trace_mod.build_engine(folder, "float32", trace.max_tokens, block_size=8, device="cpu")
    assert all(g.need.planes == 1 and g.tensor.shape[2] == 1 for g in engine.cache.groups)
    n = trace_mod.replay(engine, io.StringIO(trace.lines()), str(tmp_path), io.StringIO())
    assert n == len(trace.steps)
    got = TT.read_logits(str(tmp_path), trace, vocab)
    assert TT.compare(got, ref, 2e-5, f"{which}/{schedule}") < 2e-5
    engine.cache.check()
    assert not engine.cache.requests and engine.cache.slots.num_free == 4


def test_streams_after_every_layer_run(emulated):
    """The residual stream after each run of a layer (a repeated layer counts each time) against the plain one."""
    folder, vocab, reqs, _ = _reference("a")
    cfg, w = X.read_folder(folder)
    toks = reqs["r2"]
    want = []
    P.forward(cfg, w, toks, streams=want)
    engine = trace_mod.build_engine(folder, "float32", 64, block_size=8, device="cpu")
    seen = []
    def recording(block):
        def run(x, ctx, cache, write=True):
            y = block(x, ctx, cache, write)
            seen.append(y.clone())           # (the next layer adds into y in place)
            return y
        return run

    for layer in engine.model.layers:
        layer.block = recording(layer.block)
    engine.runner.step([StepEntry("x", toks, [0])])
    assert len(seen) == len(want) == 8
    for k, (a, b) in enumerate(zip(seen, want)):
        assert float((a.double() - b).abs().max() / b.abs().max()) < 1e-5, f"layer run {k}"


def test_odd_sizes_in_portions(emulated):
    folder, vocab, reqs, ref = _reference("odd")
    engine = trace_mod.build_engine(folder, "float32", 128, block_size=8, device="cpu")
    toks = reqs["r1"]
    got = torch.cat([engine.runner.step([StepEntry("x", toks[:9], list(range(9)))]),
                     engine.runner.step([StepEntry("x", toks[9:11], [0, 1])]),
                     engine.runner.step([StepEntry("x", toks[11:69], list(range(58)))]),
                     engine.runner.step([StepEntry("x", toks[69:], [0])])]).double()
    assert float((got - ref["r1"]).abs().max() / ref["r1"].abs().max()) < 2e-5
    engine.runner.finish("x")
    engine.cache.check()


def test_generate_greedy_matches_plain(emulated):
    folder, vocab, reqs, ref = _reference("a")
    cfg, w = X.read_folder(folder)
    prompts = [reqs["r2"], reqs["r4"], reqs["r0"][:30]]
    llm = LLM(folder, dtype="float32", device="cpu", block_size=8, num_blocks=24, max_model_len=64, max_num_seqs=2,
              max_num_batched_tokens=16, max_prefill_chunk=7)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == P.greedy(cfg, w, p, 6)
    assert not llm.engine.cache.requests


def test_command_line_info_and_random_weights(tmp_path):
    """`rvllm random-weights` writes a folder for the design from a config.json; `rvllm info` reads it back."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(X.small_a()))
    out = tmp_path / "model"
    run = lambda *a: subprocess.run([sys.executable, os.path.join(root, "bin", "rvllm"), *a], capture_output=True, text=True, timeout=300)
    p = run("random-weights", "--config", str(cfg_file), "--out", str(out), "--seed", "3")
    assert p.returncode == 0, p.stderr
    p = run("info", "--model", str(out))
    assert p.returncode == 0, p.stderr
    info = json.loads(p.stdout)
    assert info["architecture"] == "Vipelix" and info["config"]["loop"] == {"start": 1, "stop": 3, "times": 3}
    # one row per token and layer run: 56 + 3 x (32 + 32) + 56 elements of two bytes
    assert info["kv_bytes_per_token_bf16"] == 2 * (56 + 3 * (32 + 32) + 56)
    cfg, w = X.read_folder(str(out))
    table = w["l1.mlp.table"]
    assert table.dtype == torch.int32 and int(table.min()) >= 0 and int(table.max()) < 5 and bool((table[:, 0] != table[:, 1]).all())
    assert P.forward(cfg, w, [1, 2, 3]).shape == (3, 131)
