"""The Tufirax design on the engine's host side, without a GPU: configuration, tensor names, and the real
step function, cache and state manager, scheduler, trace replay and entry point driven with the torch stand-ins
for the kernels (emulated_kernels.py), against the plain implementation (plain_tufirax.py).  What is checked
here is the bookkeeping - state slots and pages that are freed and used again, portions cut anywhere, layers that
share tensors but not state; the kernels themselves are checked by the GPU tests."""
import io

import pytest
import torch

import plain_tufirax as P
import trace_tools as TT
import tufirax_tools as X
from emulated_kernels import EmulatedKernels
from model_tools import random_requests

from rvllm_b200 import ConfigError, LLM, SamplingParams, config_from_dict, kernels as kernel_pkg, load_config
from rvllm_b200.engine import trace as trace_mod
from rvllm_b200.models.decoder import expected_tensors


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
    assert spec.residual_dtype == "float32" and not spec.validate()
    assert len(spec.layers) == 3                                   # the layers that own tensors
    assert [(e.layer, e.cache) for e in spec.run_order] == [(0, 0), (1, 1), (1, 2), (2, 3), (0, 4)]
    names = set(expected_tensors(spec))
    assert {"embed", "head", "final.norm", "l0.norm1", "l1.norm1", "l1.norm2", "l1.mix.q", "l1.mix.q.norm", "l1.mix.sink",
            "l1.mix.g", "l1.mlp.gate", "l0.mix.in", "l0.mix.conv", "l0.mix.conv.b", "l0.mix.A_log", "l3.mlp.down"} <= names
    assert not any(n.startswith(("l2.", "l4.")) for n in names)    # layers that borrow have no tensors
    assert "l0.norm2" not in names                                  # no feed-forward, no second norm
    shapes = {n: ts.shape for n, ts in expected_tensors(spec).items()}
    assert shapes["l1.mix.q"] == (6 * 32, 72) and shapes["l1.mix.k"] == (2 * 32, 72) and shapes["l1.mix.g"] == (6, 72)
    assert shapes["l0.mix.in"] == (2 * 120 + 2 * 3 * 24 + 6, 72) and shapes["l0.mix.conv"] == (120 + 2 * 3 * 24, 3)
    assert shapes["l1.mix.q.norm"] == (192,) and shapes["l0.mix.norm"] == (120,)


def test_config_problems_are_collected():
    bad = X.small_a()
    bad["layers"][1]["mixer"]["vdim"] = 16          # the values are the keys: vdim = dim
    bad["layers"][1]["mixer"]["rot"]["dims"] = 40   # beyond the head
    bad["layers"][0]["mixer"]["groups"] = 4         # 6 heads do not split into 4 groups
    bad["layers"][3]["type"] = "conv"
    bad["layers"][4]["weights_of"] = 4
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    text = str(e.value)
    for piece in ("vdim", "rot.dims", "groups", "'conv'", "weights_of"):
        assert piece in text, (piece, text)
    loop = X.small_a()
    loop["layers"][1]["weights_of"] = 2             # 1 -> 2 -> 1
    with pytest.raises(ConfigError, match="circle"):
        config_from_dict(loop)


def test_architecture_key_forms():
    c = X.small_b()
    assert type(config_from_dict(c)).__name__ == "TufiraxConfig"
    c2 = dict(c)
    c2["architectures"] = [c2.pop("architecture")]
    assert config_from_dict(c2) == config_from_dict(c)


# ---------------------------------------------------------------------------------------- the plain mechanisms
def test_plain_sink_and_cap_limits():
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(9, 4, 8, generator=g, dtype=torch.float64), torch.randn(9, 2, 8, generator=g, dtype=torch.float64)
    v = torch.randn(9, 2, 8, generator=g, dtype=torch.float64)
    # no sink in effect and a cap far away: ordinary causal softmax attention
    o = P.sink_softmax_attention(q, k, v, 0.3, 1e9, torch.full((4,), -1e9, dtype=torch.float64))
    for h in range(4):
        s = torch.einsum("td,sd->ts", q[:, h], k[:, h // 2]) * 0.3
        s = s.masked_fill(torch.triu(torch.ones(9, 9, dtype=torch.bool), 1), float("-inf"))
        assert torch.allclose(o[:, h], torch.softmax(s, -1) @ v[:, h // 2], atol=1e-12)
    # a huge sink takes all the weight: the output vanishes; the first token without sink returns its own value
    o = P.sink_softmax_attention(q, k, v, 0.3, 5.0, torch.full((4,), 60.0, dtype=torch.float64))
    assert float(o.abs().max()) < 1e-15
    o = P.sink_softmax_attention(q, k, v, 0.3, 5.0, torch.full((4,), -1e9, dtype=torch.float64))
    assert torch.allclose(o[0, 3], v[0, 1])
    # the cap bounds every score: with cap c all weights of a row lie within e^(2c) of one another
    o_small = P.sink_softmax_attention(q * 100, k, v, 1.0, 1e-3, torch.full((4,), -1e9, dtype=torch.float64))
    assert torch.allclose(o_small[8, 0], v[:, 0].mean(0), atol=2e-3)


def test_plain_scan_is_the_recurrence_and_conv_is_causal():
    g = torch.Generator().manual_seed(1)
    T, H, Pd, N, G = 7, 4, 3, 5, 2
    x, B, C = (torch.randn(T, H, Pd, generator=g, dtype=torch.float64), torch.randn(T, G, N, generator=g, dtype=torch.float64),
               torch.randn(T, G, N, generator=g, dtype=torch.float64))
    dt = torch.rand(T, H, generator=g, dtype=torch.float64)
    a_log, D = torch.randn(H, generator=g, dtype=torch.float64), torch.randn(H, generator=g, dtype=torch.float64)
    y = P.selective_scan(x, B, C, dt, a_log, D, G)
    # closed form for the last token of head 3 (group 1): sum_s prod_{r>s} decay_r * dt_s (B_s . C_T) x_s + D x_T
    h, grp = 3, 1
    want = D[h] * x[-1, h]
    for s in range(T):
        decay = torch.exp(-torch.exp(a_log[h]) * dt[s + 1:, h].sum())
        want = want + decay * dt[s, h] * (B[s, grp] @ C[-1, grp]) * x[s, h]
    assert torch.allclose(y[-1, h], want, atol=1e-12)
    u = torch.randn(6, 2, generator=g, dtype=torch.float64)
    taps, bias = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64), torch.tensor([0.5, -0.5], dtype=torch.float64)
    out = P.causal_conv(u, taps, bias)
    assert torch.allclose(out[0], torch.stack([100 * u[0, 0] + 0.5, u[0, 1] - 0.5]))           # zeros before the start
    assert torch.allclose(out[3, 0], u[1, 0] + 10 * u[2, 0] + 100 * u[3, 0] + 0.5)              # last column: the current token


# ---------------------------------------------------------------------------------------- replay through the engine
LENGTHS = (41, 70, 23, 88, 1, 37)
SCHEDULES = {"whole": TT.schedule_whole, "bulk_tail": TT.schedule_bulk_tail, "portions": TT.schedule_portions,
             "mixed": TT.schedule_mixed}
_cache = {}


def _reference(which):
    if which not in _cache:
        folder = X.write_folder({"a": X.small_a, "b": X.small_b}[which](), seed=5, edit=X.lively)
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
        assert max(len(s["entries"]) for s in trace.steps) == 4 and trace.preemptions == 1     # a slot is freed and used again
    engine = trace_mod.build_engine(folder, "float32", trace.max_tokens, block_size=8, device="cpu")
    assert len(engine.cache._state) == sum(1 for l in X.read_folder(folder)[0]["layers"] if l["type"] == "mamba2")
    echo = io.StringIO()
    n = trace_mod.replay(engine, io.StringIO(trace.lines()), str(tmp_path), echo)
    assert n == len(trace.steps)
    got = TT.read_logits(str(tmp_path), trace, vocab)
    assert TT.compare(got, ref, 2e-5, f"{which}/{schedule}") < 2e-5
    engine.cache.check()
    assert not engine.cache.requests and engine.cache.slots.num_free == 4


@pytest.mark.parametrize("kind", ["mamba2", "attention"])
def test_models_of_one_kind_of_layer(emulated, kind):
    """Only state (no page group at all) or only pages (no state): the engine asks for nothing it does not need."""
    from rvllm_b200.engine.step import StepEntry
    layer = X.mamba2(ff=40) if kind == "mamba2" else X.attention(heads=2, kv_heads=1, dim=16, rot_dims=8)
    # (the borrowing layer comes FIRST in the mamba2 model: a layer may name a later one)
    layers = [X.shared(layer, 1), layer] if kind == "mamba2" else [layer, X.shared(layer, 0)]
    folder = X.write_folder(X.config(layers, width=48, vocab=97), seed=2, edit=X.lively)
    assert set(n.split(".")[0] for n in X.read_folder(folder)[1] if n.startswith("l")) == ({"l1"} if kind == "mamba2" else {"l0"})
    toks = random_requests(97, (29,), seed=1)["r0"]
    want = X.plain_logits(folder, {"x": toks})["x"]
    engine = trace_mod.build_engine(folder, "float32", 64, block_size=8, device="cpu")
    assert (len(engine.cache.groups), len(engine.cache._state)) == ((0, 2) if kind == "mamba2" else (1, 0))
    got = [engine.runner.step([StepEntry("x", toks[:11], list(range(11)))]), engine.runner.step([StepEntry("x", toks[11:28], list(range(17)))]),
           engine.runner.step([StepEntry("x", toks[28:], [0])])]
    got = torch.cat(got).double()
    assert float((got - want).abs().max() / want.abs().max()) < 2e-5
    engine.runner.finish("x")
    engine.cache.check()


def test_state_slot_is_cleared_for_its_next_request(emulated):
    """Two requests, one after the other, in an engine with ONE slot: the second starts from a zero state."""
    folder, vocab, reqs, ref = _reference("a")
    engine = trace_mod.build_engine(folder, "float32", 128, block_size=8, device="cpu", max_live=1)
    from rvllm_b200.engine.step import StepEntry
    for rid in ("r0", "r2"):
        toks = reqs[rid]
        logits = engine.runner.step([StepEntry(rid, toks, [len(toks) - 1])])
        want = ref[rid][-1]
        assert float((logits[0].double() - want).abs().max() / want.abs().max()) < 2e-5, rid
        assert any(float(t.abs().max()) > 0 for t in engine.cache._state.values())
        engine.runner.finish(rid)


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
    import json
    import os
    import subprocess
    import sys
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
    assert info["architecture"] == "Tufirax" and info["config"]["layers"][2]["weights_of"] == 1
    # two mamba2 layers of (6 heads x 24 x 20 + 2 x 264) floats, one of (4 x 40 x 33 + 4 x 212)
    assert info["state_bytes_per_request"] == 4 * (2 * (6 * 24 * 20 + 2 * 264) + (4 * 40 * 33 + 4 * 212))
    assert info["kv_bytes_per_token_bf16"] == 2 * (2 * 2 * 32 * 2)            # two attention layers: k and v of 2 heads of 32
    cfg, w = X.read_folder(str(out))
    assert P.forward(cfg, w, [1, 2, 3]).shape == (3, 211)
