"""The kernels and the whole path of the Tufirax design on the GPU, against the plain implementation
(plain_tufirax.py): every mechanism alone, then trace replay under the four schedules in both number
formats, generation through the entry point and its scheduler, and long decoding."""
import io

import numpy as np
import pytest
import torch

import plain_tufirax as P
import trace_tools as TT
import tufirax_tools as X
from gpu_tools import paged_setup, rel_err
from model_tools import random_requests

pytestmark = pytest.mark.gpu
F64 = torch.float64
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {torch.float32: 2e-5, torch.bfloat16: 1.6e-2}


@pytest.fixture(scope="module")
def K():
    from rvllm_b200.kernels import get_library
    return get_library("cuda:0")


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64) * scale


# ---------------------------------------------------------------------------------------- row kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [72, 320, 4096 + 24])
def test_residual_rmsnorm(K, dtype, cols):
    y, r, g = rnd(5, cols, seed=1, scale=3.0), rnd(5, cols, seed=2), rnd(cols, seed=3) + 1.0
    want = r + P.rms(y.float().double(), 1e-5) * g.to(dtype).double()
    res = r.float().cuda()
    out, rounded = K.residual_rmsnorm(y.float().cuda(), g.to(dtype).cuda(), 1e-5, res, dtype)
    assert out is res and rel_err(out, want) < 2e-6            # the stream is updated in place
    assert rounded.dtype == dtype and rel_err(rounded, want) < (2e-6 if dtype == torch.float32 else 5e-3)
    # without a stream: a plain norm of a float32 row into the activations' type
    n = K.rmsnorm(y.float().cuda(), g.to(dtype).cuda(), 1e-5, out_dtype=dtype)
    assert n.dtype == dtype and rel_err(n, P.rms(y.float().double(), 1e-5) * g.to(dtype).double()) < TOL[dtype] / 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gelu_gated_product(K, dtype):
    gu = rnd(7, 2 * 93, seed=4, scale=2.5)
    out = K.act_mul(gu.float().cuda(), "gelu_tanh", dtype)
    want = P.gelu_tanh(gu[:, :93].float().double()) * gu[:, 93:].float().double()
    assert out.dtype == dtype and rel_err(out, want) < TOL[dtype] / 2
    x, w = rnd(33, 64, seed=5).to(dtype), rnd(2 * 48, 64, seed=6, scale=0.2).to(dtype)
    got = K.gate_up_act(x.cuda(), w.cuda(), "gelu_tanh")
    h = x.double() @ w.double().t()
    assert rel_err(got, P.gelu_tanh(h[:, :48]) * h[:, 48:]) < TOL[dtype]


@pytest.mark.parametrize("rows", [1, 8, 40, 64, 130, 300, 1024])
def test_gelu_in_the_gated_gemm_epilogues(K, rows):
    """bfloat16 rows through the dispatch a model takes: the weight-streaming GEMM for few rows, the prefill GEMM for many
    (both apply the activation to their float accumulators), the product and the activation kernel in between."""
    x, w = rnd(rows, 256, seed=90).to(torch.bfloat16), rnd(2 * 384, 256, seed=91, scale=0.15).to(torch.bfloat16)
    h = x.double() @ w.double().t()
    want = P.gelu_tanh(h[:, :384]) * h[:, 384:]
    got = K.gate_up_act(x.cuda(), w.cuda(), "gelu_tanh")
    assert got.dtype == torch.bfloat16 and rel_err(got, want) < 6e-3
    silu = K.gate_up_act(x.cuda(), w.cuda(), "silu")
    assert rel_err(silu, P.silu(h[:, :384]) * h[:, 384:]) < 6e-3 and rel_err(silu, want) > 2e-2      # the two differ
    K.raise_on_abort()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(6, 2, 32, 16), (8, 2, 64, 64), (3, 3, 24, 2), (4, 1, 128, 96)])
def test_qk_norm_rotation_cache_write(K, dtype, nh, nkv, hd, rot):
    T, page, n_pages, eps = 11, 8, 5, 1e-5
    proj = rnd(T, (nh + nkv) * hd + nh, seed=7, scale=2.0).float()
    wq, wk = (rnd(nh * hd, seed=8) + 1.0).to(dtype), (rnd(nkv * hd, seed=9) + 1.0).to(dtype)
    pos = torch.tensor([3, 4, 5, 0, 1, 2, 3, 100, 101, 7, 8], dtype=torch.int32)
    half = rot // 2
    freq = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(half)], dtype=F64)
    ang = torch.arange(128, dtype=F64)[:, None] * freq[None, :]
    slots = torch.tensor([9, 10, 11, 0, 1, 2, 3, 30, 31, -1, 20], dtype=torch.int32)
    cache = torch.zeros((n_pages, 2, nkv, page, hd), dtype=dtype, device="cuda")
    q, gate = K.qk_norm_rope_cache_write(proj.cuda(), wq.cuda(), wk.cuda(), eps, pos.cuda(), torch.cos(ang).float().cuda(),
                                         torch.sin(ang).float().cuda(), slots.cuda(), cache, nh, nkv, hd, dtype, with_gate=True)
    pd = proj.double()
    qw, kw = nh * hd, nkv * hd
    for t in range(T):
        qn = (P.rms(pd[t:t + 1, :qw], eps) * wq.double()).view(1, nh, hd)
        kn = (P.rms(pd[t:t + 1, qw:qw + kw], eps) * wk.double()).view(1, nkv, hd)
        qr = P.rotate_leading(qn, [int(pos[t])], rot, 50.0)
        kr = P.rotate_leading(kn, [int(pos[t])], rot, 50.0)
        assert rel_err(q[t], qr.reshape(-1)) < TOL[dtype] / 2, t
        s = int(slots[t])
        if s >= 0:
            assert rel_err(cache[s // page, 0, :, s % page], kr[0]) < TOL[dtype] / 2, t
            assert rel_err(cache[s // page, 1, :, s % page], pd[t, qw:qw + kw].view(nkv, hd)) < TOL[dtype] / 2, t   # the value: k as projected
    assert rel_err(gate, torch.sigmoid(pd[:, qw + kw:])) < 2e-6
    untouched = [s for s in range(n_pages * page) if s not in set(slots.tolist())]
    assert all(float(cache[s // page, :, :, s % page].abs().max()) == 0 for s in untouched)


# ---------------------------------------------------------------------------------------- attention
def _attention_case(nh, nkv, hd, ctxs, q_lens, page, dtype, seed, far=None, sink_value=None):
    """Random q, k, v of whole sequences; `far` = (sequence, key position): that key is made to dominate the last
    query of the sequence; returns the paged cache, the metadata, q of the step's tokens, sinks, gate and the
    plain result for the step's tokens."""
    B = len(ctxs)
    qs = [rnd(c, nh, hd, seed=seed + 10 * b) for b, c in enumerate(ctxs)]
    ks = [rnd(c, nkv, hd, seed=seed + 10 * b + 1) for b, c in enumerate(ctxs)]
    vs = [rnd(c, nkv, hd, seed=seed + 10 * b + 2) for b, c in enumerate(ctxs)]
    if far is not None:
        b, j = far
        ks[b][j] = qs[b][-1].view(nkv, nh // nkv, hd)[:, 0] * 3.0          # aligned with the last query's first head of each group
        vs[b][j] = 5.0
    qs = [q.to(dtype).double() for q in qs]
    ks = [k.to(dtype).double() for k in ks]
    vs = [v.to(dtype).double() for v in vs]
    sinks = rnd(nh, seed=seed + 5, scale=1.5).float()
    if sink_value is not None:
        sinks[1] = sink_value          # (head 1: not one of the heads the far key is aligned with)
    T = sum(q_lens)
    gate = torch.rand(T, nh, generator=torch.Generator().manual_seed(seed + 6)).float()
    cache, meta = paged_setup([k.float() for k in ks], [v.float() for v in vs], q_lens, page, dtype, seed=seed)
    q_step = torch.cat([q[-n:] for q, n in zip(qs, q_lens)]).reshape(T, nh * hd)
    scale, cap = 0.17, 9.0
    want = torch.cat([P.sink_softmax_attention(q, k, v, scale, cap, sinks.double())[-n:]
                      for q, k, v, n in zip(qs, ks, vs, q_lens)]) * gate.double()[:, :, None]
    return cache, meta, q_step.to(dtype).cuda(), sinks.cuda(), gate.cuda(), want.reshape(T, nh * hd), scale, cap


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_plain_attention_kernel_with_cap_sink_gate(K, dtype):
    cache, meta, q, sinks, gate, want, scale, cap = _attention_case(6, 2, 24, [37, 5, 150], [9, 5, 1], 8, dtype, 3, far=(2, 1))
    out = K.paged_attention_plain(q, cache, meta, 6, 2, 24, scale, None, cap, sinks, gate)
    assert rel_err(out, want) < (3e-6 if dtype == torch.float32 else 6e-3)
    # each option alone is an option: none of them given equals the kernel's old behaviour
    base = K.paged_attention_plain(q, cache, meta, 6, 2, 24, scale, None)
    none = K.paged_attention_plain(q, cache, meta, 6, 2, 24, scale, None, None, None, None)
    assert torch.equal(base, none)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("page", [16, 8])
def test_tensor_core_attention_paths_with_cap_sink_gate(K, hd, page):
    """Prompt portions (the tcgen05 kernel and the mma.sync kernel) beside decoded tokens (TMA-fed and cp.async
    decode kernels, one and several key splits): a far key that dominates, placed on a page's first slot, and a
    sink that takes nearly all the weight of one head."""
    nh, nkv, dtype = 8, 2, torch.bfloat16
    ctxs, q_lens = [300, 70, 513, 64, 1], [40, 70, 1, 1, 1]
    cache, meta, q, sinks, gate, want, scale, cap = _attention_case(nh, nkv, hd, ctxs, q_lens, page, dtype, 11, far=(2, 2 * page),
                                                                    sink_value=12.0)
    x = dict(softcap=cap, sinks=sinks, gate=gate)
    ref = K.paged_attention_plain(q, cache, meta, nh, nkv, hd, scale, None, cap, sinks, gate)
    assert rel_err(ref, want) < 6e-3
    assert float(want.view(-1, nh, hd)[:, 1].abs().max()) < 0.02 * float(want.abs().max())      # head 1: the sink has the weight
    far_row = sum(q_lens[:2])                                                                   # the decoded token of sequence 2
    assert float(want.view(-1, nh, hd)[far_row, 4].mean() / gate[far_row, 4].cpu()) > 2.5        # the far key (value 5) has most of the weight
    out = K.paged_attention(q, cache, meta, nh, nkv, hd, scale, None, **x)                      # the dispatch a model takes
    assert rel_err(out, want) < 8e-3
    for name, run in {
        "tcgen05 + tma decode": lambda o: (K.attention_tcgen05(q, cache, meta, o, nh, nkv, hd, scale, None, **x),
                                           K.decode_attention(q, cache, meta, o, nh, nkv, hd, scale, None, q_filter=1, **x)),
        "flash + cp.async decode": lambda o: (K.flash_attention(q, cache, meta, o, nh, nkv, hd, scale, None, mode=0, q_filter=2, **x),
                                              K.decode_attention(q, cache, meta, o, nh, nkv, hd, scale, None, q_filter=1, tma=False, **x)),
        # (the merge of key splits writes every row of the step, so here the decoded tokens go first and the prompt
        # portions' kernel overwrites its own rows afterwards; a model's mixed steps do not split)
        "3 splits, then flash": lambda o: (K.decode_attention(q, cache, meta, o, nh, nkv, hd, scale, None, q_filter=1, num_splits=3, **x),
                                           K.flash_attention(q, cache, meta, o, nh, nkv, hd, scale, None, mode=0, q_filter=2, **x)),
        "5 splits by cp.async, then flash": lambda o: (K.decode_attention(q, cache, meta, o, nh, nkv, hd, scale, None, q_filter=1,
                                                                          num_splits=5, tma=False, **x),
                                                       K.flash_attention(q, cache, meta, o, nh, nkv, hd, scale, None, mode=0, q_filter=2, **x)),
    }.items():
        o = torch.full_like(q, float("nan"))
        run(o)
        assert torch.isfinite(o).all(), name
        assert rel_err(o, want) < 8e-3, name
    K.raise_on_abort()


def test_decode_only_step_with_splits(K):
    nh, nkv, hd, page, dtype = 8, 4, 64, 16, torch.bfloat16
    ctxs = [1000, 33, 257, 1]
    cache, meta, q, sinks, gate, want, scale, cap = _attention_case(nh, nkv, hd, ctxs, [1] * 4, page, dtype, 21, far=(0, 15))
    out = K.paged_attention(q, cache, meta, nh, nkv, hd, scale, None, softcap=cap, sinks=sinks, gate=gate)
    assert K.decode_splits(meta, nh, nkv) > 1
    assert rel_err(out, want) < 8e-3
    assert float(want.view(-1, nh, hd)[0, 0].mean() / gate[0, 0].cpu()) > 2.5
    K.raise_on_abort()


# ---------------------------------------------------------------------------------------- state-space mixer
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [1, 3, 4, 6])
def test_causal_conv_through_state(K, dtype, taps):
    C, lens, slots = 50, [23, 2, 9], [2, 0, 3]
    us = [rnd(n, C, seed=30 + i).to(dtype) for i, n in enumerate(lens)]
    w, b = rnd(C, taps, seed=40, scale=0.5).to(dtype), rnd(C, seed=41).to(dtype)
    want = [P.silu(P.causal_conv(u.double(), w.double(), b.double())) for u in us]
    conv_off = 7
    state = torch.zeros((4, conv_off + max(taps - 1, 0) * C + 3), dtype=torch.float32, device="cuda")
    state[1] = 99.0                                   # a slot nobody uses: must stay as it is
    cuts = [[5, 1, 2], [1, 1, 1], [2, 0, 6], [15, 0, 0]]          # portions down to one token, a sequence absent from a step
    at = [0, 0, 0]
    for cut in cuts:
        rows, seqs, cu, sl = [], [], [0], []
        for s, n in enumerate(cut):
            if n == 0:
                continue
            rows.append(us[s][at[s]:at[s] + n])
            seqs += [len(sl)] * n
            cu.append(cu[-1] + n)
            sl.append(slots[s])
        # one padding sequence with slot -1 at the end, as a graph bucket has
        rows.append(torch.zeros(1, C, dtype=dtype)); seqs.append(len(sl)); cu.append(cu[-1] + 1); sl.append(-1)
        proj = torch.cat([torch.zeros(len(seqs), 4, dtype=dtype), torch.cat(rows), torch.zeros(len(seqs), 2, dtype=dtype)], 1).cuda()
        out = K.causal_conv_silu(proj, 4, C, w.cuda(), b.cuda(), torch.tensor(seqs, dtype=torch.int32).cuda(),
                                 torch.tensor(cu, dtype=torch.int32).cuda(), torch.tensor(sl, dtype=torch.int32).cuda(), state, conv_off, dtype)
        r = 0
        for s, n in enumerate(cut):
            if n:
                assert rel_err(out[r:r + n], want[s][at[s]:at[s] + n]) < TOL[dtype] / 2, (cut, s)
                r += n
                at[s] += n
    assert float((state[1] - 99.0).abs().max()) == 0 and float(state[:, :conv_off].abs().max().cpu()) in (0.0, 99.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("columns", [1, 2])
@pytest.mark.parametrize("heads,Pd,N,groups", [(6, 20, 24, 3), (4, 33, 40, 1), (8, 64, 128, 2), (2, 48, 7, 2), (3, 16, 200, 1)])
def test_scan_through_state(K, dtype, heads, Pd, N, groups, columns):
    if columns == 2 and N > 128:
        pytest.skip("states beyond 128 values keep one column per thread")
    lens, slots = [37, 3, 18], [1, 3, 0]
    inner, ch = heads * Pd, heads * Pd + 2 * groups * N
    xbc = [rnd(n, ch, seed=50 + i).to(dtype) for i, n in enumerate(lens)]
    dtr = [rnd(n, heads, seed=60 + i, scale=2.0).float() for i, n in enumerate(lens)]
    dt_bias, a_log, D = rnd(heads, seed=70).float(), (rnd(heads, seed=71) - 1.0).float(), rnd(heads, seed=72).float()
    want = []
    for u, d in zip(xbc, dtr):
        n = u.shape[0]
        ud = u.double()
        want.append(P.selective_scan(ud[:, :inner].reshape(n, heads, Pd), ud[:, inner:inner + groups * N].reshape(n, groups, N),
                                     ud[:, inner + groups * N:].reshape(n, groups, N), P.softplus(d.double() + dt_bias.double()),
                                     a_log.double(), D.double(), groups).reshape(n, inner))
    state = torch.zeros((4, heads * N * Pd + 5), dtype=torch.float32, device="cuda")
    state[2] = -7.0
    cuts = [[16, 1, 2], [1, 1, 1], [3, 1, 15], [17, 0, 0]]          # 16: exactly one chunk of the kernel; then beyond it
    at = [0, 0, 0]
    for cut in cuts:
        rows, drows, cu, sl = [], [], [0], []
        for s, n in enumerate(cut):
            if n:
                rows.append(xbc[s][at[s]:at[s] + n]); drows.append(dtr[s][at[s]:at[s] + n]); cu.append(cu[-1] + n); sl.append(slots[s])
        rows.append(torch.ones(1, ch, dtype=dtype)); drows.append(torch.zeros(1, heads)); cu.append(cu[-1] + 1); sl.append(-1)
        proj = torch.cat([torch.zeros(cu[-1], 3), torch.cat(drows)], 1).cuda()
        y = K.ssm_scan(torch.cat(rows).cuda(), proj, 3, dt_bias.cuda(), a_log.cuda(), D.cuda(), torch.tensor(cu, dtype=torch.int32).cuda(),
                       torch.tensor(sl, dtype=torch.int32).cuda(), state, heads, Pd, N, groups, columns=columns)
        assert y.dtype == torch.float32 and float(y[-1].abs().max()) == 0           # the padding row
        r = 0
        for s, n in enumerate(cut):
            if n:
                assert rel_err(y[r:r + n], want[s][at[s]:at[s] + n]) < 1e-5, (cut, s)
                r += n
                at[s] += n
    assert float((state[2] + 7.0).abs().max()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,Pd,N,groups,seg", [(6, 20, 24, 3, 16), (4, 33, 40, 1, 32), (8, 64, 128, 2, 48), (2, 16, 256, 1, 16)])
def test_scan_in_segments(K, dtype, heads, Pd, N, groups, seg):
    """Long portions cut into segments that are scanned side by side and joined: the same outputs and the same final
    state as the plain recurrence, continued from a state that an earlier step left, beside a short sequence (one
    segment), a sequence of exactly two segments and a padding row; slow and fast decays."""
    lens, slots = [5 * seg + 7, 3, 2 * seg, 1], [2, 0, 3, -1]
    first = [9, 2, 0, 0]                                   # tokens that an earlier, unsegmented step brings
    inner, ch = heads * Pd, heads * Pd + 2 * groups * N
    xbc = [rnd(f + n, ch, seed=150 + i).to(dtype) for i, (f, n) in enumerate(zip(first, lens))]
    dtr = [rnd(f + n, heads, seed=160 + i, scale=2.0).float() for i, (f, n) in enumerate(zip(first, lens))]
    dt_bias, D = rnd(heads, seed=170).float(), rnd(heads, seed=172).float()
    a_log = torch.linspace(-5.0, 1.0, heads)
    want = []
    for u, d in zip(xbc, dtr):
        n, ud = u.shape[0], u.double()
        want.append(P.selective_scan(ud[:, :inner].reshape(n, heads, Pd), ud[:, inner:inner + groups * N].reshape(n, groups, N),
                                     ud[:, inner + groups * N:].reshape(n, groups, N), P.softplus(d.double() + dt_bias.double()),
                                     a_log.double(), D.double(), groups).reshape(n, inner))
    state = torch.zeros((4, heads * N * Pd + 2), dtype=torch.float32, device="cuda")
    state[1] = 3.0
    ref_state = state.clone()
    for use_segments, st in ((True, state), (False, ref_state)):
        for step, counts in enumerate((first, lens)):
            rows, drows, cu, sl, at = [], [], [0], [], []
            for s, n in enumerate(counts):
                if n:
                    a = 0 if step == 0 else first[s]
                    rows.append(xbc[s][a:a + n]); drows.append(dtr[s][a:a + n]); cu.append(cu[-1] + n); sl.append(slots[s]); at.append((s, a, n))
            proj = torch.cat(drows).cuda()
            y = K.ssm_scan(torch.cat(rows).cuda(), proj, 0, dt_bias.cuda(), a_log.cuda(), D.cuda(), torch.tensor(cu, dtype=torch.int32).cuda(),
                           torch.tensor(sl, dtype=torch.int32).cuda(), st, heads, Pd, N, groups,
                           max_q_len=max(counts) if use_segments else None, segment_tokens=seg)
            r = 0
            for s, a, n in at:
                if slots[s] >= 0:
                    assert rel_err(y[r:r + n], want[s][a:a + n]) < 2e-5, (use_segments, step, s)
                else:
                    assert float(y[r:r + n].abs().max()) == 0
                r += n
    assert rel_err(state[:, :heads * N * Pd], ref_state[:, :heads * N * Pd]) < 2e-5 and float((state[1] - 3.0).abs().max()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,parts", [(120, 4), (132, 1), (2048, 2)])
def test_gated_group_norm(K, dtype, width, parts):
    y, z, g = rnd(6, width, seed=80, scale=2.0).float(), rnd(6, width + 9, seed=81).float(), (rnd(width, seed=82) + 1).to(dtype)
    out = K.gated_group_rmsnorm(y.cuda(), z.cuda(), g.cuda(), 1e-5, parts, dtype)
    want = P.grouped_rms(y.double() * P.silu(z[:, :width].double()), parts, 1e-5) * g.double()
    assert out.dtype == dtype and rel_err(out, want) < TOL[dtype] / 2


# ---------------------------------------------------------------------------------------- the whole path
LENGTHS = {"a": (45, 170, 33, 81, 1, 138), "b": (90, 37, 700, 64, 151, 2)}      # 700: beyond two segments of the scan
SCHEDULES = {"whole": TT.schedule_whole, "bulk_tail": TT.schedule_bulk_tail, "portions": TT.schedule_portions,
             "mixed": TT.schedule_mixed}
_cache = {}


def _reference(which):
    if which not in _cache:
        from rvllm_b200 import load_config
        folder = X.write_folder({"a": X.small_a, "b": X.small_b}[which](), seed=5, edit=X.lively)
        vocab = load_config(folder).vocab_size
        reqs = random_requests(vocab, LENGTHS[which], seed=4)
        _cache[which] = (folder, vocab, reqs, X.plain_logits(folder, reqs), X.plain_logits(folder, reqs, rounded=True))
    return _cache[which][:4]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", list(SCHEDULES))
@pytest.mark.parametrize("which", ["a", "b"])
def test_replay_matches_plain(tmp_path, which, schedule, dtype):
    from rvllm_b200.engine import trace as trace_mod
    folder, vocab, reqs, ref = _reference(which)
    trace = SCHEDULES[schedule](reqs)
    block = 8 if which == "a" else 16
    if schedule == "whole":                      # once per configuration as a user runs it: a process of its own
        TT.run_trace_tool(folder, dtype, trace, str(tmp_path), block)
    else:
        engine = trace_mod.build_engine(folder, dtype, trace.max_tokens, block, graphs=schedule == "bulk_tail")
        trace_mod.replay(engine, io.StringIO(trace.lines()), str(tmp_path), io.StringIO())
        engine.cache.check()
        assert not engine.cache.requests
    got = TT.read_logits(str(tmp_path), trace, vocab)
    what = f"{which}/{schedule}/{dtype}"
    if dtype == "float32":
        TT.compare(got, ref, 1e-4, what)
    else:
        # against what storing activations in bfloat16 costs by itself on the same requests (no position beyond
        # 1.5 x its worst, the median within 1.25 x its median), and no position beyond a loose plain bound either
        TT.compare_bfloat16(got, ref, _cache[which][4], what)
        TT.compare(got, ref, 0.2, what)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_odd_shapes_whole_and_mixed(tmp_path, dtype):
    """Sizes off every fast path (see tufirax_tools.odd_shapes), whole prompts and the mixed schedule."""
    from rvllm_b200 import load_config
    from rvllm_b200.engine import trace as trace_mod
    folder = X.write_folder(X.odd_shapes(), seed=8, edit=X.lively)
    vocab = load_config(folder).vocab_size
    reqs = random_requests(vocab, (70, 150, 9, 33, 130), seed=6)
    ref = X.plain_logits(folder, reqs)
    rounded = X.plain_logits(folder, reqs, rounded=True) if dtype == "bfloat16" else None
    for name, make in (("whole", TT.schedule_whole), ("mixed", TT.schedule_mixed)):
        out = tmp_path / name
        trace = make(reqs)
        engine = trace_mod.build_engine(folder, dtype, trace.max_tokens, 16)
        trace_mod.replay(engine, io.StringIO(trace.lines()), str(out), io.StringIO())
        engine.cache.check()
        got = TT.read_logits(str(out), trace, vocab)
        if dtype == "float32":
            TT.compare(got, ref, 1e-4, f"odd/{name}")
        else:
            TT.compare_bfloat16(got, ref, rounded, f"odd/{name}")
        del engine


def test_generation_through_the_entry_point():
    """Greedy tokens through LLM.generate and its scheduler (decode steps from CUDA graphs, prompts in portions,
    more requests than slots): float32 equals the plain implementation token for token; bfloat16 may differ only
    where the plain logits' two best lie closer together than its rounding."""
    from rvllm_b200 import LLM, SamplingParams
    folder, vocab, reqs, ref = _reference("b")
    cfg, w = X.read_folder(folder)
    prompts = [reqs["r1"], reqs["r5"], reqs["r3"], reqs["r0"][:50], reqs["r4"][:100]]
    for dtype in ("float32", "bfloat16"):
        llm = LLM(folder, dtype=dtype, block_size=16, num_blocks=40, max_model_len=256, max_num_seqs=3,
                  max_num_batched_tokens=48, max_prefill_chunk=33)
        assert llm.engine.model.graph_safe
        outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True))
        assert llm.engine.runner._graphs, "decode steps were not replayed from graphs"
        for p, o in zip(prompts, outs):
            got = o.outputs[0].token_ids
            if dtype == "float32":
                assert got == P.greedy(cfg, w, p, 20)
            else:
                ids = list(p)
                for tok in got:
                    logits = P.forward(cfg, w, ids)[-1]
                    top = torch.topk(logits, 2).values
                    assert float(top[0] - top[1]) / float(logits.abs().max()) <= 6e-2 or tok == int(logits.argmax())
                    ids.append(tok)
        assert not llm.engine.cache.requests
        del llm


def test_long_decoding_keeps_state_and_cache():
    """A short prompt, then 400 tokens one by one (graphs): the last logits equal those of the whole sequence."""
    from rvllm_b200.engine import trace as trace_mod
    from rvllm_b200.engine.step import StepEntry
    folder, vocab, reqs, ref = _reference("a")
    toks = random_requests(vocab, (420,), seed=9)["r0"]
    want = X.plain_logits(folder, {"x": toks})["x"]
    engine = trace_mod.build_engine(folder, "float32", 512, 8, graphs=True)
    engine.runner.step([StepEntry("x", toks[:20], [])])
    for i in range(20, 420):
        logits = engine.runner.step([StepEntry("x", toks[i:i + 1], [0])])
        if i % 57 == 0 or i == 419:
            assert rel_err(logits[0], want[i]) < 1e-4, i
