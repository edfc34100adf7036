"""The kernels and the whole path of the Vipelix design on the GPU, against the plain implementation
(plain_vipelix.py): every mechanism alone, then trace replay under the four schedules in both number formats,
generation through the entry point and its scheduler, and long decoding."""
import io

import pytest
import torch

import plain_vipelix as P
import trace_tools as TT
import vipelix_tools as X
from gpu_tools import rel_err
from model_tools import random_requests

pytestmark = pytest.mark.gpu
F64 = torch.float64
TOL = {torch.float32: 2e-5, torch.bfloat16: 1.6e-2}


@pytest.fixture(scope="module")
def K():
    from rvllm_b200.kernels import get_library
    return get_library("cuda:0")


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64) * scale


# ---------------------------------------------------------------------------------------- row kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [44, 352, 4096 + 24])
def test_add_then_norm_for_the_next_sublayer(K, dtype, cols):
    y, r = rnd(6, cols, seed=1, scale=3.0), rnd(6, cols, seed=2)
    g1, g2 = (rnd(cols, seed=3) + 1.0).to(dtype), (rnd(cols, seed=4) + 1.0).to(dtype)
    stream = r + P.rms_norm(y.float().double(), g1.double(), 1e-5)
    res = r.float().cuda()
    out, nxt = K.residual_rmsnorm(y.float().cuda(), g1.cuda(), 1e-5, res, dtype, next_norm=(g2.cuda(), 1e-6))
    assert out is res and rel_err(out, stream) < 2e-6
    assert nxt.dtype == dtype and rel_err(nxt, P.rms_norm(stream, g2.double(), 1e-6)) < (4e-6 if dtype == torch.float32 else 5e-3)
    # without a following norm nothing but the stream comes back
    out2, none = K.residual_rmsnorm(y.float().cuda(), g1.cuda(), 1e-5, r.float().cuda(), None)
    assert none is None and rel_err(out2, stream) < 2e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stream_add_polynorm_softcap(K, dtype):
    x, e, table = rnd(5, 76, seed=5), rnd(5, 76, seed=6), rnd(3, 76, seed=7).to(dtype)
    got = K.stream_add(x.float().cuda(), e.float().cuda(), table.cuda(), 2)
    assert rel_err(got, x.float().double() + e.float().double() + table[2].double()) < 1e-6
    got = K.stream_add(x.float().cuda(), None, table.cuda(), 0)
    assert rel_err(got, x.float().double() + table[0].double()) < 1e-6
    z, coef = rnd(7, 93, seed=8, scale=2.0).float(), torch.tensor([0.7, -1.2, 0.4, 0.3])
    out = K.polynorm(z.cuda(), coef.cuda(), 1e-5, dtype)
    assert out.dtype == dtype and rel_err(out, P.polynorm(z.double(), coef.double(), 1e-5)) < TOL[dtype] / 2
    only_cube = K.polynorm(z.cuda(), torch.tensor([0.0, 0.0, 1.0, 0.0]).cuda(), 1e-5, torch.float32)
    assert rel_err(only_cube, P.unit_rms(z.double() ** 3, 1e-5)) < 1e-5
    logits = rnd(4, 131, seed=9, scale=20.0).float()
    assert rel_err(K.softcap(logits.clone().cuda(), 7.5), 7.5 * torch.tanh(logits.double() / 7.5)) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,Rd,dims,R", [(3, 24, 16, 16, 40), (4, 8, 12, 8, 20), (1, 9, 6, 6, 35), (6, 48, 32, 32, 112), (5, 10, 2, 2, 13)])
def test_latent_prepare(K, dtype, H, D, Rd, dims, R):
    T, page, n_pages, eps, base = 11, 8, 5, 1e-5, 300.0
    row = R + Rd
    proj = rnd(T, H * (D + Rd) + row + H, seed=10, scale=2.0).float()
    gamma = (rnd(R, seed=11) + 1.0).to(dtype)
    pos = torch.tensor([3, 4, 5, 0, 1, 2, 3, 100, 101, 7, 8], dtype=torch.int32)
    inv = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    ang = torch.arange(128, dtype=F64)[:, None] * inv[None, :]
    slots = torch.tensor([0, 1, 2, 16, 17, 18, 19, 30, 31, -1, 39], dtype=torch.int32)
    cache = torch.full((n_pages, 1, 1, page, row), 7.0, dtype=dtype).cuda()
    q_plain, q_row, gate = K.latent_prepare(proj.cuda(), gamma.cuda(), eps, pos.cuda(), torch.cos(ang).float().cuda(),
                                            torch.sin(ang).float().cuda(), slots.cuda(), cache, H, D, Rd, R, dtype)
    x = proj.double()
    q = x[:, :H * (D + Rd)].view(T, H, D + Rd)
    tol = 1e-6 if dtype == torch.float32 else 5e-3
    assert q_plain.shape == (T, H, D) and rel_err(q_plain, q[:, :, :D]) < tol
    assert rel_err(q_row[:, :, R:], P.turn_pairs(q[:, :, D:], pos.long(), dims, base)) < tol
    want_row = torch.cat([P.rms_norm(x[:, H * (D + Rd):H * (D + Rd) + R], gamma.double(), eps),
                          P.turn_pairs(x[:, H * (D + Rd) + R:H * (D + Rd) + row], pos.long(), dims, base)], dim=1)
    flat = cache.view(n_pages * page, row)
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            assert rel_err(flat[s], want_row[t]) < tol, t
    untouched = [s for s in range(n_pages * page) if s not in slots.tolist()]
    assert bool((flat[untouched] == 7.0).all())                     # slot -1 writes nothing, nothing else is touched
    assert rel_err(gate, torch.sigmoid(x[:, -H:])) < 1e-6 and gate.dtype == torch.float32


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,N,K_", [(1, 3, 40, 24), (70, 4, 128, 64), (130, 2, 20, 9), (33, 5, 13, 10), (257, 4, 80, 128),
                                       (300, 9, 192, 72), (1030, 3, 264, 200), (128, 2, 16, 8)])
def test_per_head_products(K, dtype, T, H, N, K_):
    """Contiguous and sliced operands.  bfloat16 with aligned rows: the tcgen05 GEMM batched over the heads from 128 rows on
    (K that is no multiple of its k block, more columns than a tile, an odd number of row blocks per head), mma.sync below;
    everything else the plain kernel."""
    x, w = rnd(T, H, K_, seed=12).to(dtype), rnd(H, N, K_, seed=13, scale=0.3).to(dtype)
    want = torch.einsum("thk,hnk->thn", x.double(), w.double())
    got = K.head_linear(x.cuda(), w.cuda(), None, out_dtype=torch.float32)
    assert got.shape == (T, H, N) and rel_err(got, want) < 1e-5
    wide_in = torch.zeros(T, H, K_ + 8, dtype=dtype).cuda()
    wide_in[:, :, :K_] = x.cuda()
    wide_out = torch.full((T, H, N + 16), 5.0, dtype=dtype).cuda()
    K.head_linear(wide_in[:, :, :K_], w.cuda(), wide_out[:, :, :N])
    assert rel_err(wide_out[:, :, :N], want) < TOL[dtype] / 2 and bool((wide_out[:, :, N:] == 5.0).all())
    K.raise_on_abort()


# ---------------------------------------------------------------------------------------- attention over cached rows
def latent_pages(rows_per_seq, q_lens, page, dtype, seed=0, spare=3):
    """Scatter whole-sequence rows [ctx, row] into shuffled pages of a one-plane cache; the last q_len tokens of a
    sequence are the step's.  Slots nobody wrote hold finite junk, as a page that is used again would."""
    from rvllm_b200.kernels import AttentionMeta
    B, row = len(rows_per_seq), rows_per_seq[0].shape[1]
    ctx = [r.shape[0] for r in rows_per_seq]
    blocks = [(c + page - 1) // page for c in ctx]
    n_pages = sum(blocks) + spare
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    cache = torch.full((n_pages, 1, 1, page, row), 3.0, dtype=torch.float32)
    table = torch.full((B, max(blocks)), -1, dtype=torch.int32)
    nxt = 0
    for b in range(B):
        for blk in range(blocks[b]):
            table[b, blk] = perm[nxt]
            lo, hi = blk * page, min(ctx[b], (blk + 1) * page)
            cache[perm[nxt], 0, 0, :hi - lo] = rows_per_seq[b][lo:hi]
            nxt += 1
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(q_lens)])
    meta = AttentionMeta(table.cuda(), torch.tensor(cu, dtype=torch.int32).cuda(), torch.tensor(ctx, dtype=torch.int32).cuda(),
                         seq.cuda(), None, B, max(q_lens), max(ctx), page, sum(1 for n in q_lens if n == 1))
    return cache.cuda().to(dtype), meta


def plain_latent(q, rows_per_seq, q_lens, vd, scale, gate):
    """q [T, H, row] float64; every token attends to the rows at positions up to its own."""
    out, t = [], 0
    for rows, n in zip(rows_per_seq, q_lens):
        ctx = rows.shape[0]
        for i in range(n):
            p = torch.softmax(q[t] @ rows[:ctx - n + i + 1].T * scale, -1)
            out.append((p @ rows[:ctx - n + i + 1, :vd]) * gate[t][:, None])
            t += 1
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,row,vd,page", [(6, 144, 112, 16), (3, 56, 40, 8), (2, 128, 96, 16), (5, 64, 48, 32), (1, 300, 260, 16),
                                           (8, 192, 128, 16), (32, 256, 192, 16), (3, 96, 64, 8), (7, 104, 32, 16), (128, 64, 64, 16)])
@pytest.mark.parametrize("q_lens,ctx", [((1, 1, 1), (257, 64, 1)), ((70, 5), (70, 133)), ((1, 40, 1, 2), (100, 300, 17, 2))])
def test_latent_attention_kernels(K, dtype, H, row, vd, page, q_lens, ctx):
    """Decoded tokens alone (key splits), prompt portions behind a prefix, and both in one step; rows of the sizes
    the tensor-core kernels are built for (tcgen05 for portions where the value is a multiple of 32, mma.sync where row and
    value are multiples of 16) and of sizes they are not (the plain kernel, rows beyond 256 elements)."""
    rows = [rnd(c, row, seed=20 + i).to(dtype).double() for i, c in enumerate(ctx)]
    T = sum(q_lens)
    q, gate = rnd(T, H, row, seed=30, scale=1.5).to(dtype), torch.rand(T, H, generator=torch.Generator().manual_seed(1))
    cache, meta = latent_pages(rows, q_lens, page, dtype)
    got = K.latent_attention(q.cuda(), cache, meta, H, row, vd, 0.11, gate=gate.cuda())
    want = plain_latent(q.double(), rows, q_lens, vd, 0.11, gate.double())
    assert got.shape == (T, H, vd) and rel_err(got, want) < (3e-5 if dtype == torch.float32 else 2e-2)
    if dtype == torch.bfloat16 and row <= 256:      # the kernels are the same function
        K.LATENT_TCGEN05 = False
        try:
            flash = K.latent_attention(q.cuda(), cache, meta, H, row, vd, 0.11, gate=gate.cuda())
            K.LATENT_FLASH = False
            slow = K.latent_attention(q.cuda(), cache, meta, H, row, vd, 0.11, gate=gate.cuda())
        finally:
            K.LATENT_FLASH = K.LATENT_TCGEN05 = True
        assert rel_err(got, slow) < 2e-2 and rel_err(flash, slow) < 2e-2
        K.raise_on_abort()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("far", [0, 1, 15, 16, 63, 64, 127, 128, 1023, 1024, 1500])
def test_one_far_key_takes_all_the_weight(K, dtype, far):
    """Among 1,600 rows one answers the query far more strongly than the rest - the first row of the sequence, a page's
    first and last slot, the edges of the kernel's tiles of 64 keys: the result is that row's leading part.  In a
    prompt portion, in a decoded token with the keys cut over CTAs, and in a mixed step."""
    H, row, vd, page, ctx = 4, 96, 64, 16, 1600
    rows = rnd(ctx, row, seed=40).to(dtype).double()
    probe = rows[far] / rows[far].norm() * 30.0                     # q . rows[far] = 30 |rows[far]|; the others stay near zero
    for q_lens, ctxs in (((1,), (ctx,)), ((90,), (ctx,)), ((1, 3), (ctx, 1580))):
        T = sum(q_lens)
        q = rnd(T, H, row, seed=41, scale=0.05).to(dtype)
        q[q_lens[0] - 1, 2] = probe.to(dtype)                       # the last token of the first sequence, head 2
        seqs = [rows[:c] for c in ctxs]
        cache, meta = latent_pages(seqs, q_lens, page, dtype, seed=far)
        got = K.latent_attention(q.cuda(), cache, meta, H, row, vd, 1.0)
        assert rel_err(got[q_lens[0] - 1, 2], rows[far, :vd]) < (1e-4 if dtype == torch.float32 else 1e-2), (q_lens, far)
        ones = torch.ones(T, H, dtype=F64)
        assert rel_err(got, plain_latent(q.double(), seqs, q_lens, vd, 1.0, ones)) < (3e-5 if dtype == torch.float32 else 2e-2)


# ---------------------------------------------------------------------------------------- experts
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,width,ff,E,top,ids", [(1, 48, 24, 5, 2, 37), (9, 44, 9, 4, 4, 37), (70, 384, 88, 12, 2, 37), (300, 64, 40, 3, 1, 37),
                                                   (513, 384, 88, 12, 3, 200), (200, 128, 264, 7, 3, 2), (1100, 256, 128, 40, 4, 1)])
def test_experts_chosen_by_table(K, dtype, T, width, ff, E, top, ids):
    """Few tokens (a kernel that streams the chosen experts' weights) and many (sorted by expert, grouped products on the
    tensor cores, in bfloat16); with two or one token id in play most experts get no row at all and one gets many tiles."""
    g = torch.Generator().manual_seed(3)
    x = rnd(T, width, seed=50).to(dtype)
    gate_up, down = rnd(E, 2 * ff, width, seed=51, scale=0.2).to(dtype), rnd(E, width, ff, seed=52, scale=0.2).to(dtype)
    table = torch.rand(ids, E, generator=g).argsort(1)[:, :top].to(torch.int32)
    tokens = torch.randint(0, ids, (T,), generator=g).to(torch.int32)
    add = rnd(T, width, seed=53).float()
    chosen = K.gather_rows(table.cuda(), tokens.cuda())
    assert chosen.dtype == torch.int32 and torch.equal(chosen.cpu(), table[tokens.long()])
    want = add.double().clone()
    for t in range(T):
        for e in table[int(tokens[t])].tolist():
            gu = gate_up[e].double() @ x[t].double()
            h = gu[:ff] * torch.sigmoid(gu[:ff]) * gu[ff:]
            want[t] += (down[e].double() @ h) / top
    got = K.moe_experts(x.cuda(), chosen, gate_up.cuda(), down.cuda(), 1.0 / top, add=add.cuda(), out_dtype=torch.float32)
    assert got.dtype == torch.float32 and rel_err(got, want) < (2e-5 if dtype == torch.float32 else 1e-2)
    bare = K.moe_experts(x.cuda(), chosen, gate_up.cuda(), down.cuda(), 1.0 / top)
    assert bare.dtype == dtype and rel_err(bare, want - add.double()) < TOL[dtype]
    K.raise_on_abort()


# ---------------------------------------------------------------------------------------- the whole path
LENGTHS = {"a": (45, 170, 33, 81, 1, 138), "b": (90, 37, 300, 64, 151, 2)}
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
        TT.compare_bfloat16(got, ref, _cache[which][4], what)
        TT.compare(got, ref, 0.2, what)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_odd_shapes_whole_and_mixed(tmp_path, dtype):
    """Sizes off every fast path (see vipelix_tools.odd_shapes), whole prompts and the mixed schedule."""
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


def test_long_decoding_keeps_every_pass_apart():
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
