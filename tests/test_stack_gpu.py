"""Layer-stack engine (Kozusun design) against the plain restatement in tests/stack_oracle.py: every mechanism alone,
whole prompts, decoding through the cache, parts of prompts, unequal batches, slot reuse, window / kept-token edges,
other sizes, and greedy generation through the engine's own entry points."""
import math

import pytest
import torch

import stack_oracle as so
from tinygpt_b200 import engine, models, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
# fp32 engines are held to summation-order noise.  bf16 engines round every activation to 8 bits of mantissa; on these
# narrow models that alone moves a logit row by up to 6 % of its spread, so the bf16 runs catch gross faults and the
# fp32 runs (same step function, cache and attention kernel) the fine ones.
TOL = {torch.float32: 3e-4, torch.bfloat16: 9e-2}


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest per-row error: rms of the difference (mean removed) over rms of the wanted row (mean removed)."""
    got, want = got.float().cpu(), want.float().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    c = want - want.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / c.pow(2).mean(-1).sqrt().clamp_min(1e-6)).max())


def make_engine(cfg, w, dtype, max_ctx=160, max_slots=4):
    spec = models.kozusun_from_config(cfg).with_ctx(max_ctx, max_slots)
    return engine.DecodeEngine(spec, models.pack_stack_weights(spec, w, device=DEV, dtype=dtype))


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ------------------------------------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("offset", [0.0, 1.0])
def test_rmsnorm_op(dtype, offset):
    g = torch.Generator().manual_seed(1)
    x, w = torch.randn(7, 100, generator=g) * 3, torch.randn(100, generator=g) * 0.2
    got = ops.stack_rmsnorm(x.to(DEV), w.to(DEV), 1e-5, offset, out_dtype=dtype)
    want = so.rms(x, 1e-5) * (offset + w)
    assert rel_err(got, want) < (1e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 13, 27), (5, 64, 64), (70, 130, 90), (3, 8, 1)])
def test_linear_op_any_shape(dtype, shape):
    M, N, K = shape
    g = torch.Generator().manual_seed(2)
    a, w, b = (torch.randn(M, K, generator=g).to(dtype), torch.randn(N, K, generator=g).to(dtype),
               torch.randn(N, generator=g))
    got = ops.stack_linear(a.to(DEV), w.to(DEV), b.to(DEV))
    want = a.float() @ w.float().T + b
    assert (got.float().cpu() - want).abs().max() < (1e-4 if dtype == torch.float32 else 0.02 * want.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_act_mul_and_rms_add_ops(dtype):
    g = torch.Generator().manual_seed(3)
    proj = (torch.randn(6, 50, generator=g) * 2).to(dtype).to(DEV)
    got = ops.stack_act_mul(proj[:, 3:23], proj[:, 27:47])
    want = so.gelu_tanh(proj[:, 3:23].float().cpu()) * proj[:, 27:47].float().cpu()
    assert (got.float().cpu() - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.03)
    x, y, w = torch.randn(4, 36, generator=g), torch.randn(4, 36, generator=g) * 5, torch.randn(36, generator=g)
    got = ops.stack_rms_add(x.clone().to(DEV), y.to(DEV), w.to(DEV), 1e-5, 0.3)
    assert (got.cpu() - (x + 0.3 * so.rms(y, 1e-5) * w)).abs().max() < 1e-5


def _attention_case(dtype, *, heads, kv_heads, dim, vdim, window, keep_first, n_ctx, query_pos, hot_key, gate=False):
    """One query at position query_pos in slot 1 of a 2-slot cache whose rows 0 … n_ctx-1 are filled; the query and
    key `hot_key` (every head) are scaled so that this one score dominates if — and only if — the key is visible."""
    g = torch.Generator().manual_seed(4)
    nk, nv = kv_heads * dim, kv_heads * vdim
    n_in = heads * dim + nk + nv + heads
    off_k, off_v, off_g = heads * dim, heads * dim + nk, heads * dim + nk + nv
    proj = torch.randn(n_ctx, n_in, generator=g) * 0.3
    u = torch.randn(dim, generator=g)
    u = u / u.norm()
    proj[hot_key, off_k:off_k + nk] = (u * 6).repeat(kv_heads)
    proj[query_pos, :heads * dim] = (u * 6).repeat(heads)
    proj = proj.to(dtype)
    kc = torch.zeros(2, n_ctx + 3, nk, dtype=dtype, device=DEV)
    vc = torch.zeros(2, n_ctx + 3, nv, dtype=dtype, device=DEV)
    slot = torch.ones(n_ctx, dtype=torch.int32, device=DEV)
    pos = torch.arange(n_ctx, dtype=torch.int32, device=DEV)
    kw = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim)
    ops.stack_kv_store(kc, vc, proj.to(DEV), off_k, off_v, slot, pos, **kw)
    assert float(kc[0].abs().max()) == 0.0            # the other slot stays untouched
    q = proj[query_pos:query_pos + 1].to(DEV)
    out = ops.stack_attention(q, 0, off_g, kc, vc, slot[:1], pos[query_pos:query_pos + 1], scale=1.0, window=window,
                              keep_first=keep_first, out_gate=gate, **kw).float().cpu()[0]
    # plain reference, key by key
    p = proj.float()
    want = torch.zeros(heads, vdim)
    for h in range(heads):
        kv = h // (heads // kv_heads)
        js = [j for j in range(n_ctx) if so.sees(query_pos, j, window, keep_first)]
        s = torch.stack([(p[query_pos, h * dim:(h + 1) * dim] * p[j, off_k + kv * dim: off_k + (kv + 1) * dim]).sum()
                         for j in js])
        pr = torch.softmax(s, 0)
        want[h] = sum(pr[n] * p[j, off_v + kv * vdim: off_v + (kv + 1) * vdim] for n, j in enumerate(js))
        if gate:
            want[h] = want[h] * torch.sigmoid(p[query_pos, off_g + h])
    hot_v = p[hot_key, off_v:off_v + vdim]
    return out.view(heads, vdim), want, hot_v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", [
    # (window, keep_first, n_ctx, query, hot key, visible?)
    (16, 4, 300, 299, 284, True),    # last key inside the window
    (16, 4, 300, 299, 283, False),   # first key outside it
    (16, 4, 300, 299, 3, True),      # last kept first token, far away among hundreds
    (16, 4, 300, 299, 4, False),     # first token that is not kept
    (16, 4, 300, 299, 299, True),    # the query's own position
    (16, 4, 12, 11, 0, True),        # window not yet full: everything visible
    (16, 0, 40, 39, 0, False),       # nothing kept
    (1, 2, 40, 39, 38, False),       # window of one token: only itself and the kept ones
    (1, 2, 40, 39, 1, True),
    (33, 40, 100, 70, 39, True),     # kept prefix longer than the window, overlapping it
    (33, 40, 100, 99, 40, False),
    (64, 3, 100, 35, 0, True),       # window longer than the context so far
])
def test_attention_window_edges(dtype, case):
    window, keep, n_ctx, qpos, hot, visible = case
    out, want, hot_v = _attention_case(dtype, heads=4, kv_heads=2, dim=24, vdim=12, window=window, keep_first=keep,
                                       n_ctx=n_ctx, query_pos=qpos, hot_key=hot)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (out - want).abs().max() < tol
    # the crafted score: a visible hot key owns the output of head 0, an invisible one leaves no trace
    near = (out[0] - hot_v).abs().max() < 0.05
    assert bool(near) == visible


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(1, 1, 8, 8), (6, 3, 20, 36), (8, 8, 64, 64), (2, 1, 128, 100), (3, 1, 5, 3)])
def test_attention_head_shapes_and_gate(dtype, sizes):
    heads, kv_heads, dim, vdim = sizes
    out, want, _ = _attention_case(dtype, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, window=9, keep_first=2,
                                   n_ctx=50, query_pos=49, hot_key=45, gate=True)
    assert (out - want).abs().max() < (2e-5 if dtype == torch.float32 else 2e-2)


# ----------------------------------------------------------------------------------------------- whole model paths
CFG_A = dict(layers=[dict(heads=4, kv_heads=2, dim=16, vdim=8, size=6, keep_first=2, ff=48),
                     dict(heads=4, kv_heads=2, dim=16, vdim=8, size=6, keep_first=2, ff=48),
                     dict(heads=2, kv_heads=1, dim=24, vdim=32, size=9, keep_first=0, ff=40)],
             loop=(0, 2, 2))


@pytest.fixture(scope="module")
def model_a():
    cfg = so.make_config(**CFG_A)
    w = so.make_weights(cfg, seed=5)
    toks = tokens(41, cfg["vocab"], 6)
    return cfg, w, toks, so.forward(cfg, w, toks)


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompt_every_position(model_a, dtype):
    cfg, w, toks, want = model_a
    eng = make_engine(cfg, w, dtype)
    got = eng.step([(0, toks, list(range(len(toks))))])
    assert rel_err(got, want) < TOL[dtype]
    # the engine's reference-shaped entry point gives the same rows (bf16 logits)
    eng.reset_cache()
    ids = torch.tensor([toks], dtype=torch.int64, device=DEV)
    lg = eng.forward(ids, all_positions=True)[0]
    assert rel_err(lg, want) < max(TOL[dtype], 2e-2)
    eng.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_then_token_by_token(model_a, dtype):
    cfg, w, toks, want = model_a
    eng = make_engine(cfg, w, dtype)
    n0 = 5
    rows = [eng.step([(2, toks[:n0], list(range(n0)))])]
    for t in range(n0, len(toks)):                      # decoding walks the window (6, 9) over decoded tokens
        rows.append(eng.step([(2, [toks[t]], [0])]))
    assert eng.slot_position(2) == len(toks)
    assert rel_err(torch.cat(rows), want) < TOL[dtype]
    eng.close()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2, 2, 2, 35], [1, 7, 33], [13, 2, 26], [39, 2], [3] * 13 + [2]])
def test_prompt_in_parts(model_a, dtype, cuts):
    cfg, w, toks, want = model_a
    assert sum(cuts) == len(toks)
    eng = make_engine(cfg, w, dtype)
    rows, at = [], 0
    for c in cuts:
        rows.append(eng.step([(0, toks[at:at + c], list(range(c)))]))
        at += c
    assert rel_err(torch.cat(rows), want) < TOL[dtype]
    eng.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batch_equals_each_alone(model_a, dtype):
    cfg, w, _, _ = model_a
    lens = [1, 23, 9, 40]
    seqs = [tokens(n + 6, cfg["vocab"], 10 + i) for i, n in enumerate(lens)]
    wants = [so.forward(cfg, w, s) for s in seqs]
    eng = make_engine(cfg, w, dtype)
    # the prompts together in one step (slots in scrambled order), then six decode steps together
    order = [3, 0, 2, 1]
    got = eng.step([(order[i], seqs[i][:lens[i]], list(range(lens[i]))) for i in range(4)])
    at = 0
    for i, n in enumerate(lens):
        assert rel_err(got[at:at + n], wants[i][:n]) < TOL[dtype], f"prompt {i}"
        at += n
    for t in range(6):
        got = eng.step([(order[i], [seqs[i][lens[i] + t]], [0]) for i in range(4)])
        for i in range(4):
            assert rel_err(got[i:i + 1], wants[i][lens[i] + t: lens[i] + t + 1]) < TOL[dtype], f"decode {t} of {i}"
    eng.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_shorter_requests_leave_and_slots_are_reused(model_a, dtype):
    cfg, w, _, _ = model_a
    eng = make_engine(cfg, w, dtype, max_slots=2)
    pool = eng.slots
    a, b, c = (tokens(n, cfg["vocab"], 20 + n) for n in (30, 12, 17))
    wa, wb, wc = (so.forward(cfg, w, s) for s in (a, b, c))
    sa, sb = pool.acquire("a"), pool.acquire("b")
    eng.step([(sa, a[:10], []), (sb, b[:10], [])])
    for t in range(10, 12):
        eng.step([(sa, [a[t]], []), (sb, [b[t]], [])])
    eng.release(pool.release("b"))                       # b is over; a goes on alone
    with pytest.raises(Exception):
        pool.slot("b")
    sc = pool.acquire("c")                               # c takes b's slot, whose rows still hold b's keys
    assert sc == sb and eng.slot_position(sc) == 0
    got = eng.step([(sa, a[12:14], [0, 1]), (sc, c, list(range(len(c))))])
    assert rel_err(got[:2], wa[12:14]) < TOL[dtype]
    assert rel_err(got[2:], wc) < TOL[dtype]
    got = eng.step([(sa, a[14:], list(range(16)))])
    assert rel_err(got, wa[14:]) < TOL[dtype]
    with pytest.raises(Exception):
        eng.step([(5, [1], [0])])                        # a slot the engine does not have
    eng.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_past_window_and_kept_tokens(dtype):
    cfg = so.make_config(layers=[dict(heads=2, kv_heads=2, dim=8, vdim=8, size=5, keep_first=3, ff=24)] * 2, side_dim=4)
    w = so.make_weights(cfg, seed=7)
    toks = tokens(90, cfg["vocab"], 8)
    want = so.forward(cfg, w, toks)
    eng = make_engine(cfg, w, dtype)
    rows = [eng.step([(1, toks[:2], [0, 1])])]           # the first tokens of a sequence, then 88 single steps
    for t in range(2, 90):
        rows.append(eng.step([(1, [toks[t]], [0])]))
    assert rel_err(torch.cat(rows), want) < TOL[dtype]
    eng.close()


OTHER = {
    "no loop, no side, one layer without ff": dict(
        layers=[dict(heads=2, kv_heads=1, dim=8, vdim=16, size=4, keep_first=1, ff=None),
                dict(heads=3, kv_heads=3, dim=12, vdim=12, size=50, keep_first=0, ff=20)], side_dim=0),
    "loop in the middle, once": dict(
        layers=[dict(heads=2, kv_heads=2, dim=8, vdim=8, size=7, keep_first=2, ff=16)] * 3, loop=(1, 2, 1)),
    "loop over everything, three passes": dict(
        layers=[dict(heads=4, kv_heads=1, dim=8, vdim=4, size=3, keep_first=5, ff=16)], loop=(0, 1, 3)),
    "loop at the end, odd sizes": dict(
        width=52, vocab=77, side_dim=5,
        layers=[dict(heads=3, kv_heads=1, dim=10, vdim=6, size=8, keep_first=1, ff=22),
                dict(heads=5, kv_heads=5, dim=4, vdim=7, size=2, keep_first=0, ff=9)], loop=(1, 2, 2)),
    "multipliers of one": dict(
        embed_scale=1.0, residual_mult=1.0, side_dim=8,
        layers=[dict(heads=1, kv_heads=1, dim=32, vdim=32, size=1, keep_first=1, ff=8, scale=1.0)] * 2),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(OTHER))
def test_other_sizes_and_layer_orders(dtype, name):
    cfg = so.make_config(**OTHER[name])
    w = so.make_weights(cfg, seed=9)
    toks = tokens(26, cfg["vocab"], 11)
    want = so.forward(cfg, w, toks)
    eng = make_engine(cfg, w, dtype)
    got = torch.cat([eng.step([(0, toks[:17], list(range(17)))])] +
                    [eng.step([(0, [toks[t]], [0])]) for t in range(17, 26)])
    assert rel_err(got, want) < TOL[dtype]
    eng.close()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd", [64, 128])
def test_long_prompts_big_heads_and_split_keys(dtype, hd):
    """Head sizes the tensor-core prompt attention takes (bf16), windows whose edges cross its 64-key tiles, kept tokens
    in a tile of their own, and decode steps whose key lists are long enough to be split over CTAs."""
    cfg = so.make_config(width=64, vocab=80, side_dim=8, loop=(0, 1, 2),
                         layers=[dict(heads=2, kv_heads=1, dim=hd, vdim=hd, size=70, keep_first=5, ff=32),
                                 dict(heads=2, kv_heads=2, dim=hd, vdim=hd, size=300, keep_first=0, ff=32)])
    w = so.make_weights(cfg, seed=12)
    n0, n1 = 171, 8
    toks = tokens(n0 + n1, cfg["vocab"], 13)
    short = tokens(20, cfg["vocab"], 14)
    want, want_short = so.forward(cfg, w, toks), so.forward(cfg, w, short)
    eng = make_engine(cfg, w, dtype, max_ctx=420)
    # a long and a short prompt together, the long one cut so that its second part starts inside a tile
    got = eng.step([(0, toks[:100], list(range(100))), (1, short[:17], list(range(17)))])
    assert rel_err(got[:100], want[:100]) < TOL[dtype]
    assert rel_err(got[100:], want_short[:17]) < TOL[dtype]
    got = eng.step([(0, toks[100:n0], list(range(n0 - 100))), (1, short[17:], [0, 1, 2])])
    assert rel_err(got[:n0 - 100], want[100:n0]) < TOL[dtype]
    assert rel_err(got[n0 - 100:], want_short[17:]) < TOL[dtype]
    eng.release(1)
    rows = [eng.step([(0, [toks[t]], [0])]) for t in range(n0, n0 + n1)]
    assert rel_err(torch.cat(rows), want[n0:]) < TOL[dtype]
    eng.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_steps_longer_than_one_pass_and_unordered_wants(dtype):
    """A step of more rows than one pass through the layers takes (4 096) is cut by the engine; the rows around the cut
    agree with the same prompt fed in two steps, and wanted places come back in the order they were asked for."""
    cfg = so.make_config(width=32, vocab=50, side_dim=4, loop=(0, 1, 2),
                         layers=[dict(heads=2, kv_heads=1, dim=8, vdim=8, size=16, keep_first=2, ff=16)])
    w = so.make_weights(cfg, seed=30)
    toks = tokens(4200, cfg["vocab"], 31)
    want = [4199, 0, 4096, 4095, 4097, 17, 2100, 4094]
    eng = make_engine(cfg, w, dtype, max_ctx=4300, max_slots=2)
    one = eng.step([(0, toks, want)])
    a = eng.step([(1, toks[:2100], [0, 17])])
    b = eng.step([(1, toks[2100:], [k - 2100 for k in (4199, 4096, 4095, 4097, 2100, 4094)])])
    two = torch.stack([b[0], a[0], b[1], b[2], b[3], a[1], b[4], b[5]])
    assert rel_err(one, two) < (1e-5 if dtype == torch.float32 else 3e-2)
    # the first rows also against the restatement
    ref = so.forward(cfg, w, toks[:18])
    assert rel_err(one[[1, 5]], ref[[0, 17]]) < TOL[dtype]
    eng.close()


def test_fast_products_agree_with_the_general_kernels(monkeypatch):
    """bf16: the GEMV / tcgen05 / tensor-core-attention routes against the same engine held on the general kernels
    (B200_STACK_PLAIN=1) — same rounding points up to summation order, so far tighter than against the fp32 restatement."""
    cfg = so.make_config(width=128, vocab=160, side_dim=64, loop=(0, 1, 2),
                         layers=[dict(heads=4, kv_heads=2, dim=64, vdim=64, size=40, keep_first=3, ff=96),
                                 dict(heads=2, kv_heads=1, dim=128, vdim=128, size=200, keep_first=0, ff=64)])
    w = so.make_weights(cfg, seed=21)
    toks = tokens(150, cfg["vocab"], 22)

    def run():
        eng = make_engine(cfg, w, torch.bfloat16, max_ctx=300)
        out = [eng.step([(0, toks[:140], list(range(140)))])] + [eng.step([(0, [t], [0])]) for t in toks[140:]]
        eng.close()
        return torch.cat(out)

    fast = run()
    monkeypatch.setenv("B200_STACK_PLAIN", "1")
    plain = run()
    assert rel_err(fast, plain) < 3e-2


def test_residual_stream_mechanisms_show_in_the_logits():
    """Each constant matters: dropping the kept tokens, shifting the window by one, dropping the side input or the loop's
    re-read of the embedding moves the oracle's logits by far more than the engine's distance to the true design."""
    cfg = so.make_config(**CFG_A)
    w = so.make_weights(cfg, seed=5)
    toks = tokens(30, cfg["vocab"], 6)
    want = so.forward(cfg, w, toks)
    eng = make_engine(cfg, w, torch.float32)
    err = rel_err(eng.step([(0, toks, list(range(30)))]), want)
    eng.close()
    import copy
    for what in ("keep", "window", "side", "loop"):
        c = copy.deepcopy(cfg)
        ww = dict(w)
        if what == "keep":
            for L in c["layers"]:
                L["mixer"]["mask"]["keep_first"] = 0
        elif what == "window":
            for L in c["layers"]:
                L["mixer"]["mask"]["size"] += 1
        elif what == "side":
            ww["side.embed"] = torch.zeros_like(w["side.embed"])
        else:
            ww["loop.in"] = torch.cat([w["loop.in"][:, :c["width"]], torch.zeros_like(w["loop.in"][:, c["width"]:])], 1)
        assert rel_err(so.forward(c, ww, toks), want) > 50 * err, what


# ---------------------------------------------------------------------- generation through the engine's entry points
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_single_and_ragged(model_a, dtype):
    cfg, w, toks, _ = model_a
    eng = make_engine(cfg, w, dtype)
    prompt, n = toks[:9], 12
    want, margins = so.greedy(cfg, w, prompt, n)
    got = eng.generate_sync(prompt, n).tolist()
    tol = 0.02 if dtype == torch.float32 else 0.5
    for i in range(n):                                   # equal up to the first step that is too close to call
        if margins[i] < tol:
            break
        assert got[i] == want[i], f"step {i}: {got[i]} vs {want[i]} (margin {margins[i]:.3f})"
    # unequal prompts together: generate_sync_batch takes the ragged path (no padding), each like generating alone
    prompts = [toks[:9], toks[3:5], toks[10:31]]
    outs = eng.generate_sync_batch(prompts, 6).tolist()
    for p, o in zip(prompts, outs):
        w1, m1 = so.greedy(cfg, w, p, 6)
        for i in range(6):
            if m1[i] < tol:
                break
            assert o[i] == w1[i]
    # the device sampler with top_k = 1 is greedy too
    eng.set_sampler(temperature=0.7, top_k=1)
    assert eng.generate_sync(prompt, 4).tolist()[:1] == got[:1]
    eng.close()


def test_context_overflow_is_refused(model_a):
    cfg, w, toks, _ = model_a
    eng = make_engine(cfg, w, torch.bfloat16, max_ctx=16)
    eng.step([(0, toks[:16], [])])
    with pytest.raises(Exception):
        eng.step([(0, [1], [0])])
    eng.close()
