"""Silatar design in the layer-stack engine against the plain restatement in tests/silatar_oracle.py: every mechanism
alone (layer norm, clamped gated unit, rotary table, latent attention with crafted far keys, the mLSTM recurrence and its
carried state, routed experts), whole prompts, decoding through cache and state, prompts cut into portions, unequal
batches, slots given back and used again, long decoding, other sizes and layer orders, greedy generation through the
engine's own entry points."""
import math

import pytest
import torch

import silatar_oracle as so
from tinygpt_b200 import engine, models, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
# fp32 engines are held to summation-order noise.  bf16 engines round every activation to 8 bits of mantissa, and a token
# whose two best router scores are closer than that rounding may go to another expert than in the fp32 restatement — which
# then colours every later position through the recurrent state.  So against the restatement the bf16 runs are held to the
# median row and to most rows (gross faults), the fp32 runs of the same step function to every row (fine faults), and the
# bf16 kernels' own paths (weight-streaming products, tensor-core products, general kernels) to each other.
TOL = {torch.float32: 3e-4, torch.bfloat16: 9e-2}


def row_err(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: rms of the difference (mean removed) over rms of the wanted row (mean removed)."""
    got, want = got.float().cpu(), want.float().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    c = want - want.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / c.pow(2).mean(-1).sqrt().clamp_min(1e-6)


def assert_close(got, want, dtype, what=""):
    e = row_err(got, want)
    if dtype == torch.float32:
        assert float(e.max()) < TOL[dtype], f"{what}: worst row {float(e.max()):.2e} at {int(e.argmax())}"
    else:
        assert bool(torch.isfinite(got.float()).all()), what
        assert float(e.median()) < TOL[dtype] and float((e < TOL[dtype]).float().mean()) >= 0.6, \
            f"{what}: {int((e >= TOL[dtype]).sum())} of {len(e)} rows off, median {float(e.median()):.2e}"


ROT = {"base": 10000.0, "dims": 8, "scaling": {"factor": 8.0, "fast": 16.0, "original": 64, "slow": 2.0}}


def latent(heads=3, dim=12, rot_dim=8, vdim=20, kv_rank=40, rot=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": 1.0 / math.sqrt(dim + rot_dim)}
    if rot_dim > 0:
        m["rot"] = dict(rot or ROT)
    return {"type": "latent_attention", "mixer": m}


def mlstm(heads=3, dim=16, vdim=24, cap=12.0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def dense(ff=72):
    return {"ff": ff, "kind": "dense"}


def moe(experts=6, top=2, ff=24, limit=1.5, shared=(40, 2.5)):
    d = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        d["shared"] = {"ff": shared[0], "limit": shared[1]}
    return d


def config(layers, width=64, vocab=96, loop=None, softcap=20.0, eps=1e-5):
    cfg = {"architecture": "Silatar", "layers": [dict(mix, mlp=mlp) for mix, mlp in layers], "logit_softcap": softcap,
           "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def base_config():
    return config([(latent(), moe()), (mlstm(), dense()), (latent(heads=2, dim=8, rot_dim=10, vdim=12, kv_rank=24), dense(40)),
                   (mlstm(heads=2, dim=8, vdim=40), moe(experts=5, top=3, ff=16, shared=None))], loop=(1, 3, 2))


def make(cfg, dtype, seed=0, max_ctx=160, max_slots=4):
    spec = models.silatar_from_config(cfg).with_ctx(max_ctx, max_slots)
    w = models.synth_silatar_weights(spec, seed=seed)
    eng = engine.DecodeEngine(spec, models.pack_weights(spec, w, device=DEV, dtype=dtype))
    return eng, {k: v.float() for k, v in w.items()}


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ------------------------------------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_norm_ops(dtype):
    g = torch.Generator().manual_seed(1)
    x, w = torch.randn(9, 100, generator=g) * 3 + 1.5, 1 + torch.randn(100, generator=g) * 0.2
    got = ops.stack_norm(x.to(DEV), w.to(DEV), 1e-5, "layer", out_dtype=dtype)
    assert float(row_err(got, so.layer_norm(x, w, 1e-5)).max()) < (1e-6 if dtype == torch.float32 else 5e-3)
    y = torch.randn(9, 100, generator=g) * 7 - 2
    got = ops.stack_norm_add(x.clone().to(DEV), y.to(DEV), w.to(DEV), 1e-5, "layer")
    assert (got.cpu() - (x + so.layer_norm(y, w, 1e-5))).abs().max() < 1e-5
    got = ops.stack_norm(x.to(DEV), w.to(DEV), 1e-5, "rms", out_dtype=torch.float32)
    assert (got.cpu() - so.unit_rms(x, 1e-5) * w).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_clamped_gated_unit_and_erf_gelu(dtype):
    g = torch.Generator().manual_seed(2)
    gu = (torch.randn(7, 2 * 19, generator=g) * 3).to(dtype)
    got = ops.stack_glu_clamp(gu.to(DEV), 1.75)
    gg, uu = gu.float()[:, :19].clamp(max=1.75), gu.float()[:, 19:].clamp(-1.75, 1.75)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1)
    assert (got.float().cpu() - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.04)
    z = (torch.randn(5, 33, generator=g) * 2).to(dtype)
    want = 0.5 * z.float() * (1 + torch.erf(z.float() / math.sqrt(2)))
    assert (ops.stack_act(z.to(DEV), "gelu_erf").float().cpu() - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.03)


def _selector_latent(dtype, mixer, n, seed, eps=1e-5):
    """A latent-attention case whose input rows ARE the projections: w_q / w_dkv pick columns of h, w_o is the identity.
    → (h [n, nq + nd], oracle weights, op weights)"""
    g = torch.Generator().manual_seed(seed)
    H, dn, dr, dv, r = (mixer[k] for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    nq, nd = H * (dn + dr), r + dr
    w = {"q": torch.eye(nq + nd)[:nq], "dkv": torch.eye(nq + nd)[nq:], "dkv.norm": 1 + 0.2 * torch.randn(r, generator=g),
         "uk": torch.randn(H * dn, r, generator=g) * 0.3, "uv": torch.randn(H * dv, r, generator=g) * 0.3,
         "o": torch.eye(H * dv)}
    w = {k: v.to(dtype).float() for k, v in w.items()}
    h = torch.randn(n, nq + nd, generator=g).to(dtype).float()
    return h, w


def _run_latent_op(h, w, mixer, dtype, steps, max_ctx, slot=1, eps=1e-5):
    """Feeds h's rows through the op in the given portions (all in cache slot `slot` of 3) → [n, heads·vdim]."""
    H, dn, dr, dv, r = (mixer[k] for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    rot = models._rotary_from_config(mixer["rot"])
    cache = torch.zeros(3, max_ctx, r + dr, dtype=dtype, device=DEV)
    kw = dict(heads=H, dim=dn, rot_dim=dr, vdim=dv, kv_rank=r, scale=mixer["scale"], rot_dims=rot.dims,
              c_norm=w["dkv.norm"].to(DEV), uk_t=w["uk"].view(H, dn, r).transpose(1, 2).contiguous().to(dtype).to(DEV),
              uv=w["uv"].to(dtype).to(DEV), rot_table=rot.table(max_ctx).to(DEV), eps=eps)
    out, at = [], 0
    for n in steps:
        rows = h[at:at + n].to(dtype).to(DEV)
        pos = torch.arange(at, at + n, dtype=torch.int32, device=DEV)
        out.append(ops.stack_latent_attention(rows, H * (dn + dr), cache, torch.full((n,), slot, dtype=torch.int32, device=DEV),
                                              pos, **kw))
        at += n
    return torch.cat(out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rot", [ROT, {"base": 500.0, "dims": 4}, {"base": 10000.0, "dims": 6, "scaling": {
    "factor": 2.0, "fast": 4.0, "original": 32, "slow": 1.0}}])
def test_latent_attention_op(dtype, rot):
    mixer = latent(heads=3, dim=12, rot_dim=8, vdim=20, kv_rank=40, rot=rot)["mixer"]
    h, w = _selector_latent(dtype, mixer, 45, seed=3)
    want = so.latent_attention(h, w, "", mixer, 1e-5)
    for steps in ([45], [40, 1, 1, 1, 1, 1], [2, 13, 30]):
        got = _run_latent_op(h, w, mixer, dtype, steps, max_ctx=64)
        assert float(row_err(got, want).max()) < (2e-5 if dtype == torch.float32 else 4e-2), steps


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_latent_attention_far_key_stands_out(dtype, decode):
    """300 positions; the query of the last one is aimed, through uk of head 1, at the latent of position 3, so that this
    one score dominates: a key list that starts late, ends early or skips rows changes the output outright."""
    mixer = latent(heads=2, dim=10, rot_dim=4, vdim=16, kv_rank=36, rot={"base": 100.0, "dims": 4})["mixer"]
    n, far = 300, 3
    h, w = _selector_latent(dtype, mixer, n, seed=4)
    H, dn, dr, r = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["kv_rank"]
    nq = H * (dn + dr)
    c_far = so.unit_rms(h[far:far + 1, nq:nq + r], 1e-5)[0] * w["dkv.norm"]
    aim = w["uk"].view(H, dn, r)[1] @ c_far
    h[n - 1, (dn + dr):(dn + dr) + dn] = (aim * (25.0 / mixer["scale"] / float(aim @ aim))).to(dtype).float()
    want = so.latent_attention(h, w, "", mixer, 1e-5)
    pr = torch.softmax(torch.tensor([float((h[n - 1, (dn + dr):(dn + dr) + dn] @ (w["uk"].view(H, dn, r)[1] @ (
        so.unit_rms(h[j:j + 1, nq:nq + r], 1e-5)[0] * w["dkv.norm"]))) * mixer["scale"]) for j in range(n)]), 0)
    assert float(pr[far]) > 0.5      # the crafted score does dominate the plain part
    got = _run_latent_op(h, w, mixer, dtype, [n - 1, 1] if decode else [n], max_ctx=320)
    assert float(row_err(got[-1:], want[-1:]).max()) < (2e-5 if dtype == torch.float32 else 4e-2)
    assert float(row_err(got, want).max()) < (2e-5 if dtype == torch.float32 else 4e-2)


def _mlstm_case(dtype, H, dk, dv, n, seed, cap):
    g = torch.Generator().manual_seed(seed)
    proj = torch.randn(n, 2 * H * dk + H * dv, generator=g).to(dtype)
    gates = torch.randn(n, 2 * H, generator=g) * 6 + torch.tensor([0.0] * H + [3.0] * H)
    p = proj.float()
    q = p[:, :H * dk].view(n, H, dk) * dk ** -0.5
    k, v = p[:, H * dk:2 * H * dk].view(n, H, dk), p[:, 2 * H * dk:].view(n, H, dv)
    want = so.mlstm_cell(q, k, v, so.capped(gates[:, :H], cap), torch.nn.functional.logsigmoid(so.capped(gates[:, H:], cap)))
    return proj, gates, want


def _mlstm_out(raw, dv):
    return raw[..., :dv] / (torch.maximum(raw[..., dv].abs(), torch.exp(-raw[..., dv + 1])) + 1e-6).unsqueeze(-1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(3, 16, 24), (1, 40, 7), (2, 33, 64), (4, 8, 9)])
def test_mlstm_recurrence_op_and_carried_state(dtype, sizes):
    H, dk, dv = sizes
    n, cap = 70, 9.0
    proj, gates, want = _mlstm_case(dtype, H, dk, dv, n, seed=5, cap=cap)
    kw = dict(heads=H, dim=dk, vdim=dv, gate_cap=cap)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    for steps in ([n], [n - 9] + [1] * 9, [2, 30, 38]):
        state = ops.stack_mlstm_state(3, H, dk, dv, DEV)
        state.fill_(7.0)                      # whatever an earlier sequence left: position 0 starts from zero
        out, at = [], 0
        for c in steps:
            raw = ops.stack_mlstm(proj[at:at + c].to(DEV), 0, H * dk, 2 * H * dk, gates[at:at + c].to(DEV), state, i32([0]), i32([c]),
                                  i32([2] * c), i32(list(range(at, at + c))), **kw)
            out.append(_mlstm_out(raw.cpu(), dv))
            at += c
        err = (torch.cat(out) - want).abs().max() / want.abs().max()
        assert float(err) < (2e-5 if dtype == torch.float32 else 1e-4), (steps, float(err))   # the recurrence is fp32 either way


@pytest.mark.parametrize("dtype", DTYPES)
def test_mlstm_sequences_side_by_side(dtype):
    """Three sequences of unequal length in one launch, in scrambled slots, against each alone."""
    H, dk, dv, cap = 2, 16, 20, 15.0
    lens = [5, 1, 17]
    cases = [_mlstm_case(dtype, H, dk, dv, n, seed=10 + i, cap=cap) for i, n in enumerate(lens)]
    proj, gates = torch.cat([c[0] for c in cases]), torch.cat([c[1] for c in cases])
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    slots, row0 = [2, 0, 1], [0, 5, 6]
    state = ops.stack_mlstm_state(3, H, dk, dv, DEV)
    raw = ops.stack_mlstm(proj.to(DEV), 0, H * dk, 2 * H * dk, gates.to(DEV), state, i32(row0), i32(lens),
                          i32(sum(([s] * n for s, n in zip(slots, lens)), [])), i32(sum((list(range(n)) for n in lens), [])),
                          heads=H, dim=dk, vdim=dv, gate_cap=cap)
    got = _mlstm_out(raw.cpu(), dv)
    want = torch.cat([c[2] for c in cases])
    assert float((got - want).abs().max() / want.abs().max()) < 1e-4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(6, 2, 24), (5, 1, 16), (9, 9, 8), (33, 4, 40)])
def test_routed_experts_op(dtype, shape):
    E, top, ff = shape
    W, n = 48, 37
    g = torch.Generator().manual_seed(6)
    w = {"router": torch.randn(E, W, generator=g) * 0.5}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = torch.randn(ff, W, generator=g) * 0.3, torch.randn(ff, W, generator=g) * 0.3
        w[f"e{e}.down"] = torch.randn(W, ff, generator=g) * 0.3
    w = {k: v.to(dtype).float() for k, v in w.items()}
    h = torch.randn(n, W, generator=g).to(dtype).float()
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": 1.25}}
    want = so.moe_ff(h, w, "", mlp)
    idx, val = so.routing(h, w, "", top)
    t = lambda v: v.to(dtype).to(DEV)
    y, chosen, scores = ops.stack_moe(t(h), t(w["router"]),
                                      t(torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)])),
                                      t(torch.stack([w[f"e{e}.down"] for e in range(E)])), top, 1.25)
    assert torch.equal(chosen.cpu().long().sort(-1).values, idx.sort(-1).values)
    assert (scores.cpu().sort(-1).values - val.sort(-1).values).abs().max() < 1e-5
    assert float(row_err(y, want).max()) < (2e-5 if dtype == torch.float32 else 3e-2)


# ------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompt(dtype):
    cfg = base_config()
    eng, w = make(cfg, dtype)
    toks = tokens(50, cfg["vocab"], 7)
    got = eng.step([(0, toks, list(range(50)))])
    assert_close(got, so.forward(cfg, w, toks), dtype, "whole prompt")
    assert_close(got[:3], so.forward(cfg, w, toks)[:3], dtype, "first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_then_token_by_token_and_long_decode(dtype):
    cfg = base_config()
    eng, w = make(cfg, dtype)
    toks = tokens(120, cfg["vocab"], 8)
    want = so.forward(cfg, w, toks)
    rows = [eng.step([(2, toks[:30], list(range(30)))])]
    for t in range(30, 120):
        rows.append(eng.step([(2, [toks[t]], [0])]))
    assert_close(torch.cat(rows), want, dtype, "prefill + 90 decode steps")
    assert eng.slot_position(2) == 120


@pytest.mark.parametrize("dtype", DTYPES)
def test_from_the_first_token_one_by_one(dtype):
    cfg = base_config()
    eng, w = make(cfg, dtype)
    toks = tokens(20, cfg["vocab"], 9)
    rows = [eng.step([(1, [t], [0])]) for t in toks]
    assert_close(torch.cat(rows), so.forward(cfg, w, toks), dtype, "one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2, 2, 2, 44], [33, 2, 15], [1, 48, 1], [17, 16, 17]])
def test_prompt_in_portions(dtype, cuts):
    cfg = base_config()
    eng, w = make(cfg, dtype)
    toks = tokens(sum(cuts), cfg["vocab"], 10)
    rows, at = [], 0
    for c in cuts:
        rows.append(eng.step([(0, toks[at:at + c], list(range(c)))]))
        at += c
    assert_close(torch.cat(rows), so.forward(cfg, w, toks), dtype, f"portions {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batch_against_each_alone_then_decoded_together(dtype):
    cfg = base_config()
    eng, w = make(cfg, dtype)
    lens, new = [1, 37, 9], 12
    seqs = [tokens(n + new, cfg["vocab"], 20 + i) for i, n in enumerate(lens)]
    want = [so.forward(cfg, w, s) for s in seqs]
    slots = [3, 0, 2]
    got = eng.step([(sl, s[:n], list(range(n))) for sl, s, n in zip(slots, seqs, lens)])
    at = 0
    for i, n in enumerate(lens):
        assert_close(got[at:at + n], want[i][:n], dtype, f"batched prompt {i}")
        at += n
    live = [0, 1, 2]
    for t in range(new):
        if t == 5:                       # the middle request ends early; its slot goes back
            eng.release(slots[1])
            live = [0, 2]
        got = eng.step([(slots[i], [seqs[i][lens[i] + t]], [0]) for i in live])
        for r, i in enumerate(live):
            assert_close(got[r:r + 1], want[i][lens[i] + t:lens[i] + t + 1], dtype, f"batched decode {i} step {t}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_slot_given_back_and_used_again(dtype):
    cfg = base_config()
    eng, w = make(cfg, dtype, max_slots=2)
    a, b = tokens(40, cfg["vocab"], 30), tokens(25, cfg["vocab"], 31)
    eng.step([(0, a, [])])
    eng.step([(1, b[:10], [])])
    eng.release(0)
    got = eng.step([(0, b, list(range(25))), (1, b[10:], list(range(15)))])   # slot 0 again, from position 0
    want = so.forward(cfg, w, b)
    assert_close(got[:25], want, dtype, "reused slot")
    assert_close(got[25:], want[10:], dtype, "the other slot went on")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["no_loop", "loop_all", "loop_tail", "no_mlp", "top1_no_shared", "odd_sizes", "one_head",
                                  "plain_rotary", "wide_latent", "no_rotary"])
def test_other_orders_and_sizes(dtype, case):
    if case == "no_loop":
        cfg = config([(mlstm(), moe()), (latent(), dense())])
    elif case == "loop_all":
        cfg = config([(latent(), dense()), (mlstm(), moe(top=1))], loop=(0, 2, 3))
    elif case == "loop_tail":
        cfg = config([(mlstm(), dense()), (latent(), moe()), (latent(), dense())], loop=(2, 3, 2))
    elif case == "no_mlp":
        cfg = config([(latent(), None), (mlstm(), None), (latent(), dense())], softcap=5.0)
    elif case == "top1_no_shared":
        cfg = config([(latent(), moe(experts=3, top=1, shared=None)), (mlstm(), moe(experts=2, top=2, shared=(8, 0.5)))])
    elif case == "odd_sizes":
        cfg = config([(latent(heads=5, dim=7, rot_dim=6, vdim=9, kv_rank=33, rot={"base": 77.0, "dims": 2}), dense(50)),
                      (mlstm(heads=3, dim=11, vdim=13, cap=4.0), moe(experts=7, top=3, ff=10, shared=(9, 1.0)))], width=60,
                     vocab=77, eps=1e-3)
    elif case == "one_head":
        cfg = config([(latent(heads=1, dim=32, rot_dim=16, vdim=48, kv_rank=64, rot=dict(ROT, dims=16)), dense(64)),
                      (mlstm(heads=1, dim=64, vdim=32), dense(32))], width=128)
    elif case == "wide_latent":      # a latent wider than the split-key decode kernel takes
        cfg = config([(latent(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=544, rot={"base": 100.0, "dims": 4}), dense(32)),
                      (mlstm(heads=1, dim=8, vdim=8), None)])
    elif case == "no_rotary":        # no rotated part at all
        cfg = config([(latent(heads=2, dim=16, rot_dim=0, vdim=8, kv_rank=24), dense(32)), (mlstm(), dense())])
    else:
        cfg = config([(latent(rot={"base": 1000.0, "dims": 8}), dense()), (mlstm(), dense())])
    eng, w = make(cfg, dtype, seed=3)
    toks = tokens(34, cfg["vocab"], 40)
    want = so.forward(cfg, w, toks)
    rows = [eng.step([(1, toks[:20], list(range(20)))]), eng.step([(1, toks[20:23], [0, 1, 2])])]
    rows += [eng.step([(1, [t], [0])]) for t in toks[23:]]
    assert_close(torch.cat(rows), want, dtype, case)


@pytest.mark.parametrize("dtype", DTYPES)
def test_expert_layers_of_unequal_count_share_the_engine(dtype):
    """Eight experts in one layer, three in the next, and prompt after prompt through the same engine: what one layer's
    routing leaves behind must not reach the other's.  Every prompt must come out as from an engine that has seen nothing
    before (both number formats), and as the restatement has it (fp32)."""
    cfg = config([(latent(), moe(experts=8, top=2, ff=16, shared=None)), (mlstm(), moe(experts=3, top=2, ff=24))], loop=(0, 2, 2))
    eng, w = make(cfg, dtype, seed=5)
    for seed, n in ((1, 60), (2, 24), (3, 41), (4, 12)):
        toks = tokens(n, cfg["vocab"], seed)
        got = eng.step([(0, toks, list(range(n)))])
        eng.release(0)
        fresh, _ = make(cfg, dtype, seed=5)
        alone = fresh.step([(0, toks, list(range(n)))])
        fresh.close()
        assert float(row_err(got, alone).max()) < 1e-5, f"prompt of {n} after others"
        if dtype == torch.float32:
            assert_close(got, so.forward(cfg, w, toks), dtype, f"prompt of {n}")


def test_the_constants_matter():
    """Moving one constant of the design moves the logits: none of them is ignored on the way to the engine."""
    cfg = base_config()
    toks = tokens(30, cfg["vocab"], 50)
    eng, _ = make(cfg, torch.float32)
    ref = eng.step([(0, toks, list(range(30)))]).cpu()
    eng.close()

    def moved(edit):
        c = base_config()
        edit(c)
        e, _ = make(c, torch.float32)
        out = e.step([(0, toks, list(range(30)))]).cpu()
        e.close()
        return float(row_err(out, ref).max())

    def set_(path, v):
        def f(c):
            d = c
            for k in path[:-1]:
                d = d[k]
            d[path[-1]] = v
        return f

    L = ["layers"]
    for path, v in [(L + [0, "mixer", "scale"], 0.5), (L + [0, "mixer", "rot", "base"], 50.0),
                    (L + [0, "mixer", "rot", "scaling", "factor"], 2.0), (L + [0, "mixer", "rot", "scaling", "slow"], 8.0),
                    (L + [0, "mixer", "rot", "dims"], 4), (L + [1, "mixer", "gate_cap"], 2.0),
                    (L + [0, "mlp", "expert", "limit"], 0.2), (L + [0, "mlp", "shared", "limit"], 0.2),
                    (L + [0, "mlp", "router", "top"], 1), (["logit_softcap"], 3.0), (["norm", "eps"], 1e-1),
                    (["loop", "times"], 1)]:
        assert moved(set_(path, v)) > 1e-3, path


def test_bf16_paths_agree_with_each_other():
    """Sizes the fast paths take (multiples of 8; 32 and more rows for the tensor-core products and the per-expert products,
    16 and more rows of a sequence with dim + rot_dim == vdim == 64 for the tensor-core prompt attention over expanded keys,
    up to 8 rows for the weight-streaming products and the split-key decode attention): the same prompt whole, in portions,
    token by token and beside other requests."""
    cfg = config([(latent(heads=2, dim=32, rot_dim=32, vdim=64, kv_rank=64, rot=dict(ROT, dims=32)),
                   moe(experts=8, top=2, ff=64, shared=(64, 2.0))),
                  (mlstm(heads=2, dim=32, vdim=32), dense(128)),
                  (latent(heads=4, dim=16, rot_dim=8, vdim=16, kv_rank=64), dense(64))], width=128, vocab=160, loop=(0, 2, 2))
    eng, w = make(cfg, torch.bfloat16, max_ctx=256)
    toks = tokens(100, cfg["vocab"], 90)
    whole = eng.step([(0, toks, list(range(100)))])
    assert_close(whole, so.forward(cfg, w, toks), torch.bfloat16, "whole")
    eng.release(0)
    parts = torch.cat([eng.step([(0, toks[:64], list(range(64)))]), eng.step([(0, toks[64:96], list(range(32)))]),
                       eng.step([(0, toks[96:], list(range(4)))])])
    other = tokens(40, cfg["vocab"], 91)
    eng.step([(1, toks[:60], []), (2, other, [])])
    single = torch.cat([eng.step([(1, [t], [0]), (2, [other[i % 40]], [])])[:1] for i, t in enumerate(toks[60:])])
    for name, got, ref in (("portions", parts, whole), ("decoded beside another", single, whole[60:])):
        e = row_err(got, ref)
        assert float((e < 3e-2).float().mean()) >= 0.9 and float(e.median()) < 1e-2, (name, float(e.median()), float(e.max()))


# ------------------------------------------------------------------------------------------- generation
def test_greedy_generation_through_the_engine():
    cfg = config([(latent(), dense()), (mlstm(), moe())], loop=(0, 2, 2))
    eng, w = make(cfg, torch.float32)
    prompt, new = tokens(11, cfg["vocab"], 60), 9
    seq = list(prompt)
    for _ in range(new):
        seq.append(int(so.forward(cfg, w, seq)[-1].argmax()))
    assert eng.generate_sync(prompt, new).tolist() == seq[len(prompt):]
    prompts = [tokens(4, cfg["vocab"], 61), tokens(13, cfg["vocab"], 62), tokens(7, cfg["vocab"], 63)]
    want = []
    for p in prompts:
        s = list(p)
        for _ in range(6):
            s.append(int(so.forward(cfg, w, s)[-1].argmax()))
        want.append(s[len(p):])
    assert eng.generate_sync_batch(prompts, 6).tolist() == want
    with pytest.raises(Exception):      # a recurrent state cannot be rewound into the middle of a sequence
        eng.seek(3)


def test_bf16_generation_runs_and_is_deterministic():
    cfg = base_config()
    eng, _ = make(cfg, torch.bfloat16)
    prompt = tokens(40, cfg["vocab"], 70)
    a = eng.generate_sync(prompt, 24).tolist()
    b = eng.generate_sync(prompt, 24).tolist()
    assert a == b and all(0 <= t < cfg["vocab"] for t in a)


def test_context_overflow_is_refused():
    cfg = config([(latent(), dense())])
    eng, _ = make(cfg, torch.float32, max_ctx=16)
    with pytest.raises(Exception):
        eng.step([(0, tokens(17, cfg["vocab"], 80), [])])
