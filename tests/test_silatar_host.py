"""Host side of the Silatar design (no GPU): config reader and registry, run order, merged layouts, rotary frequencies
against the restatement, checkpoint round trip through the loader, and the restatement's own sanity."""
import math

import pytest
import torch

import silatar_oracle as so
from tinygpt_b200 import loader, models

ROT = {"base": 10000.0, "dims": 8, "scaling": {"factor": 8.0, "fast": 16.0, "original": 64, "slow": 2.0}}


def cfg_small():
    return {"architecture": "Silatar", "width": 40, "vocab": 50, "logit_softcap": 12.0, "norm": {"eps": 1e-4},
            "loop": {"start": 1, "stop": 3, "times": 3},
            "layers": [
                {"type": "mlstm", "mixer": {"heads": 2, "dim": 6, "vdim": 10, "gate_cap": 7.0}, "mlp": None},
                {"type": "latent_attention",
                 "mixer": {"heads": 3, "dim": 5, "rot_dim": 8, "vdim": 7, "kv_rank": 12, "scale": 0.3, "rot": ROT},
                 "mlp": {"kind": "moe", "expert": {"ff": 9, "limit": 1.5}, "router": {"experts": 4, "top": 2},
                         "shared": {"ff": 11, "limit": 2.0}}},
                {"type": "mlstm", "mixer": {"heads": 1, "dim": 16, "vdim": 8, "gate_cap": 15.0},
                 "mlp": {"kind": "dense", "ff": 30}},
                {"type": "latent_attention",
                 "mixer": {"heads": 2, "dim": 4, "rot_dim": 6, "vdim": 4, "kv_rank": 9, "scale": 0.5,
                           "rot": {"base": 100.0, "dims": 4}},
                 "mlp": {"kind": "moe", "expert": {"ff": 5, "limit": 0.7}, "router": {"experts": 3, "top": 1}}}]}


def test_registry_reads_the_config_and_writes_it_back():
    cfg = cfg_small()
    spec = models.ARCHITECTURES["Silatar"](cfg)
    assert spec.architecture == "Silatar" and spec.block == "sandwich" and spec.norm_kind == "layer"
    assert [r[0] for r in spec.runs()] == [0, 1, 2, 1, 2, 1, 2, 3] == so.layer_runs(cfg)
    assert not any(mix for _, mix in spec.runs())          # nothing happens between passes
    assert spec.layers[1].latent.rot.factor == 8.0 and spec.layers[3].latent.rot.factor == 0.0
    assert spec.layers[1].moe.shared_ff == 11 and spec.layers[3].moe.shared_ff == 0 and spec.layers[0].ff == 0
    assert models.silatar_from_config(models.silatar_config(spec)) == spec
    for bad in ({"type": "attention"}, {"mlp": {"kind": "gated"}}):
        c = cfg_small()
        c["layers"][1].update(bad)
        with pytest.raises(ValueError):
            models.silatar_from_config(c)
    c = cfg_small()
    c["loop"]["stop"] = 9
    with pytest.raises(ValueError):
        models.silatar_from_config(c)


@pytest.mark.parametrize("rot", [ROT, {"base": 100.0, "dims": 4}, {"base": 500000.0, "dims": 32, "scaling": {
    "factor": 16.0, "fast": 8.0, "original": 512, "slow": 0.5}}])
def test_rotary_frequencies_and_table_match_the_restatement(rot):
    spec = models._rotary_from_config(rot)
    f, mag = spec.frequencies()
    f0, mag0 = so.rotary_frequencies(rot)
    assert torch.allclose(torch.from_numpy(f), f0, rtol=1e-12, atol=0) and abs(mag - mag0) < 1e-12
    tab = spec.table(70)
    v = torch.randn(70, rot["dims"] + 3, dtype=torch.float64)
    want = so.rotate(v, torch.arange(70), rot)
    a, b = v[:, 0:rot["dims"]:2], v[:, 1:rot["dims"]:2]
    c, s = tab[..., 0].double(), tab[..., 1].double()
    assert (a * c - b * s - want[:, 0:rot["dims"]:2]).abs().max() < 1e-5
    assert (b * c + a * s - want[:, 1:rot["dims"]:2]).abs().max() < 1e-5
    assert torch.equal(want[:, rot["dims"]:], v[:, rot["dims"]:])      # the rest passes unchanged


def test_merged_layouts_and_packed_weights():
    spec = models.silatar_from_config(cfg_small())
    w = models.synth_silatar_weights(spec, seed=1)
    assert set(w) == set(models.silatar_tensor_shapes(spec))
    pk = models.pack_weights(spec, w, device="cpu", dtype=torch.float32)
    lay = spec.mix_layout(1)                                  # latent attention: [q | down]
    a = spec.layers[1].latent
    assert lay.off_k % 8 == 0 and lay.n_in % 8 == 0 and lay.k_out == a.heads * a.vdim
    assert torch.equal(pk["l1.w_in"][:a.heads * (a.dim + a.rot_dim)], w["l1.mix.q"].float())
    assert torch.equal(pk["l1.w_in"][lay.off_k:lay.off_k + a.kv_rank + a.rot_dim], w["l1.mix.dkv"].float())
    assert float(pk["l1.w_in"][a.heads * (a.dim + a.rot_dim):lay.off_k].abs().sum()) == 0.0
    uk = w["l1.mix.uk"].float().view(a.heads, a.dim, a.kv_rank)
    assert torch.equal(pk["l1.uk_t"], uk.transpose(1, 2).contiguous())
    lay = spec.mix_layout(0)                                  # mLSTM: [q | k | v | out gate | gates]
    m = spec.layers[0].mlstm
    assert torch.equal(pk["l0.w_in"][lay.off_gate + m.heads:lay.off_gate + 2 * m.heads], w["l0.mix.f"].float())
    assert torch.equal(pk["l0.b_in"][lay.off_gate:lay.off_gate + m.heads], w["l0.mix.i.b"].float())
    assert float(pk["l0.b_in"][:lay.off_gate].abs().sum()) == 0.0
    mo = spec.layers[1].moe
    assert pk["l1.w_exp_in"].shape == (mo.experts, 2 * mo.expert_ff, spec.width)
    assert torch.equal(pk["l1.w_exp_in"][2, mo.expert_ff:], w["l1.mlp.e2.up"].float())
    assert torch.equal(pk["l1.w_ff_in"][2 * mo.shared_ff], w["l1.mlp.shared.sg"].float()[0])
    assert "l3.w_ff_in" not in pk and "l0.ff_norm" not in pk and "l2.w_ff_in" in pk
    assert spec.weight_params() > 0


def test_checkpoint_round_trip_through_the_loader(tmp_path):
    spec = models.silatar_from_config(cfg_small())
    w = models.synth_silatar_weights(spec, seed=2)
    models.save_stack_checkpoint(spec, w, str(tmp_path))
    assert loader.is_stack_model(tmp_path)
    spec2, pk = loader.load_model(tmp_path, device="cpu", dtype=torch.float32, max_ctx=99, max_slots=3)
    assert spec2 == spec.with_ctx(99, 3)
    want = models.pack_weights(spec, w, device="cpu", dtype=torch.float32)
    assert set(pk) == set(want) and all(torch.equal(pk[k], want[k]) for k in want)
    (tmp_path / "config.json").write_text((tmp_path / "config.json").read_text().replace('"kv_rank": 12', '"kv_rank": 13'))
    with pytest.raises(loader.LoaderError):
        loader.load_model(tmp_path, device="cpu", dtype=torch.float32)


def test_restatement_is_causal_and_its_state_is_what_the_equations_say():
    cfg = cfg_small()
    spec = models.silatar_from_config(cfg)
    w = {k: v.double() for k, v in models.synth_silatar_weights(spec, seed=3).items()}
    g = torch.Generator().manual_seed(4)
    toks = torch.randint(0, cfg["vocab"], (19,), generator=g).tolist()
    full = so.forward(cfg, w, toks)
    assert (so.forward(cfg, w, toks[:11]) - full[:11]).abs().max() < 1e-9
    assert float(full.abs().max()) < cfg["logit_softcap"]
    # a memory that forgets nothing and takes everything in with weight 1 is the plain sum of k vᵀ
    T, H, dk, dv = 6, 1, 3, 2
    q, k, v = torch.randn(T, H, dk, dtype=torch.float64), torch.randn(T, H, dk, dtype=torch.float64), torch.randn(T, H, dv, dtype=torch.float64)
    out = so.mlstm_cell(q, k, v, torch.zeros(T, H, dtype=torch.float64), torch.zeros(T, H, dtype=torch.float64))
    S = sum(torch.outer(k[t, 0], v[t, 0]) for t in range(T))
    n = k[:, 0].sum(0)
    assert (out[-1, 0] - S.T @ q[-1, 0] / (max(abs(float(n @ q[-1, 0])), 1.0) + 1e-6)).abs().max() < 1e-12
    # routing: the weight multiplies the expert's input
    h = torch.randn(3, cfg["width"], dtype=torch.float64)
    idx, val = so.routing(h, w, "l3.mlp.", 1)
    one = so.expert(val[0, 0] * h[:1], w, f"l3.mlp.e{int(idx[0, 0])}.", 0.7)
    assert (so.moe_ff(h, w, "l3.mlp.", cfg["layers"][3]["mlp"])[0] - one[0]).abs().max() < 1e-12
