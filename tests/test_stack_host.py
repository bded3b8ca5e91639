"""Host side of the layer-stack models (no GPU): config reader and registry, run order, weight layout, checkpoint
loading, the slot pool, and the plain restatement's own masks."""
import json
import struct

import pytest
import torch

import stack_oracle as so
from tinygpt_b200 import engine, loader, models


def test_config_reader_takes_every_size_from_the_config():
    cfg = so.make_config(width=40, vocab=51, side_dim=3, embed_scale=2.5, residual_mult=0.7, eps=3e-6, loop=(1, 3, 4),
                         layers=[dict(heads=6, kv_heads=3, dim=10, vdim=14, size=11, keep_first=5, ff=24, scale=0.37),
                                 dict(heads=2, kv_heads=1, dim=8, vdim=8, size=2, keep_first=0, ff=None),
                                 dict(heads=1, kv_heads=1, dim=4, vdim=6, size=100, keep_first=9, ff=8)])
    spec = models.ARCHITECTURES[cfg["architecture"]](cfg)
    assert (spec.width, spec.vocab, spec.side_dim, spec.embed_scale, spec.residual_mult, spec.norm_eps) == \
           (40, 51, 3, 2.5, 0.7, 3e-6)
    assert spec.norm_offset == 1.0 and (spec.loop_start, spec.loop_stop, spec.loop_times) == (1, 3, 4)
    a = spec.layers[0].attn
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.keep_first) == (6, 3, 10, 14, 11, 5)
    assert abs(a.scale - 0.37) < 1e-7 and spec.layers[1].ff == 0 and spec.layers[2].ff == 8
    assert models.kozusun_from_config(models.kozusun_config(spec)) == spec
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["type"] = "recurrent"
    with pytest.raises(ValueError):
        models.kozusun_from_config(bad)


def test_run_order_matches_the_plain_order():
    for loop in (None, (0, 2, 3), (1, 2, 1), (2, 4, 2), (0, 4, 2)):
        cfg = so.make_config(layers=[dict(heads=1, kv_heads=1, dim=4, vdim=4, size=2, keep_first=0, ff=4)] * 4, loop=loop)
        assert models.kozusun_from_config(cfg).runs() == so.layer_order(cfg)


def test_visibility_rule():
    a = models.AttnSpec(1, 1, 4, 4, 1.0, window=5, keep_first=2)
    for i in range(20):
        for j in range(20):
            assert a.visible(i, j) == so.sees(i, j, 5, 2)
    assert so.sees(10, 6, 5, 2) and not so.sees(10, 5, 5, 2) and so.sees(10, 1, 5, 2) and not so.sees(10, 2, 5, 2)


def test_packed_layout_holds_every_checkpoint_tensor():
    cfg = so.make_config(width=24, vocab=30, side_dim=3, loop=(0, 1, 2),
                         layers=[dict(heads=3, kv_heads=1, dim=5, vdim=7, size=4, keep_first=1, ff=10),
                                 dict(heads=2, kv_heads=2, dim=4, vdim=4, size=4, keep_first=1, ff=None)])
    w = so.make_weights(cfg, seed=1)
    spec = models.kozusun_from_config(cfg)
    assert set(models.kozusun_tensor_shapes(spec)) == set(w)
    assert all(tuple(w[k].shape) == v for k, v in models.kozusun_tensor_shapes(spec).items())
    for dtype in (torch.bfloat16, torch.float32):
        pk = models.pack_stack_weights(spec, w, device="cpu", dtype=dtype)
        for i in range(2):
            lay, a, p = spec.layout(i), spec.layers[i].attn, f"l{i}."
            assert all(o % 8 == 0 for o in (lay.off_k, lay.off_v, lay.off_g, lay.off_gate, lay.off_up, lay.n_in, lay.off_act))
            wi, bi, wo = pk[p + "w_in"], pk[p + "b_in"], pk[p + "w_out"]
            assert wi.dtype == dtype and bi.dtype == torch.float32 and wi.shape == (lay.n_in, 24)
            assert torch.equal(wi[lay.off_k:lay.off_k + a.kv_heads * a.dim].float(), w[p + "mix.k"].float())
            assert torch.equal(bi[lay.off_v:lay.off_v + a.kv_heads * a.vdim], w[p + "mix.v.b"].float())
            assert torch.equal(wi[lay.off_g:lay.off_g + a.heads].float(), w[p + "mix.g"].float())
            assert torch.equal(wo[:, :a.heads * a.vdim].float(), w[p + "mix.o"].float())
            used = a.heads * a.dim + a.kv_heads * (a.dim + a.vdim) + a.heads + 2 * spec.layers[i].ff
            assert int((wi.float().abs().sum(1) > 0).sum()) == used      # padding rows are zero
        assert torch.equal(pk["l0.w_out"][:, spec.layout(0).off_act:spec.layout(0).off_act + 10].float(),
                           w["l0.mlp.down"].float())


def _write_safetensors(path, tensors):
    header, blobs, off = {}, [], 0
    for k, t in tensors.items():
        raw = t.contiguous().view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


def test_checkpoint_directory_round_trip(tmp_path):
    cfg = so.make_config(loop=(0, 1, 2))
    w = so.make_weights(cfg, seed=2)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    _write_safetensors(tmp_path / "model.safetensors", w)
    assert loader.is_stack_model(tmp_path)
    spec, pk = loader.load_model(tmp_path, device="cpu", dtype=torch.float32, max_ctx=77, max_slots=3)
    assert spec.max_ctx == 77 and spec.max_slots == 3 and spec.architecture == "Kozusun"
    want = models.pack_stack_weights(spec, w, device="cpu", dtype=torch.float32)
    assert set(pk) == set(want) and all(torch.equal(pk[k], want[k]) for k in pk)
    del w["l1.mix.g"]
    _write_safetensors(tmp_path / "model.safetensors", w)
    with pytest.raises(loader.LoaderError):
        loader.load_model(tmp_path, device="cpu")
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nonesuch"}))
    assert not loader.is_stack_model(tmp_path)


def test_slot_pool_hands_freed_slots_out_again():
    pool = engine.SequenceSlots(3)
    assert [pool.acquire(n) for n in "abc"] == [0, 1, 2] and pool.acquire("b") == 1
    with pytest.raises(Exception):
        pool.acquire("d")
    assert pool.release("b") == 1 and "b" not in pool and len(pool) == 2
    assert pool.acquire("d") == 1
    pool.release("a"), pool.release("d")
    assert pool.acquire("e") == 0 and pool.acquire("f") == 1


def test_plain_model_is_causal_and_windowed():
    """The restatement itself: logits at a position do not change with later tokens, and not with tokens that have
    left every layer's reach."""
    cfg = so.make_config(layers=[dict(heads=2, kv_heads=1, dim=8, vdim=8, size=3, keep_first=1, ff=16)] * 2, side_dim=4)
    w = so.make_weights(cfg, seed=3)
    a = [5, 9, 2, 7, 7, 1, 30, 4, 8, 6, 11, 3]
    b = list(a)
    b[-1] = 40
    la, lb = so.forward(cfg, w, a), so.forward(cfg, w, b)
    assert torch.equal(la[:-1], lb[:-1]) and not torch.equal(la[-1], lb[-1])
    c = list(a)
    c[2] = 41        # position 2 is neither kept nor within two layers × window 3 of position 11
    assert torch.allclose(so.forward(cfg, w, c)[-1], la[-1], atol=1e-6)
    c = list(a)
    c[0] = 41        # position 0 is kept
    assert not torch.allclose(so.forward(cfg, w, c)[-1], la[-1], atol=1e-4)
