"""Host side of the Tokatar path without a GPU: configuration reading and validation, the registry and the mixer table, the
frequency tables against the restatement, and the restatement itself (mask by blocks, the 1 in the denominator, rotation)."""
import json
import math

import pytest
import torch

import tokatar_oracle as to


def _cfg():
    layers = [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 10},
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 0.5, "softcap": 7.0, "mask": {"size": 5},
                   "rot": {"base": 100.0, "dims": 2, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 16}}}},
        {"type": "attention_2", "mlp": None,
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 2, "scale": 0.4, "mask": {"size": 3},
                   "rot": {"base": 50.0, "dims": 4}}},
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 7},
         "mixer": {"heads": 2, "dim": 3, "rot_dim": 2, "vdim": 3, "kv_rank": 5, "scale": 0.45, "rot": {"base": 9.0, "dims": 2}}}]
    return {"architecture": "Tokatar", "vocab": 11, "width": 12, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
            "layers": layers}


def test_config_round_trip():
    from llark_b200.models.tokatar import TokatarConfig

    c = TokatarConfig.from_dict(_cfg())
    assert (c.vocab, c.width, c.eps, c.embedding_scale) == (11, 12, 1e-5, 2.0)
    assert [l.type for l in c.layers] == ["attention", "attention_2", "latent_attention"] and c.layers[1].mlp is None
    assert TokatarConfig.from_dict(json.loads(json.dumps(c.to_dict()))).to_dict() == c.to_dict()


@pytest.mark.parametrize("bad", [
    lambda d: d.update(architecture="Other"),
    lambda d: d["layers"][0].update(type="hgrn2"),
    lambda d: d["layers"][0]["mlp"].update(kind="moe"),
    lambda d: d.update(layers=[]),
])
def test_config_validation(bad):
    from llark_b200.models.tokatar import TokatarConfig

    d = json.loads(json.dumps(_cfg()))
    bad(d)
    with pytest.raises(ValueError):
        TokatarConfig.from_dict(d)


def test_registry_and_tables():
    from llark_b200.mixers import FEED_FORWARDS, MIXERS
    from llark_b200.models.registry import model_class_for
    from llark_b200.models.tokatar import FEED_FORWARD_KINDS, MIXER_TYPES

    assert model_class_for({"architecture": "Tokatar"}).__name__ == "TokatarForCausalLM"
    assert set(MIXER_TYPES.values()) <= set(MIXERS) and set(FEED_FORWARD_KINDS.values()) <= set(FEED_FORWARDS)
    vrot, plain = MIXERS["rotary_attention_vrot"].Weights, MIXERS["rotary_attention"].Weights
    assert (vrot.biases, vrot.whole_norm, vrot.interleaved, vrot.rotate_values, vrot.plus_one) == (True,) * 5
    assert (plain.biases, plain.whole_norm, plain.interleaved, plain.rotate_values, plain.plus_one) == (False,) * 5
    lat = MIXERS["latent_attention_causal"].Weights
    assert lat.halves and lat.gate_per_head and not MIXERS["latent_attention"].Weights.halves


@pytest.mark.parametrize("dims,base,scaling", [
    (8, 100.0, None), (40, 1e4, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}),
    (16, 30.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 40}), (6, 5e5, {"factor": 2.0, "low": 2.0, "high": 3.0, "original": 10})])
def test_frequency_table(dims, base, scaling):
    from llark_b200.mixers import rotary_frequencies

    f, mult = rotary_frequencies(dims, base, scaling)
    want = to.frequencies(dims, base)
    if scaling:
        want = to.scaled_frequencies(want, scaling)
    assert mult == 1.0 and f.shape == (dims // 2,)
    assert torch.allclose(f, want, rtol=1e-12, atol=0.0)


def test_frequency_bands():
    """Short waves keep their frequency, long waves are slowed by the factor, the band between lies between."""
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 40}
    f = to.frequencies(16, 30.0)
    g = to.scaled_frequencies(f, sc)
    wave = 2 * math.pi / f
    kinds = set()
    for i in range(8):
        if wave[i] < 10.0:
            assert g[i] == f[i]
            kinds.add("kept")
        elif wave[i] > 40.0:
            assert g[i] == f[i] / 4.0
            kinds.add("slowed")
        else:
            assert f[i] / 4.0 < g[i] < f[i]
            kinds.add("blended")
    assert kinds == {"kept", "slowed", "blended"}


def test_restated_mask_and_denominator():
    m = to.visible(7, 3)
    assert m[2].tolist() == [True, True, True, False, False, False, False]
    assert m[3].tolist() == [False, False, False, True, False, False, False]
    assert m[6].tolist() == [False] * 6 + [True]
    assert to.visible(4)[3].all() and not to.visible(4)[0, 1]
    q = torch.zeros(1, 1, 2, dtype=torch.float64)
    v = torch.ones(1, 1, 3, dtype=torch.float64)
    assert torch.allclose(to.attend(q, q, v, 1.0, to.visible(1), plus_one=True), torch.full((1, 1, 3), 0.5, dtype=torch.float64))
    assert torch.allclose(to.attend(q, q, v, 1.0, to.visible(1)), v)


def test_restated_rotation_is_relative_and_undone_by_its_inverse():
    g = torch.Generator().manual_seed(0)
    x, y = torch.randn(1, 1, 6, generator=g, dtype=torch.float64), torch.randn(1, 1, 6, generator=g, dtype=torch.float64)
    f = to.frequencies(4, 10.0)
    for layout in ("halves", "interleaved"):
        a = (to.turn(x, torch.tensor([9]), f, layout) * to.turn(y, torch.tensor([4]), f, layout)).sum()
        b = (to.turn(x, torch.tensor([25]), f, layout) * to.turn(y, torch.tensor([20]), f, layout)).sum()
        assert abs(a - b) < 1e-12
        back = to.turn(to.turn(x, torch.tensor([9]), f, layout), torch.tensor([9]), f, layout, sign=-1.0)
        assert torch.allclose(back, x)
        assert torch.equal(to.turn(x, torch.tensor([9]), f, layout)[..., 4:], x[..., 4:])  # the rest of the head passes


def test_restated_model_runs_and_is_causal():
    cfg = _cfg()
    W = to.random_weights(cfg, seed=0)
    toks = [1, 5, 3, 9, 0, 2, 7, 7, 4]
    full, res = to.forward(cfg, W, toks, return_residuals=True)
    assert full.shape == (9, 11) and len(res) == 3
    assert torch.allclose(to.forward(cfg, W, toks[:5]), full[:5], atol=1e-12)


def test_checkpoint_container_keeps_single_numbers(tmp_path):
    """Norm weights of this design are tensors without an axis; the container's writer and reader keep them so."""
    from llark_b200.safetensors_io import load_file, save_file

    W = {k: v.to(torch.bfloat16) for k, v in to.random_weights(_cfg(), seed=1).items()}
    save_file(W, str(tmp_path / "m.safetensors"))
    back = load_file(str(tmp_path / "m.safetensors"))
    assert set(back) == set(W)
    assert back["l0.norm1"].shape == () and back["final.norm"].shape == ()
    assert all(torch.equal(back[k], W[k]) for k in W)
