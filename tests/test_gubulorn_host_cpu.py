"""Host side of the Gubulorn path without a GPU: configuration reading and validation, the registry and the tables of
mixers and feed-forwards, the slot cache's per-position stores (growth keeps entries in place), the restatement's router."""
import json

import pytest
import torch

import gubulorn_oracle as go


def _cfg():
    moe = {"kind": "moe", "expert": {"ff": 8},
           "router": {"experts": 3, "identity": 1, "top": 2, "groups": {"count": 2, "keep": 1}}}
    layers = [
        {"type": "delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "conv": 2}, "mlp": None},
        {"type": "parallel", "mlp": moe,
         "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 0.3, "q_temp": {"coef": 0.2, "every": 5}},
                   "right": {"heads": 2, "vdim": 3, "state": 5, "groups": 1, "norm_groups": 2, "conv": 3}}},
        {"type": "delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 4, "conv": 4},
         "mlp": {"kind": "dense", "ff": 10, "limit": 1.5}}]
    return {"architecture": "Gubulorn", "vocab": 11, "width": 12, "norm": {"eps": 1e-5}, "postln_alpha": 2.5,
            "logit_scale": 0.5, "logit_softcap": 9.0, "layers": layers}


def test_config_round_trip():
    from llark_b200.models.gubulorn import GubulornConfig

    c = GubulornConfig.from_dict(_cfg())
    assert (c.vocab, c.width, c.eps, c.alpha, c.logit_scale, c.logit_softcap) == (11, 12, 1e-5, 2.5, 0.5, 9.0)
    assert [l.type for l in c.layers] == ["delta", "parallel", "delta"] and c.layers[0].mlp is None
    assert GubulornConfig.from_dict(json.loads(json.dumps(c.to_dict()))).to_dict() == c.to_dict()
    d = _cfg()
    d["logit_softcap"] = None
    assert GubulornConfig.from_dict(d).logit_softcap is None


@pytest.mark.parametrize("bad", [
    lambda d: d.update(architecture="Other"),
    lambda d: d["layers"][0].update(type="hgrn2"),
    lambda d: d["layers"][1]["mlp"].update(kind="relu"),
    lambda d: d.update(logit_softcap=0.0),
])
def test_config_validation(bad):
    from llark_b200.models.gubulorn import GubulornConfig

    d = json.loads(json.dumps(_cfg()))
    bad(d)
    with pytest.raises(ValueError):
        GubulornConfig.from_dict(d)


def test_registry_and_tables():
    from llark_b200.mixers import FEED_FORWARDS, MIXERS
    from llark_b200.models.gubulorn import FEED_FORWARD_KINDS
    from llark_b200.models.registry import model_class_for

    assert model_class_for({"architecture": "Gubulorn"}).__name__ == "GubulornForCausalLM"
    assert {"delta", "parallel", "sink_attention", "ssd"} <= set(MIXERS)
    for kind in FEED_FORWARD_KINDS.values():
        assert hasattr(FEED_FORWARDS[kind], "post_norm")
    assert all(hasattr(MIXERS[t], "branches") for t in ("delta", "parallel", "sink_attention", "ssd"))


def test_per_position_stores_grow_in_place():
    from llark_b200.state_cache import StateCache

    cache = StateCache("cpu", n_slots=2, positions=4)
    hk = cache.add_store((3,), torch.float32, zero_on_alloc=False, per_position=True)
    hs = cache.add_store((2, 2), torch.float32, zero_on_alloc=True)
    a = cache.alloc()
    assert cache.view(hk).shape == (2, 4, 3) and cache.view(hs).shape == (2, 2, 2)
    cache.view(hk)[a] = torch.arange(12.0).reshape(4, 3)
    cache.view(hs)[a] = 7.0
    cache.reserve_positions(4)
    assert cache.positions == 4
    cache.reserve_positions(9)
    assert cache.positions == 16 and cache.view(hk).shape == (2, 16, 3)
    assert torch.equal(cache.view(hk)[a, :4], torch.arange(12.0).reshape(4, 3))
    assert torch.equal(cache.view(hs)[a], torch.full((2, 2), 7.0))
    b = cache.alloc()
    c = cache.alloc()  # a third slot: every store doubles along the slots, entries stay
    assert cache.n_slots == 4 and cache.view(hk).shape == (4, 16, 3) and len({a, b, c}) == 3
    assert torch.equal(cache.view(hk)[a, :4], torch.arange(12.0).reshape(4, 3))
    assert cache.bytes_per_slot() == (16 * 3 + 4) * 4
    plain = StateCache("cpu", n_slots=1)
    plain.add_store((2,), torch.float32, zero_on_alloc=True)
    plain.alloc()
    plain.reserve_positions(10_000)  # nothing per position: nothing to do
    assert not plain.has_per_position


def test_restated_router_shuts_groups_out_with_minus_infinity():
    """Two groups of two, one kept: with every choice score negative the kept group's members must win, not the others'."""
    z = torch.tensor([[2.0, 1.0, 0.0, -1.0]], dtype=torch.float64)
    corr = torch.tensor([-1.0, -0.9, -0.2, -0.95], dtype=torch.float64)
    ids, wts = go.route(z, corr, 2, 2, 1)
    s = torch.softmax(z, -1)
    # choice scores: group 0 = {s0 - 1, s1 - 0.9}, group 1 = {s2 - 0.2, s3 - 0.95}: group 1 has the best single score
    assert sorted(ids[0].tolist()) == [2, 3]
    assert torch.allclose(wts[0].sort().values, s[0, [2, 3]].sort().values)
