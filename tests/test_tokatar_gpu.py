"""Tokatar on the GPU against the plain restatement in tests/tokatar_oracle.py (float64 on the CPU): every mechanism alone
through its op or its mixer class, then the whole model through the engine's step function, the slot cache, the scheduler,
generate() and the command-line tools. Configurations are small and deliberately unlike each other: key heads shared by
all, by two or by none, key and value sizes that differ (scalar attention route) or agree at a multiple of 16 (tensor-core
route), rotation over a part of the head and over all of it, with and without rescaled frequencies and soft cap, blocks of
1 to 100 positions and attention without a mask, layers without a feed-forward, every mixer first or last."""
import math

import pytest
import torch

import tokatar_oracle as to

pytestmark = pytest.mark.gpu
F32, F64, BF16 = torch.float32, torch.float64, torch.bfloat16


def _dev():
    return torch.device("cuda:0")


def _layout(lens, pos0, slots):
    from llark_b200.state_cache import StepLayout

    return StepLayout(lens, pos0, slots, _dev())


def _rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return ((a - b).norm() / (b.norm() + 1e-30)).item()


def _logit_err(got, want):
    """Difference of logits with the mean over the vocabulary taken off, rms, relative to the rms of the expected ones:
    the largest over the positions."""
    d = got.double().cpu() - want.double().cpu()
    d = d - d.mean(dim=-1, keepdim=True)
    w = want.double().cpu()
    w = w - w.mean(dim=-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()).max().item()


def _tol(dtype):
    return 1e-4 if dtype == F32 else 6e-2


# ------------------------------------------------------------------------------------------------ configurations
def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def _att(heads, kv, dim, vdim, size, rot, softcap=None, scale=None, mlp=None, kind="attention"):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": rot, "scale": scale or 1.0 / math.sqrt(dim)}
    if size:
        m["mask"] = {"size": size}
    if softcap:
        m["softcap"] = softcap
    return {"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": mlp} if mlp else None}


def _att2(heads, kv, dim, vdim, size, rot, scale=None, mlp=None):
    return _att(heads, kv, dim, vdim, size, rot, scale=scale, mlp=mlp, kind="attention_2")


def _lat(heads, dim, rot_dim, vdim, rank, base, scale=None, mlp=None):
    return {"type": "latent_attention", "mlp": {"kind": "dense", "ff": mlp} if mlp else None,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                      "rot": {"base": base, "dims": rot_dim}, "scale": scale or 1.0 / math.sqrt(dim + rot_dim)}}


def _cfg(layers, vocab=97, width=72, eps=1e-5, scale=3.0):
    return {"architecture": "Tokatar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": layers}


CONFIGS = {
    # every size differs from every other: rotation over half of the head with rescaled frequencies (all three bands are
    # hit: original 40), soft cap that bites, blocks of 24 and of 7 positions, key heads shared by two and by none, values
    # narrower than keys, a latent wider than the heads, the last layer without a feed-forward
    "mixed": _cfg([_att(4, 2, 16, 12, 24, _rot(100.0, 8, (4.0, 1.0, 4.0, 40)), softcap=2.0, mlp=40),
                   _att2(3, 3, 10, 6, 7, _rot(50.0, 10), mlp=31),
                   _lat(3, 6, 4, 5, 12, 30.0, mlp=20),
                   _att(2, 1, 6, 8, 5, _rot(10.0, 6))]),
    # latent attention first, nothing a multiple of 4 but the rotated parts, blocks of ONE position (a token sees only
    # itself) and a block longer than any test sequence, attention without any mask, rescaled frequencies on the value
    # rotating attention (the values keep the plain ones), embedding scale 1, a large eps
    "odd_sizes": _cfg([_lat(3, 5, 2, 7, 9, 7.0, mlp=23),
                       _att2(3, 1, 6, 10, 1, _rot(20.0, 4, (2.0, 1.0, 2.0, 16)), mlp=11),
                       _att(3, 3, 10, 5, None, _rot(1000.0, 2)),
                       _att2(2, 2, 6, 2, 1000, _rot(3.0, 6), mlp=17)],
                      vocab=33, width=51, eps=1e-3, scale=1.0),
    # sizes of the tensor-core route: head size 32 with one key head and blocks of 64 (a key tile) and of 100, value
    # rotation at head size 16 in interleaved pairs, a latent row of 24 + 8 = 32
    "tiles": _cfg([_att(2, 1, 32, 32, 64, _rot(10000.0, 32, (8.0, 1.0, 4.0, 64)), softcap=30.0, mlp=64),
                   _att2(4, 2, 16, 16, 100, _rot(500.0, 8), mlp=48),
                   _lat(2, 16, 8, 16, 24, 100.0, mlp=32),
                   _att(4, 4, 16, 16, 33, _rot(77.0, 16), mlp=24)],
                  vocab=50, width=80),
}


def _model(cfg, W, dtype):
    from llark_b200.models.tokatar import TokatarConfig, TokatarForCausalLM

    return TokatarForCausalLM(TokatarConfig.from_dict(cfg), W, device="cuda:0", dtype=dtype)


def _tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class _Stores:
    """Stand-in cache for a mixer used alone: slot stores filled with garbage."""

    def __init__(self, n_slots=4, positions=512):
        self.t, self.n, self.positions = [], n_slots, positions

    def add_store(self, shape, dtype, zero_on_alloc, per_position=False):
        fill = 0.0 if zero_on_alloc else float("nan")
        lead = (self.positions,) if per_position else ()
        self.t.append(torch.full((self.n,) + lead + tuple(shape), fill, device=_dev(), dtype=dtype))
        return len(self.t) - 1

    def view(self, h):
        return self.t[h]


def _mixer_class(kind):
    from llark_b200.mixers import MIXERS
    from llark_b200.models.tokatar import MIXER_TYPES

    return MIXERS[MIXER_TYPES[kind]]


def _run_mixer(kind, W, spec, width, h, portions, act, eps=1e-5, slot=2, max_positions=None):
    """h [T, width] through the mixer of layer type `kind` cut into `portions` (one request in `slot`)."""
    cls = _mixer_class(kind)
    weights = cls.Weights({k: v.to(F32) for k, v in W.items()}, "m.", spec, width, _dev(), act)
    stores = _Stores()
    mixer = cls(weights, stores, eps, act, max_positions)
    outs, at = [], 0
    for n in portions:
        st = _layout([n], [at], [slot])
        outs.append(mixer.forward(h[at:at + n].to(_dev(), act).contiguous(), st, stores).cpu())
        at += n
    assert at == h.shape[0]
    return torch.cat(outs)


def _oracle_mixer(kind, h, W, spec, eps=1e-5):
    return to.mixer(kind, h, W, "m.", spec, eps)


def _mixer_weights(layer, width, seed):
    """The tensors of one layer's mixer from the random checkpoint maker, under the prefix 'm.'."""
    W = to.random_weights(_cfg([layer], width=width), seed=seed)
    return {"m." + k[len("l0.mix."):]: v for k, v in W.items() if k.startswith("l0.mix.")}


PORTIONS = ([150], [1] * 150, [100] + [1] * 50, [31, 2, 2, 65, 1, 1, 30, 18])


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("C", [51, 72, 1024, 2048, 4100, 8196])
def test_gate_norm_scale_and_sum_with_the_next_input_norm(C):
    from llark_b200 import ops

    g = torch.Generator().manual_seed(C)
    n = 13
    x, y = torch.randn(n, C, generator=g, dtype=F64), 5.0 * torch.randn(n, C, generator=g, dtype=F64)
    pre = 2.0 * torch.randn(n, C + 8, generator=g, dtype=F64)  # the gate is a column slice of a wider projection
    ls, gb, gn = torch.randn(C, generator=g, dtype=F64), 0.7, 1.3
    gated = y * torch.sigmoid(pre[:, 8:])
    want = x + to.scalar_norm(gated, gb, 1e-5) * ls
    want_plain = x + to.scalar_norm(y, gb, 1e-5) * ls
    want_next = to.scalar_norm(want, gn, 1e-5)
    d = _dev()
    w_post = (ls * gb).to(d, F32).contiguous()
    w_next = torch.full((C,), gn, device=d, dtype=F32)
    pre_d = pre.to(d, F32)
    for act in (F32, BF16):
        got, nxt = ops.seq_gated_norm_add(x.to(d, F32), y.to(d, F32), w_post, 1e-5, gate=pre_d[:, 8:], w_next=w_next, act=act)
        assert _rel(got, want) < 1e-6
        assert nxt.dtype == act and _rel(nxt, want_next) < (1e-6 if act == F32 else 4e-3)
    assert _rel(ops.seq_gated_norm_add(x.to(d, F32), y.to(d, F32), w_post, 1e-5, gate=pre_d[:, 8:]), want) < 1e-6
    assert _rel(ops.seq_gated_norm_add(x.to(d, F32), y.to(d, F32), w_post, 1e-5), want_plain) < 1e-6
    # a gate that starts on an odd column (no 16-byte alignment) takes the scalar route
    got = ops.seq_gated_norm_add(x.to(d, F32), y.to(d, F32), w_post, 1e-5, gate=pre_d[:, 7:7 + C])
    assert _rel(got, x + to.scalar_norm(y * torch.sigmoid(pre[:, 7:7 + C]), gb, 1e-5) * ls) < 1e-6


@pytest.mark.parametrize("H,G,D,E,n_rot,interleaved,norm,vrot", [
    (4, 2, 16, 12, 8, False, False, False), (3, 3, 10, 6, 10, True, True, True), (2, 1, 6, 8, 0, False, True, False),
    (3, 1, 32, 32, 32, True, False, True), (5, 5, 7, 4, 6, False, True, True), (2, 2, 24, 16, 16, False, True, True),
    (3, 1, 12, 8, 4, True, True, True), (2, 1, 64, 64, 64, False, False, False)])
def test_projection_norm_and_rotation_of_queries_keys_and_values(H, G, D, E, n_rot, interleaved, norm, vrot):
    from llark_b200 import ops

    g = torch.Generator().manual_seed(H * D + E)
    T, pos0 = 9, 37
    n = H * D + G * D + G * E
    wq, wk = 1.0 + 0.3 * torch.randn(H * D, generator=g, dtype=F64), 1.0 + 0.3 * torch.randn(G * D, generator=g, dtype=F64)
    f = to.frequencies(n_rot, 50.0) if n_rot else torch.zeros(0, dtype=F64)
    fv = to.frequencies(E, 50.0)
    layout = "interleaved" if interleaved else "halves"
    pos = torch.arange(pos0, pos0 + T)
    d = _dev()
    st = _layout([T], [pos0], [0])
    for off in (3, 4):  # columns in front of q: an odd offset takes the scalar kernel, a multiple of four the 16-byte one
        src = torch.randn(T, n + off + (-(n + off)) % 4, generator=g, dtype=F64)
        q, k, v = src[:, off:off + H * D], src[:, off + H * D:off + (H + G) * D], src[:, off + (H + G) * D:off + n]
        if norm:
            q, k = to.rms(q, 1e-5) * wq, to.rms(k, 1e-5) * wk
        q, k = to.turn(q.reshape(T, H, D), pos, f, layout), to.turn(k.reshape(T, G, D), pos, f, layout)
        v = v.reshape(T, G, E)
        if vrot:
            v = to.turn(v, pos, fv, layout)
        for act in (F32, BF16):
            gq, gk, gv = ops.seq_qkv_rotary(src.to(d, F32), off, off + H * D, off + (H + G) * D, H, G, D, E, 1e-5, act, st,
                                            wq=wq.to(d, F32) if norm else None, wk=wk.to(d, F32) if norm else None,
                                            qk_freq=f.to(d, F32) if n_rot else None, qk_interleaved=interleaved,
                                            v_freq=fv.to(d, F32) if vrot else None, v_interleaved=interleaved)
            tol = 2e-6 if act == F32 else 4e-3
            assert _rel(gq, q.reshape(T, -1)) < tol and _rel(gk, k.reshape(T, -1)) < tol and _rel(gv, v.reshape(T, -1)) < tol


LAYERS_ALONE = {
    "attention": [_att(4, 2, 16, 12, 24, _rot(100.0, 8, (4.0, 1.0, 4.0, 40)), softcap=2.0),
                  _att(3, 1, 6, 5, 7, _rot(9.0, 6)), _att(2, 2, 32, 32, 64, _rot(1e4, 16), softcap=30.0),
                  _att(4, 1, 16, 16, 33, _rot(77.0, 16, (8.0, 1.0, 4.0, 64))), _att(2, 1, 10, 6, None, _rot(50.0, 4)),
                  _att(2, 2, 16, 16, None, _rot(50.0, 16))],
    "attention_2": [_att2(3, 3, 10, 6, 7, _rot(50.0, 10)), _att2(4, 2, 16, 16, 100, _rot(500.0, 8)),
                    _att2(3, 1, 6, 10, 1, _rot(20.0, 4, (2.0, 1.0, 2.0, 16))), _att2(2, 1, 32, 32, 48, _rot(1e4, 32)),
                    _att2(2, 2, 64, 64, 70, _rot(1e3, 64))],
    "latent_attention": [_lat(3, 6, 4, 5, 12, 30.0), _lat(2, 16, 8, 16, 24, 100.0), _lat(3, 5, 2, 7, 9, 7.0),
                         _lat(4, 32, 16, 24, 48, 3e4)],
}


@pytest.mark.parametrize("kind,index", [(k, i) for k in sorted(LAYERS_ALONE) for i in range(len(LAYERS_ALONE[k]))])
def test_mixer_alone_in_one_step_in_portions_and_token_by_token(kind, index):
    layer = LAYERS_ALONE[kind][index]
    C = 40
    W = _mixer_weights(layer, C, seed=index)
    h = torch.randn(150, C, generator=torch.Generator().manual_seed(4), dtype=F64).to(BF16).to(F64)
    want = _oracle_mixer(kind, h, W, layer["mixer"])
    for portions in PORTIONS:
        assert _rel(_run_mixer(kind, W, layer["mixer"], C, h, portions, F32), want) < 2e-5, portions
    for portions in ([150], [31, 2, 2, 65, 1, 1, 30, 18]):  # bfloat16: the tensor-core kernel where the sizes allow it
        assert _rel(_run_mixer(kind, W, layer["mixer"], C, h, portions, BF16), want) < 2e-2, portions


def test_the_mixer_also_projects_the_layers_gate_in_its_input_product():
    """`side`: rows of another matrix (and its bias) ride in front of q | k | v | g; the mixer's own result does not change."""
    C = 40
    for kind, layer in (("attention", LAYERS_ALONE["attention"][0]), ("attention_2", LAYERS_ALONE["attention_2"][0]),
                        ("latent_attention", LAYERS_ALONE["latent_attention"][0])):
        W = _mixer_weights(layer, C, seed=3)
        g = torch.Generator().manual_seed(5)
        W["x.rg"], W["x.rg.b"] = torch.randn(C, C, generator=g, dtype=F64).to(BF16).to(F64), torch.randn(C, generator=g, dtype=F64)
        h = torch.randn(20, C, generator=g, dtype=F64).to(BF16).to(F64)
        cls = _mixer_class(kind)
        weights = cls.Weights({k: v.to(F32) for k, v in W.items()}, "m.", layer["mixer"], C, _dev(), F32, side=("x.rg", "x.rg.b"))
        stores = _Stores()
        mixer = cls(weights, stores, 1e-5, F32, None)
        y = mixer.forward(h.to(_dev(), F32), _layout([20], [0], [1]), stores)
        assert _rel(y, _oracle_mixer(kind, h, W, layer["mixer"])) < 2e-5
        assert _rel(mixer.side, h @ W["x.rg"].T + W["x.rg.b"]) < 1e-5


# ------------------------------------------------------------------------------------------------ keys at edges and far away
def _needle(kind, T, H, G, D, E, n_rot, size, far, seed, query_sign=1.0):
    """Projections that ARE the input (identity weights): queries and keys are random directions except that the last
    query of every head points along the key at position `far` in the entries that are not rotated (its rotated entries
    are zero); that key's value stands out. With a score scale of 3 the aligned pair scores about 3 (D - n_rot), every
    other about +-3 sqrt(D): the far key takes nearly all of the softmax if the mask lets it be seen."""
    g = torch.Generator().manual_seed(seed)
    C = H * D + G * D + G * E + H * E
    h = torch.randn(T, C, generator=g, dtype=F64)
    k_off, v_off = H * D, (H + G) * D
    for hd in range(H):
        kv = hd // (H // G)
        h[T - 1, hd * D:(hd + 1) * D] = query_sign * h[far, k_off + kv * D:k_off + (kv + 1) * D]
        h[T - 1, hd * D:hd * D + n_rot] = 0.0
    h[far, v_off:v_off + G * E] = 50.0 + torch.arange(G * E, dtype=F64)
    h[:, v_off + G * E:] = 4.0  # gates wide open
    eye = torch.eye(C, dtype=F64)
    W = {"m.q": eye[:k_off], "m.k": eye[k_off:v_off], "m.v": eye[v_off:v_off + G * E], "m.g": eye[v_off + G * E:],
         "m.o": eye[:, :H * E].clone()}
    if kind == "attention_2":
        zeros = lambda n: torch.zeros(n, dtype=F64)  # noqa: E731
        W.update({"m.q.b": zeros(H * D), "m.k.b": zeros(G * D), "m.v.b": zeros(G * E),
                  "m.q.norm": torch.ones(H * D, dtype=F64), "m.k.norm": torch.ones(G * D, dtype=F64)})
    spec = _att(H, G, D, E, size, _rot(100.0, n_rot), scale=3.0, kind=kind)["mixer"]
    return h.to(BF16).to(F64), W, spec, C


def _visible(T, far, size):
    return size is None or (T - 1) // size == far // size


@pytest.mark.parametrize("kind", ["attention", "attention_2"])
@pytest.mark.parametrize("size,far", [(64, 319), (64, 320), (64, 321), (64, 383), (100, 299), (100, 300), (33, 362), (33, 363),
                                      (None, 0), (None, 1), (None, 255), (None, 256), (500, 0), (500, 63), (500, 64)])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_keys_just_inside_and_just_outside_the_block_and_far_back(kind, size, far, dtype):
    """The query is the last of 384 tokens. The key sits at the first position of the query's block (seen), one before it
    (not seen), one after it, right before the query, at a key tile's edge (32 for the scalar kernel, 64 for the tensor-core
    kernel), or at the edge of the per-position store's first 256 entries when there is no mask."""
    T, H, G, D, E = 384, 2, 1, 16, 16
    h, W, spec, C = _needle(kind, T, H, G, D, E, 4, size, far, seed=far)
    want = _oracle_mixer(kind, h, W, spec)
    seen = _visible(T, far, size)
    assert (want[T - 1].abs().max() > 35.0) == seen  # the read-out is the needle's value, or nothing like it
    for portions in ([384], [383, 1], [256, 100, 27, 1], [200] + [1] * 184, [300, 2, 2] + [1] * 80):
        got = _run_mixer(kind, W, spec, C, h, portions, dtype)
        assert _rel(got[T - 1], want[T - 1]) < (1e-4 if dtype == F32 else 2e-2), portions
        assert _rel(got, want) < (1e-4 if dtype == F32 else 3e-2), portions


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_block_edges_pass_under_decoded_tokens_and_the_ring_is_no_longer_than_the_requests_bound(dtype):
    """Blocks of 24 positions over 130 tokens of which the last 100 are decoded: four block starts fall among the decoded
    tokens. With a bound of 16 positions per request the ring is shorter than a block."""
    layer = _att(4, 2, 16, 16, 24, _rot(100.0, 8), softcap=20.0)
    C = 40
    W = _mixer_weights(layer, C, seed=1)
    h = torch.randn(130, C, generator=torch.Generator().manual_seed(2), dtype=F64).to(BF16).to(F64)
    want = _oracle_mixer("attention", h, W, layer["mixer"])
    for portions in ([30] + [1] * 100, [23] + [1] * 107, [24, 24, 1, 23, 2, 22] + [1] * 34):
        assert _rel(_run_mixer("attention", W, layer["mixer"], C, h, portions, dtype), want) < (2e-5 if dtype == F32 else 2e-2)
    got = _run_mixer("attention", W, layer["mixer"], C, h[:16], [10, 1, 1, 4], dtype, max_positions=16)
    assert _rel(got, want[:16]) < (2e-5 if dtype == F32 else 2e-2)


def test_the_one_in_the_denominator_takes_the_weight_when_every_score_is_low():
    """Queries that point AWAY from every key of their block: all scores are far below zero, the softmax weights are all
    but zero and so is the output, where a plain softmax would still hand out weights that sum to one."""
    T, H, G, D, E = 80, 2, 2, 16, 16
    for dtype in (F32, BF16):
        h, W, spec, C = _needle("attention_2", T, H, G, D, E, 0, 40, 50, seed=1)
        k = h[:, H * D:(H + G) * D].reshape(T, G, D)
        h[40:, :H * D] = (-4.0 * k[40:].mean(0, keepdim=True).sign()).reshape(1, -1) * k[40:].abs().reshape(T - 40, -1)
        h = h.to(BF16).to(F64)
        want = _oracle_mixer("attention_2", h, W, spec)
        plain = to.attention_mixer(h, W, "m.", spec)
        for portions in ([80], [79, 1], [40] + [1] * 40):
            got = _run_mixer("attention_2", W, spec, C, h, portions, dtype)
            assert torch.isfinite(got).all()
            assert (got.double() - want).abs().max() < (1e-4 if dtype == F32 else 0.3)
    # the first token sees only itself: weight e^s / (1 + e^s), not 1
    assert _rel(want[0], plain[0]) > 1e-3


@pytest.mark.parametrize("far", [0, 1, 31, 32, 63, 64, 255, 256, 300])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_latent_attention_reaches_a_latent_far_back(far, dtype):
    """Identity expansions: every head's key IS the normed latent and so is its value. The last query points along the
    latent at position `far`, 350 or more tokens earlier; the read-out is that latent."""
    T, H, R, P = 400, 2, 12, 4
    g = torch.Generator().manual_seed(far)
    C = H * (R + P) + R + P + H
    h = torch.randn(T, C, generator=g, dtype=F64)
    lat0 = H * (R + P)
    unit = h[far, lat0:lat0 + R] / h[far, lat0:lat0 + R].pow(2).mean().sqrt()
    for hd in range(H):
        h[T - 1, hd * (R + P):hd * (R + P) + R] = unit
        h[T - 1, hd * (R + P) + R:(hd + 1) * (R + P)] = 0.0
    h[:, lat0 + R + P:] = 4.0
    eye = torch.eye(C, dtype=F64)
    W = {"m.q": eye[:lat0], "m.dkv": eye[lat0:lat0 + R + P], "m.g": eye[lat0 + R + P:], "m.dkv.norm": torch.ones(R, dtype=F64),
         "m.uk": torch.eye(R, dtype=F64).repeat(H, 1), "m.uv": torch.eye(R, dtype=F64).repeat(H, 1),
         "m.o": eye[:, :H * R].clone()}
    spec = _lat(H, R, P, R, R, 40.0, scale=3.0)["mixer"]
    h = h.to(BF16).to(F64)
    want = _oracle_mixer("latent_attention", h, W, spec)
    near = want[T - 1, :R] / torch.sigmoid(torch.tensor(4.0, dtype=F64))
    assert _rel(near, to.rms(h[far, lat0:lat0 + R], 1e-5)) < 0.05  # the read-out is the far latent
    for portions in ([400], [399, 1], [256, 100, 43, 1], [200] + [1] * 200):
        got = _run_mixer("latent_attention", W, spec, C, h, portions, dtype)
        assert _rel(got[T - 1], want[T - 1]) < (1e-4 if dtype == F32 else 2e-2), portions
        assert _rel(got, want) < (1e-4 if dtype == F32 else 3e-2), portions


def test_rotation_makes_scores_depend_on_the_distance_only():
    """The same 40 inputs at positions 0.. and at positions 24..: with blocks of 24 positions and rotation on, the outputs
    of the last 16 tokens (a whole block start later) agree, because q.k depends on i - j alone and the values are turned back."""
    C = 40
    for kind, layer in (("attention", _att(2, 1, 16, 16, 24, _rot(30.0, 16))), ("attention_2", _att2(2, 2, 16, 16, 24, _rot(30.0, 16)))):
        W = _mixer_weights(layer, C, seed=2)
        h = torch.randn(40, C, generator=torch.Generator().manual_seed(3), dtype=F64).to(BF16).to(F64)
        a = _run_mixer(kind, W, layer["mixer"], C, h, [40], F32)
        pad = torch.randn(24, C, generator=torch.Generator().manual_seed(4), dtype=F64).to(BF16).to(F64)
        b = _run_mixer(kind, W, layer["mixer"], C, torch.cat([pad, h]), [64], F32)
        assert _rel(b[24 + 24:], a[24:]) < 2e-5
        assert _rel(b[24:24 + 24], a[:24]) < 2e-5


# ------------------------------------------------------------------------------------------------ whole model
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_every_layer(name):
    cfg = CONFIGS[name]
    W = to.random_weights(cfg, seed=1)
    toks = _tokens(75, cfg["vocab"], 1)
    want, want_layers = to.forward(cfg, W, toks, return_residuals=True)
    m = _model(cfg, W, F32)
    cache = m.new_cache()
    logits, res = m.engine.step(cache, [cache.alloc()], [toks], want=[list(range(75))], return_residuals=True)
    assert len(res) == len(want_layers)
    for i, r in enumerate(res):
        assert _rel(r, want_layers[i]) < 2e-5, f"residual after layer {i}"
    assert _logit_err(logits, want) < 1e-4
    m16 = _model(cfg, W, BF16)
    c16 = m16.new_cache()
    got16 = m16.engine.step(c16, [c16.alloc()], [toks], want=[list(range(75))])
    assert _logit_err(got16, want) < _tol(BF16)


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_prefill_portions_and_decoding_agree(name, dtype):
    """The same 90 tokens: in one step; as a prompt and then token by token; token by token from the start; in portions
    of 7, 2, 2, 30, 1, 1, 2, ..."""
    cfg = CONFIGS[name]
    W = to.random_weights(cfg, seed=3)
    toks = _tokens(90, cfg["vocab"], 2)
    m = _model(cfg, W, dtype)
    want = to.forward(cfg, W, toks)

    def run(portions):
        cache = m.new_cache()
        s = cache.alloc()
        out, at = [], 0
        for n in portions:
            out.append(m.engine.step(cache, [s], [toks[at:at + n]], want=[list(range(n))]))
            at += n
        assert at == 90 and cache.length[s] == 90
        return torch.cat(out)

    whole = run([90])
    assert _logit_err(whole, want) < _tol(dtype)
    for portions in ([30] + [1] * 60, [1] * 90, [7, 2, 2, 30, 1, 1, 2, 3, 2, 40]):
        got = run(portions)
        assert _logit_err(got, want) < _tol(dtype)
        assert _logit_err(got, whole) < _tol(dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_unequal_batch_equals_each_request_alone_and_slots_are_reused(dtype):
    cfg = CONFIGS["mixed"]
    W = to.random_weights(cfg, seed=4)
    m = _model(cfg, W, dtype)
    prompts = [_tokens(n, cfg["vocab"], 10 + n) for n in (1, 33, 5, 70, 12)]
    tails = [_tokens(6, cfg["vocab"], 50 + i) for i in range(5)]
    stop_after = [2, 6, 1, 4, 6]  # decode steps each request takes part in

    def alone(cache, i):
        s = cache.alloc()
        out = [m.engine.step(cache, [s], [prompts[i]], want=[list(range(len(prompts[i])))])]
        for k in range(stop_after[i]):
            out.append(m.engine.step(cache, [s], [[tails[i][k]]]))
        cache.release(s)
        return torch.cat(out)

    cache = m.new_cache(n_slots=2)  # five requests: the stores have to grow while two are live
    ref = [alone(cache, i) for i in range(5)]  # one after the other: the same slot again and again
    assert cache.allocs == 5 and cache.n_slots == 2 and not cache.in_use()
    slots = [cache.alloc() for _ in range(5)]  # together, in slots that hold the leftovers of the runs above
    assert cache.n_slots >= 5
    got = [[] for _ in range(5)]
    lg = m.engine.step(cache, slots, prompts, want=[list(range(len(p))) for p in prompts])
    r = 0
    for i, p in enumerate(prompts):
        got[i].append(lg[r:r + len(p)])
        r += len(p)
    live = list(range(5))
    for k in range(6):
        live = [i for i in live if stop_after[i] > k]
        lg = m.engine.step(cache, [slots[i] for i in live], [[tails[i][k]] for i in live])
        for j, i in enumerate(live):
            got[i].append(lg[j:j + 1])
        for i in list(live):
            if stop_after[i] == k + 1:
                cache.release(slots[i])
    for i in range(5):
        assert _logit_err(torch.cat(got[i]), ref[i]) < _tol(dtype), i
    want0 = to.forward(cfg, W, prompts[3] + tails[3][:4])
    assert _logit_err(ref[3], want0) < _tol(dtype)
    assert not cache.in_use()


def test_per_position_stores_grow_and_slots_are_reused():
    """A cache that starts with room for 8 positions and 1 slot: requests of 100 and 37 tokens in portions, two at a time."""
    cfg = CONFIGS["mixed"]
    W = to.random_weights(cfg, seed=2)
    m = _model(cfg, W, F32)
    a, b = _tokens(100, cfg["vocab"], 1), _tokens(37, cfg["vocab"], 2)
    want_a, want_b = to.forward(cfg, W, a), to.forward(cfg, W, b)
    cache = m.new_cache(n_slots=1)
    assert cache.has_per_position
    cache.positions = 8  # before the first alloc: the stores are built this small
    sa = cache.alloc()
    got_a = [m.engine.step(cache, [sa], [a[:5]], want=[list(range(5))])]
    assert cache.positions == 8
    sb = cache.alloc()
    lg = m.engine.step(cache, [sa, sb], [a[5:30], b[:20]], want=[list(range(25)), list(range(20))])
    got_a.append(lg[:25])
    got_b = [lg[25:]]
    assert cache.positions == 32 and cache.n_slots == 2
    for t in range(20, 37):
        lg = m.engine.step(cache, [sb, sa], [[b[t]], [a[30 + t - 20]]])
        got_b.append(lg[:1])
        got_a.append(lg[1:])
    cache.release(sb)
    got_a.append(m.engine.step(cache, [sa], [a[47:]], want=[list(range(53))]))
    assert cache.positions == 128
    assert _logit_err(torch.cat(got_a), want_a) < 1e-4 and _logit_err(torch.cat(got_b), want_b) < 1e-4
    sc = cache.alloc()  # the slot b left, with b's keys still in it
    assert sc == sb
    assert _logit_err(m.engine.step(cache, [sc], [b], want=[list(range(37))]), want_b) < 1e-4


@pytest.mark.parametrize("name", ["mixed", "odd_sizes"])
def test_first_tokens_of_a_sequence(name):
    """Position 0 alone, and every prompt length up to a little beyond the first block edges."""
    cfg = CONFIGS[name]
    W = to.random_weights(cfg, seed=6)
    m = _model(cfg, W, F32)
    toks = _tokens(12, cfg["vocab"], 6)
    want = to.forward(cfg, W, toks)
    cache = m.new_cache()
    for n in range(1, 13):
        s = cache.alloc()
        got = m.engine.step(cache, [s], [toks[:n]], want=[list(range(n))])
        assert _logit_err(got, want[:n]) < 1e-4, n
        cache.release(s)


def test_long_prompt_and_long_decoding():
    """520 tokens, the last 140 decoded one by one: block edges at multiples of 64, 100 and 33 fall into the prompt and into
    the decoded tokens, the tiled kernels see prompts longer than their tiles, the per-position stores grow twice."""
    cfg = CONFIGS["tiles"]
    W = to.random_weights(cfg, seed=7)
    toks = _tokens(520, cfg["vocab"], 7)
    want = to.forward(cfg, W, toks)
    for dtype in (F32, BF16):
        m = _model(cfg, W, dtype)
        cache = m.new_cache()
        s = cache.alloc()
        idx = [0, 1, 32, 33, 62, 63, 64, 65, 99, 100, 101, 127, 128, 299, 300, 379]
        out = [m.engine.step(cache, [s], [toks[:380]], want=[idx])]
        for t in range(380, 520):
            out.append(m.engine.step(cache, [s], [[toks[t]]]))
        assert cache.positions >= 520
        assert _logit_err(torch.cat(out), want[idx + list(range(380, 520))]) < _tol(dtype)


def _random_config(seed):
    """A configuration drawn at random: 2 to 5 layers of any kind in any order, widths and head sizes on and off the
    16-byte and tensor-core routes, key heads that divide the heads, blocks from 1 position to more than the sequence or no
    mask at all, rotation over the whole head or a part, with or without rescaled frequencies and soft cap."""
    import random

    r = random.Random(seed)
    layers = []
    for _ in range(r.randint(2, 5)):
        kind = r.choice(["attention", "attention_2", "latent_attention"])
        ff = r.choice([40, 64, 100]) if r.random() < 0.8 else None
        if kind == "latent_attention":
            layers.append(_lat(r.choice([1, 2, 3, 4, 8]), r.choice([6, 8, 16, 32]), r.choice([2, 4, 8, 16]), r.choice([8, 12, 24, 32]),
                               r.choice([12, 24, 48, 56]), r.choice([100.0, 3e4, 1e6]), mlp=ff))
            continue
        H = r.choice([1, 2, 4, 6, 8])
        G = r.choice([g for g in (1, 2, 3, 4, 6, 8) if H % g == 0])
        D = r.choice([8, 12, 16, 32, 64, 80])
        E = r.choice([D, D, 16, 24, 64])
        scaling = (r.choice([2.0, 4.0, 8.0]), 1.0, r.choice([2.0, 4.0]), r.choice([16, 64, 4096])) if r.random() < 0.5 else None
        rot = _rot(r.choice([100.0, 1e4, 3e5]), r.choice([D, D, D // 4 * 2, 4]), scaling)
        size = r.choice([None, 1, 3, 16, 50, 64, 65, 128, 1000])
        softcap = r.choice([5.0, 30.0]) if kind == "attention" and r.random() < 0.7 else None
        layers.append(_att(H, G, D, E, size, rot, softcap=softcap, scale=r.choice([None, 0.1, 0.3]), mlp=ff, kind=kind))
    return _cfg(layers, vocab=r.choice([37, 100, 256]), width=r.choice([48, 51, 64, 100, 136]), eps=r.choice([1e-5, 1e-6]),
                scale=r.choice([1.0, 8.0]))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed):
    """Each request alone in one step, as a prompt with its last tokens decoded, and three unequal requests together."""
    cfg = _random_config(seed)
    W = to.random_weights(cfg, seed=seed)
    reqs = [_tokens(n, cfg["vocab"], seed + n) for n in (5, 70, 150)]
    want = [to.forward(cfg, W, q) for q in reqs]
    for dtype in (F32, BF16):
        m = _model(cfg, W, dtype)
        if seed % 2:
            m.engine.max_positions = 200  # rings no longer than the request may grow
        cache = m.new_cache(n_slots=2)
        tol = 1e-4 if dtype == F32 else 0.1
        for q, w in zip(reqs, want):
            s = cache.alloc()
            assert _logit_err(m.engine.step(cache, [s], [q], want=[list(range(len(q)))]), w) < tol
            cache.release(s)
            cut = max(1, len(q) - 30)
            s = cache.alloc()
            out = [m.engine.step(cache, [s], [q[:cut]], want=[list(range(cut))])]
            out += [m.engine.step(cache, [s], [[t]]) for t in q[cut:]]
            cache.release(s)
            assert _logit_err(torch.cat(out), w) < tol
        slots = [cache.alloc() for _ in reqs]
        cuts = [max(1, len(q) - 4) for q in reqs]
        lg = m.engine.step(cache, slots, [q[:c] for q, c in zip(reqs, cuts)], want=[list(range(c)) for c in cuts])
        outs, at = [], 0
        for c in cuts:
            outs.append([lg[at:at + c]])
            at += c
        for k in range(4):
            lg = m.engine.step(cache, slots, [[q[c + k]] for q, c in zip(reqs, cuts)])
            for i in range(3):
                outs[i].append(lg[i:i + 1])
        for i in range(3):
            assert _logit_err(torch.cat(outs[i]), want[i]) < tol


def test_checkpoint_folder_registry_and_greedy_generation(tmp_path):
    """config.json + model.safetensors -> the registry picks the class; generate() and the scheduler reproduce the
    restatement's greedy continuation (fp32, so that the argmax is the restatement's)."""
    import json

    from llark_b200.models.registry import load_model
    from llark_b200.safetensors_io import save_file
    from llark_b200.scheduler import BatchScheduler, Request

    cfg = CONFIGS["mixed"]
    W = to.random_weights(cfg, seed=8)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(BF16) for k, v in W.items()}, str(tmp_path / "model.safetensors"))
    m = load_model(str(tmp_path), dtype=F32)
    assert type(m).__name__ == "TokatarForCausalLM"

    def oracle_greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(to.forward(cfg, W, seq)[-1].argmax()))
        return seq

    prompts = [_tokens(9, cfg["vocab"], 1), _tokens(9, cfg["vocab"], 2)]
    want = [oracle_greedy(p, 12) for p in prompts]
    out = m.generate(input_ids=torch.tensor(prompts, device="cuda:0"), max_new_tokens=12)
    assert out.tolist() == want
    reqs = [Request(prompt=prompts[0], max_new_tokens=12), Request(prompt=prompts[1][:4], max_new_tokens=5),
            Request(prompt=prompts[1], max_new_tokens=12, eos_token_id=[want[1][9 + 3]])]
    sched = BatchScheduler(m.engine, max_batch=2)
    for r in reqs:
        sched.submit(r)
    sched.run()
    assert reqs[0].output == want[0][9:]
    assert reqs[1].output == oracle_greedy(prompts[1][:4], 5)[4:]
    first_eos = want[1][9:].index(want[1][9 + 3])
    assert reqs[2].output == want[1][9:9 + first_eos + 1]
    assert all(r.finished for r in reqs) and not sched.cache.in_use()


def test_command_line_and_trace_runner(tmp_path, monkeypatch, capsys):
    """generate_cli (scheduler, greedy) and the trace runner (given tokens step by step: two requests start together with
    unequal prompts, decode together, one ends earlier, a third starts later in the slot that was given back)."""
    import io
    import json

    import numpy as np

    from llark_b200 import generate_cli, trace_runner
    from llark_b200.safetensors_io import save_file

    cfg = CONFIGS["odd_sizes"]
    W = to.random_weights(cfg, seed=9)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(BF16) for k, v in W.items()}, str(tmp_path / "model.safetensors"))
    V = cfg["vocab"]
    a, b, c = _tokens(40, V, 1), _tokens(9, V, 2), _tokens(21, V, 3)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]},
                                     {"id": "b", "tokens": b[:5], "want": []}], "end": []}]
    for k in range(4):
        steps.append({"step": 1 + k, "entries": [{"id": "a", "tokens": [a[30 + k]], "want": [0]},
                                                 {"id": "b", "tokens": [b[5 + k]], "want": [0]}],
                      "end": ["b"] if k == 3 else []})
    steps.append({"step": 5, "entries": [{"id": "c", "tokens": c, "want": [20]}], "end": ["c"]})
    steps.append({"step": 6, "entries": [{"id": "a", "tokens": a[34:], "want": [5]}], "end": ["a"]})
    out = tmp_path / "out"
    monkeypatch.setattr("sys.stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps)))
    assert trace_runner.main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(out), "--max-tokens", "80"]) == 0
    printed = capsys.readouterr().out.split("\n")
    assert [l for l in printed if l.startswith("done")] == ["done %d" % i for i in range(7)]
    la, lb, lc = to.forward(cfg, W, a), to.forward(cfg, W, b), to.forward(cfg, W, c)

    def rows(i):
        return torch.from_numpy(np.fromfile(out / ("%d.f32" % i), dtype="<f4").reshape(-1, V).copy())

    assert _logit_err(rows(0), la[[0, 29]]) < 1e-4
    for k in range(4):
        assert _logit_err(rows(1 + k), torch.stack([la[30 + k], lb[5 + k]])) < 1e-4
    assert _logit_err(rows(5), lc[[20]]) < 1e-4
    assert _logit_err(rows(6), la[[39]]) < 1e-4

    prompts = tmp_path / "p.jsonl"
    prompts.write_text(json.dumps({"id": "x", "tokens": a[:7], "max_new_tokens": 6}) + "\n" +
                       json.dumps({"tokens": b[:3]}) + "\n")
    assert generate_cli.main(["--model", str(tmp_path), "--prompts", str(prompts), "--dtype", "float32",
                              "--max-new-tokens", "4"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().split("\n")]

    def oracle_greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(to.forward(cfg, W, seq)[-1].argmax()))
        return seq[len(prompt):]

    assert lines == [{"id": "x", "tokens": oracle_greedy(a[:7], 6)}, {"id": "1", "tokens": oracle_greedy(b[:3], 4)}]
