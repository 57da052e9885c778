"""Gubulorn on the GPU against the plain restatement in tests/gubulorn_oracle.py (float64 on the CPU): every mechanism
alone through its op or its mixer class, then the whole model through the engine's step function, the slot cache, the
scheduler, generate() and the command-line tools. Configurations are small and deliberately unlike each other: key heads
shared by several heads or by none, key and value sizes that differ (scalar attention route) or agree at a multiple of 16
(tensor-core route), state-space groups and norm parts of 1 and more, 1 to 5 convolution taps, routers with and without
pass-through experts, with one group or several, layers without a feed-forward, either mixer first or last."""
import math

import pytest
import torch

import gubulorn_oracle as go

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


def _logit_err(got, want, worst=1.0):
    """Difference of logits with the mean over the vocabulary taken off, rms, relative to the rms of the expected ones:
    the largest over the positions, or (worst < 1) the value that this share of the positions stays under. The bfloat16
    comparisons allow a tenth of the positions to be off: a router whose choice scores nearly tie may pick the other
    expert once its input is rounded, which the 32-bit comparisons (every position) do not suffer from."""
    d = got.double().cpu() - want.double().cpu()
    d = d - d.mean(dim=-1, keepdim=True)
    w = want.double().cpu()
    w = w - w.mean(dim=-1, keepdim=True)
    e = d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()
    return e.max().item() if worst >= 1.0 else torch.quantile(e, worst).item()


def _share(dtype):
    return 1.0 if dtype == F32 else 0.9


# ------------------------------------------------------------------------------------------------ configurations
def _moe(experts, identity, top, groups, keep, ff):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _delta(heads, kv, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mlp": mlp, "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def _left(heads, kv, dim, vdim, every, coef=0.4, scale=None):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale or 1.0 / math.sqrt(dim),
            "q_temp": {"coef": coef, "every": every}}


def _right(heads, vdim, state, groups, norm_groups, conv):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def _par(left, right, mlp=None):
    return {"type": "parallel", "mlp": mlp, "mixer": {"left": left, "right": right}}


def _cfg(layers, vocab=97, width=72, eps=1e-5, alpha=2.0, logit_scale=0.5, softcap=20.0):
    return {"architecture": "Gubulorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha,
            "logit_scale": logit_scale, "logit_softcap": softcap, "layers": layers}


CONFIGS = {
    # every size differs from every other; attention on the tensor-core route (dim = vdim = 16) with key heads shared by
    # two; temperature steps every 7 positions; router with three groups of which two are kept and one pass-through expert;
    # the last layer has no feed-forward
    "mixed": _cfg([_par(_left(4, 2, 16, 16, 7), _right(3, 10, 12, 1, 3, 2), mlp=_moe(5, 1, 2, 3, 2, 20)),
                   _delta(4, 2, 8, 12, 3, mlp=_dense(40, 1.0)),
                   _par(_left(3, 3, 10, 6, 5, coef=1.0), _right(4, 6, 8, 2, 1, 4), mlp=_moe(4, 0, 1, 1, 1, 9)),
                   _delta(2, 1, 20, 6, 2)]),
    # delta first and last, nothing a multiple of 4 (scalar routes everywhere), five taps and one tap (no convolution),
    # one key / value head for all query heads, as many norm parts as heads, two pass-through experts of four outputs,
    # a soft cap that bites
    "odd_sizes": _cfg([_delta(3, 1, 10, 7, 5, mlp=_moe(2, 2, 2, 2, 2, 11)),
                       _par(_left(3, 1, 6, 5, 3), _right(3, 5, 9, 3, 3, 1), mlp=_dense(23, 0.5)),
                       _delta(3, 3, 6, 10, 1, mlp=_moe(5, 1, 3, 6, 4, 7))],
                      vocab=33, width=51, eps=1e-3, alpha=1.0, logit_scale=2.0, softcap=3.0),
    # wide heads (state rows split over several lanes), a state size of 128, attention head size 32 on the tensor-core
    # route with a temperature step at 64 (the key tile's edge), no soft cap
    "wide_heads": _cfg([_par(_left(2, 1, 32, 32, 64), _right(2, 24, 128, 1, 2, 3), mlp=_moe(6, 2, 4, 4, 3, 24)),
                        _delta(2, 1, 144, 40, 4, mlp=_dense(64, 4.0))],
                       vocab=50, width=80, alpha=4.0, softcap=None),
}


def _model(cfg, W, dtype):
    from llark_b200.models.gubulorn import GubulornConfig, GubulornForCausalLM

    return GubulornForCausalLM(GubulornConfig.from_dict(cfg), W, device="cuda:0", dtype=dtype)


def _tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class _Stores:
    """Stand-in cache for a mixer used alone: slot stores filled with garbage except where alloc() would zero them."""

    def __init__(self, n_slots=4, positions=512):
        self.t, self.n, self.positions = [], n_slots, positions

    def add_store(self, shape, dtype, zero_on_alloc, per_position=False):
        fill = 0.0 if zero_on_alloc else float("nan")
        lead = (self.positions,) if per_position else ()
        self.t.append(torch.full((self.n,) + lead + tuple(shape), fill, device=_dev(), dtype=dtype))
        return len(self.t) - 1

    def view(self, h):
        return self.t[h]


def _run_mixer(cls, W, spec, width, h, portions, act, eps=1e-5, slot=2):
    """h [T, width] through mixer `cls` cut into `portions` (one request in `slot`)."""
    weights = cls.Weights({k: v.to(F32) for k, v in W.items()}, "m.", spec, width, _dev(), act)
    stores = _Stores()
    mixer = cls(weights, stores, eps, act, None)
    outs, at = [], 0
    for n in portions:
        st = _layout([n], [at], [slot])
        outs.append(mixer.forward(h[at:at + n].to(_dev(), act).contiguous(), st, stores).cpu())
        at += n
    assert at == h.shape[0]
    return torch.cat(outs)


def _mixer_weights(cfg_layer, width, seed):
    """The tensors of one layer's mixer from the random checkpoint maker, under the prefix 'm.'."""
    cfg = _cfg([cfg_layer], width=width)
    W = go.random_weights(cfg, seed=seed)
    return {"m." + k[len("l0.mix."):]: v for k, v in W.items() if k.startswith("l0.mix.")}


PORTIONS = ([67], [1] * 67, [40] + [1] * 27, [5, 2, 2, 31, 1, 1, 2, 23])


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("C", [51, 72, 1024])
def test_norm_after_the_sum(C):
    """alpha x + half the sum of two normed branches + chosen experts, one of which hands x through; then the norm."""
    from llark_b200 import ops

    g = torch.Generator().manual_seed(C)
    T, top, n_real = 9, 3, 4
    x, y1, y2 = (torch.randn(T, C, generator=g, dtype=F64) for _ in range(3))
    w, w1, w2 = (1.0 + 0.2 * torch.randn(C, generator=g, dtype=F64) for _ in range(3))
    z = torch.randn(T * top, C, generator=g, dtype=F64)
    pos_of = torch.randperm(T * top, generator=g).reshape(T, top)
    wts = torch.rand(T, top, generator=g, dtype=F64)
    ids = torch.randint(0, n_real + 2, (T, top), generator=g)
    eps, alpha = 1e-4, 3.0
    f = 0.5 * (go.rms(y1, eps) * w1 + go.rms(y2, eps) * w2)
    for t in range(T):
        for k in range(top):
            f[t] += wts[t, k] * (x[t] if ids[t, k] >= n_real else z[pos_of[t, k]])
    want = go.rms(alpha * x + f, eps) * w
    d = lambda t, dt=F32: t.to(_dev(), dt).contiguous()
    got, got16 = ops.seq_post_norm(d(x), alpha, d(w), eps, y1=d(y1), w1=d(w1), y2=d(y2), w2=d(w2), branch_scale=0.5,
                                   z=d(z), pos_of=d(pos_of, torch.int32), wts=d(wts), ids=d(ids, torch.int32),
                                   n_real=n_real, act=BF16)
    assert _rel(got, want) < 2e-6 and got16.dtype == BF16 and _rel(got16, want) < 4e-3
    plain = ops.seq_post_norm(d(x), alpha, d(w), eps, y1=d(y1))
    assert _rel(plain, go.rms(alpha * x + y1, eps) * w) < 2e-6
    assert _rel(ops.seq_post_norm(d(x), 1.0, d(w), eps), go.rms(x, eps) * w) < 2e-6


def test_clamped_gated_unit_and_logit_cap():
    from llark_b200 import ops

    g = torch.Generator().manual_seed(0)
    gu = torch.randn(7, 2 * 13, generator=g, dtype=F64) * 3.0
    lim = 1.5
    a, u = torch.clamp(gu[:, :13], max=lim), torch.clamp(gu[:, 13:], -lim, lim)
    want = a * torch.sigmoid(1.702 * a) * (u + 1.0)
    assert (a == lim).any() and (u == -lim).any() and (u == lim).any() and (gu[:, :13] < -lim).any()
    assert _rel(ops.seq_glu_clamped(gu.to(_dev(), F32), lim), want) < 1e-6
    z = torch.randn(5, 11, generator=g, dtype=F64) * 40.0
    got = ops.seq_logit_cap_(z.to(_dev(), F32).clone(), 0.25, 6.0)
    assert _rel(got, 6.0 * torch.tanh(z * 0.25 / 6.0)) < 1e-6
    assert _rel(ops.seq_logit_cap_(z.to(_dev(), F32).clone(), 0.25, None), z * 0.25) < 1e-7


@pytest.mark.parametrize("n,top,groups,keep", [(16, 4, 4, 3), (6, 2, 3, 2), (5, 3, 1, 1), (12, 1, 6, 1), (40, 8, 5, 2)])
def test_router_chooses_on_corrected_scores_and_weighs_with_plain_ones(n, top, groups, keep):
    """Corrections around -0.3 make most choice scores negative: a group that is shut out must count as minus infinity,
    not as zero, or it would win."""
    from llark_b200 import ops

    g = torch.Generator().manual_seed(n)
    z = torch.randn(300, n, generator=g, dtype=F64) * 2.0
    corr = (-0.3 + 0.2 * torch.randn(n, generator=g, dtype=F64)).to(BF16).to(F64)
    ids, wts = go.route(z.to(F32).to(F64), corr, top, groups, keep)
    got_ids, got_w = ops.seq_moe_route(z.to(_dev(), F32), groups, keep, top, 1.0, softmax_bias=True,
                                       correction=corr.to(_dev(), F32))
    assert (go.route(z, corr, top, groups, keep)[1] + corr[ids]).min() < 0  # negative choice scores do occur
    same = (got_ids.cpu().long() == ids).all(dim=1)
    assert same.float().mean() > 0.99  # a near tie may fall the other way in 32-bit
    assert _rel(got_w.cpu()[same], wts[same]) < 1e-5
    assert (wts.sum(dim=1) < 0.999).any()  # not renormalised


@pytest.mark.parametrize("dtype,n_tok", [(F32, 50), (BF16, 50), (F32, 3), (BF16, 1)])
def test_experts_with_pass_through(dtype, n_tok):
    from llark_b200.mixers import FEED_FORWARDS

    C = 40
    mlp = _moe(5, 3, 3, 4, 3, 12)
    cfg = _cfg([_delta(1, 1, 4, 4, 1, mlp=mlp)], width=C)
    W = go.random_weights(cfg, seed=5)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(n_tok, C, generator=g, dtype=F64).to(BF16).to(F64)
    wn = 1.0 + W["l0.norm2"]
    want = go.rms(2.0 * x + go.moe(x, W, "l0.mlp.", mlp), 1e-5) * wn
    ids = go.route(x @ W["l0.mlp.router"].T, W["l0.mlp.correction"], 3, 4, 3)[0]
    if n_tok > 10:
        assert (ids >= 5).any() and (ids < 5).any()
    ff_cls = FEED_FORWARDS["moe_softmax_bias"]
    ff = ff_cls(ff_cls.Weights({k: v.to(F32) for k, v in W.items()}, "l0.mlp.", mlp, C, _dev(), dtype), dtype)
    got, got_act = ff.post_norm(x.to(_dev(), F32), x.to(_dev(), dtype), 2.0, wn.to(_dev(), F32), 1e-5, dtype)
    assert got_act.dtype == dtype
    assert _rel(got, want) < (1e-5 if dtype == F32 else 2e-2)


@pytest.mark.parametrize("taps,bias", [(1, True), (2, False), (3, True), (4, True), (5, True)])
def test_conv_with_bias_carries_its_inputs_across_steps(taps, bias):
    from llark_b200 import ops

    g = torch.Generator().manual_seed(taps)
    n_ch, T = 37, 90
    src = torch.randn(T, n_ch + 6, generator=g, dtype=F64)
    w = torch.randn(n_ch, taps, generator=g, dtype=F64)
    b = torch.randn(n_ch, generator=g, dtype=F64) if bias else None
    want = go.silu(go.causal_conv(src[:, 3:3 + n_ch], w, b))
    for portions in ([90], [1] * 90, [2, 70, 1, 1, 3, 13]):
        carry = torch.zeros(3, max(taps - 1, 1), n_ch, device=_dev(), dtype=F32)
        out, at = [], 0
        for n in portions:
            s = src[at:at + n].to(_dev(), F32).contiguous()
            out.append(ops.seq_conv_act(s[:, 3:3 + n_ch], w.to(_dev(), F32), carry, _layout([n], [at], [1]), silu=True,
                                        bias=b.to(_dev(), F32) if bias else None))
            at += n
        assert _rel(torch.cat(out), want) < 2e-6, portions


@pytest.mark.parametrize("H,G,D,E,conv", [(4, 2, 8, 12, 3), (3, 1, 10, 7, 5), (2, 2, 144, 40, 2), (1, 1, 64, 64, 4)])
def test_delta_mixer(H, G, D, E, conv):
    from llark_b200.mixers import MIXERS

    layer = _delta(H, G, D, E, conv)
    C = 56
    W = _mixer_weights(layer, C, seed=H + D)
    h = torch.randn(67, C, generator=torch.Generator().manual_seed(2), dtype=F64).to(BF16).to(F64)
    want = go.delta_mixer(h, W, "m.", layer["mixer"], 1e-5)
    for portions in PORTIONS:
        assert _rel(_run_mixer(MIXERS["delta"], W, layer["mixer"], C, h, portions, F32), want) < 2e-5, portions
    assert _rel(_run_mixer(MIXERS["delta"], W, layer["mixer"], C, h, PORTIONS[3], BF16), want) < 2e-2


@pytest.mark.parametrize("H,E,N,G,NG,conv", [(3, 10, 12, 1, 3, 2), (4, 6, 8, 2, 1, 4), (3, 5, 9, 3, 3, 1), (2, 24, 128, 1, 2, 3),
                                             (6, 16, 32, 2, 4, 5)])
def test_state_space_mixer(H, E, N, G, NG, conv):
    from llark_b200.mixers import MIXERS

    layer = _par(_left(1, 1, 4, 4, 3), _right(H, E, N, G, NG, conv))
    C = 56
    W = {k.replace("m.right.", "m."): v for k, v in _mixer_weights(layer, C, seed=H + N).items() if ".right." in k}
    h = torch.randn(67, C, generator=torch.Generator().manual_seed(3), dtype=F64).to(BF16).to(F64)
    want = go.state_space_mixer(h, W, "m.", layer["mixer"]["right"], 1e-5)
    for portions in PORTIONS:
        assert _rel(_run_mixer(MIXERS["ssd"], W, layer["mixer"]["right"], C, h, portions, F32), want) < 2e-5, portions
    assert _rel(_run_mixer(MIXERS["ssd"], W, layer["mixer"]["right"], C, h, PORTIONS[3], BF16), want) < 2e-2


@pytest.mark.parametrize("H,G,D,E,every", [(4, 2, 16, 16, 7), (3, 1, 6, 5, 3), (2, 2, 32, 32, 64), (3, 3, 10, 6, 1), (2, 1, 64, 48, 32)])
def test_sink_attention_mixer(H, G, D, E, every):
    from llark_b200.mixers import MIXERS

    layer = _par(_left(H, G, D, E, every, coef=0.8), _right(1, 4, 4, 1, 1, 2))
    C, T = 56, 150
    W = {k.replace("m.left.", "m."): v for k, v in _mixer_weights(layer, C, seed=H + D).items() if ".left." in k}
    h = torch.randn(T, C, generator=torch.Generator().manual_seed(4), dtype=F64).to(BF16).to(F64)
    want = go.sink_attention(h, W, "m.", layer["mixer"]["left"], 1e-5)
    for portions in ([150], [1] * 150, [100] + [1] * 50, [31, 2, 2, 65, 1, 1, 30, 18]):
        assert _rel(_run_mixer(MIXERS["sink_attention"], W, layer["mixer"]["left"], C, h, portions, F32), want) < 2e-5
    for portions in ([150], [31, 2, 2, 65, 1, 1, 30, 18]):  # bfloat16: the tensor-core kernel where the sizes allow it
        assert _rel(_run_mixer(MIXERS["sink_attention"], W, layer["mixer"]["left"], C, h, portions, BF16), want) < 2e-2


def _needle(T, H, G, D, E, far, sink, seed):
    """Projections that ARE the input (identity weights): queries and keys are random directions except that the last
    query of every head points along the key at position `far`; that key's value stands out. With a score scale of 3 the
    aligned pair's score is about 3 D, every other about +-3 sqrt(D): the far key takes nearly all of the softmax, unless
    the sink (when it is large) takes it."""
    g = torch.Generator().manual_seed(seed)
    C = H * D + G * D + G * E + H
    h = torch.randn(T, C, generator=g, dtype=F64)
    k_off, v_off = H * D, (H + G) * D
    for hd in range(H):
        kv = hd // (H // G)
        h[T - 1, hd * D:(hd + 1) * D] = h[far, k_off + kv * D:k_off + (kv + 1) * D]
    h[far, v_off:v_off + G * E] = 50.0 + torch.arange(G * E, dtype=F64)
    h[:, v_off + G * E:] = 4.0  # gates wide open
    eye = torch.eye(C, dtype=F64)
    W = {"m.q": eye[:k_off], "m.k": eye[k_off:v_off], "m.v": eye[v_off:v_off + G * E], "m.g": eye[v_off + G * E:],
         "m.q.norm": torch.ones(D, dtype=F64), "m.k.norm": torch.ones(D, dtype=F64),
         "m.sink": torch.full((H,), float(sink), dtype=F64), "m.o": eye[:, :H * E].clone()}
    spec = {"heads": H, "kv_heads": G, "dim": D, "vdim": E, "scale": 3.0, "q_temp": {"coef": 0.0, "every": 1}}
    return h.to(BF16).to(F64), W, spec, C


@pytest.mark.parametrize("far", [0, 1, 31, 32, 63, 64, 255, 256, 300])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_attention_reaches_a_key_far_back_in_prompts_and_in_decoding(far, dtype):
    """The key sits at the start, next to a key tile's edge (32 for the scalar kernel, 64 for the tensor-core kernel) or at
    the edge of the per-position store's first 256 entries; the query comes 350 or more tokens later."""
    from llark_b200.mixers import MIXERS

    T, H, G, D, E = 400, 2, 1, 16, 16
    h, W, spec, C = _needle(T, H, G, D, E, far, sink=-2.0, seed=far)
    want = go.sink_attention(h, W, "m.", spec, 1e-5)
    assert want[T - 1].abs().max() > 40.0  # the read-out is the needle's value
    tol = 1e-4 if dtype == F32 else 2e-2
    for portions in ([400], [399, 1], [256, 100, 43, 1], [200] + [1] * 200):
        got = _run_mixer(MIXERS["sink_attention"], W, spec, C, h, portions, dtype)
        assert _rel(got[T - 1], want[T - 1]) < tol, portions
        assert _rel(got, want) < (1e-4 if dtype == F32 else 3e-2), portions


def test_a_large_sink_takes_the_weight_of_every_key():
    from llark_b200.mixers import MIXERS

    T, H, G, D, E = 80, 2, 2, 16, 16
    for dtype in (F32, BF16):
        for sink in (60.0, 200.0):  # about the needle's score; far beyond every score
            h, W, spec, C = _needle(T, H, G, D, E, 5, sink=sink, seed=1)
            want = go.sink_attention(h, W, "m.", spec, 1e-5)
            for portions in ([80], [79, 1]):
                got = _run_mixer(MIXERS["sink_attention"], W, spec, C, h, portions, dtype)
                assert torch.isfinite(got).all()
                assert (got.double() - want).abs().max() < (1e-3 if dtype == F32 else 0.5) * max(want.abs().max(), 1.0)
        assert want.abs().max() < 1e-6  # sink 200: every output is all but zero


@pytest.mark.parametrize("portions", [[300], [1] * 300, [250] + [1] * 50])
def test_recurrent_states_keep_a_value_for_hundreds_of_steps(portions):
    """A write at the start, then decays of almost one: the read-out at the end is the value written 298 steps earlier.
    Through the delta scan with the correction (one decay per head) and without it (state-space rule)."""
    from llark_b200 import ops

    T, H, D, E = 300, 2, 8, 6
    g = torch.Generator().manual_seed(0)
    key = torch.zeros(T, H, D, dtype=F64)
    key[:, :, 1] = 1.0           # later tokens write and read along another direction
    key[1, :, 0], key[1, :, 1] = 1.0, 0.0
    q = key.clone()
    q[T - 1, :, 0], q[T - 1, :, 1] = 1.0, 0.0
    v = torch.randn(T, H, E, generator=g, dtype=F64)
    dec = torch.full((T, H), -12.0, dtype=F64)      # softplus ~ 6e-6: decay 0.999994 per step
    beta = torch.full((T, H), 8.0, dtype=F64)       # sigmoid ~ 1
    zeros = torch.zeros(H, dtype=F64)
    d = lambda t: t.to(_dev(), F32).contiguous()
    for rule, correct in ((ops.DELTA_GATED_SCALAR, True), (ops.DELTA_STATE_SPACE, False)):
        state = torch.zeros(3, H, D, E, device=_dev(), dtype=F32)
        out, at = [], 0
        for n in portions:
            sl = slice(at, at + n)
            vec = ops.seq_delta_prep(rule, d(q[sl].reshape(n, H * D)), d(key[sl].reshape(n, H * D)), d(dec[sl]),
                                     d(beta[sl]), H, H, D, dec_bias=d(zeros), rate_log=d(zeros))
            out.append(ops.seq_delta_scan(vec, d(v[sl].reshape(n, H * E)), state, _layout([n], [at], [1]), H, D, E,
                                          correct=correct))
            at += n
        last = torch.cat(out)[T - 1].double().cpu().reshape(H, E)
        if correct:  # unit keys: the state along direction 0 holds beta * v_1 / sqrt(D) for q scaled by 1 / sqrt(D)
            want = v[1] * torch.sigmoid(torch.tensor(8.0, dtype=F64)) / math.sqrt(D)
        else:        # state-space rule: dt * v_1 with dt = softplus(-12)
            want = v[1] * math.log1p(math.exp(-12.0))
        assert ((last - want).norm() / want.norm()).item() < 5e-3, rule


def test_per_position_stores_grow_and_slots_are_reused():
    """A cache that starts with room for 8 positions and 1 slot: requests of 100 tokens in portions, two at a time."""
    cfg = CONFIGS["mixed"]
    W = go.random_weights(cfg, seed=2)
    m = _model(cfg, W, F32)
    from llark_b200.state_cache import StateCache

    a, b = _tokens(100, cfg["vocab"], 1), _tokens(37, cfg["vocab"], 2)
    want_a, want_b = go.forward(cfg, W, a), go.forward(cfg, W, b)
    cache = m.new_cache(n_slots=1)
    assert isinstance(cache, StateCache) and cache.has_per_position
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
    sc = cache.alloc()  # the slot b left, with b's keys and states still in it
    assert sc == sb
    assert _logit_err(m.engine.step(cache, [sc], [b], want=[list(range(37))]), want_b) < 1e-4


# ------------------------------------------------------------------------------------------------ whole model
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_every_layer(name):
    cfg = CONFIGS[name]
    W = go.random_weights(cfg, seed=1)
    toks = _tokens(75, cfg["vocab"], 1)
    want, want_layers = go.forward(cfg, W, toks, return_residuals=True)
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
    assert _logit_err(got16, want, 0.9) < 8e-2


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_prefill_portions_and_decoding_agree(name, dtype):
    """The same 90 tokens: in one step; as a prompt and then token by token; token by token from the start; in portions
    of 7, 2, 2, 30, 1, 1, 2, ..."""
    cfg = CONFIGS[name]
    W = go.random_weights(cfg, seed=3)
    toks = _tokens(90, cfg["vocab"], 2)
    m = _model(cfg, W, dtype)
    want = go.forward(cfg, W, toks)

    def run(portions):
        cache = m.new_cache()
        s = cache.alloc()
        out, at = [], 0
        for n in portions:
            out.append(m.engine.step(cache, [s], [toks[at:at + n]], want=[list(range(n))]))
            at += n
        assert at == 90 and cache.length[s] == 90
        return torch.cat(out)

    tol = 1e-4 if dtype == F32 else 8e-2
    whole = run([90])
    assert _logit_err(whole, want, _share(dtype)) < tol
    for portions in ([30] + [1] * 60, [1] * 90, [7, 2, 2, 30, 1, 1, 2, 3, 2, 40]):
        got = run(portions)
        assert _logit_err(got, want, _share(dtype)) < tol
        assert _logit_err(got, whole, _share(dtype)) < (1e-4 if dtype == F32 else 8e-2)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_unequal_batch_equals_each_request_alone_and_slots_are_reused(dtype):
    cfg = CONFIGS["mixed"]
    W = go.random_weights(cfg, seed=4)
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
        assert _logit_err(torch.cat(got[i]), ref[i], _share(dtype)) < (1e-4 if dtype == F32 else 8e-2), i
    want0 = go.forward(cfg, W, prompts[3] + tails[3][:4])
    assert _logit_err(ref[3], want0, _share(dtype)) < (1e-4 if dtype == F32 else 8e-2)
    assert not cache.in_use()


@pytest.mark.parametrize("name", ["mixed", "odd_sizes"])
def test_first_tokens_of_a_sequence(name):
    """Position 0 alone, and every prompt length up to a little beyond the taps and the first temperature steps."""
    cfg = CONFIGS[name]
    W = go.random_weights(cfg, seed=6)
    m = _model(cfg, W, F32)
    toks = _tokens(12, cfg["vocab"], 6)
    want = go.forward(cfg, W, toks)
    cache = m.new_cache()
    for n in range(1, 13):
        s = cache.alloc()
        got = m.engine.step(cache, [s], [toks[:n]], want=[list(range(n))])
        assert _logit_err(got, want[:n]) < 1e-4, n
        cache.release(s)


def test_long_prompt_and_long_decoding():
    """520 tokens, the last 140 decoded one by one: the temperature steps at 64, 128, ... fall into the prompt and into the
    decoded tokens, the recurrent states run for hundreds of steps, the tiled kernels see prompts longer than their tiles,
    the per-position stores grow twice."""
    cfg = CONFIGS["wide_heads"]
    W = go.random_weights(cfg, seed=7)
    toks = _tokens(520, cfg["vocab"], 7)
    want = go.forward(cfg, W, toks)
    for dtype, tol in ((F32, 1e-4), (BF16, 8e-2)):
        m = _model(cfg, W, dtype)
        cache = m.new_cache()
        s = cache.alloc()
        idx = [0, 1, 62, 63, 64, 65, 126, 127, 128, 300, 379]
        out = [m.engine.step(cache, [s], [toks[:380]], want=[idx])]
        for t in range(380, 520):
            out.append(m.engine.step(cache, [s], [[toks[t]]]))
        assert cache.positions >= 520
        assert _logit_err(torch.cat(out), want[idx + list(range(380, 520))], _share(dtype)) < tol


def test_checkpoint_folder_registry_and_greedy_generation(tmp_path):
    """config.json + model.safetensors -> the registry picks the class; generate() and the scheduler reproduce the
    restatement's greedy continuation (fp32, so that the argmax is the restatement's)."""
    import json

    from llark_b200.models.registry import load_model
    from llark_b200.safetensors_io import save_file
    from llark_b200.scheduler import BatchScheduler, Request

    cfg = CONFIGS["mixed"]
    W = go.random_weights(cfg, seed=8)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(BF16) for k, v in W.items()}, str(tmp_path / "model.safetensors"))
    m = load_model(str(tmp_path), dtype=F32)
    assert type(m).__name__ == "GubulornForCausalLM"

    def oracle_greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(go.forward(cfg, W, seq)[-1].argmax()))
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
    W = go.random_weights(cfg, seed=9)
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
    la, lb, lc = go.forward(cfg, W, a), go.forward(cfg, W, b), go.forward(cfg, W, c)

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
            seq.append(int(go.forward(cfg, W, seq)[-1].argmax()))
        return seq[len(prompt):]

    assert lines == [{"id": "x", "tokens": oracle_greedy(a[:7], 6)}, {"id": "1", "tokens": oracle_greedy(b[:3], 4)}]
