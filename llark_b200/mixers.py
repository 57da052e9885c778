"""Sequence mixers and feed-forwards of layer-list decoders on the generation path, by the `type` / `kind` names a
model's configuration uses. Each class packs its weights once (projections that read the same input become ONE matrix,
as the Llama path fuses q|k|v and gate|up), registers its per-request stores with the StateCache, and runs one packed
step through the C-ABI ops. Weights and state are separate objects: a layer that reuses another layer's weights gets
the same packed weights and stores of its own.

    "attention"  GatedWindowAttention   sliding-window softmax attention, per-head RMS norm of q and k, values = the
                                        un-normed keys, per-head temperature, sigmoid output gate
    "hgrn2"      GatedLinearRecurrence  HGRN2: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T silu(q)_t, forget
                                        gate with a learned lower bound, per-head RMS norm of o
    "dense"      ReluSquaredFF          down(relu(up x)^2)
    "latent_attention"  LatentWindowAttention   keys and values of all heads expanded from one low-rank latent per token plus
                                        one rotated key part shared by the heads (interleaved rotary pairs, optional
                                        YaRN blend of the frequencies); only the latent and that part are cached, the
                                        expansions are folded into the query and the output; sliding window, sigmoid gate
    "channel_delta"     GatedDeltaRule  S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q with a decay per head and
                                        key channel, unit q / k behind a short convolution + SiLU, gated per-head RMS norm
    "general_delta"     GeneralizedDeltaRule    S <- diag(w) S - (a u)(u^T S) + k v^T, u the unit key; o = S^T r
    "moe"        RoutedExperts          sigmoid router, group-limited top-k, weighted sum of small SwiGLU experts
    "delta"      ScalarGatedDeltaRule   the gated delta rule with ONE decay per head and a SiLU output gate
    "sink_attention"  SinkAttention     causal softmax attention over everything before (or a window), grouped key / value
                                        heads, per-head RMS norm of q and k, no rotation, a query temperature that grows
                                        with the position, a learned sink term in every softmax denominator, one sigmoid
                                        gate per head; keys and values live in per-position stores that grow
    "ssd"        StateSpaceDuality      Mamba-2: S <- exp(-exp(A) dt) S + dt B x^T, y = S^T C + D x behind a short
                                        convolution of x | B | C, SiLU gate in front of a grouped RMS norm
    "parallel"   ParallelMixers         a sink_attention ("left") and an ssd ("right") side by side on the same input,
                                        one fused input projection; the layer takes half the sum of their RMS-normed outputs
    "clamped_glu"  ClampedGluFF         down(min(g, l) * sigmoid(1.702 min(g, l)) * (clamp(u, -l, l) + 1))
    "moe_softmax_bias"  BiasedSoftmaxExperts  softmax router whose choice is made on score + a stored correction (groups
                                        ranked by their best), weights = plain scores, and trailing experts without
                                        weights that hand their input through

    "rotary_attention"  RotaryAttention   grouped-query softmax attention with rotary positions on q and k (halves or
                                        interleaved pairs, part of the head, optionally rescaled frequencies), optional
                                        soft cap of the scores, a mask by blocks of positions (or a window, or none: the
                                        keys then live in per-position stores), element-wise sigmoid gate
    "rotary_attention_vrot"  ValueRotaryAttention   the same with biased projections, an RMS norm over the WHOLE q and k
                                        projections, interleaved pairs, values that are stored rotated by their own position
                                        (the head outputs are turned back by the query's) and a 1 in every softmax denominator
    "latent_attention_causal"  LatentCausalAttention   latent attention over everything before (per-position store), rotary
                                        halves, one gate per head

Mixers that take `side=(matrix name, bias name)` compute that projection of their input inside their fused input GEMM and
leave it in `self.side` (fp32 view) after forward(): a layer's gate on the sublayer's result reads the same input.

A mixer's `branches(x_act, st, cache)` returns ([(output fp32, norm weight or None), ...], scale): what the layer's residual
kernel adds up (each output first RMS-normed with its weight when there is one). The default is the one output of forward().
"""
import math

import torch

from . import ops

F32 = torch.float32


def _vec(w, name, dev):
    return w[name].to(device=dev, dtype=F32).contiguous()


def _mat(w, name, dev, act):
    return w[name].to(device=dev, dtype=act).contiguous()


def _pad_rows(m, multiple=8):
    """Zero rows up to a multiple: keeps fused projections of odd total width on the tensor-core path (16-byte rows)."""
    pad = (-m.shape[0]) % multiple
    if not pad:
        return m.contiguous()
    return torch.cat([m, torch.zeros((pad, m.shape[1]), device=m.device, dtype=m.dtype)]).contiguous()


class _OneBranch:
    def branches(self, x_act, st, cache):
        return [(self.forward(x_act, st, cache), None)], 1.0


class GatedWindowAttentionWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        H, D = int(spec["heads"]), int(spec["dim"])
        G = int(spec.get("kv_heads", H))
        if H % G:
            raise ValueError("heads must be a multiple of kv_heads")
        if int(spec.get("vdim", D)) != D:
            raise ValueError("the values of this mixer are its keys: vdim must equal dim")
        self.H, self.G, self.D = H, G, D
        self.window = int(spec["mask"]["size"])
        # one projection for q | k | gate; the gate has no bias
        self.w_qkg = torch.cat([_mat(w, pfx + "q", dev, act), _mat(w, pfx + "k", dev, act), _mat(w, pfx + "g", dev, act)])
        self.b_qkg = torch.cat([_vec(w, pfx + "q.b", dev), _vec(w, pfx + "k.b", dev),
                                torch.zeros(H * D, device=dev, dtype=F32)])
        self.q_off, self.k_off, self.g_off = 0, H * D, (H + G) * D
        self.q_norm, self.k_norm = _vec(w, pfx + "q.norm", dev), _vec(w, pfx + "k.norm", dev)
        self.scale_h = (float(spec["scale"]) * _vec(w, pfx + "temp", dev)).contiguous()  # score scale per head
        self.w_o = _mat(w, pfx + "o", dev, act)
        for t, shape in ((self.w_qkg, ((2 * H + G) * D, width)), (self.w_o, (width, H * D)), (self.q_norm, (D,)),
                         (self.k_norm, (D,)), (self.scale_h, (H,))):
            if tuple(t.shape) != shape:
                raise ValueError(f"{pfx}: tensor of shape {tuple(t.shape)}, expected {shape}")


class GatedWindowAttention:
    Weights = GatedWindowAttentionWeights

    def __init__(self, weights, cache, eps, act, max_positions):
        self.w, self.eps, self.act = weights, float(eps), act
        w = weights
        self.cap = max(1, min(w.window, int(max_positions)))  # ring entries per request
        self.h_k = cache.add_store((self.cap, w.G * w.D), act, zero_on_alloc=False)
        self.h_v = cache.add_store((self.cap, w.G * w.D), act, zero_on_alloc=False)

    def forward(self, hc, st, cache):
        w = self.w
        kring, vring = cache.view(self.h_k), cache.view(self.h_v)
        qkg = ops.linear(hc, w.w_qkg, bias=w.b_qkg, out_dtype=F32)
        single = st.max_len == 1
        qn, kn, vr = ops.seq_qk_headnorm(qkg, w.q_off, w.k_off, w.q_norm, w.k_norm, w.H, w.G, w.D, self.eps, self.act,
                                         st=st, kring=kring if single else None, vring=vring if single else None,
                                         cap=self.cap)
        gate = qkg[:, w.g_off:]
        o = ops.seq_swa_attn(qn, kn, vr, kring, vring, gate, qkg.stride(0), w.scale_h, st, w.H, w.G, w.D, w.D,
                             w.window, self.cap, from_ring_only=single)
        if not single:
            ops.seq_kv_ring_write(kn, vr, kring, vring, st, self.cap)
        return ops.linear(o, w.w_o, out_dtype=F32)


class GatedLinearRecurrenceWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        H, D = int(spec["heads"]), int(spec["dim"])
        E = int(spec.get("vdim", D))
        self.H, self.D, self.E = H, D, E
        self.w_qfv = torch.cat([_mat(w, pfx + "q", dev, act), _mat(w, pfx + "f", dev, act), _mat(w, pfx + "v", dev, act)])
        self.b_qfv = torch.cat([torch.zeros(H * D, device=dev, dtype=F32), _vec(w, pfx + "f.b", dev),
                                torch.zeros(H * E, device=dev, dtype=F32)])
        self.q_off, self.f_off, self.v_off = 0, H * D, 2 * H * D
        self.lower = _vec(w, pfx + "lower", dev)
        self.norm = _vec(w, pfx + "norm", dev)
        self.w_o = _mat(w, pfx + "o", dev, act)
        for t, shape in ((self.w_qfv, (2 * H * D + H * E, width)), (self.w_o, (width, H * E)), (self.lower, (H * D,)),
                         (self.norm, (E,))):
            if tuple(t.shape) != shape:
                raise ValueError(f"{pfx}: tensor of shape {tuple(t.shape)}, expected {shape}")


class GatedLinearRecurrence:
    Weights = GatedLinearRecurrenceWeights

    def __init__(self, weights, cache, eps, act, max_positions):
        self.w, self.eps, self.act = weights, float(eps), act
        self.h_state = cache.add_store((weights.H, weights.D, weights.E), F32, zero_on_alloc=True)

    def forward(self, hc, st, cache):
        w = self.w
        qfv = ops.linear(hc, w.w_qfv, bias=w.b_qfv, out_dtype=F32)
        o_raw = ops.seq_glr_scan(qfv, w.q_off, w.f_off, w.v_off, w.lower, cache.view(self.h_state), st, w.H, w.D, w.E)
        o = ops.seq_head_rmsnorm(o_raw, w.norm, w.E, self.eps, self.act)
        return ops.linear(o, w.w_o, out_dtype=F32)


class ReluSquaredFFWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        F = int(spec["ff"])
        self.w_up, self.w_down = _mat(w, pfx + "up", dev, act), _mat(w, pfx + "down", dev, act)
        if tuple(self.w_up.shape) != (F, width) or tuple(self.w_down.shape) != (width, F):
            raise ValueError(f"{pfx}: feed-forward tensors do not fit ff = {F}")


class ReluSquaredFF:
    Weights = ReluSquaredFFWeights

    def __init__(self, weights, act):
        self.w, self.act = weights, act

    def forward(self, x_act):
        u = ops.linear(x_act, self.w.w_up, out_dtype=self.act)
        return ops.linear(ops.seq_relu2(u), self.w.w_down, out_dtype=F32)


WINDOW_ALL = 1 << 30  # "window" of an attention that sees every earlier position


def _expect(pfx, pairs):
    for t, shape in pairs:
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"{pfx}: tensor of shape {tuple(t.shape)}, expected {tuple(shape)}")


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2 (float64). `scaling` = {factor, original, low, high}: rescaled in three bands of
    the wavelength (see below). `scaling` = {factor, original, fast, slow}: blended the YaRN way: with where(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(where(fast)), 0),
    hi = min(ceil(where(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency is
    f_i / factor * ramp_i + f_i (1 - ramp_i); cos and sin are then multiplied by 0.1 ln(factor) + 1. Returns
    (frequencies as a float64 tensor, that multiplier)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if "low" in scaling or "high" in scaling:
        # rescaling in three bands of the wavelength l = 2 pi / f: l < original / high keeps f, l > original / low gets
        # f / factor, between them s = (original / l - low) / (high - low) blends (1 - s) f / factor + s f
        low, high = float(scaling["low"]), float(scaling["high"])
        wave = 2.0 * math.pi / f
        s = ((original / wave - low) / (high - low)).clamp(0.0, 1.0) if high != low else torch.zeros_like(f)
        mid = (1.0 - s) * f / factor + s * f
        return torch.where(wave < original / high, f, torch.where(wave > original / low, f / factor, mid)), 1.0

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class LatentWindowAttentionWeights:
    halves = False         # rotary pairs (i, i + n/2) instead of (2i, 2i + 1)
    gate_per_head = False  # the gate projection has one row per head instead of one per output channel

    def __init__(self, w, pfx, spec, width, dev, act, side=None):
        H, Dn, P, E, R = (int(spec[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
        self.H, self.Dn, self.P, self.E, self.R = H, Dn, P, E, R
        mask = spec.get("mask") or {}
        self.window = int(mask["size"]) if mask.get("size") else None  # None: every earlier position
        rot = spec.get("rot") or {}
        n_rot = int(rot.get("dims", P))
        if n_rot % 2 or n_rot > P:
            raise ValueError(f"{pfx}: rot.dims must be even and at most rot_dim")
        if n_rot:
            f, self.mult = rotary_frequencies(n_rot, rot["base"], rot.get("scaling"))
            self.freqs = f.to(device=dev, dtype=F32).contiguous()
        else:
            self.freqs, self.mult = None, 1.0
        # one projection for (side |) q | latent + shared rotated key part | gate
        n_gate = H if self.gate_per_head else H * E
        parts = [_mat(w, pfx + "q", dev, act), _mat(w, pfx + "dkv", dev, act), _mat(w, pfx + "g", dev, act)]
        _expect(pfx, ((parts[0], (H * (Dn + P), width)), (parts[1], (R + P, width)), (parts[2], (n_gate, width))))
        self.side_n, self.b_in = 0, None
        if side is not None:
            parts.insert(0, _mat(w, side[0], dev, act))
            self.side_n = parts[0].shape[0]
            _expect(pfx, ((parts[0], (self.side_n, width)),))
        self.q_off = self.side_n
        self.q_n, self.lat_off = H * (Dn + P), self.q_off + H * (Dn + P)
        self.g_off = self.lat_off + R + P
        self.n_in = self.g_off + n_gate
        self.w_in = _pad_rows(torch.cat(parts))
        if side is not None and side[1] is not None:
            self.b_in = torch.zeros(self.w_in.shape[0], device=dev, dtype=F32)
            self.b_in[:self.side_n] = _vec(w, side[1], dev)
        self.norm = _vec(w, pfx + "dkv.norm", dev)
        uk, uv = _mat(w, pfx + "uk", dev, act), _mat(w, pfx + "uv", dev, act)
        _expect(pfx, ((uk, (H * Dn, R)), (uv, (H * E, R)), (self.norm, (R,))))
        self.uk_t = uk.view(H, Dn, R).transpose(1, 2).contiguous()  # [H, R, Dn]: folds W_uk into the query
        self.uv = uv.view(H, E, R).contiguous()                     # [H, E, R]: unfolds the latent-space output
        self.scale_h = torch.full((H,), float(spec["scale"]), device=dev, dtype=F32)
        self.w_o = _mat(w, pfx + "o", dev, act)
        _expect(pfx, ((self.w_o, (width, H * E)),))


class LatentWindowAttention:
    Weights = LatentWindowAttentionWeights

    def __init__(self, weights, cache, eps, act, max_positions=None):
        self.w, self.eps, self.act = weights, float(eps), act
        self.side = None
        w = weights
        if w.window is None:  # one entry per position, grown by the cache
            self.cap = None
            self.h_ring = cache.add_store((w.R + w.P,), act, zero_on_alloc=False, per_position=True)
        else:
            self.cap = max(1, min(w.window, int(max_positions))) if max_positions else max(1, w.window)
            self.h_ring = cache.add_store((self.cap, w.R + w.P), act, zero_on_alloc=False)

    def forward(self, hc, st, cache):
        w = self.w
        W = w.R + w.P
        ring = cache.view(self.h_ring)
        cap = self.cap if self.cap is not None else cache.positions
        pin = ops.linear(hc, w.w_in, bias=w.b_in, out_dtype=F32)
        self.side = pin[:, :w.side_n] if w.side_n else None
        q, lat, gate = pin[:, w.q_off:w.lat_off], pin[:, w.lat_off:w.g_off], pin[:, w.g_off:w.n_in]
        single = st.max_len == 1
        ckr, qf = ops.seq_latent_prep(q, lat, w.norm, w.freqs, w.mult, st, w.H, w.Dn, w.P, w.R, self.eps, self.act,
                                      ring=ring if single else None, cap=cap, halves=w.halves)
        ops.seq_head_linear(q, w.Dn + w.P, w.uk_t, qf, W, N=w.R, K=w.Dn)
        # one shared key head whose rows [latent | rotated part] are also the values; output columns >= R are unused. A
        # gate of one number per head commutes with the unfolding and is applied here, an element-wise one after it.
        o = ops.seq_swa_attn(qf, ckr, ckr, ring, ring, gate if w.gate_per_head else None,
                             pin.stride(0) if w.gate_per_head else 0, w.scale_h, st, w.H, 1, W, W,
                             w.window or WINDOW_ALL, cap, from_ring_only=single, gate_per_head=w.gate_per_head)
        if not single:
            ops.seq_kv_ring_write(ckr, None, ring, None, st, cap)
        og = torch.empty((st.n_tok, w.H * w.E), device=hc.device, dtype=self.act)
        ops.seq_head_linear(o, W, w.uv, og, w.E, N=w.E, K=w.R, gate=None if w.gate_per_head else gate)
        return ops.linear(og, w.w_o, out_dtype=F32)


class LatentCausalAttentionWeights(LatentWindowAttentionWeights):
    halves = True
    gate_per_head = True


class LatentCausalAttention(LatentWindowAttention):
    Weights = LatentCausalAttentionWeights


class GatedDeltaRuleWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        H, D = int(spec["heads"]), int(spec["dim"])
        G, E = int(spec.get("kv_heads", H)), int(spec.get("vdim", D))
        if H % G:
            raise ValueError("heads must be a multiple of kv_heads")
        self.H, self.G, self.D, self.E = H, G, D, E
        a1, g1 = _mat(w, pfx + "a1", dev, act), _mat(w, pfx + "g1", dev, act)
        self.ra, self.rg = a1.shape[0], g1.shape[0]
        # one projection for q | k | v | beta, one for the two low-rank bottlenecks
        self.w_in = torch.cat([_mat(w, pfx + "q", dev, act), _mat(w, pfx + "k", dev, act), _mat(w, pfx + "v", dev, act),
                               _mat(w, pfx + "b", dev, act)])
        self.w_low = torch.cat([a1, g1])
        self.n_conv, self.b_off = 2 * G * D + H * E, 2 * G * D + H * E
        self.conv = torch.cat([_vec(w, pfx + "q.conv", dev), _vec(w, pfx + "k.conv", dev), _vec(w, pfx + "v.conv", dev)])
        self.taps = self.conv.shape[1]
        if "conv" in spec and int(spec["conv"]) != self.taps:
            raise ValueError(f"{pfx}: convolution tensors do not fit conv = {spec['conv']}")
        self.a2, self.g2 = _mat(w, pfx + "a2", dev, act), _mat(w, pfx + "g2", dev, act)
        self.dt_bias, self.rate_log = _vec(w, pfx + "dt_bias", dev), _vec(w, pfx + "A_log", dev)
        self.norm = _vec(w, pfx + "norm", dev)
        self.w_o = _mat(w, pfx + "o", dev, act)
        _expect(pfx, ((self.w_in, (self.n_conv + H, width)), (self.w_low, (self.ra + self.rg, width)),
                      (self.conv, (self.n_conv, self.taps)), (self.a2, (H * D, self.ra)), (self.g2, (H * E, self.rg)),
                      (self.dt_bias, (H * D,)), (self.rate_log, (H,)), (self.norm, (E,)), (self.w_o, (width, H * E))))


class GatedDeltaRule:
    Weights = GatedDeltaRuleWeights

    def __init__(self, weights, cache, eps, act, max_positions=None):
        self.w, self.eps, self.act = weights, float(eps), act
        w = weights
        self.h_state = cache.add_store((w.H, w.D, w.E), F32, zero_on_alloc=True)
        self.h_carry = cache.add_store((max(w.taps - 1, 1), w.n_conv), F32, zero_on_alloc=True)

    def forward(self, hc, st, cache):
        w = self.w
        GD = w.G * w.D
        pin = ops.linear(hc, w.w_in, out_dtype=F32)
        low = ops.linear(hc, w.w_low, out_dtype=self.act)
        dec = ops.linear(low[:, :w.ra], w.a2, out_dtype=F32)
        gate = ops.linear(low[:, w.ra:], w.g2, out_dtype=F32)
        cv = ops.seq_conv_act(pin[:, :w.n_conv], w.conv, cache.view(self.h_carry), st, silu=True)
        vec = ops.seq_delta_prep(ops.DELTA_GATED, cv[:, :GD], cv[:, GD:2 * GD], dec, pin[:, w.b_off:], w.H, w.G, w.D,
                                 dec_bias=w.dt_bias, rate_log=w.rate_log)
        o = ops.seq_delta_scan(vec, cv[:, 2 * GD:], cache.view(self.h_state), st, w.H, w.D, w.E)
        on = ops.seq_head_norm_gate(o, w.norm, w.H, w.E, self.eps, self.act, gate=gate)
        return ops.linear(on, w.w_o, out_dtype=F32)


class GeneralizedDeltaRuleWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        H, D = int(spec["heads"]), int(spec["dim"])
        self.H, self.D = H, D
        HD = H * D
        # one projection for r | k | v | removal rate | gate; the rate has a bias
        self.w_in = torch.cat([_mat(w, pfx + n, dev, act) for n in ("r", "k", "v", "a", "g")])
        zero = torch.zeros(HD, device=dev, dtype=F32)
        self.b_in = torch.cat([zero, zero, zero, _vec(w, pfx + "a.b", dev), zero])
        self.w1, self.w2, self.w0 = _mat(w, pfx + "w1", dev, act), _mat(w, pfx + "w2", dev, act), _vec(w, pfx + "w0", dev)
        self.norm = _vec(w, pfx + "norm", dev)
        self.w_o = _mat(w, pfx + "o", dev, act)
        rw = self.w1.shape[0]
        _expect(pfx, ((self.w_in, (5 * HD, width)), (self.b_in, (5 * HD,)), (self.w1, (rw, width)), (self.w2, (HD, rw)),
                      (self.w0, (HD,)), (self.norm, (HD,)), (self.w_o, (width, HD))))


class GeneralizedDeltaRule:
    Weights = GeneralizedDeltaRuleWeights

    def __init__(self, weights, cache, eps, act, max_positions=None):
        self.w, self.eps, self.act = weights, float(eps), act
        self.h_state = cache.add_store((weights.H, weights.D, weights.D), F32, zero_on_alloc=True)

    def forward(self, hc, st, cache):
        w = self.w
        HD = w.H * w.D
        pin = ops.linear(hc, w.w_in, bias=w.b_in, out_dtype=F32)
        low = ops.seq_tanh(ops.linear(hc, w.w1, out_dtype=F32), self.act)
        dec = ops.linear(low, w.w2, bias=w.w0, out_dtype=F32)
        vec = ops.seq_delta_prep(ops.DELTA_GENERALIZED, pin[:, :HD], pin[:, HD:2 * HD], dec, pin[:, 3 * HD:4 * HD], w.H,
                                 w.H, w.D)
        o = ops.seq_delta_scan(vec, pin[:, 2 * HD:3 * HD], cache.view(self.h_state), st, w.H, w.D, w.D)
        on = ops.seq_head_norm_gate(o, w.norm, w.H, w.D, self.eps, self.act, gate=pin[:, 4 * HD:], w_per_head=True)
        return ops.linear(on, w.w_o, out_dtype=F32)


class ScalarGatedDeltaRuleWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        H, D = int(spec["heads"]), int(spec["dim"])
        G, E = int(spec.get("kv_heads", H)), int(spec.get("vdim", D))
        if H % G:
            raise ValueError("heads must be a multiple of kv_heads")
        self.H, self.G, self.D, self.E = H, G, D, E
        # one projection for q | k | v | beta | decay | gate
        parts = [_mat(w, pfx + n, dev, act) for n in ("q", "k", "v", "b", "a", "g")]
        self.n_conv = 2 * G * D + H * E
        self.b_off, self.a_off, self.g_off = self.n_conv, self.n_conv + H, self.n_conv + 2 * H
        self.n_in = self.g_off + H * E
        _expect(pfx, ((torch.cat(parts), (self.n_in, width)),))
        self.w_in = _pad_rows(torch.cat(parts))
        self.conv = torch.cat([_vec(w, pfx + "q.conv", dev), _vec(w, pfx + "k.conv", dev), _vec(w, pfx + "v.conv", dev)])
        self.taps = self.conv.shape[1]
        if "conv" in spec and int(spec["conv"]) != self.taps:
            raise ValueError(f"{pfx}: convolution tensors do not fit conv = {spec['conv']}")
        self.dt_bias, self.rate_log = _vec(w, pfx + "dt_bias", dev), _vec(w, pfx + "A_log", dev)
        self.norm = _vec(w, pfx + "norm", dev)
        self.w_o = _mat(w, pfx + "o", dev, act)
        _expect(pfx, ((self.conv, (self.n_conv, self.taps)), (self.dt_bias, (H,)), (self.rate_log, (H,)), (self.norm, (E,)),
                      (self.w_o, (width, H * E))))


class ScalarGatedDeltaRule(_OneBranch):
    Weights = ScalarGatedDeltaRuleWeights

    def __init__(self, weights, cache, eps, act, max_positions=None):
        self.w, self.eps, self.act = weights, float(eps), act
        w = weights
        self.h_state = cache.add_store((w.H, w.D, w.E), F32, zero_on_alloc=True)
        self.h_carry = cache.add_store((max(w.taps - 1, 1), w.n_conv), F32, zero_on_alloc=True)

    def forward(self, hc, st, cache):
        return self.mix(ops.linear(hc, self.w.w_in, out_dtype=F32), st, cache)

    def mix(self, pin, st, cache):
        w = self.w
        GD = w.G * w.D
        cv = ops.seq_conv_act(pin[:, :w.n_conv], w.conv, cache.view(self.h_carry), st, silu=True)
        vec = ops.seq_delta_prep(ops.DELTA_GATED_SCALAR, cv[:, :GD], cv[:, GD:2 * GD], pin[:, w.a_off:w.a_off + w.H],
                                 pin[:, w.b_off:w.b_off + w.H], w.H, w.G, w.D, dec_bias=w.dt_bias, rate_log=w.rate_log)
        o = ops.seq_delta_scan(vec, cv[:, 2 * GD:], cache.view(self.h_state), st, w.H, w.D, w.E)
        on = ops.seq_head_norm_gate(o, w.norm, w.H, w.E, self.eps, self.act, gate=pin[:, w.g_off:w.n_in], gate_silu=True)
        return ops.linear(on, w.w_o, out_dtype=F32)


class SinkAttentionWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        H, D = int(spec["heads"]), int(spec["dim"])
        G, E = int(spec.get("kv_heads", H)), int(spec.get("vdim", D))
        if H % G:
            raise ValueError("heads must be a multiple of kv_heads")
        self.H, self.G, self.D, self.E = H, G, D, E
        mask = spec.get("mask") or {}
        self.window = int(mask["size"]) if mask.get("size") else None  # None: every earlier position
        temp = spec.get("q_temp") or {}
        self.temp_coef, self.temp_every = float(temp.get("coef", 0.0)), int(temp.get("every", 0))
        if self.temp_every < 0:
            raise ValueError(f"{pfx}: q_temp.every must be positive")
        # one projection for q | k | v | gate (one gate number per head)
        parts = [_mat(w, pfx + n, dev, act) for n in ("q", "k", "v", "g")]
        self.k_off, self.v_off, self.g_off = H * D, (H + G) * D, (H + G) * D + G * E
        self.n_in = self.g_off + H
        _expect(pfx, ((torch.cat(parts), (self.n_in, width)),))
        self.w_in = _pad_rows(torch.cat(parts))
        self.q_norm, self.k_norm = _vec(w, pfx + "q.norm", dev), _vec(w, pfx + "k.norm", dev)
        self.sink = _vec(w, pfx + "sink", dev) if pfx + "sink" in w else None
        self.scale_h = torch.full((H,), float(spec["scale"]), device=dev, dtype=F32)
        self.w_o = _mat(w, pfx + "o", dev, act)
        _expect(pfx, ((self.q_norm, (D,)), (self.k_norm, (D,)), (self.w_o, (width, H * E))))
        if self.sink is not None:
            _expect(pfx, ((self.sink, (H,)),))


class SinkAttention(_OneBranch):
    Weights = SinkAttentionWeights

    def __init__(self, weights, cache, eps, act, max_positions=None):
        self.w, self.eps, self.act = weights, float(eps), act
        w = weights
        if w.window is None:  # one entry per position, grown by the cache
            self.h_k = cache.add_store((w.G * w.D,), act, zero_on_alloc=False, per_position=True)
            self.h_v = cache.add_store((w.G * w.E,), act, zero_on_alloc=False, per_position=True)
            self.ring = None
        else:
            self.ring = max(1, min(w.window, int(max_positions))) if max_positions else max(1, w.window)
            self.h_k = cache.add_store((self.ring, w.G * w.D), act, zero_on_alloc=False)
            self.h_v = cache.add_store((self.ring, w.G * w.E), act, zero_on_alloc=False)

    def forward(self, hc, st, cache):
        return self.mix(ops.linear(hc, self.w.w_in, out_dtype=F32), st, cache)

    def mix(self, pin, st, cache):
        w = self.w
        kring, vring = cache.view(self.h_k), cache.view(self.h_v)
        cap = self.ring if self.ring is not None else cache.positions
        single = st.max_len == 1
        qn, kn, vv = ops.seq_qkv_headnorm(pin, 0, w.k_off, w.v_off, w.q_norm, w.k_norm, w.H, w.G, w.D, w.E, self.eps,
                                          self.act, st, kring=kring if single else None, vring=vring if single else None,
                                          cap=cap, temp_coef=w.temp_coef, temp_every=w.temp_every)
        o = ops.seq_swa_attn(qn, kn, vv, kring, vring, pin[:, w.g_off:w.n_in], pin.stride(0), w.scale_h, st, w.H, w.G, w.D,
                             w.E, w.window or WINDOW_ALL, cap, from_ring_only=single, sink=w.sink, gate_per_head=True)
        if not single:
            ops.seq_kv_ring_write(kn, vv, kring, vring, st, cap)
        return ops.linear(o, w.w_o, out_dtype=F32)


class RotaryAttentionWeights:
    biases = False            # q, k and v projections have biases (`<name>.b`)
    whole_norm = False        # RMS norm over the whole q and k projections (weights `q.norm`, `k.norm`) before rotation
    interleaved = False       # rotary pairs (2i, 2i + 1) instead of (i, i + n/2)
    rotate_values = False     # values are stored rotated by their position over all of vdim; outputs are turned back
    plus_one = False          # a 1 joins every softmax denominator (a key of score 0 without a value)
    mask_kind = "chunk"       # what mask.size means: "chunk" = blocks of positions counted from 0, "window" = sliding

    def __init__(self, w, pfx, spec, width, dev, act, side=None):
        H, D = int(spec["heads"]), int(spec["dim"])
        G, E = int(spec.get("kv_heads", H)), int(spec.get("vdim", D))
        if H % G:
            raise ValueError(f"{pfx}: heads must be a multiple of kv_heads")
        self.H, self.G, self.D, self.E = H, G, D, E
        mask = spec.get("mask") or {}
        self.span = int(mask["size"]) if mask.get("size") else None  # None: every earlier position
        if self.span is not None and self.span <= 0:
            raise ValueError(f"{pfx}: mask.size must be positive")
        cap = spec.get("softcap")
        self.softcap = float(cap) if cap else 0.0
        rot = spec.get("rot") or {}
        n_rot = int(rot.get("dims", D)) if rot else 0
        if n_rot % 2 or n_rot > D:
            raise ValueError(f"{pfx}: rot.dims must be even and at most dim")
        self.qk_freq = None
        if n_rot:
            f, mult = rotary_frequencies(n_rot, rot["base"], rot.get("scaling"))
            if mult != 1.0:
                raise ValueError(f"{pfx}: this mixer takes no magnitude factor on the rotation")
            self.qk_freq = f.to(device=dev, dtype=F32).contiguous()
        self.v_freq = None
        if self.rotate_values:
            if E % 2:
                raise ValueError(f"{pfx}: rotated values need an even vdim")
            self.v_freq = rotary_frequencies(E, rot["base"])[0].to(device=dev, dtype=F32).contiguous()
        # one projection for (side |) q | k | v | gate
        names = ("q", "k", "v", "g")
        parts = [_mat(w, pfx + n, dev, act) for n in names]
        _expect(pfx, ((parts[0], (H * D, width)), (parts[1], (G * D, width)), (parts[2], (G * E, width)),
                      (parts[3], (H * E, width))))
        bias = [(_vec(w, pfx + n + ".b", dev) if self.biases and n != "g" else torch.zeros(m.shape[0], device=dev, dtype=F32))
                for n, m in zip(names, parts)]
        self.side_n = 0
        if side is not None:
            parts.insert(0, _mat(w, side[0], dev, act))
            self.side_n = parts[0].shape[0]
            _expect(pfx, ((parts[0], (self.side_n, width)),))
            bias.insert(0, _vec(w, side[1], dev) if side[1] is not None else torch.zeros(self.side_n, device=dev, dtype=F32))
        self.q_off = self.side_n
        self.k_off, self.v_off, self.g_off = self.q_off + H * D, self.q_off + (H + G) * D, self.q_off + (H + G) * D + G * E
        self.n_in = self.g_off + H * E
        self.w_in = _pad_rows(torch.cat(parts))
        self.b_in = None
        if self.biases or (side is not None and side[1] is not None):
            self.b_in = torch.zeros(self.w_in.shape[0], device=dev, dtype=F32)
            self.b_in[:self.n_in] = torch.cat(bias)
        self.q_norm = self.k_norm = None
        if self.whole_norm:
            self.q_norm, self.k_norm = _vec(w, pfx + "q.norm", dev), _vec(w, pfx + "k.norm", dev)
            _expect(pfx, ((self.q_norm, (H * D,)), (self.k_norm, (G * D,))))
        self.sink = torch.zeros(H, device=dev, dtype=F32) if self.plus_one else None  # exp(0) in the denominator
        self.scale_h = torch.full((H,), float(spec["scale"]), device=dev, dtype=F32)
        self.w_o = _mat(w, pfx + "o", dev, act)
        _expect(pfx, ((self.w_o, (width, H * E)),))


class RotaryAttention(_OneBranch):
    Weights = RotaryAttentionWeights

    def __init__(self, weights, cache, eps, act, max_positions=None):
        self.w, self.eps, self.act = weights, float(eps), act
        self.side = None
        w = weights
        if w.span is None:  # one entry per position, grown by the cache
            self.ring = None
            self.h_k = cache.add_store((w.G * w.D,), act, zero_on_alloc=False, per_position=True)
            self.h_v = cache.add_store((w.G * w.E,), act, zero_on_alloc=False, per_position=True)
        else:  # the keys a query sees never outnumber mask.size: a ring, entry = position % size
            self.ring = max(1, min(w.span, int(max_positions))) if max_positions else w.span
            self.h_k = cache.add_store((self.ring, w.G * w.D), act, zero_on_alloc=False)
            self.h_v = cache.add_store((self.ring, w.G * w.E), act, zero_on_alloc=False)

    def forward(self, hc, st, cache):
        w = self.w
        pin = ops.linear(hc, w.w_in, bias=w.b_in, out_dtype=F32)
        self.side = pin[:, :w.side_n] if w.side_n else None
        kring, vring = cache.view(self.h_k), cache.view(self.h_v)
        cap = self.ring if self.ring is not None else cache.positions
        single = st.max_len == 1
        q, k, v = ops.seq_qkv_rotary(pin, w.q_off, w.k_off, w.v_off, w.H, w.G, w.D, w.E, self.eps, self.act, st,
                                     wq=w.q_norm, wk=w.k_norm, qk_freq=w.qk_freq, qk_interleaved=w.interleaved,
                                     v_freq=w.v_freq, v_interleaved=w.interleaved,
                                     kring=kring if single else None, vring=vring if single else None, cap=cap)
        chunk = w.span if (w.span is not None and w.mask_kind == "chunk") else 0
        window = w.span if (w.span is not None and w.mask_kind == "window") else WINDOW_ALL
        o = ops.seq_swa_attn(q, k, v, kring, vring, pin[:, w.g_off:w.n_in], pin.stride(0), w.scale_h, st, w.H, w.G, w.D,
                             w.E, window, cap, from_ring_only=single, sink=w.sink, chunk=chunk, softcap=w.softcap,
                             vfreq=w.v_freq, v_interleaved=w.interleaved)
        if not single:
            ops.seq_kv_ring_write(k, v, kring, vring, st, cap)
        return ops.linear(o, w.w_o, out_dtype=F32)


class ValueRotaryAttentionWeights(RotaryAttentionWeights):
    biases = True
    whole_norm = True
    interleaved = True
    rotate_values = True
    plus_one = True


class ValueRotaryAttention(RotaryAttention):
    Weights = ValueRotaryAttentionWeights


class StateSpaceDualityWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        H, E, N = int(spec["heads"]), int(spec["vdim"]), int(spec["state"])
        G, NG = int(spec.get("groups", 1)), int(spec.get("norm_groups", 1))
        if H % G or (H * E) % NG:
            raise ValueError(f"{pfx}: heads must be a multiple of groups, heads * vdim of norm_groups")
        self.H, self.E, self.N, self.G, self.NG = H, E, N, G, NG
        inner = self.inner = H * E
        self.n_conv = inner + 2 * G * N
        self.n_in = 2 * inner + 2 * G * N + H  # gate | x | B | C | step size
        w_in = _mat(w, pfx + "in", dev, act)
        _expect(pfx, ((w_in, (self.n_in, width)),))
        self.w_in = _pad_rows(w_in)
        self.conv, self.conv_b = _vec(w, pfx + "conv", dev), _vec(w, pfx + "conv.b", dev)
        self.taps = self.conv.shape[1]
        if "conv" in spec and int(spec["conv"]) != self.taps:
            raise ValueError(f"{pfx}: convolution tensor does not fit conv = {spec['conv']}")
        self.dt_bias, self.rate_log, self.skip = (_vec(w, pfx + n, dev) for n in ("dt_bias", "A_log", "D"))
        self.norm = _vec(w, pfx + "norm", dev)
        self.w_o = _mat(w, pfx + "o", dev, act)
        _expect(pfx, ((self.conv, (self.n_conv, self.taps)), (self.conv_b, (self.n_conv,)), (self.dt_bias, (H,)),
                      (self.rate_log, (H,)), (self.skip, (H,)), (self.norm, (inner,)), (self.w_o, (width, inner))))


class StateSpaceDuality(_OneBranch):
    Weights = StateSpaceDualityWeights

    def __init__(self, weights, cache, eps, act, max_positions=None):
        self.w, self.eps, self.act = weights, float(eps), act
        w = weights
        self.h_state = cache.add_store((w.H, w.N, w.E), F32, zero_on_alloc=True)
        self.h_carry = cache.add_store((max(w.taps - 1, 1), w.n_conv), F32, zero_on_alloc=True)

    def forward(self, hc, st, cache):
        return self.mix(ops.linear(hc, self.w.w_in, out_dtype=F32), st, cache)

    def mix(self, pin, st, cache):
        w = self.w
        inner, GN = w.inner, w.G * w.N
        gate, step = pin[:, :inner], pin[:, inner + w.n_conv:w.n_in]
        cv = ops.seq_conv_act(pin[:, inner:inner + w.n_conv], w.conv, cache.view(self.h_carry), st, silu=True,
                              bias=w.conv_b)
        xs, write, read = cv[:, :inner], cv[:, inner:inner + GN], cv[:, inner + GN:]
        vec = ops.seq_delta_prep(ops.DELTA_STATE_SPACE, read, write, step, None, w.H, w.G, w.N, dec_bias=w.dt_bias,
                                 rate_log=w.rate_log)
        o = ops.seq_delta_scan(vec, xs, cache.view(self.h_state), st, w.H, w.N, w.E, correct=False)
        y = ops.seq_skip_gate_group_norm(o, xs, w.skip, gate, w.norm, w.H, w.E, w.NG, self.eps, self.act)
        return ops.linear(y, w.w_o, out_dtype=F32)


class ParallelMixersWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        self.left = SinkAttentionWeights(w, pfx + "left.", spec["left"], width, dev, act)
        self.right = StateSpaceDualityWeights(w, pfx + "right.", spec["right"], width, dev, act)
        self.left_out, self.right_out = _vec(w, pfx + "left.out", dev), _vec(w, pfx + "right.out", dev)
        _expect(pfx, ((self.left_out, (width,)), (self.right_out, (width,))))
        # both read the same input: one projection (each side's rows are already padded to 16-byte multiples)
        self.n_left = self.left.w_in.shape[0]
        self.w_in = torch.cat([self.left.w_in, self.right.w_in]).contiguous()


class ParallelMixers:
    Weights = ParallelMixersWeights

    def __init__(self, weights, cache, eps, act, max_positions=None):
        self.w = weights
        self.left = SinkAttention(weights.left, cache, eps, act, max_positions)
        self.right = StateSpaceDuality(weights.right, cache, eps, act, max_positions)

    def branches(self, hc, st, cache):
        w = self.w
        pin = ops.linear(hc, w.w_in, out_dtype=F32)
        yl = self.left.mix(pin[:, :w.n_left], st, cache)
        yr = self.right.mix(pin[:, w.n_left:], st, cache)
        return [(yl, w.left_out), (yr, w.right_out)], 0.5


class ClampedGluFFWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        F = int(spec["ff"])
        self.ff, self.limit = F, float(spec["limit"])
        gate, up = _mat(w, pfx + "gate", dev, act), _mat(w, pfx + "up", dev, act)
        self.w_down = _mat(w, pfx + "down", dev, act)
        _expect(pfx, ((gate, (F, width)), (up, (F, width)), (self.w_down, (width, F))))
        self.w_gu = torch.cat([gate, up]).contiguous()


class ClampedGluFF:
    Weights = ClampedGluFFWeights

    def __init__(self, weights, act):
        self.w, self.act = weights, act

    def forward(self, x_act):
        gu = ops.linear(x_act, self.w.w_gu, out_dtype=self.act)
        return ops.linear(ops.seq_glu_clamped(gu, self.w.limit), self.w.w_down, out_dtype=F32)

    def post_norm(self, x, x_act, alpha, w_norm, eps, act):
        """rmsnorm(alpha x + ff(x)) * w_norm -> (fp32, copy in act)."""
        return ops.seq_post_norm(x, alpha, w_norm, eps, y1=self.forward(x_act), act=act)


class RoutedExpertsWeights:
    softmax_bias = False  # True: softmax scores, choice on score + `correction`, plain scores as weights

    def __init__(self, w, pfx, spec, width, dev, act):
        r = spec["router"]
        self.n, self.top = int(r["experts"]), int(r["top"])
        self.n_id = int(r.get("identity", 0))  # trailing router outputs without weights: they hand their input through
        n_all = self.n_all = self.n + self.n_id
        groups = r.get("groups") or {"count": 1, "keep": 1}
        self.n_groups, self.keep, self.scale = int(groups["count"]), int(groups["keep"]), float(r.get("scale", 1.0))
        ff = int(spec["expert"]["ff"])
        self.ff = ff
        if n_all % self.n_groups or not 0 < self.keep <= self.n_groups or self.top > self.keep * (n_all // self.n_groups):
            raise ValueError(f"{pfx}: router groups do not fit experts / top")
        self.router = _vec(w, pfx + "router", dev)  # the router runs in fp32 whatever the serving dtype
        # A checkpoint stores bf16, so the router's weights usually ARE bf16 numbers. The product of two bf16 numbers is
        # exact in fp32, so on bf16 activations the tensor-core GEMM with its fp32 accumulator computes the same sums of
        # exact products as the fp32 kernel does, in another order. Rows padded with zeros to a whole 64-wide tile.
        self.router_act = None
        if act == torch.bfloat16 and bool((self.router.to(act).to(F32) == self.router).all()):
            pad = (-n_all) % 64
            self.router_act = torch.cat([self.router.to(act), torch.zeros((pad, width), device=dev, dtype=act)]).contiguous()
        self.w_gate_up = torch.stack([torch.cat([_mat(w, f"{pfx}e{e}.gate", dev, act), _mat(w, f"{pfx}e{e}.up", dev, act)])
                                      for e in range(self.n)]).contiguous()
        self.w_down = torch.stack([_mat(w, f"{pfx}e{e}.down", dev, act) for e in range(self.n)]).contiguous()
        self.correction = _vec(w, pfx + "correction", dev) if self.softmax_bias else None
        _expect(pfx, ((self.router, (n_all, width)), (self.w_gate_up, (self.n, 2 * ff, width)),
                      (self.w_down, (self.n, width, ff))))
        if self.correction is not None:
            _expect(pfx, ((self.correction, (n_all,)),))


class RoutedExperts:
    """Feed-forward whose result is added to the residual together with the mixer's (side-by-side sublayers)."""
    Weights = RoutedExpertsWeights

    def __init__(self, weights, act):
        self.w, self.act = weights, act

    def route(self, x_act):
        w = self.w
        if w.router_act is not None:
            logits = ops.linear(x_act, w.router_act, out_dtype=F32)[:, :w.n_all]
        else:
            logits = ops.linear_w32(x_act, w.router)
        return ops.seq_moe_route(logits, w.n_groups, w.keep, w.top, w.scale, softmax_bias=w.softmax_bias,
                                 correction=w.correction)

    def residual(self, x, y, x_act):
        """x + (y + experts(x_act)): fp32 residual sum with the mixer's output y."""
        w = self.w
        if w.n_id:
            raise ValueError("experts that hand their input through need the norm-after-sum residual (post_norm)")
        ids, wts = self.route(x_act)
        z, pos_of = ops.seq_moe_experts(x_act, ids, w.w_gate_up, w.w_down)
        return ops.seq_residual_combine(x, y, z, pos_of, wts, w.top)

    def post_norm(self, x, x_act, alpha, w_norm, eps, act):
        """rmsnorm(alpha x + experts(x)) * w_norm -> (fp32, copy in act); the weighted sum over a token's choices is taken
        inside the norm kernel, in the order of the choices."""
        w = self.w
        ids, wts = self.route(x_act)
        z, pos_of = ops.seq_moe_experts(x_act, ids, w.w_gate_up, w.w_down, n_through=w.n_id)
        return ops.seq_post_norm(x, alpha, w_norm, eps, z=z, pos_of=pos_of, wts=wts, ids=ids, n_real=w.n, act=act)


class BiasedSoftmaxExpertsWeights(RoutedExpertsWeights):
    softmax_bias = True


class BiasedSoftmaxExperts(RoutedExperts):
    Weights = BiasedSoftmaxExpertsWeights


MIXERS = {"attention": GatedWindowAttention, "hgrn2": GatedLinearRecurrence, "latent_attention": LatentWindowAttention,
          "channel_delta": GatedDeltaRule, "general_delta": GeneralizedDeltaRule, "delta": ScalarGatedDeltaRule,
          "sink_attention": SinkAttention, "ssd": StateSpaceDuality, "parallel": ParallelMixers,
          "rotary_attention": RotaryAttention, "rotary_attention_vrot": ValueRotaryAttention,
          "latent_attention_causal": LatentCausalAttention}
FEED_FORWARDS = {"dense": ReluSquaredFF, "moe": RoutedExperts, "clamped_glu": ClampedGluFF,
                 "moe_softmax_bias": BiasedSoftmaxExperts}
