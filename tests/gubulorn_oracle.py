"""Plain, slow restatement of the Gubulorn decoder for the tests: one function per mechanism, whole sequences only (no
cache, no batching, no kernels), PyTorch on the CPU in whatever float dtype the weights come in (the tests use float64).
Nothing here is imported by the package and nothing of the package is imported here.

Notation: T tokens, C = width, H heads, G key/value heads (or state-space groups), D = per-head key size, E = per-head
value size, N = state size. Weights are a dict name -> tensor with linear weights stored [out, in]; `m` is a mixer's
dictionary of sizes.
"""
import math

import torch


# ------------------------------------------------------------------------------------------------ elementwise pieces
def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight sits around zero."""
    return rms(x, eps) * (1.0 + w)


def unit(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + eps)


def causal_conv(h, w, bias=None):
    """h [T, n], w [n, taps]: c_t = sum_j w[:, j] h_(t - taps + 1 + j) (+ bias), zeros before the start."""
    T, n = h.shape
    taps = w.shape[1]
    c = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                c[t] = c[t] + w[:, j] * h[s]
    if bias is not None:
        c = c + bias
    return c


# ------------------------------------------------------------------------------------------------ mixer "delta"
def scalar_gated_delta_recurrence(q, k, v, beta, g):
    """q, k [T, H, D], v [T, H, E], beta, g [T, H]. Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, H, D = q.shape
    E = v.shape[2]
    S = torch.zeros(H, D, E, dtype=q.dtype)
    o = torch.zeros(T, H, E, dtype=q.dtype)
    for t in range(T):
        for h in range(H):
            S[h] = g[t, h] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, h])
            S[h] = S[h] + torch.outer(k[t, h], u)
            o[t, h] = S[h].T @ q[t, h]
    return o


def delta_mixer(h, W, pfx, m, eps):
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ W[pfx + "q"].T, W[pfx + "q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(h @ W[pfx + "k"].T, W[pfx + "k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(h @ W[pfx + "v"].T, W[pfx + "v.conv"])).reshape(T, H, E)
    q = unit(q) * D ** -0.5
    k = unit(k)
    rep = H // G
    q = q.repeat_interleave(rep, dim=1)
    k = k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ W[pfx + "b"].T)
    g = torch.exp(-torch.exp(W[pfx + "A_log"]) * softplus(h @ W[pfx + "a"].T + W[pfx + "dt_bias"]))
    o = scalar_gated_delta_recurrence(q, k, v, beta, g)
    o = rms(o, eps) * W[pfx + "norm"]
    o = o * silu(h @ W[pfx + "g"].T).reshape(T, H, E)
    return o.reshape(T, H * E) @ W[pfx + "o"].T


# ------------------------------------------------------------------------------------------------ mixer "parallel"
def sink_attention(h, W, pfx, m, eps):
    """Full causal softmax attention: head norms on q and k, a temperature on q that grows with the position in steps,
    one extra term exp(sink_h) in every softmax denominator, one sigmoid gate per head on the output."""
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ W[pfx + "q"].T).reshape(T, H, D)
    k = (h @ W[pfx + "k"].T).reshape(T, G, D)
    v = (h @ W[pfx + "v"].T).reshape(T, G, E)
    q = rms(q, eps) * W[pfx + "q.norm"]
    k = rms(k, eps) * W[pfx + "k.norm"]
    pos = torch.arange(T)
    temp = 1.0 + m["q_temp"]["coef"] * torch.log(torch.floor((pos + 1) / m["q_temp"]["every"]).to(h.dtype) + 1.0)
    q = q * temp[:, None, None]
    gate = torch.sigmoid(h @ W[pfx + "g"].T)
    out = torch.zeros(T, H, E, dtype=h.dtype)
    rep = H // G
    for hd in range(H):
        kv = hd // rep
        s = (q[:, hd] @ k[:, kv].T) * m["scale"]
        for i in range(T):
            row = s[i, :i + 1]
            top = torch.maximum(row.max(), W[pfx + "sink"][hd])
            e = torch.exp(row - top)
            den = e.sum() + torch.exp(W[pfx + "sink"][hd] - top)
            out[i, hd] = (e / den) @ v[:i + 1, kv]
    out = out * gate[:, :, None]
    return out.reshape(T, H * E) @ W[pfx + "o"].T


def state_space_recurrence(x, B, Cm, dt, a_log, Dskip):
    """x [T, H, E], B, Cm [T, H, N] (already spread to heads), dt [T, H]: S = exp(-exp(a_log) dt) S + dt B x^T,
    y = S^T C + Dskip x."""
    T, H, E = x.shape
    N = B.shape[2]
    S = torch.zeros(H, N, E, dtype=x.dtype)
    y = torch.zeros(T, H, E, dtype=x.dtype)
    for t in range(T):
        for h in range(H):
            S[h] = torch.exp(-torch.exp(a_log[h]) * dt[t, h]) * S[h] + dt[t, h] * torch.outer(B[t, h], x[t, h])
            y[t, h] = S[h].T @ Cm[t, h] + Dskip[h] * x[t, h]
    return y


def state_space_mixer(h, W, pfx, m, eps):
    H, E, N, G, NG = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    T = h.shape[0]
    inner = H * E
    p = h @ W[pfx + "in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[pfx + "conv"], W[pfx + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, E)
    rep = H // G
    B = xbc[:, inner:inner + G * N].reshape(T, G, N).repeat_interleave(rep, dim=1)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N).repeat_interleave(rep, dim=1)
    dt = softplus(dt + W[pfx + "dt_bias"])
    y = state_space_recurrence(x, B, Cm, dt, W[pfx + "A_log"], W[pfx + "D"]).reshape(T, inner)
    y = y * silu(z)
    y = rms(y.reshape(T, NG, inner // NG), eps).reshape(T, inner) * W[pfx + "norm"]
    return y @ W[pfx + "o"].T


def parallel_mixer(h, W, pfx, m, eps):
    left = sink_attention(h, W, pfx + "left.", m["left"], eps)
    right = state_space_mixer(h, W, pfx + "right.", m["right"], eps)
    return 0.5 * (rms(left, eps) * W[pfx + "left.out"] + rms(right, eps) * W[pfx + "right.out"])


# ------------------------------------------------------------------------------------------------ feed-forwards
def dense_ff(h, W, pfx, mlp):
    lim = mlp["limit"]
    g = torch.clamp(h @ W[pfx + "gate"].T, max=lim)
    u = torch.clamp(h @ W[pfx + "up"].T, min=-lim, max=lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[pfx + "down"].T


def route(z, correction, top, n_groups, keep):
    """z [T, n] router logits -> (ids [T, top], weights [T, top]): softmax scores, the choice is made on score +
    correction inside the `keep` groups whose best choice score is largest, the weights are the plain scores."""
    T, n = z.shape
    s = torch.softmax(z, dim=-1)
    c = s + correction
    per = n // n_groups
    best = c.reshape(T, n_groups, per).max(dim=-1).values
    kept = torch.topk(best, keep, dim=-1).indices
    allowed = torch.zeros(T, n_groups, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    allowed = allowed.repeat_interleave(per, dim=1)
    c = torch.where(allowed, c, torch.full_like(c, -math.inf))
    ids = torch.topk(c, top, dim=-1).indices
    return ids, torch.gather(s, 1, ids)


def moe(h, W, pfx, mlp):
    r = mlp["router"]
    n_real, n_id = r["experts"], r.get("identity", 0)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    z = h @ W[pfx + "router"].T
    ids, wts = route(z, W[pfx + "correction"], r["top"], groups["count"], groups["keep"])
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(ids[t, j])
            if e >= n_real:
                assert e < n_real + n_id
                y[t] = y[t] + wts[t, j] * h[t]
            else:
                a = silu(W[f"{pfx}e{e}.gate"] @ h[t]) * (W[f"{pfx}e{e}.up"] @ h[t])
                y[t] = y[t] + wts[t, j] * (W[f"{pfx}e{e}.down"] @ a)
    return y


# ------------------------------------------------------------------------------------------------ the model
def forward(cfg, W, tokens, return_residuals=False):
    """Logits [T, vocab] of one sequence (cfg: the configuration as a dict)."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = norm_one_plus(W["embed"][torch.as_tensor(tokens)], W["embed.norm"], eps)
    residuals = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "delta":
            y = delta_mixer(x, W, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(x, W, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = norm_one_plus(alpha * x + y, W[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            f = dense_ff(x, W, p + "mlp.", mlp) if mlp["kind"] == "dense" else moe(x, W, p + "mlp.", mlp)
            x = norm_one_plus(alpha * x + f, W[p + "norm2"], eps)
        residuals.append(x)
    z = (norm_one_plus(x, W["final.norm"], eps) @ W["head"].T) * cfg["logit_scale"]
    cap = cfg["logit_softcap"]
    z = cap * torch.tanh(z / cap)
    return (z, residuals) if return_residuals else z
