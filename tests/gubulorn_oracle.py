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
    cap = cfg.get("logit_softcap")
    if cap is not None:
        z = cap * torch.tanh(z / cap)
    return (z, residuals) if return_residuals else z


# ------------------------------------------------------------------------------------------------ random checkpoints
def random_weights(cfg, seed=0, dtype=torch.float64):
    """Random weights of a configuration, rounded to bfloat16 (what a checkpoint stores) and returned in `dtype`. Router
    corrections are large enough to make choice scores negative; sinks, skips and decays are of order one."""
    g = torch.Generator().manual_seed(seed)
    C, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, out, inp, scale=1.0):
        W[name] = torch.randn(out, inp, generator=g) * scale / math.sqrt(inp)

    def vec(name, n, mean=0.0, std=1.0):
        W[name] = mean + std * torch.randn(n, generator=g)

    W["embed"] = torch.randn(V, C, generator=g)
    mat("head", V, C, 2.0)
    vec("embed.norm", C, 0.0, 0.1)
    vec("final.norm", C, 0.0, 0.1)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", C, 0.0, 0.1)
        x = p + "mix."
        if L["type"] == "delta":
            H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * E)):
                mat(x + n, rows, C, 2.0)
                W[x + n + ".conv"] = torch.randn(rows, m["conv"], generator=g) * 0.5
            mat(x + "b", H, C)
            mat(x + "a", H, C)
            W[x + "A_log"] = torch.rand(H, generator=g) * 2.0 - 2.0
            vec(x + "dt_bias", H, -1.0, 1.0)
            vec(x + "norm", E, 1.0, 0.1)
            mat(x + "g", H * E, C)
            mat(x + "o", C, H * E)
        else:
            a, b = m["left"], m["right"]
            H, G, D, E = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            mat(x + "left.q", H * D, C, 2.0)
            mat(x + "left.k", G * D, C, 2.0)
            mat(x + "left.v", G * E, C)
            vec(x + "left.q.norm", D, 1.0, 0.2)
            vec(x + "left.k.norm", D, 1.0, 0.2)
            vec(x + "left.sink", H, 0.5, 1.0)
            mat(x + "left.g", H, C, 2.0)
            mat(x + "left.o", C, H * E)
            vec(x + "left.out", C, 1.0, 0.1)
            Hs, Es, N, Gs = b["heads"], b["vdim"], b["state"], b["groups"]
            inner, nc = Hs * Es, Hs * Es + 2 * Gs * N
            mat(x + "right.in", 2 * inner + 2 * Gs * N + Hs, C, 1.5)
            W[x + "right.conv"] = torch.randn(nc, b["conv"], generator=g) * 0.5
            vec(x + "right.conv.b", nc, 0.0, 0.3)
            vec(x + "right.dt_bias", Hs, -1.0, 1.0)
            W[x + "right.A_log"] = torch.rand(Hs, generator=g) * 2.0 - 2.0
            vec(x + "right.D", Hs, 1.0, 0.5)
            vec(x + "right.norm", inner, 1.0, 0.1)
            mat(x + "right.o", C, inner)
            vec(x + "right.out", C, 1.0, 0.1)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        vec(p + "norm2", C, 0.0, 0.1)
        if mlp["kind"] == "dense":
            mat(p + "mlp.gate", mlp["ff"], C, 2.0)
            mat(p + "mlp.up", mlp["ff"], C, 2.0)
            mat(p + "mlp.down", C, mlp["ff"])
        else:
            r = mlp["router"]
            n_all = r["experts"] + r.get("identity", 0)
            mat(p + "mlp.router", n_all, C, 2.0)
            vec(p + "mlp.correction", n_all, -0.05, 0.15)
            for e in range(r["experts"]):
                mat(f"{p}mlp.e{e}.gate", mlp["expert"]["ff"], C)
                mat(f"{p}mlp.e{e}.up", mlp["expert"]["ff"], C)
                mat(f"{p}mlp.e{e}.down", C, mlp["expert"]["ff"])
    return {k: v.to(torch.bfloat16).to(dtype) for k, v in W.items()}
