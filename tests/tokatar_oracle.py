"""Plain, slow restatement of the Tokatar decoder for the tests: one function per mechanism, whole sequences only (no
cache, no batching, no kernels), PyTorch on the CPU in whatever float dtype the weights come in (the tests use float64).
Nothing here is imported by the package and nothing of the package is imported here.

Notation: T tokens, C = width, H query heads, G key / value heads, D = per-head query / key size, E = per-head value size,
R = latent size, P = rotated part of a latent-attention head. Weights are a dict name -> tensor, linear weights stored
[out, in]; `m` is a mixer's dictionary of sizes and constants as the configuration carries it.
"""
import math

import torch


# ------------------------------------------------------------------------------------------------ small pieces
def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is ONE number for all coordinates."""
    return rms(x, eps) * g


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def frequencies(dims, base):
    """f_i = base^(-2 i / dims) for the dims / 2 pairs."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return float(base) ** (-2.0 * i / dims)


def scaled_frequencies(f, scaling):
    """The three-band rescaling of rotary frequencies by wavelength: short waves keep f, long waves get f / factor, the
    band between is blended linearly in original / wavelength."""
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for i in range(f.numel()):
        wave = 2.0 * math.pi / float(f[i])
        if wave < original / high:
            continue
        if wave > original / low:
            out[i] = f[i] / factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = (1.0 - s) * f[i] / factor + s * f[i]
    return out


def turn(x, positions, f, layout, sign=1.0):
    """Rotates the first 2 * len(f) entries of the last axis of x [T, ..., n]; row t by positions[t] * f_i * sign.
    layout "halves": entry i pairs with i + len(f); "interleaved": entry 2 i with 2 i + 1. The rest passes."""
    n_pairs = f.numel()
    if n_pairs == 0:
        return x
    ang = positions.to(torch.float64)[:, None] * f[None, :] * sign          # [T, pairs]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [n_pairs]
    co, si = torch.cos(ang).to(x.dtype).view(shape), torch.sin(ang).to(x.dtype).view(shape)
    out = x.clone()
    if layout == "halves":
        u, v = x[..., :n_pairs], x[..., n_pairs:2 * n_pairs]
        out[..., :n_pairs] = u * co - v * si
        out[..., n_pairs:2 * n_pairs] = v * co + u * si
    elif layout == "interleaved":
        u, v = x[..., 0:2 * n_pairs:2], x[..., 1:2 * n_pairs:2]
        out[..., 0:2 * n_pairs:2] = u * co - v * si
        out[..., 1:2 * n_pairs:2] = v * co + u * si
    else:
        raise ValueError(layout)
    return out


def visible(T, chunk=None):
    """[T, T] boolean: query i sees key j. Causal; with `chunk` only inside the block of `chunk` positions that holds i,
    blocks counted from position 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if chunk:
        ok = ok & (i // chunk == j // chunk)
    return ok


def attend(q, k, v, scale, mask, softcap=None, plus_one=False):
    """q [T, H, D], k [T, G, D], v [T, G, E] -> [T, H, E]. Scores scaled, optionally squashed by cap * tanh(s / cap);
    softmax over the visible keys, with `plus_one` a 1 joins the denominator (a key of score 0 that carries no value)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~mask, -math.inf)
        top = s.max(dim=-1, keepdim=True).values
        if plus_one:
            top = torch.clamp(top, min=0.0)
        e = torch.exp(s - top)
        den = e.sum(dim=-1, keepdim=True)
        if plus_one:
            den = den + torch.exp(-top)
        out[:, h] = (e / den) @ v[:, g]
    return out


def _rot_freqs(m, dims_default):
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", dims_default))
    if not dims:
        return torch.zeros(0, dtype=torch.float64)
    f = frequencies(dims, rot["base"])
    if rot.get("scaling"):
        f = scaled_frequencies(f, rot["scaling"])
    return f


# ------------------------------------------------------------------------------------------------ mixer "attention"
def attention_mixer(h, W, pfx, m):
    """Grouped-query attention, rotary positions in halves on q and k, soft-capped scores, chunked mask, plain softmax,
    element-wise sigmoid gate before the output matrix."""
    T = h.shape[0]
    H, G, D, E = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    f = _rot_freqs(m, D)
    q = turn((h @ W[pfx + "q"].T).view(T, H, D), pos, f, "halves")
    k = turn((h @ W[pfx + "k"].T).view(T, G, D), pos, f, "halves")
    v = (h @ W[pfx + "v"].T).view(T, G, E)
    chunk = (m.get("mask") or {}).get("size")
    o = attend(q, k, v, float(m["scale"]), visible(T, chunk), softcap=m.get("softcap"))
    o = o.reshape(T, H * E) * torch.sigmoid(h @ W[pfx + "g"].T)
    return o @ W[pfx + "o"].T


# ------------------------------------------------------------------------------------------------ mixer "attention_2"
def attention_2_mixer(h, W, pfx, m, eps):
    """Biased projections, RMS norm of the WHOLE q and k projections, interleaved rotary pairs, values rotated by their own
    position and the head outputs turned back by the query's, chunked mask, softmax with 1 added to the denominator,
    element-wise sigmoid gate."""
    T = h.shape[0]
    H, G, D, E = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = rms(h @ W[pfx + "q"].T + W[pfx + "q.b"], eps) * W[pfx + "q.norm"]
    k = rms(h @ W[pfx + "k"].T + W[pfx + "k.b"], eps) * W[pfx + "k.norm"]
    v = (h @ W[pfx + "v"].T + W[pfx + "v.b"]).view(T, G, E)
    f = _rot_freqs(m, D)
    q = turn(q.view(T, H, D), pos, f, "interleaved")
    k = turn(k.view(T, G, D), pos, f, "interleaved")
    fv = frequencies(E, m["rot"]["base"])
    v = turn(v, pos, fv, "interleaved")
    chunk = (m.get("mask") or {}).get("size")
    o = attend(q, k, v, float(m["scale"]), visible(T, chunk), plus_one=True)
    o = turn(o, pos, fv, "interleaved", sign=-1.0)
    o = o.reshape(T, H * E) * torch.sigmoid(h @ W[pfx + "g"].T)
    return o @ W[pfx + "o"].T


# ------------------------------------------------------------------------------------------------ mixer "latent_attention"
def latent_attention_mixer(h, W, pfx, m, eps):
    """Keys and values of every head are expansions of one normed latent per token; one rotated key part is shared by the
    heads. Causal over everything before, plain softmax, one sigmoid gate per head."""
    T = h.shape[0]
    H, D, P, E, R = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    pos = torch.arange(T)
    f = _rot_freqs(m, P)
    q = (h @ W[pfx + "q"].T).view(T, H, D + P)
    q_plain, q_rot = q[..., :D], turn(q[..., D:].contiguous(), pos, f, "halves")
    down = h @ W[pfx + "dkv"].T
    c = rms(down[:, :R], eps) * W[pfx + "dkv.norm"]
    k_rot = turn(down[:, R:].contiguous().view(T, 1, P), pos, f, "halves")[:, 0]
    k_plain = (c @ W[pfx + "uk"].T).view(T, H, D)
    v = (c @ W[pfx + "uv"].T).view(T, H, E)
    mask = visible(T)
    gate = torch.sigmoid(h @ W[pfx + "g"].T)                                # [T, H]
    out = torch.zeros(T, H, E, dtype=h.dtype)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * float(m["scale"])
        s = s.masked_fill(~mask, -math.inf)
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, hd] * gate[:, hd:hd + 1]
    return out.reshape(T, H * E) @ W[pfx + "o"].T


# ------------------------------------------------------------------------------------------------ feed-forward, layer, model
def dense_ff(h, W, pfx):
    return relu_squared(h @ W[pfx + "up"].T) @ W[pfx + "down"].T


def sublayer(x, h, y, W, p, k, eps):
    """x + ls_k * norm_kb(y * sigmoid(rg_k h + b)): the sublayer's result y, gated by its own input h, normed, scaled."""
    y = y * torch.sigmoid(h @ W[f"{p}rg{k}"].T + W[f"{p}rg{k}.b"])
    return x + scalar_norm(y, W[f"{p}norm{k}b"], eps) * W[f"{p}ls{k}"]


def mixer(kind, h, W, pfx, m, eps):
    if kind == "attention":
        return attention_mixer(h, W, pfx, m)
    if kind == "attention_2":
        return attention_2_mixer(h, W, pfx, m, eps)
    if kind == "latent_attention":
        return latent_attention_mixer(h, W, pfx, m, eps)
    raise ValueError(kind)


def forward(cfg, W, tokens, return_residuals=False):
    """cfg: the configuration as a dict; tokens: list of ids -> logits [T, vocab] (and the stream after every layer)."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    residuals = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = scalar_norm(x, W[p + "norm1"], eps)
        x = sublayer(x, h, mixer(layer["type"], h, W, p + "mix.", layer["mixer"], eps), W, p, 1, eps)
        if layer.get("mlp"):
            h = scalar_norm(x, W[p + "norm2"], eps)
            x = sublayer(x, h, dense_ff(h, W, p + "mlp."), W, p, 2, eps)
        residuals.append(x)
    logits = scalar_norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, residuals) if return_residuals else logits


# ------------------------------------------------------------------------------------------------ random checkpoints
def random_weights(cfg, seed=0, dtype=torch.float64):
    """Random weights of every tensor a configuration names, as bf16 numbers held in `dtype` (a checkpoint stores bf16)."""
    gen = torch.Generator().manual_seed(seed)
    C, V = int(cfg["width"]), int(cfg["vocab"])
    W = {}

    def mat(name, n_out, n_in, gain=1.0):
        W[name] = torch.randn(n_out, n_in, generator=gen) * (gain / math.sqrt(n_in))

    def vec(name, n, mean=0.0, spread=1.0):
        W[name] = mean + spread * torch.randn(n, generator=gen)

    def scalar(name, mean=1.0, spread=0.2):
        W[name] = (mean + spread * torch.randn((), generator=gen)).reshape(())

    W["embed"] = torch.randn(V, C, generator=gen) / float(cfg["embedding"]["scale"])
    mat("head", V, C)
    scalar("final.norm")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm1b"):
            scalar(p + n)
        vec(p + "ls1", C, 0.5, 0.2)
        mat(p + "rg1", C, C)
        vec(p + "rg1.b", C, 0.5, 0.5)
        x = p + "mix."
        if layer["type"] in ("attention", "attention_2"):
            H, G, D, E = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            mat(x + "q", H * D, C, 2.0), mat(x + "k", G * D, C, 2.0), mat(x + "v", G * E, C), mat(x + "g", H * E, C)
            mat(x + "o", C, H * E)
            if layer["type"] == "attention_2":
                vec(x + "q.b", H * D, 0.0, 0.3), vec(x + "k.b", G * D, 0.0, 0.3), vec(x + "v.b", G * E, 0.0, 0.3)
                vec(x + "q.norm", H * D, 1.0, 0.3), vec(x + "k.norm", G * D, 1.0, 0.3)
        else:
            H, D, P, E, R = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
            mat(x + "q", H * (D + P), C, 2.0), mat(x + "dkv", R + P, C, 2.0), vec(x + "dkv.norm", R, 1.0, 0.3)
            mat(x + "uk", H * D, R), mat(x + "uv", H * E, R), mat(x + "g", H, C), mat(x + "o", C, H * E)
        if layer.get("mlp"):
            F = int(layer["mlp"]["ff"])
            for n in ("norm2", "norm2b"):
                scalar(p + n)
            vec(p + "ls2", C, 0.5, 0.2)
            mat(p + "rg2", C, C)
            vec(p + "rg2.b", C, 0.5, 0.5)
            mat(p + "mlp.up", F, C, 1.5), mat(p + "mlp.down", C, F)
    return {k: v.to(torch.bfloat16).to(dtype) for k, v in W.items()}
