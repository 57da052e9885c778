"""Generation throughput of the Kelutar path beside the Llama path at equal size (`bench.py --workload generation`), of
Golavik beside Kelutar (`generation-golavik`), of Gubulorn beside Golavik (`generation-gubulorn`) and of Tokatar beside an
all-attention Kelutar (`generation-tokatar`).

Random weights, synthetic token ids. For each size: prefill tokens/s (a packed batch of whole prompts) and decode tokens/s
(one token per request and step, after a prompt of `context` tokens) for both decoders, plus a per-op table: every op
of one prefill step and one decode step is bracketed by CUDA events on the launching stream (the ops module's functions
are wrapped for the duration), its algorithmic bytes and FLOPs are counted from the shapes, and its distance from the
roofline max(bytes / measured copy bandwidth, FLOPs / measured bf16 peak) is reported, so that each Kelutar kernel can be
read against the like kernel of the Llama path. Timing: >= 3 warm-up steps, an L2 flush (a 256 MB fill) between timed
steps, CUDA events, synchronised on both sides."""
import json
import math
import os
import time

import torch

BF16, F32 = torch.bfloat16, torch.float32

# (name, width, layers, heads, head dim, window, ff, vocab): layers repeat hgrn2, hgrn2, hgrn2, attention(+ff)
SIZES = [
    ("w2048", 2048, 8, 16, 128, 1024, 8192, 32000),
    ("w4096", 4096, 4, 32, 128, 2048, 11008, 32000),
]


def kelutar_config(width, layers, heads, dim, window, ff, vocab, max_positions):
    ls = []
    for i in range(layers):
        if i % 4 == 3:
            ls.append({"type": "attention", "mixer": {"heads": heads, "kv_heads": heads, "dim": dim, "vdim": dim,
                                                      "mask": {"size": window}, "scale": 1.0 / math.sqrt(dim)},
                       "mlp": {"kind": "dense", "ff": ff}})
        else:
            ls.append({"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": dim}, "mlp": None})
    return {"architecture": "Kelutar", "vocab": vocab, "width": width, "max_positions": max_positions,
            "embedding": {"scale": math.sqrt(width)}, "norm": {"eps": 1e-5}, "canon": {"taps": 4}, "layers": ls}


def kelutar_random_weights(cfg, device, seed=0):
    g = torch.Generator(device=device).manual_seed(seed)
    C = cfg["width"]

    def mat(o, i, s=None):
        return (torch.randn(o, i, device=device, generator=g) * (s or 1.0 / math.sqrt(i))).to(BF16)

    def vec(n, mean=1.0, s=0.1):
        return (mean + torch.randn(n, device=device, generator=g) * s).to(BF16)

    W = {"embed": mat(cfg["vocab"], C, 1.0 / math.sqrt(C)), "pos": mat(cfg["max_positions"], C, 0.5),
         "final.norm": vec(C), "head": mat(cfg["vocab"], C)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = "l%d." % i, layer["mixer"]
        H, D = m["heads"], m["dim"]
        W[p + "norm1"], W[p + "canon1"] = vec(C), mat(C, cfg["canon"]["taps"], 0.3)
        if layer["type"] == "attention":
            G = m["kv_heads"]
            W.update({p + "mix.q": mat(H * D, C), p + "mix.q.b": vec(H * D, 0.0), p + "mix.k": mat(G * D, C),
                      p + "mix.k.b": vec(G * D, 0.0), p + "mix.q.norm": vec(D), p + "mix.k.norm": vec(D),
                      p + "mix.temp": vec(H), p + "mix.g": mat(H * D, C), p + "mix.o": mat(C, H * D)})
        else:
            E = m["vdim"]
            W.update({p + "mix.q": mat(H * D, C), p + "mix.f": mat(H * D, C), p + "mix.v": mat(H * E, C),
                      p + "mix.f.b": vec(H * D, 1.0, 1.0), p + "mix.lower": vec(H * D, 0.5, 0.1).clamp(0, 0.95),
                      p + "mix.norm": vec(E), p + "mix.o": mat(C, H * E)})
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            W.update({p + "norm2": vec(C), p + "mlp.up": mat(F, C), p + "mlp.down": mat(C, F)})
    return W


def llama_model(width, layers, heads, ff, vocab, max_positions):
    from llark_b200.models.llamav2 import WrappedLlamav2Config, WrappedLlamav2ForCausalLM

    hf = WrappedLlamav2Config(hidden_size=width, intermediate_size=ff, num_hidden_layers=layers,
                              num_attention_heads=heads, num_key_value_heads=heads, vocab_size=vocab,
                              max_position_embeddings=max_positions, rms_norm_eps=1e-5)
    hf.mm_hidden_size = 64
    old = torch.get_default_dtype()
    torch.set_default_dtype(BF16)
    try:
        with torch.device("cuda"):
            model = WrappedLlamav2ForCausalLM(hf)
    finally:
        torch.set_default_dtype(old)
    return model.to(BF16).eval()


class _Flush:
    def __init__(self):
        self.buf = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)

    def __call__(self):
        self.buf.fill_(1)


def timed(fn, warmup, iters, flush, setup=None):
    """Median ms of fn() over iters, each after setup() and an L2 flush, CUDA events on the current stream."""
    ms = []
    for i in range(warmup + iters):
        if setup is not None:
            setup()
        flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            ms.append(e0.elapsed_time(e1))
    ms.sort()
    return ms[len(ms) // 2]


class OpTimer:
    """Wraps the named functions of llark_b200.ops with CUDA-event brackets while active."""

    def __init__(self, names):
        from llark_b200 import ops

        self.ops, self.names, self.saved, self.records, self.depth = ops, names, {}, [], 0

    def __enter__(self):
        for n in self.names:
            f = getattr(self.ops, n)
            self.saved[n] = f

            def wrap(*a, __f=f, __n=n, **k):
                if self.depth:  # an op that another timed op calls is part of that one
                    return __f(*a, **k)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                self.depth += 1
                try:
                    out = __f(*a, **k)
                finally:
                    self.depth -= 1
                e1.record()
                self.records.append((__n, e0, e1, a, k, out))
                return out

            setattr(self.ops, n, wrap)
        return self

    def __exit__(self, *exc):
        for n, f in self.saved.items():
            setattr(self.ops, n, f)
        torch.cuda.synchronize()


def _nbytes(x):
    if torch.is_tensor(x):
        return x.numel() * x.element_size()
    if isinstance(x, (tuple, list)):
        return sum(_nbytes(y) for y in x)
    return 0


def _op_work(name, a, k, out, ctx):
    """(algorithmic bytes, FLOPs) of one recorded call. Stores that are only partly touched (rings, states, KV caches)
    are counted by what the op has to read and write, the rest by the tensors handed in and out."""
    if name in ("linear", "gemm", "gemv"):
        x, w = a[0], a[1]
        M, K = x.shape[0], x.shape[1]
        N = k.get("N") or w.shape[0]
        return _nbytes(x) + N * K * w.element_size() + _nbytes(out), 2.0 * M * N * K
    if name == "seq_swa_attn":
        qn, st, H, G, D, E, window = a[0], a[8], a[9], a[10], a[11], a[12], a[13]
        chunk = k.get("chunk") or 0
        if chunk:  # a query sees its own block of positions up to itself; the step reads its blocks' keys once
            keys = sum((p0 + i) % chunk + 1 for p0, n in zip(st.pos0_host, st.lens) for i in range(n))
            kv_once = sum(n + min(p0 % chunk, p0) for p0, n in zip(st.pos0_host, st.lens)) * G * (D + E) * 2
            return 2 * _nbytes(qn) + kv_once + st.n_tok * H * E * 4, 2.0 * keys * H * (D + E)
        keys = sum(min(window, p0 + i + 1) for p0, n in zip(st.pos0_host, st.lens) for i in range(n))
        kv_once = sum(min(n + min(window, p0), n + window) for p0, n in zip(st.pos0_host, st.lens)) * G * (D + E) * 2
        return 2 * _nbytes(qn) + kv_once + st.n_tok * H * E * 4, 2.0 * keys * H * (D + E)
    if name == "attn_fwd":
        qkv, B, S, NH, D = a[0], a[2], a[3], a[4], a[5]
        return _nbytes(qkv) + B * S * NH * D * 2, 4.0 * B * NH * D * S * (S + 1) / 2
    if name == "attn_decode":
        q, lens_ctx = a[0], ctx["context"]
        B, H = q.shape
        return 2 * B * lens_ctx * H * 2 + 2 * _nbytes(q), 4.0 * B * lens_ctx * H
    if name == "seq_glr_scan":
        src, state, st, H, D, E = a[0], a[5], a[6], a[7], a[8], a[9]
        return _nbytes(src) + 2 * st.n_seq * H * D * E * 4 + st.n_tok * H * E * 4, 5.0 * st.n_tok * H * D * E
    if name == "seq_delta_scan":
        vec, v, state, st, H, D, E = a[0], a[1], a[2], a[3], a[4], a[5], a[6]
        per = 9.0 if k.get("correct", True) else 5.0  # without the correction: decay, write and read-out only
        return (_nbytes(vec) + st.n_tok * H * E * 8 + 2 * st.n_seq * H * D * E * 4), per * st.n_tok * H * D * E
    if name == "seq_moe_experts":
        x, ids, wgu, wd = a[0], a[1], a[2], a[3]
        n_ent, (n_exp, ff2, C) = ids.numel(), wgu.shape
        hit = min(n_exp, n_ent)
        return (hit * (ff2 * C + C * ff2 // 2) * wgu.element_size() + n_ent * C * (x.element_size() + 4)
                + n_ent * ff2 * x.element_size()), 2.0 * n_ent * 3 * (ff2 // 2) * C
    if name == "seq_head_linear":
        x, w, y, N, K = a[0], a[2], a[3], k["N"], k["K"]
        M, H = x.shape[0], w.shape[0]
        return M * H * (K * x.element_size() + N * y.element_size()) + _nbytes(w), 2.0 * M * H * N * K
    if name == "seq_short_conv":
        return _nbytes(a[0]) + _nbytes(out), 0.0
    if name == "seq_qk_headnorm":
        return _nbytes(a[0]) * 2 // 3 + _nbytes(out), 0.0
    if name == "seq_qkv_rotary":  # reads the q | k | v columns of the fused projection, writes them in the activation dtype
        return 3 * _nbytes(out), 0.0
    if name == "seq_kv_ring_write":
        return 2 * (_nbytes(a[0]) + _nbytes(a[1])), 0.0
    if name == "embed_splice_fwd":
        return 2 * _nbytes(a[6]), 0.0
    if name == "seq_embed":
        return 3 * _nbytes(out), 0.0
    if name == "rope_":
        return 2 * _nbytes(a[0]) * 2 // 3, 0.0
    tensors = [x for x in a if torch.is_tensor(x)] + [v for v in k.values() if torch.is_tensor(v)]
    return sum(_nbytes(t) for t in tensors) + (_nbytes(out) if not any(out is t for t in tensors) else 0), 0.0


def op_table(records, ctx, peaks):
    bw, fl = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    agg = {}
    for name, e0, e1, a, k, out in records:
        if name == "gemm" and ctx.get("skip_gemm"):
            continue  # already inside `linear`
        ms = e0.elapsed_time(e1)
        nb, flops = _op_work(name, a, k, out, ctx)
        if name == "linear":
            name = "linear_rows" if a[0].shape[0] <= 8 else "linear_tcgen05"
        if name == "gemm":
            name = "gemm_tcgen05"
        d = agg.setdefault(name, {"calls": 0, "ms": 0.0, "bytes": 0, "flops": 0.0, "roof_ms": 0.0})
        d["calls"] += 1
        d["ms"] += ms
        d["bytes"] += nb
        d["flops"] += flops
        d["roof_ms"] += max(nb / bw, flops / fl) * 1e3
    for d in agg.values():
        d["of_roofline"] = round(d["roof_ms"] / d["ms"], 4) if d["ms"] > 0 else None
        d["ms"], d["roof_ms"] = round(d["ms"], 4), round(d["roof_ms"], 4)
        d["gb_s"] = round(d["bytes"] / (d["ms"] * 1e-3) / 1e9, 1) if d["ms"] > 0 else None
        d["tflops"] = round(d["flops"] / (d["ms"] * 1e-3) / 1e12, 2) if d["ms"] > 0 else None
        del d["bytes"], d["flops"]
    return agg


KELUTAR_OPS = ["linear", "seq_embed", "seq_short_conv", "seq_add_rmsnorm", "seq_rmsnorm_rows", "seq_relu2",
               "seq_qk_headnorm", "seq_swa_attn", "seq_kv_ring_write", "seq_glr_scan", "seq_head_rmsnorm"]
LLAMA_OPS = ["gemm", "gemv", "rmsnorm_fwd", "rope_", "attn_fwd", "attn_decode", "swiglu_fwd", "embed_splice_fwd"]


GOLAVIK_OPS = ["linear", "linear_w32", "seq_embed", "seq_short_conv", "seq_group_rmsnorm", "seq_residual_combine",
               "seq_conv_act", "seq_delta_prep", "seq_delta_scan", "seq_head_norm_gate", "seq_latent_prep",
               "seq_head_linear", "seq_swa_attn", "seq_kv_ring_write", "seq_moe_route", "seq_moe_experts", "seq_tanh"]

# (name, width, layers, heads, head dim, window, experts, top, expert ff, latent rank, rotated size, vocab): layers repeat
# latent_attention, channel_delta, general_delta, channel_delta, each with a routed feed-forward; the Kelutar model beside it
# has the same width, layer count, heads and window, and a dense feed-forward of top x expert-ff rows on its attention layers
GOLAVIK_SIZES = [
    ("g2048", 2048, 4, 16, 128, 1024, 32, 4, 1024, 192, 64, 32000),
    ("g4096", 4096, 4, 32, 128, 2048, 64, 6, 1024, 192, 64, 32000),
]


def golavik_config(width, layers, heads, dim, window, experts, top, ff, rank, rot, vocab):
    moe = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": 8, "keep": 4}}}
    kinds = [
        {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": dim, "kv_rank": rank,
                                               "scale": 1.0 / math.sqrt(dim + rot), "mask": {"size": window},
                                               "rot": {"base": 10000.0, "dims": rot,
                                                       "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0,
                                                                   "slow": 1.0}}}},
        {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": heads, "dim": dim, "vdim": dim, "conv": 4}},
        {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}},
        {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": heads, "dim": dim, "vdim": dim, "conv": 4}}]
    return {"architecture": "Golavik", "vocab": vocab, "width": width, "norm": {"eps": 1e-5, "groups": 2},
            "canon": {"taps": 4}, "loop": None,
            "layers": [dict(kinds[i % 4], mlp=moe) for i in range(layers)]}


def golavik_random_weights(cfg, device, seed=0, low_rank=64):
    g = torch.Generator(device=device).manual_seed(seed)
    C = cfg["width"]

    def mat(o, i, s=None):
        return (torch.randn(o, i, device=device, generator=g) * (s or 1.0 / math.sqrt(i))).to(BF16)

    def vec(n, mean=1.0, s=0.1):
        return (mean + torch.randn(n, device=device, generator=g) * s).to(BF16)

    W = {"embed": mat(cfg["vocab"], C, 1.0 / math.sqrt(C)), "final.norm": vec(C)}
    taps = cfg["canon"]["taps"]
    for i, layer in enumerate(cfg["layers"]):
        p, m = "l%d." % i, layer["mixer"]
        x = p + "mix."
        W[p + "norm1"], W[p + "canon1"], W[p + "canon2"] = vec(C), mat(C, taps, 0.3), mat(C, taps, 0.3)
        H, D = m["heads"], m["dim"]
        if layer["type"] == "latent_attention":
            P, E, R = m["rot_dim"], m["vdim"], m["kv_rank"]
            W.update({x + "q": mat(H * (D + P), C), x + "dkv": mat(R + P, C), x + "dkv.norm": vec(R),
                      x + "uk": mat(H * D, R), x + "uv": mat(H * E, R), x + "g": mat(H * E, C), x + "o": mat(C, H * E)})
        elif layer["type"] == "channel_delta":
            G, E = m["kv_heads"], m["vdim"]
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * E)):
                W[x + n], W[x + n + ".conv"] = mat(rows, C), mat(rows, m["conv"], 0.5)
            W.update({x + "b": mat(H, C), x + "A_log": vec(H, -1.0, 0.5), x + "norm": vec(E), x + "a1": mat(low_rank, C),
                      x + "a2": mat(H * D, low_rank), x + "dt_bias": vec(H * D, -1.0, 1.0), x + "g1": mat(low_rank, C),
                      x + "g2": mat(H * E, low_rank), x + "o": mat(C, H * E)})
        else:
            for n in ("r", "k", "v", "a", "g"):
                W[x + n] = mat(H * D, C)
            W.update({x + "a.b": vec(H * D, 0.0, 0.5), x + "w1": mat(low_rank, C), x + "w2": mat(H * D, low_rank),
                      x + "w0": vec(H * D, -0.5, 1.0), x + "norm": vec(H * D), x + "o": mat(C, H * D)})
        r, f = layer["mlp"]["router"], layer["mlp"]["expert"]["ff"]
        W[p + "mlp.router"] = mat(r["experts"], C)
        for e in range(r["experts"]):
            W.update({"%smlp.e%d.gate" % (p, e): mat(f, C), "%smlp.e%d.up" % (p, e): mat(f, C),
                      "%smlp.e%d.down" % (p, e): mat(C, f)})
    return W


def bench_native(tag, eng, op_names, out, vocab, peaks, steps, warmup, flush, g, prefill_batch, prompt, decode_batches,
                 context):
    """Prefill and decode timings and op tables of one native decoder (an engine with step / new_cache) into out."""
    state = {}

    def setup_prefill():
        state["cache"] = eng.new_cache(n_slots=prefill_batch)
        state["slots"] = [state["cache"].alloc() for _ in range(prefill_batch)]

    toks = torch.randint(0, vocab, (prefill_batch, prompt), generator=torch.Generator().manual_seed(0)).tolist()
    ms = timed(lambda: eng.step(state["cache"], state["slots"], toks), warmup, steps, flush, setup=setup_prefill)
    out["prefill"][tag + "_tokens_per_s"] = round(prefill_batch * prompt / ms * 1e3, 1)
    out["prefill"][tag + "_ms"] = round(ms, 3)
    for _ in range(2):  # the second pass is the one that is read: no first-use cost of the wrappers
        setup_prefill()
        with OpTimer(op_names) as t:
            eng.step(state["cache"], state["slots"], toks)
    out["prefill"][tag + "_ops"] = op_table(t.records, {}, peaks)
    state.clear()
    for B in decode_batches:
        cache = eng.new_cache(n_slots=B)
        slots = [cache.alloc() for _ in range(B)]
        eng.step(cache, slots, torch.randint(0, vocab, (B, context), generator=g).tolist())
        nxt = torch.randint(0, vocab, (B, 1), generator=g).tolist()
        ms = timed(lambda: eng.step(cache, slots, nxt), warmup, max(steps, 10), flush)
        out["decode"]["%s_b%d_tokens_per_s" % (tag, B)] = round(B / ms * 1e3, 1)
        out["decode"]["%s_b%d_ms" % (tag, B)] = round(ms, 3)
        if B == decode_batches[-1] or B == 8:
            for _ in range(2):
                with OpTimer(op_names) as t:
                    eng.step(cache, slots, nxt)
            out["decode"]["%s_b%d_ops" % (tag, B)] = op_table(t.records, {"context": context}, peaks)
        del cache
    torch.cuda.empty_cache()


def bench_size_golavik(name, width, layers, heads, dim, window, experts, top, ff, rank, rot, vocab, peaks, steps, warmup,
                       prefill_batch=4, prompt=2048, decode_batches=(1, 8, 32), context=1024):
    """Golavik beside Kelutar (the closest existing decoder: a layer list of recurrences and window attention on the same
    step function, cache and linears) at equal width, layer count, heads and window."""
    from llark_b200.models.golavik import GolavikConfig, GolavikForCausalLM
    from llark_b200.models.kelutar import KelutarConfig, KelutarForCausalLM

    flush = _Flush()
    out = {"size": name, "width": width, "layers": layers, "heads": heads, "head_dim": dim, "window": window,
           "experts": experts, "top": top, "expert_ff": ff, "kv_rank": rank, "rot_dim": rot, "vocab": vocab,
           "prefill": {"batch": prefill_batch, "prompt": prompt}, "decode": {"context": context}}
    g = torch.Generator().manual_seed(0)
    cfg = golavik_config(width, layers, heads, dim, window, experts, top, ff, rank, rot, vocab)
    gm = GolavikForCausalLM(GolavikConfig.from_dict(cfg), golavik_random_weights(cfg, "cuda"), dtype=BF16)
    bench_native("golavik", gm.engine, GOLAVIK_OPS, out, vocab, peaks, steps, warmup, flush, g, prefill_batch, prompt,
                 decode_batches, context)
    del gm
    torch.cuda.empty_cache()
    kcfg = kelutar_config(width, layers, heads, dim, window, top * ff, vocab, max(prompt, context) + 64)
    km = KelutarForCausalLM(KelutarConfig.from_dict(kcfg), kelutar_random_weights(kcfg, "cuda"), dtype=BF16)
    bench_native("kelutar", km.engine, KELUTAR_OPS, out, vocab, peaks, steps, warmup, flush, g, prefill_batch, prompt,
                 decode_batches, context)
    del km
    torch.cuda.empty_cache()
    return out


def run_golavik(args, peaks, peaks_kind, emit):
    from llark_b200 import ops

    ops.init()
    t0 = time.time()
    sizes = [s for s in GOLAVIK_SIZES if not os.environ.get("LLARK_BENCH_SIZE") or s[0] == os.environ["LLARK_BENCH_SIZE"]]
    results = [bench_size_golavik(*s, peaks=peaks, steps=args.steps, warmup=max(args.warmup, 3)) for s in sizes]
    head = results[0]
    emit({"metric": "generation tokens/s, Golavik beside Kelutar at equal size (prefill of %d x %d tokens)"
                    % (head["prefill"]["batch"], head["prefill"]["prompt"]),
          "value": head["prefill"]["golavik_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
          "warmup": max(args.warmup, 3), "ms_per_step": head["prefill"]["golavik_ms"], "higher_is_better": True,
          "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights",
          "config": {"model": "Golavik " + head["size"], "l2": "256 MB fill between timed steps",
                     "peaks": peaks_kind, "hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"]},
          "sizes": results, "wall_s": round(time.time() - t0, 1)})


GUBULORN_OPS = ["linear", "linear_w32", "seq_embed", "seq_post_norm", "seq_rmsnorm_rows", "seq_conv_act", "seq_delta_prep",
                "seq_delta_scan", "seq_head_norm_gate", "seq_skip_gate_group_norm", "seq_qkv_headnorm", "seq_swa_attn",
                "seq_kv_ring_write", "seq_moe_route", "seq_moe_experts", "seq_glu_clamped", "seq_logit_cap_"]

# (name, width, layers, heads, head dim, experts, pass-through experts, top, expert ff, state-space heads, state size,
# vocab): layers repeat delta, parallel, parallel, delta, each with a routed feed-forward except the first (a clamped gated
# unit of top x expert-ff rows); the state-space side has heads of 64 channels. The Golavik model beside it has the same
# width, layer count, heads, head size, experts, top and expert ff, and a window as long as the prompt.
GUBULORN_SIZES = [
    ("u2048", 2048, 4, 16, 128, 32, 8, 4, 1024, 64, 128, 32000),
    ("u4096", 4096, 4, 32, 128, 64, 8, 6, 1024, 128, 128, 32000),
]


def gubulorn_config(width, layers, heads, dim, experts, through, top, ff, ss_heads, state, vocab):
    moe = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "identity": through, "top": top, "groups": {"count": 8, "keep": 4}}}
    delta = {"type": "delta", "mixer": {"heads": heads, "kv_heads": heads, "dim": dim, "vdim": dim, "conv": 4}}
    par = {"type": "parallel",
           "mixer": {"left": {"heads": heads, "kv_heads": max(heads // 4, 1), "dim": dim, "vdim": dim,
                              "scale": 1.0 / math.sqrt(dim), "q_temp": {"coef": 0.1, "every": 512}},
                     "right": {"heads": ss_heads, "vdim": 64, "state": state, "groups": 8, "norm_groups": 8, "conv": 4}}}
    kinds = [delta, par, par, delta]
    ls = [dict(kinds[i % 4], mlp=moe) for i in range(layers)]
    ls[0]["mlp"] = {"kind": "dense", "ff": top * ff, "limit": 7.0}
    return {"architecture": "Gubulorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "postln_alpha": 2.0,
            "logit_scale": 1.0, "logit_softcap": 30.0, "layers": ls}


def gubulorn_random_weights(cfg, device, seed=0):
    g = torch.Generator(device=device).manual_seed(seed)
    C = cfg["width"]

    def mat(o, i, s=None):
        return (torch.randn(o, i, device=device, generator=g) * (s or 1.0 / math.sqrt(i))).to(BF16)

    def vec(n, mean=1.0, s=0.1):
        return (mean + torch.randn(n, device=device, generator=g) * s).to(BF16)

    W = {"embed": mat(cfg["vocab"], C, 1.0), "embed.norm": vec(C, 0.0), "final.norm": vec(C, 0.0),
         "head": mat(cfg["vocab"], C)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = "l%d." % i, layer["mixer"]
        x = p + "mix."
        W[p + "norm1"], W[p + "norm2"] = vec(C, 0.0), vec(C, 0.0)
        if layer["type"] == "delta":
            H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * E)):
                W[x + n], W[x + n + ".conv"] = mat(rows, C), mat(rows, m["conv"], 0.5)
            W.update({x + "b": mat(H, C), x + "a": mat(H, C), x + "A_log": vec(H, -1.0, 0.5), x + "dt_bias": vec(H, -1.0, 1.0),
                      x + "norm": vec(E), x + "g": mat(H * E, C), x + "o": mat(C, H * E)})
        else:
            a, b = m["left"], m["right"]
            H, G, D, E = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            W.update({x + "left.q": mat(H * D, C), x + "left.k": mat(G * D, C), x + "left.v": mat(G * E, C),
                      x + "left.q.norm": vec(D), x + "left.k.norm": vec(D), x + "left.sink": vec(H, 0.0, 1.0),
                      x + "left.g": mat(H, C), x + "left.o": mat(C, H * E), x + "left.out": vec(C)})
            Hs, Es, N, Gs = b["heads"], b["vdim"], b["state"], b["groups"]
            inner, nc = Hs * Es, Hs * Es + 2 * Gs * N
            W.update({x + "right.in": mat(2 * inner + 2 * Gs * N + Hs, C), x + "right.conv": mat(nc, b["conv"], 0.5),
                      x + "right.conv.b": vec(nc, 0.0, 0.3), x + "right.dt_bias": vec(Hs, -1.0, 1.0),
                      x + "right.A_log": vec(Hs, -1.0, 0.5), x + "right.D": vec(Hs), x + "right.norm": vec(inner),
                      x + "right.o": mat(C, inner), x + "right.out": vec(C)})
        mlp = layer["mlp"]
        if mlp["kind"] == "dense":
            W.update({p + "mlp.gate": mat(mlp["ff"], C), p + "mlp.up": mat(mlp["ff"], C), p + "mlp.down": mat(C, mlp["ff"])})
        else:
            r, f = mlp["router"], mlp["expert"]["ff"]
            W[p + "mlp.router"] = mat(r["experts"] + r["identity"], C)
            W[p + "mlp.correction"] = vec(r["experts"] + r["identity"], 0.0, 0.01)
            for e in range(r["experts"]):
                W.update({"%smlp.e%d.gate" % (p, e): mat(f, C), "%smlp.e%d.up" % (p, e): mat(f, C),
                          "%smlp.e%d.down" % (p, e): mat(C, f)})
    return W


def bench_size_gubulorn(name, width, layers, heads, dim, experts, through, top, ff, ss_heads, state, vocab, peaks, steps,
                        warmup, prefill_batch=4, prompt=2048, decode_batches=(1, 8, 32), context=1024):
    """Gubulorn beside Golavik (the closest existing decoder: delta-rule scans, attention over a per-slot store and routed
    experts on the same step function, cache and linears) at equal width, layer count, heads, experts and expert size."""
    from llark_b200.models.golavik import GolavikConfig, GolavikForCausalLM
    from llark_b200.models.gubulorn import GubulornConfig, GubulornForCausalLM

    flush = _Flush()
    out = {"size": name, "width": width, "layers": layers, "heads": heads, "head_dim": dim, "experts": experts,
           "pass_through_experts": through, "top": top, "expert_ff": ff, "state_space_heads": ss_heads, "state": state,
           "vocab": vocab, "prefill": {"batch": prefill_batch, "prompt": prompt}, "decode": {"context": context}}
    g = torch.Generator().manual_seed(0)
    cfg = gubulorn_config(width, layers, heads, dim, experts, through, top, ff, ss_heads, state, vocab)
    um = GubulornForCausalLM(GubulornConfig.from_dict(cfg), gubulorn_random_weights(cfg, "cuda"), dtype=BF16)
    um.engine.max_positions = max(prompt, context) + 64
    bench_native("gubulorn", um.engine, GUBULORN_OPS, out, vocab, peaks, steps, warmup, flush, g, prefill_batch, prompt,
                 decode_batches, context)
    del um
    torch.cuda.empty_cache()
    gcfg = golavik_config(width, layers, heads, dim, max(prompt, context), experts, top, ff, 192, 64, vocab)
    gm = GolavikForCausalLM(GolavikConfig.from_dict(gcfg), golavik_random_weights(gcfg, "cuda"), dtype=BF16)
    bench_native("golavik", gm.engine, GOLAVIK_OPS, out, vocab, peaks, steps, warmup, flush, g, prefill_batch, prompt,
                 decode_batches, context)
    del gm
    torch.cuda.empty_cache()
    return out


def run_gubulorn(args, peaks, peaks_kind, emit):
    from llark_b200 import ops

    ops.init()
    t0 = time.time()
    sizes = [s for s in GUBULORN_SIZES if not os.environ.get("LLARK_BENCH_SIZE") or s[0] == os.environ["LLARK_BENCH_SIZE"]]
    results = [bench_size_gubulorn(*s, peaks=peaks, steps=args.steps, warmup=max(args.warmup, 3)) for s in sizes]
    head = results[0]
    emit({"metric": "generation tokens/s, Gubulorn beside Golavik at equal size (prefill of %d x %d tokens)"
                    % (head["prefill"]["batch"], head["prefill"]["prompt"]),
          "value": head["prefill"]["gubulorn_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
          "warmup": max(args.warmup, 3), "ms_per_step": head["prefill"]["gubulorn_ms"], "higher_is_better": True,
          "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights",
          "config": {"model": "Gubulorn " + head["size"], "l2": "256 MB fill between timed steps",
                     "peaks": peaks_kind, "hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"]},
          "sizes": results, "wall_s": round(time.time() - t0, 1)})


TOKATAR_OPS = ["linear", "seq_embed", "seq_group_rmsnorm", "seq_gated_norm_add", "seq_relu2", "seq_qkv_rotary", "seq_swa_attn",
               "seq_kv_ring_write", "seq_latent_prep", "seq_head_linear"]

# (name, width, layers, heads, key/value heads, head dim, block of positions, ff, latent rank, rotated size, vocab): layers
# repeat attention, attention_2, latent_attention, attention, each with a dense feed-forward; the Kelutar model beside it has
# an attention layer with the same feed-forward in EVERY place (same width, layer count, heads, key / value heads, and a
# window as long as the block)
TOKATAR_SIZES = [
    ("t2048", 2048, 8, 16, 4, 128, 2048, 8192, 192, 64, 32000),
    ("t4096", 4096, 4, 32, 8, 128, 2048, 11008, 192, 64, 32000),
]


def tokatar_config(width, layers, heads, kv, dim, block, ff, rank, rot, vocab):
    mlp = {"kind": "dense", "ff": ff}
    scale = 1.0 / math.sqrt(dim)
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "mask": {"size": block}, "scale": scale,
                     "softcap": 30.0, "rot": {"base": 100000.0, "dims": dim,
                                              "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    att2 = {"type": "attention_2", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": heads, "dim": dim, "vdim": dim, "mask": {"size": block}, "scale": scale,
                      "rot": {"base": 1000000.0, "dims": dim}}}
    lat = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": dim, "kv_rank": rank,
                     "scale": 1.0 / math.sqrt(dim + rot), "rot": {"base": 10000.0, "dims": rot}}}
    return {"architecture": "Tokatar", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"scale": math.sqrt(width)}, "layers": [(att, att2, lat, att)[i % 4] for i in range(layers)]}


def tokatar_random_weights(cfg, device, seed=0):
    g = torch.Generator(device=device).manual_seed(seed)
    C = cfg["width"]

    def mat(o, i, s=None):
        return (torch.randn(o, i, device=device, generator=g) * (s or 1.0 / math.sqrt(i))).to(BF16)

    def vec(n, mean=1.0, s=0.1):
        return (mean + torch.randn(n, device=device, generator=g) * s).to(BF16)

    def one(mean=1.0):
        return vec(1, mean).reshape(())

    W = {"embed": mat(cfg["vocab"], C, 1.0 / math.sqrt(C)), "final.norm": one(), "head": mat(cfg["vocab"], C)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = "l%d." % i, layer["mixer"]
        for k in ("1", "2"):
            W.update({p + "norm" + k: one(), p + "norm" + k + "b": one(), p + "ls" + k: vec(C, 0.5), p + "rg" + k: mat(C, C),
                      p + "rg" + k + ".b": vec(C, 0.5, 0.5)})
        H, D, E = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "latent_attention":
            R, P = m["kv_rank"], m["rot_dim"]
            W.update({p + "mix.q": mat(H * (D + P), C), p + "mix.dkv": mat(R + P, C), p + "mix.dkv.norm": vec(R),
                      p + "mix.uk": mat(H * D, R), p + "mix.uv": mat(H * E, R), p + "mix.g": mat(H, C),
                      p + "mix.o": mat(C, H * E)})
        else:
            G = m["kv_heads"]
            W.update({p + "mix.q": mat(H * D, C), p + "mix.k": mat(G * D, C), p + "mix.v": mat(G * E, C),
                      p + "mix.g": mat(H * E, C), p + "mix.o": mat(C, H * E)})
            if layer["type"] == "attention_2":
                W.update({p + "mix.q.b": vec(H * D, 0.0), p + "mix.k.b": vec(G * D, 0.0), p + "mix.v.b": vec(G * E, 0.0),
                          p + "mix.q.norm": vec(H * D), p + "mix.k.norm": vec(G * D)})
        F = layer["mlp"]["ff"]
        W.update({p + "mlp.up": mat(F, C), p + "mlp.down": mat(C, F)})
    return W


def kelutar_attention_config(width, layers, heads, kv, dim, window, ff, vocab, max_positions):
    """A Kelutar model whose every layer is its window attention with a dense feed-forward."""
    cfg = kelutar_config(width, layers, heads, dim, window, ff, vocab, max_positions)
    cfg["layers"] = [{"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim,
                                                     "mask": {"size": window}, "scale": 1.0 / math.sqrt(dim)},
                      "mlp": {"kind": "dense", "ff": ff}} for _ in range(layers)]
    return cfg


def bench_size_tokatar(name, width, layers, heads, kv, dim, block, ff, rank, rot, vocab, peaks, steps, warmup,
                       prefill_batch=4, prompt=2048, decode_batches=(1, 8, 32), context=1024):
    """Tokatar beside Kelutar with attention in every layer (the closest existing decoder: the same attention kernels,
    squared-ReLU feed-forward, step function, cache and linears) at equal width, layer count, heads and feed-forward."""
    from llark_b200.models.kelutar import KelutarConfig, KelutarForCausalLM
    from llark_b200.models.tokatar import TokatarConfig, TokatarForCausalLM

    flush = _Flush()
    out = {"size": name, "width": width, "layers": layers, "heads": heads, "kv_heads": kv, "head_dim": dim, "block": block,
           "ff": ff, "kv_rank": rank, "rot_dim": rot, "vocab": vocab,
           "prefill": {"batch": prefill_batch, "prompt": prompt}, "decode": {"context": context}}
    g = torch.Generator().manual_seed(0)
    cfg = tokatar_config(width, layers, heads, kv, dim, block, ff, rank, rot, vocab)
    tm = TokatarForCausalLM(TokatarConfig.from_dict(cfg), tokatar_random_weights(cfg, "cuda"), dtype=BF16)
    tm.engine.max_positions = max(prompt, context) + 64
    bench_native("tokatar", tm.engine, TOKATAR_OPS, out, vocab, peaks, steps, warmup, flush, g, prefill_batch, prompt,
                 decode_batches, context)
    del tm
    torch.cuda.empty_cache()
    kcfg = kelutar_attention_config(width, layers, heads, kv, dim, block, ff, vocab, max(prompt, context) + 64)
    km = KelutarForCausalLM(KelutarConfig.from_dict(kcfg), kelutar_random_weights(kcfg, "cuda"), dtype=BF16)
    bench_native("kelutar", km.engine, KELUTAR_OPS, out, vocab, peaks, steps, warmup, flush, g, prefill_batch, prompt,
                 decode_batches, context)
    del km
    torch.cuda.empty_cache()
    return out


def run_tokatar(args, peaks, peaks_kind, emit):
    from llark_b200 import ops

    ops.init()
    t0 = time.time()
    sizes = [s for s in TOKATAR_SIZES if not os.environ.get("LLARK_BENCH_SIZE") or s[0] == os.environ["LLARK_BENCH_SIZE"]]
    results = [bench_size_tokatar(*s, peaks=peaks, steps=args.steps, warmup=max(args.warmup, 3)) for s in sizes]
    head = results[0]
    emit({"metric": "generation tokens/s, Tokatar beside an all-attention Kelutar at equal size (prefill of %d x %d tokens)"
                    % (head["prefill"]["batch"], head["prefill"]["prompt"]),
          "value": head["prefill"]["tokatar_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
          "warmup": max(args.warmup, 3), "ms_per_step": head["prefill"]["tokatar_ms"], "higher_is_better": True,
          "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights",
          "config": {"model": "Tokatar " + head["size"], "l2": "256 MB fill between timed steps",
                     "peaks": peaks_kind, "hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"]},
          "sizes": results, "wall_s": round(time.time() - t0, 1)})


def bench_size(name, width, layers, heads, dim, window, ff, vocab, peaks, steps, warmup, prefill_batch=4,
               prompt=2048, decode_batches=(1, 8, 32), context=1024):
    from llark_b200.models.kelutar import KelutarConfig, KelutarForCausalLM

    flush = _Flush()
    max_pos = max(prompt, context) + 64
    out = {"size": name, "width": width, "layers": layers, "heads": heads, "head_dim": dim, "window": window, "ff": ff,
           "vocab": vocab, "prefill": {"batch": prefill_batch, "prompt": prompt}, "decode": {"context": context}}
    g = torch.Generator().manual_seed(0)
    ids_prefill = torch.randint(0, vocab, (prefill_batch, prompt), generator=g)
    # ------------------------------------------------------------------ Kelutar
    cfg = kelutar_config(width, layers, heads, dim, window, ff, vocab, max_pos)
    km = KelutarForCausalLM(KelutarConfig.from_dict(cfg), kelutar_random_weights(cfg, "cuda"), dtype=BF16)
    eng = km.engine
    state = {}

    def k_setup_prefill():
        state["cache"] = eng.new_cache(n_slots=prefill_batch)
        state["slots"] = [state["cache"].alloc() for _ in range(prefill_batch)]

    toks = ids_prefill.tolist()
    ms = timed(lambda: eng.step(state["cache"], state["slots"], toks), warmup, steps, flush, setup=k_setup_prefill)
    out["prefill"]["kelutar_tokens_per_s"] = round(prefill_batch * prompt / ms * 1e3, 1)
    out["prefill"]["kelutar_ms"] = round(ms, 3)
    for _ in range(2):  # the second pass is the one that is read: no first-use cost of the wrappers
        k_setup_prefill()
        with OpTimer(KELUTAR_OPS) as t:
            eng.step(state["cache"], state["slots"], toks)
    out["prefill"]["kelutar_ops"] = op_table(t.records, {}, peaks)
    for B in decode_batches:
        cache = eng.new_cache(n_slots=B)
        slots = [cache.alloc() for _ in range(B)]
        eng.step(cache, slots, torch.randint(0, vocab, (B, context), generator=g).tolist())
        nxt = torch.randint(0, vocab, (B, 1), generator=g).tolist()
        ms = timed(lambda: eng.step(cache, slots, nxt), warmup, max(steps, 10), flush)
        out["decode"]["kelutar_b%d_tokens_per_s" % B] = round(B / ms * 1e3, 1)
        out["decode"]["kelutar_b%d_ms" % B] = round(ms, 3)
        if B == decode_batches[-1] or B == 8:
            for _ in range(2):
                with OpTimer(KELUTAR_OPS) as t:
                    eng.step(cache, slots, nxt)
            out["decode"]["kelutar_b%d_ops" % B] = op_table(t.records, {"context": context}, peaks)
    del km, eng, cache
    torch.cuda.empty_cache()
    # ------------------------------------------------------------------ Llama path at equal size
    lm = llama_model(width, layers, heads, ff, vocab, max_pos)
    le = lm.engine
    dev = torch.device("cuda")
    ids_dev = ids_prefill.to(dev)

    def l_setup_prefill():
        state["lc"] = le.new_cache(prefill_batch, max_pos, dev)

    ms = timed(lambda: le.prefill(ids_dev, None, state["lc"]), warmup, steps, flush, setup=l_setup_prefill)
    out["prefill"]["llama_tokens_per_s"] = round(prefill_batch * prompt / ms * 1e3, 1)
    out["prefill"]["llama_ms"] = round(ms, 3)
    for _ in range(2):
        l_setup_prefill()
        with OpTimer(LLAMA_OPS) as t:
            le.prefill(ids_dev, None, state["lc"])
    out["prefill"]["llama_ops"] = op_table(t.records, {}, peaks)
    for B in decode_batches:
        lc = le.new_cache(B, max_pos, dev)
        le.prefill(torch.randint(0, vocab, (B, context), generator=g).to(dev), None, lc)
        nxt = torch.randint(0, vocab, (B, 1), generator=g).to(dev)

        def l_step():
            lc.length = context
            le.decode_step(nxt, lc)

        ms = timed(l_step, warmup, max(steps, 10), flush)
        out["decode"]["llama_b%d_tokens_per_s" % B] = round(B / ms * 1e3, 1)
        out["decode"]["llama_b%d_ms" % B] = round(ms, 3)
        if B == decode_batches[-1] or B == 8:
            for _ in range(2):
                with OpTimer(LLAMA_OPS) as t:
                    l_step()
            out["decode"]["llama_b%d_ops" % B] = op_table(t.records, {"context": context}, peaks)
    del lm, le, lc
    torch.cuda.empty_cache()
    return out


def run(args, peaks, peaks_kind, emit):
    from llark_b200 import ops

    ops.init()
    t0 = time.time()
    sizes = [s for s in SIZES if not os.environ.get("LLARK_BENCH_SIZE") or s[0] == os.environ["LLARK_BENCH_SIZE"]]
    results = [bench_size(*s, peaks=peaks, steps=args.steps, warmup=max(args.warmup, 3)) for s in sizes]
    head = results[0]
    emit({"metric": "generation tokens/s, Kelutar beside the Llama path at equal size (prefill of %d x %d tokens)"
                    % (head["prefill"]["batch"], head["prefill"]["prompt"]),
          "value": head["prefill"]["kelutar_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
          "warmup": max(args.warmup, 3), "ms_per_step": head["prefill"]["kelutar_ms"], "higher_is_better": True,
          "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights",
          "config": {"model": "Kelutar " + head["size"], "l2": "256 MB fill between timed steps",
                     "peaks": peaks_kind, "hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"]},
          "sizes": results, "wall_s": round(time.time() - t0, 1)})
