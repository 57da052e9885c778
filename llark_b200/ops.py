"""Thin torch-tensor wrappers over the C-ABI (include/llark_b200.h).

PyTorch is plumbing here: it owns device memory and the current stream; every op below passes raw device
pointers + the stream to libllark_b200.so. There is no eager/PyTorch fallback: on a machine without the built
extension or without a GPU these raise.
"""
import ctypes
import math

import torch

from ._lib import EPI_QUICK_GELU, EPI_ROPE, EPI_SWIGLU_BWD, GemmEpilogue, check, lib

BF16 = torch.bfloat16

# bench.py sets this to a list: every gemm() launch then appends (start_event, end_event, flops, shape) recorded on the
# launching stream, which is how the roofline of the dominant kernel is measured live inside the timed region.
GEMM_PROFILE = None


_INITED = False


def init():
    """llark_init(): the one-time allocation + synchronisation of the library (tile-counter ring, TMA encoder), on the
    current device. Called once before the first GEMM so that no op of the hot loop allocates or synchronises."""
    global _INITED
    if not _INITED:
        check(lib().llark_init(), "llark_init")
        _INITED = True


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _req(t, dtype=None):
    if not t.is_cuda:
        raise RuntimeError("llark_b200 ops need CUDA tensors (no CPU fallback)")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"expected {dtype}, got {t.dtype}")
    return t


def gemm(a, b, *, a_mn=False, b_mn=False, M=None, N=None, K=None, out=None, out_dtype=None, bias=None,
         residual=None, lda=None, ldb=None, ldc=None, ldr=None, max_ctas=0, quick_gelu=False, rope=None,
         swiglu_bwd=None):
    """C[M,N] = A[M,K] @ B[N,K]^T (+bias) (+residual), optionally with one fused epilogue (llark_gemm_ex):

    quick_gelu=True            C = quick_gelu(acc + bias)
    rope=(cos, sin, S, cols)   columns [0, cols) rotated per 128-wide head, position = row % S (fused-QKV projection)
    swiglu_bwd=gu              acc is d(act) [M, I]; `out` must be the dgu buffer [M, 2I]: out = (dgate | dup)

    a: [M,K] (a_mn=False) or [K,M] (a_mn=True); b: [N,K] (b_mn=False) or [K,N] (b_mn=True); row-major with
    leading dimension = last-dim stride unless lda/ldb given. bf16 inputs use kind::f16, fp32 inputs kind::tf32.
    """
    _req(a), _req(b)
    if not _INITED:
        init()
    in_fp32 = a.dtype == torch.float32
    if a.dtype != b.dtype or a.dtype not in (BF16, torch.float32):
        raise TypeError("gemm inputs must both be bf16 or both fp32")
    if M is None:
        M = a.shape[1] if a_mn else a.shape[0]
    if K is None:
        K = a.shape[0] if a_mn else a.shape[1]
    if N is None:
        N = b.shape[1] if b_mn else b.shape[0]
    lda = lda if lda is not None else a.stride(0)
    ldb = ldb if ldb is not None else b.stride(0)
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype or (torch.float32 if in_fp32 else BF16))
    ldc = ldc if ldc is not None else out.stride(0)
    c_fp32 = out.dtype == torch.float32
    if residual is not None:
        if residual.dtype != out.dtype:
            raise TypeError("residual dtype must equal output dtype")
        ldr = ldr if ldr is not None else residual.stride(0)
    else:
        ldr = 0
    bias_fp32 = bias is not None and bias.dtype == torch.float32
    prof = GEMM_PROFILE
    if prof is not None:
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
    ep = None
    if quick_gelu:
        ep = GemmEpilogue(EPI_QUICK_GELU, None, None, 0, 0, 0)
    elif rope is not None:
        cos_t, sin_t, S_rope, cols = rope
        ep = GemmEpilogue(EPI_ROPE, cos_t.data_ptr(), sin_t.data_ptr(), 0, int(S_rope), int(cols))
    elif swiglu_bwd is not None:
        ep = GemmEpilogue(EPI_SWIGLU_BWD, swiglu_bwd.data_ptr(), None, swiglu_bwd.stride(0), 0, 0)
    if ep is None:
        rc = lib().llark_gemm(_p(a), int(a_mn), lda, _p(b), int(b_mn), ldb, _p(out), ldc, int(c_fp32), _p(bias),
                              int(bias_fp32), _p(residual), ldr, M, N, K, int(in_fp32), max_ctas, _stream())
    else:
        rc = lib().llark_gemm_ex(_p(a), int(a_mn), lda, _p(b), int(b_mn), ldb, _p(out), ldc, int(c_fp32), _p(bias),
                                 int(bias_fp32), _p(residual), ldr, M, N, K, int(in_fp32), max_ctas, ctypes.byref(ep),
                                 _stream())
    check(rc, f"llark_gemm(M={M},N={N},K={K})")
    if prof is not None:
        e1.record()
        prof.append((e0, e1, 2.0 * M * N * K, (M, N, K, int(a_mn), int(b_mn))))
    return out


def cast_f32_to_bf16(x, out=None):
    _req(x, torch.float32)
    x = x.contiguous()
    out = out if out is not None else torch.empty(x.shape, device=x.device, dtype=BF16)
    check(lib().llark_cast_f32_to_bf16(_p(x), _p(out), x.numel(), _stream()), "cast_f32_to_bf16")
    return out


def cast_bf16_to_f32(x, out=None):
    _req(x, BF16)
    x = x.contiguous()
    out = out if out is not None else torch.empty(x.shape, device=x.device, dtype=torch.float32)
    check(lib().llark_cast_bf16_to_f32(_p(x), _p(out), x.numel(), _stream()), "cast_bf16_to_f32")
    return out


def splice_scan(ids, start_id, end_id, frames, start_pos, flags):
    B, S = ids.shape
    check(lib().llark_splice_scan(_p(ids), B, S, start_id, end_id, _p(frames), _p(start_pos), _p(flags), _stream()),
          "splice_scan")


def embed_splice_fwd(ids, table, audio, audio_off, frames, start_pos, out):
    B, S = ids.shape
    H = table.shape[1]
    check(lib().llark_embed_splice_fwd(_p(ids), _p(table), _p(audio), _p(audio_off), _p(frames), _p(start_pos),
                                       _p(out), B, S, H, table.shape[0], _stream()), "embed_splice_fwd")
    return out


def embed_splice_bwd(ids, dout, daudio, audio_off, frames, start_pos, dtable, vocab, detach_text):
    B, S = ids.shape
    H = dout.shape[-1]
    check(lib().llark_embed_splice_bwd(_p(ids), _p(dout), _p(daudio), _p(audio_off), _p(frames), _p(start_pos),
                                       _p(dtable), B, S, H, vocab, int(detach_text), _stream()), "embed_splice_bwd")


def rmsnorm_fwd(x, w, eps, y=None, rstd=None):
    rows, H = x.shape
    y = y if y is not None else torch.empty_like(x)
    check(lib().llark_rmsnorm_fwd(_p(x), _p(w), _p(y), _p(rstd), rows, H, eps, _stream()), "rmsnorm_fwd")
    return y


def rmsnorm_bwd(x, w, dy, rstd, dres, dx, dw, accumulate_dw, workspace):
    rows, H = x.shape
    need = lib().llark_rmsnorm_bwd_workspace(rows, H)
    if workspace.numel() * workspace.element_size() < need:
        raise RuntimeError("rmsnorm_bwd workspace too small")
    check(lib().llark_rmsnorm_bwd(_p(x), _p(w), _p(dy), _p(rstd), _p(dres), _p(dx), _p(dw), int(accumulate_dw), rows,
                                  H, _p(workspace), _stream()), "rmsnorm_bwd")
    return dx


def rope_(qkv, cos_t, sin_t, S, n_heads, D, inverse=False):
    rows = qkv.shape[0]
    check(lib().llark_rope(_p(qkv), _p(cos_t), _p(sin_t), rows, S, n_heads, D, qkv.stride(0), int(inverse), _stream()),
          "rope")
    return qkv


def swiglu_fwd(gu, act=None):
    rows, I2 = gu.shape
    act = act if act is not None else torch.empty((rows, I2 // 2), device=gu.device, dtype=BF16)
    check(lib().llark_swiglu_fwd(_p(gu), _p(act), rows, I2 // 2, _stream()), "swiglu_fwd")
    return act


def swiglu_bwd(gu, dact, dgu=None):
    rows, I2 = gu.shape
    dgu = dgu if dgu is not None else torch.empty_like(gu)
    check(lib().llark_swiglu_bwd(_p(gu), _p(dact), _p(dgu), rows, I2 // 2, _stream()), "swiglu_bwd")
    return dgu


def attn_fwd(qkv, key_mask, B, S, n_heads, head_dim, out=None, lse=None):
    out = out if out is not None else torch.empty((B * S, n_heads * head_dim), device=qkv.device, dtype=BF16)
    lse = lse if lse is not None else torch.empty((B, n_heads, S), device=qkv.device, dtype=torch.float32)
    check(lib().llark_attn_fwd(_p(qkv), _p(key_mask), _p(out), _p(lse), B, S, n_heads, head_dim,
                               1.0 / math.sqrt(head_dim), _stream()), "attn_fwd")
    return out, lse


def attn_decode(q, k_cache, v_cache, lens, n_heads, head_dim, out=None):
    """One query token per row against the KV cache: q [B, H], caches [B, s_max, H], lens int32 [B] -> out [B, H]."""
    B, s_max = k_cache.shape[0], k_cache.shape[1]
    out = out if out is not None else torch.empty((B, n_heads * head_dim), device=q.device, dtype=BF16)
    check(lib().llark_attn_decode(_p(q), _p(k_cache), _p(v_cache), _p(lens), _p(out), B, s_max, n_heads, head_dim,
                                  1.0 / math.sqrt(head_dim), _stream()), "attn_decode")
    return out


def attn_bwd(qkv, key_mask, out, dout, lse, B, S, n_heads, head_dim, dqkv=None, workspace=None, rope=None):
    """dqkv = (dq | dk | dv). rope=(cos, sin) (bf16 [>= S, head_dim]): the inverse rotary embedding of the dq | dk heads is
    fused into the backward kernels (llark_attn_bwd_rope), bit-identical to attn_bwd followed by rope_(inverse=True)."""
    dqkv = dqkv if dqkv is not None else torch.empty_like(qkv)
    need = lib().llark_attn_bwd_workspace(B, S, n_heads)
    if workspace is None:
        workspace = torch.empty(need, device=qkv.device, dtype=torch.uint8)
    if rope is not None:
        cos_t, sin_t = rope
        check(lib().llark_attn_bwd_rope(_p(qkv), _p(key_mask), _p(out), _p(dout), _p(lse), _p(dqkv), B, S, n_heads,
                                        head_dim, 1.0 / math.sqrt(head_dim), _p(_req(cos_t, BF16)), _p(_req(sin_t, BF16)),
                                        _p(workspace), _stream()), "attn_bwd_rope")
        return dqkv
    check(lib().llark_attn_bwd(_p(qkv), _p(key_mask), _p(out), _p(dout), _p(lse), _p(dqkv), B, S, n_heads, head_dim,
                               1.0 / math.sqrt(head_dim), _p(workspace), _stream()), "attn_bwd")
    return dqkv


def gemv(x, w, bias=None, residual=None, out=None, N=None):
    """y[M, N] = x[M, K] @ w[N, K]^T (+ bias) (+ residual) for M <= 8 rows: the weight-streaming kernel of the decode step
    (csrc/gemv.cu). `out` may be wider than N (padded logits buffer)."""
    M, K = x.shape
    N = int(N) if N is not None else w.shape[0]
    out = out if out is not None else torch.empty((M, N), device=x.device, dtype=BF16)
    check(lib().llark_gemv(_p(x), x.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), _p(bias), _p(residual),
                           residual.stride(0) if residual is not None else 0, M, N, K, _stream()), "gemv")
    return out


# ------------------------------------------------------------------------------------------------ MPT variant (staged)
def attn_alibi_fwd(qkv, key_mask, B, S, n_heads, head_dim, slopes, out=None, lse=None):
    out = out if out is not None else torch.empty((B * S, n_heads * head_dim), device=qkv.device, dtype=BF16)
    lse = lse if lse is not None else torch.empty((B, n_heads, S), device=qkv.device, dtype=torch.float32)
    check(lib().llark_attn_alibi_fwd(_p(qkv), _p(key_mask), _p(out), _p(lse), _p(slopes), B, S, n_heads, head_dim,
                                     1.0 / math.sqrt(head_dim), _stream()), "attn_alibi_fwd")
    return out, lse


def attn_alibi_bwd(qkv, key_mask, out, dout, lse, B, S, n_heads, head_dim, slopes, dqkv=None):
    dqkv = dqkv if dqkv is not None else torch.empty_like(qkv)
    ws = torch.empty(lib().llark_attn_bwd_workspace(B, S, n_heads), device=qkv.device, dtype=torch.uint8)
    check(lib().llark_attn_alibi_bwd(_p(qkv), _p(key_mask), _p(out), _p(dout), _p(lse), _p(dqkv), _p(slopes), B, S,
                                     n_heads, head_dim, 1.0 / math.sqrt(head_dim), _p(ws), _stream()), "attn_alibi_bwd")
    return dqkv


def ln_fwd(x, w, eps, mean=None, rstd=None, out=None, out_dtype=BF16):
    """Bias-free LayerNorm of the rows of a [rows, W] bf16 view (row stride = x.stride(0)); out may be a strided view."""
    rows, W = x.shape
    out = out if out is not None else torch.empty((rows, W), device=x.device, dtype=BF16)
    check(lib().llark_ln_fwd(_p(x), x.stride(0), _p(w), _p(out), out.stride(0), _p(mean), _p(rstd), rows, W, eps,
                             _stream()), "ln_fwd")
    return out


def ln_bwd(x, w, dy, mean, rstd, dres, dx, dw, accumulate_dw):
    rows, W = x.shape
    ws = torch.empty(lib().llark_ln_bwd_workspace(rows, W), device=x.device, dtype=torch.uint8) if dw is not None else None
    check(lib().llark_ln_bwd(_p(x), x.stride(0), _p(w), _p(dy), dy.stride(0), _p(mean), _p(rstd), _p(dres), _p(dx),
                             dx.stride(0), _p(dw), int(accumulate_dw), rows, W, _p(ws), _stream()), "ln_bwd")
    return dx


def gelu_fwd(u, out=None):
    out = out if out is not None else torch.empty_like(u)
    check(lib().llark_gelu_fwd(_p(u), _p(out), u.numel(), _stream()), "gelu_fwd")
    return out


def gelu_bwd(u, dh, out=None):
    out = out if out is not None else torch.empty_like(u)
    check(lib().llark_gelu_bwd(_p(u), _p(dh), _p(out), u.numel(), _stream()), "gelu_bwd")
    return out


def colsum(x, out, accumulate=False):
    rows, H = x.shape
    check(lib().llark_colsum(_p(x), _p(out), rows, H, int(accumulate), _stream()), "colsum")
    return out


def ce_fwd(logits, ldv, V, labels, B, S, row_loss, row_lse, loss_out):
    check(lib().llark_ce_fwd(_p(logits), ldv, V, _p(labels), B, S, _p(row_loss), _p(row_lse), _p(loss_out), _stream()),
          "ce_fwd")


def ce_bwd(logits, ldv, V, labels, B, S, row_lse, loss_out, gscale_ptr, gscale, dlogits):
    check(lib().llark_ce_bwd(_p(logits), ldv, V, _p(labels), B, S, _p(row_lse), _p(loss_out), _p(gscale_ptr),
                             float(gscale), _p(dlogits), _stream()), "ce_bwd")


def grad_sumsq(g, out, accumulate, workspace):
    check(lib().llark_grad_sumsq(_p(g), g.numel(), _p(out), int(accumulate), _p(workspace), _stream()), "grad_sumsq")


def adamw_step(p, g, m, v, sumsq, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, max_norm=0.0,
               zero_grad=False):
    check(lib().llark_adamw_step(_p(p), _p(g), _p(m), _p(v), p.numel(), _p(sumsq), lr, beta1, beta2, eps, weight_decay,
                                 step, grad_scale, max_norm, int(zero_grad), _stream()), "adamw_step")


# ------------------------------------------------------------------------------------------------ Jukebox front end
def jb_conv_down(x, w, b):
    N, c_in, T = x.shape
    c_out = w.shape[0]
    y = torch.empty((N, c_out, T // 2), device=x.device, dtype=torch.float32)
    check(lib().llark_jb_conv_down(_p(x), _p(w), _p(b), _p(y), N, c_in, c_out, T, _stream()), "jb_conv_down")
    return y


def jb_resblock(x, w1, b1, w2, b2, dilation):
    N, C, T = x.shape
    y = torch.empty_like(x)
    check(lib().llark_jb_resblock(_p(x), _p(w1), _p(b1), _p(w2), _p(b2), _p(y), N, T, dilation, _stream()),
          "jb_resblock")
    return y


def jb_conv_k3(x, w, b):
    N, c_in, T = x.shape
    c_out = w.shape[0]
    y = torch.empty((N, c_out, T), device=x.device, dtype=torch.float32)
    check(lib().llark_jb_conv_k3(_p(x), _p(w), _p(b), _p(y), N, c_in, c_out, T, _stream()), "jb_conv_k3")
    return y


def jb_vq_encode(x, codebook):
    N, E, T = x.shape
    codes = torch.empty((N, T), device=x.device, dtype=torch.int64)
    check(lib().llark_jb_vq_encode(_p(x), _p(codebook), _p(codes), N, T, codebook.shape[0], _stream()), "jb_vq_encode")
    return codes


def layernorm_fwd(x, gamma, beta, eps=1e-5, out_dtype=torch.float32, out=None):
    rows, W = x.shape
    out = out if out is not None else torch.empty((rows, W), device=x.device, dtype=out_dtype)
    check(lib().llark_layernorm_fwd(_p(x), _p(gamma), _p(beta), _p(out), int(out.dtype == BF16), rows, W, eps,
                                    _stream()), "layernorm_fwd")
    return out


def jb_embed_tokens(codes, emb, y_cond, pos_emb, x_cond):
    N, T = codes.shape
    W = emb.shape[1]
    out = torch.empty((N * T, W), device=codes.device, dtype=torch.float32)
    check(lib().llark_jb_embed_tokens(_p(codes), _p(emb), _p(y_cond), _p(pos_emb), _p(x_cond), _p(out), N, T, W,
                                      _stream()), "jb_embed_tokens")
    return out


def jb_sparse_attn(qkv, N, T, heads, dh, block, pattern, out=None, out_dtype=torch.float32, exact=False):
    """Factored attention of the prior. Default: the tensor-core kernel (TF32 operands, fp32 accumulate, fp32 or bf16
    output); exact=True (or a geometry outside that kernel's envelope) runs the fp32 SIMT kernel (fp32 output)."""
    own = out is None
    if own:
        out = torch.empty((N * T, heads * dh), device=qkv.device, dtype=torch.float32 if exact else out_dtype)
    if not exact:
        rc = lib().llark_jb_sparse_attn_tc(_p(qkv), _p(out), int(out.dtype == BF16), N, T, heads, dh, block, pattern,
                                           _stream())
        if rc != -1:  # LLARK_EINVAL = outside the envelope -> SIMT kernel below
            check(rc, "jb_sparse_attn_tc")
            return out
        if out.dtype != torch.float32:
            if not own:
                raise TypeError("the SIMT factored-attention kernel writes fp32")
            out = torch.empty((N * T, heads * dh), device=qkv.device, dtype=torch.float32)  # caller casts
    check(lib().llark_jb_sparse_attn(_p(qkv), _p(out), N, T, heads, dh, block, pattern, _stream()), "jb_sparse_attn")
    return out


def quick_gelu(x, out=None):
    out = out if out is not None else torch.empty_like(x)
    check(lib().llark_quick_gelu(_p(x), _p(out), x.numel(), _stream()), "quick_gelu")
    return out


def add3(a, b, c=None, out=None):
    out = out if out is not None else torch.empty_like(a)
    check(lib().llark_add3(_p(a), _p(b), _p(c), _p(out), a.numel(), _stream()), "add3")
    return out


def jb_label_cond(total_row, abs_table, rel_table, abs_bins, rel_bins):
    """x_cond [T, W] = (total_row + abs_table[abs_bins]) + rel_table[rel_bins] (fp32 tables, int32 bins on the device)."""
    T, W = abs_bins.numel(), abs_table.shape[1]
    out = torch.empty((T, W), device=abs_table.device, dtype=torch.float32)
    check(lib().llark_jb_label_cond(_p(_req(total_row, torch.float32)), _p(_req(abs_table, torch.float32)),
                                    _p(_req(rel_table, torch.float32)), _p(_req(abs_bins, torch.int32)),
                                    _p(_req(rel_bins, torch.int32)), _p(out), T, W, _stream()), "jb_label_cond")
    return out


def jb_pool_batched(acts, T_valid, frame):
    """acts fp32 [N, T, W] (contiguous) -> [N, T_valid // frame, W]: windowed mean over time of every clip, one launch."""
    _req(acts, torch.float32)
    N, T, W = acts.shape
    if not acts.is_contiguous() or T_valid > T:
        raise ValueError("jb_pool_batched needs a contiguous [N, T, W] tensor with T >= T_valid")
    out = torch.empty((N, T_valid // frame, W), device=acts.device, dtype=torch.float32)
    check(lib().llark_jb_pool_batched(_p(acts), _p(out), N, T * W, T_valid, W, frame, _stream()), "jb_pool_batched")
    return out


def jb_pool(acts, T_valid, frame):
    W = acts.shape[1]
    out = torch.empty((T_valid // frame, W), device=acts.device, dtype=torch.float32)
    check(lib().llark_jb_pool(_p(acts), _p(out), T_valid, W, frame, _stream()), "jb_pool")
    return out


# ------------------------------------------------------------------------------------------------ fp32 verification path
def _f32(t):
    return _req(t, torch.float32)


def v32_split_tf32(x):
    x = _f32(x).contiguous()
    hi, lo = torch.empty_like(x), torch.empty_like(x)
    check(lib().llark_v32_split_tf32(_p(x), _p(hi), _p(lo), x.numel(), _stream()), "v32_split_tf32")
    return hi, lo


def v32_embed_splice_fwd(ids, table, audio, audio_off, frames, start_pos, out):
    B, S = ids.shape
    H = table.shape[1]
    check(lib().llark_v32_embed_splice_fwd(_p(ids), _p(_f32(table)), _p(audio), _p(audio_off), _p(frames), _p(start_pos),
                                           _p(_f32(out)), B, S, H, table.shape[0], _stream()), "v32_embed_splice_fwd")
    return out


def v32_rmsnorm_fwd(x, w, eps):
    rows, H = x.shape
    y = torch.empty_like(_f32(x))
    check(lib().llark_v32_rmsnorm_fwd(_p(x), _p(_f32(w)), _p(y), rows, H, eps, _stream()), "v32_rmsnorm_fwd")
    return y


def v32_rope_(qkv, cos_t, sin_t, S, n_rot_heads, D):
    check(lib().llark_v32_rope(_p(_f32(qkv)), _p(_f32(cos_t)), _p(_f32(sin_t)), qkv.shape[0], S, n_rot_heads, D,
                               qkv.stride(0), _stream()), "v32_rope")
    return qkv


def v32_swiglu_fwd(gu):
    rows, I2 = gu.shape
    act = torch.empty((rows, I2 // 2), device=gu.device, dtype=torch.float32)
    check(lib().llark_v32_swiglu_fwd(_p(_f32(gu)), _p(act), rows, I2 // 2, _stream()), "v32_swiglu_fwd")
    return act


def v32_attn_fwd(qkv, key_mask, B, S, n_heads, head_dim):
    out = torch.empty((B * S, n_heads * head_dim), device=qkv.device, dtype=torch.float32)
    check(lib().llark_v32_attn_fwd(_p(_f32(qkv)), _p(key_mask), _p(out), B, S, n_heads, head_dim,
                                   1.0 / math.sqrt(head_dim), _stream()), "v32_attn_fwd")
    return out


def v32_ce_fwd(logits, V, labels, B, S):
    row_loss = torch.empty(B * S, device=logits.device, dtype=torch.float32)
    loss_out = torch.empty(2, device=logits.device, dtype=torch.float32)
    check(lib().llark_v32_ce_fwd(_p(_f32(logits)), logits.stride(0), V, _p(labels), B, S, _p(row_loss), _p(loss_out),
                                 _stream()), "v32_ce_fwd")
    return loss_out[0]


# ------------------------------------------------------------------------------------------------ generation path of
# layer-list decoders (csrc/seq_ops.cu, csrc/seq_mixers.cu). `st` is a llark_b200.state_cache.StepLayout: the packed
# step (tok_seq, cu, pos0, slot on the device). The residual stream is fp32; `act` is torch.bfloat16 or torch.float32.
def _actf(dtype):
    if dtype not in (BF16, torch.float32):
        raise TypeError(f"activation dtype must be bfloat16 or float32, got {dtype}")
    return int(dtype == torch.float32)


# rows up to which a linear is the weight-streaming kernel (the activations then sit in L1 / L2, the op is a pure read
# of the weight matrix); above it the tcgen05 GEMM core (bf16, at least one 64-wide tile in N and K, rows that TMA can
# address) or the tiled SIMT kernel (fp32 mode, small or odd shapes)
LINEAR_ROWS_MAX = 8
LINEAR_STATS = {"rows": 0, "tcgen05": 0, "simt": 0}


def linear(a, w, bias=None, out_dtype=None, out=None):
    """y[M, N] = a[M, K] @ w[N, K]^T (+ bias fp32 [N]); a and w both bf16 or both fp32 (true fp32 arithmetic, no TF32);
    output bf16 or fp32."""
    _req(a), _req(w)
    if a.dtype != w.dtype:
        raise TypeError("linear: activation and weight dtypes differ")
    in_fp32 = _actf(a.dtype)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError("linear: inner sizes differ")
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype or a.dtype)
    c_fp32 = _actf(out.dtype)
    if bias is not None:
        _req(bias, torch.float32)
    vec = 4 if c_fp32 else 8
    if M <= LINEAR_ROWS_MAX:
        LINEAR_STATS["rows"] += 1
        check(lib().llark_linear_rows(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), c_fp32, _p(bias),
                                      M, N, K, in_fp32, _stream()), "linear_rows")
    elif (not in_fp32 and K >= 64 and N >= 64 and K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and out.stride(0) % vec == 0
          and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0):
        LINEAR_STATS["tcgen05"] += 1
        gemm(a, w, bias=bias, out=out, M=M, N=N, K=K)
    else:
        LINEAR_STATS["simt"] += 1
        check(lib().llark_linear_simt(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), c_fp32, _p(bias),
                                      M, N, K, in_fp32, _stream()), "linear_simt")
    return out


def seq_embed(ids, st, table, pos_table, scale):
    """ids int32 [n_tok] -> x fp32 [n_tok, C] = table[id] * scale + pos_table[position]."""
    _req(ids, torch.int32)
    C = table.shape[1]
    x = torch.empty((st.n_tok, C), device=table.device, dtype=torch.float32)
    check(lib().llark_seq_embed(_p(ids), _p(st.tok_seq), _p(st.cu), _p(st.pos0), _p(table), _p(pos_table), float(scale),
                                _p(x), st.n_tok, C, _actf(table.dtype), _stream()), "seq_embed")
    return x


def seq_short_conv(h, w, tail, st, act):
    """h fp32 [n_tok, C], w fp32 [C, taps], tail fp32 [slots, taps-1, C] (updated) -> h + conv(h) in `act`."""
    _req(h, torch.float32), _req(w, torch.float32)
    C, taps = w.shape
    y = torch.empty((st.n_tok, C), device=h.device, dtype=act)
    inline = int(st.max_len == 1)
    check(lib().llark_seq_short_conv(_p(h), _p(w), _p(tail), _p(st.tok_seq), _p(st.cu), _p(st.slot), _p(y), st.n_tok, C,
                                     taps, inline, _actf(act), _stream()), "seq_short_conv")
    if not inline and taps > 1:
        check(lib().llark_seq_conv_tail(_p(h), _p(tail), _p(st.cu), _p(st.slot), st.n_seq, C, taps, _stream()),
              "seq_conv_tail")
    return y


def seq_add_rmsnorm(x, y, w, eps, act=None):
    """x + rmsnorm(y) * w (fp32, new tensor); with `act` also a copy of the result in that dtype."""
    _req(x, torch.float32), _req(y, torch.float32), _req(w, torch.float32)
    rows, C = x.shape
    out = torch.empty_like(x)
    xa = torch.empty((rows, C), device=x.device, dtype=act) if act is not None else None
    check(lib().llark_seq_add_rmsnorm(_p(x), _p(y), _p(w), _p(out), _p(xa), rows, C, float(eps),
                                      _actf(act) if act is not None else 0, _stream()), "seq_add_rmsnorm")
    return (out, xa) if act is not None else out


def seq_gated_norm_add(x, y, w, eps, gate=None, w_next=None, act=None):
    """x + rmsnorm(y * sigmoid(gate)) * w (fp32, new tensor; gate fp32, a column slice is fine); with w_next also
    rmsnorm(result) * w_next in `act`: the input of the next sublayer."""
    _req(x, torch.float32), _req(y, torch.float32), _req(w, torch.float32)
    rows, C = x.shape
    if not y.is_contiguous() or y.shape != x.shape:
        raise ValueError("seq_gated_norm_add: y must be contiguous and of the stream's shape")
    if gate is not None:
        _req(gate, torch.float32)
        if gate.shape != x.shape or gate.stride(1) != 1:
            raise ValueError("seq_gated_norm_add: gate must be [rows, C] with unit column stride")
    out = torch.empty_like(x)
    xa = torch.empty((rows, C), device=x.device, dtype=act) if w_next is not None else None
    check(lib().llark_seq_gated_norm_add(_p(x), _p(y), _p(gate), gate.stride(0) if gate is not None else 0, _p(w),
                                         _p(w_next), _p(out), _p(xa), rows, C, float(eps),
                                         _actf(act) if w_next is not None else 0, _stream()), "seq_gated_norm_add")
    return (out, xa) if w_next is not None else out


def seq_rmsnorm_rows(x, rows, w, eps, act):
    _req(x, torch.float32), _req(w, torch.float32)
    n = rows.numel() if rows is not None else x.shape[0]
    C = x.shape[1]
    out = torch.empty((n, C), device=x.device, dtype=act)
    check(lib().llark_seq_rmsnorm_rows(_p(x), _p(rows), _p(w), _p(out), n, C, float(eps), _actf(act), _stream()),
          "seq_rmsnorm_rows")
    return out


def seq_relu2(u):
    y = torch.empty_like(u)
    check(lib().llark_seq_relu2(_p(u), _p(y), u.numel(), _actf(u.dtype), _stream()), "seq_relu2")
    return y


def seq_qk_headnorm(src, q_off, k_off, wq, wk, H, G, D, eps, act, st=None, kring=None, vring=None, cap=0):
    """src fp32 [n_tok, ld] -> (qn [n_tok, H*D], kn [n_tok, G*D], vraw [n_tok, G*D]) in `act`; with kring / vring the
    k rows also go straight into the rings (steps of one token per request)."""
    _req(src, torch.float32)
    n = src.shape[0]
    qn = torch.empty((n, H * D), device=src.device, dtype=act)
    kn = torch.empty((n, G * D), device=src.device, dtype=act)
    vr = torch.empty((n, G * D), device=src.device, dtype=act)
    check(lib().llark_seq_qk_headnorm(_p(src), src.stride(0), q_off, k_off, _p(wq), _p(wk), _p(qn), _p(kn), _p(vr),
                                      _p(kring), _p(vring), _p(st.tok_seq) if st else None, _p(st.cu) if st else None,
                                      _p(st.pos0) if st else None, _p(st.slot) if st else None, n, H, G, D, cap,
                                      float(eps), _actf(act), _stream()), "seq_qk_headnorm")
    return qn, kn, vr


def seq_qkv_headnorm(src, q_off, k_off, v_off, wq, wk, H, G, D, E, eps, act, st, kring=None, vring=None, cap=0,
                     temp_coef=0.0, temp_every=0):
    """As seq_qk_headnorm with values of their own (E columns per key / value head at v_off, copied un-normed) and an
    optional temperature on the query that grows with the position: 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)."""
    _req(src, torch.float32)
    n = src.shape[0]
    qn = torch.empty((n, H * D), device=src.device, dtype=act)
    kn = torch.empty((n, G * D), device=src.device, dtype=act)
    vv = torch.empty((n, G * E), device=src.device, dtype=act)
    check(lib().llark_seq_qkv_headnorm(_p(src), src.stride(0), q_off, k_off, v_off, _p(wq), _p(wk), _p(qn), _p(kn), _p(vv),
                                       _p(kring), _p(vring), _p(st.tok_seq), _p(st.cu), _p(st.pos0), _p(st.slot), n, H, G,
                                       D, E, cap, float(eps), float(temp_coef), int(temp_every), _actf(act), _stream()),
          "seq_qkv_headnorm")
    return qn, kn, vv


SWA_MMA_MIN_LEN = 16  # shortest longest-request of a step that goes to the tensor-core attention kernel


def seq_swa_attn(qn, kn, vv, kring, vring, gate, gate_ld, scale_h, st, H, G, D, E, window, cap, from_ring_only, sink=None,
                 gate_per_head=False, chunk=0, softcap=0.0, vfreq=None, v_interleaved=False):
    """Softmax attention of a packed step over the last `window` positions (rings of `cap` entries per slot hold what
    earlier steps brought). sink fp32 [H]: one more term exp(sink_h) of the denominator; gate_per_head: gate [n_tok, H].
    chunk > 0: instead of the window the query sees the earlier positions of its own block of `chunk` positions (blocks
    counted from position 0 of the sequence). softcap > 0: score <- softcap * tanh(score / softcap). vfreq fp32 [E / 2]:
    the values were stored rotated by their own position; each head's weighted sum is turned back by the query's."""
    out = torch.empty((st.n_tok, H * E), device=qn.device, dtype=qn.dtype)
    if sink is not None:
        _req(sink, torch.float32)
    if vfreq is not None:
        _req(vfreq, torch.float32)
        if vfreq.numel() != E // 2:
            raise ValueError("seq_swa_attn: one frequency per pair of value channels")
    if (qn.dtype == BF16 and not from_ring_only and st.max_len >= SWA_MMA_MIN_LEN and D == E and D % 16 == 0
            and D <= 256 and (gate is None or gate_per_head or gate_ld % 2 == 0)
            and (vfreq is None or v_interleaved or D in (64, 128, 256))):
        # prompts and portions: 64-query tiles on the tensor cores; single tokens, fp32 and odd head sizes stay SIMT
        check(lib().llark_seq_swa_attn_mma(_p(qn), _p(kn), _p(vv), _p(kring), _p(vring), _p(gate), gate_ld, _p(scale_h),
                                           _p(out), _p(st.cu), _p(st.pos0), _p(st.slot), st.n_seq, st.max_len, H, G, D,
                                           window, cap, _p(sink), int(gate_per_head), int(chunk), float(softcap or 0.0),
                                           _p(vfreq), int(v_interleaved), _stream()), "seq_swa_attn_mma")
        return out
    check(lib().llark_seq_swa_attn(_p(qn), _p(kn), _p(vv), _p(kring), _p(vring), _p(gate), gate_ld, _p(scale_h), _p(out),
                                   _p(st.tok_seq), _p(st.cu), _p(st.pos0), _p(st.slot), st.n_tok, H, G, D, E, window, cap,
                                   int(from_ring_only), _p(sink), int(gate_per_head), int(chunk), float(softcap or 0.0),
                                   _p(vfreq), int(v_interleaved), _actf(qn.dtype), _stream()),
          "seq_swa_attn")
    return out


def seq_qkv_rotary(src, q_off, k_off, v_off, H, G, D, E, eps, act, st, wq=None, wk=None, qk_freq=None, qk_interleaved=False,
                   v_freq=None, v_interleaved=False, kring=None, vring=None, cap=0):
    """src fp32 [n_tok, ld] -> (q [n_tok, H*D], k [n_tok, G*D], v [n_tok, G*E]) in `act`. wq / wk: RMS norm over the whole
    q / k projection with weights [H*D] / [G*D]. qk_freq fp32 [n_rot / 2]: the first n_rot entries of each q / k head are
    rotated by position * frequency (pairs (i, i + n_rot/2), or (2i, 2i+1) when interleaved). v_freq fp32 [E / 2]: the
    value heads are rotated the same way over all of E. With kring / vring the k / v rows also go straight into the rings
    (steps of one token per request)."""
    _req(src, torch.float32)
    n = src.shape[0]
    qn = torch.empty((n, H * D), device=src.device, dtype=act)
    kn = torch.empty((n, G * D), device=src.device, dtype=act)
    vv = torch.empty((n, G * E), device=src.device, dtype=act)
    n_rot = 2 * qk_freq.numel() if qk_freq is not None else 0
    if v_freq is not None and v_freq.numel() != E // 2:
        raise ValueError("seq_qkv_rotary: one frequency per pair of value channels")
    check(lib().llark_seq_qkv_rotary(_p(src), src.stride(0), q_off, k_off, v_off, _p(wq), _p(wk), _p(qk_freq), n_rot,
                                     int(qk_interleaved), _p(v_freq), int(v_interleaved), _p(qn), _p(kn), _p(vv), _p(kring),
                                     _p(vring), _p(st.tok_seq), _p(st.cu), _p(st.pos0), _p(st.slot), n, H, G, D, E, int(cap),
                                     float(eps), _actf(act), _stream()), "seq_qkv_rotary")
    return qn, kn, vv


def seq_kv_ring_write(kn, vv, kring, vring, st, cap):
    """Rows of this step into the rings; vv = vring = None when the keys are their own values (one ring)."""
    check(lib().llark_seq_kv_ring_write(_p(kn), _p(vv), _p(kring), _p(vring), _p(st.tok_seq), _p(st.cu), _p(st.pos0),
                                        _p(st.slot), st.n_tok, kn.shape[1], vv.shape[1] if vv is not None else 1, cap,
                                        _actf(kn.dtype), _stream()),
          "seq_kv_ring_write")


GLR_CHUNK = 256        # rows per work item when a long prompt is scanned in chunks
GLR_CHUNK_MIN_LEN = 512  # shortest longest-request of a step that is scanned in chunks


def seq_glr_scan(src, q_off, f_off, v_off, lower, state, st, H, D, E):
    """src fp32 [n_tok, ld] -> o_raw fp32 [n_tok, H*E]; state fp32 [slots, H, D, E] read and written back. Steps with a
    long request run in three passes over chunks of GLR_CHUNK rows (local states from zero; combine; outputs), which
    gives the scan as many independent work items as there are chunks."""
    _req(src, torch.float32), _req(state, torch.float32)
    o = torch.empty((st.n_tok, H * E), device=src.device, dtype=torch.float32)
    L = lib()
    if st.max_len < GLR_CHUNK_MIN_LEN:
        check(L.llark_seq_glr_scan(_p(src), src.stride(0), q_off, f_off, v_off, _p(lower), _p(state), _p(state), None,
                                   _p(o), _p(st.cu), _p(st.lens_dev), _p(st.slot), _p(st.slot), st.n_seq, H, D, E,
                                   _stream()), "seq_glr_scan")
        return o
    ch = st.chunks(GLR_CHUNK)
    cstate = torch.empty((ch.n_items, H, D, E), device=src.device, dtype=torch.float32)
    cdecay = torch.empty((ch.n_items, H, D), device=src.device, dtype=torch.float32)
    check(L.llark_seq_glr_scan(_p(src), src.stride(0), q_off, f_off, v_off, _p(lower), None, _p(cstate), _p(cdecay), None,
                               _p(ch.row0), _p(ch.n), _p(ch.minus1), _p(ch.index), ch.n_items, H, D, E, _stream()),
          "seq_glr_scan(local)")
    check(L.llark_seq_glr_combine(_p(state), _p(cstate), _p(cdecay), _p(ch.seq_item0), _p(st.slot), st.n_seq, H, D, E,
                                  _stream()), "seq_glr_combine")
    check(L.llark_seq_glr_scan(_p(src), src.stride(0), q_off, f_off, v_off, _p(lower), _p(cstate), _p(state), None, _p(o),
                               _p(ch.row0), _p(ch.n), _p(ch.index), _p(ch.last_slot), ch.n_items, H, D, E, _stream()),
          "seq_glr_scan(outputs)")
    return o


def seq_head_rmsnorm(x, w, E, eps, act):
    """x fp32 [n_tok, H*E]: RMS norm of every E-wide head with the shared weight w fp32 [E] -> `act`."""
    _req(x, torch.float32)
    out = torch.empty(x.shape, device=x.device, dtype=act)
    check(lib().llark_seq_head_rmsnorm(_p(x), _p(w), _p(out), x.numel() // E, E, float(eps), _actf(act), _stream()),
          "seq_head_rmsnorm")
    return out


# ------------------------------------------------------------------------------------------------ further parts of
# layer-list decoders: grouped RMS norm, the residual of side-by-side sublayers, delta-rule recurrences
# (csrc/seq_delta.cu), latent attention (csrc/seq_latent.cu), routed mixture of experts (csrc/seq_moe.cu)
def linear_w32(a, w, bias=None):
    """a [M, K] (bf16 or fp32) @ w fp32 [N, K]^T -> fp32 [M, N]: fp32 arithmetic on 32-bit weights (router logits)."""
    _req(a), _req(w, torch.float32)
    M, K = a.shape
    N = w.shape[0]
    out = torch.empty((M, N), device=a.device, dtype=torch.float32)
    check(lib().llark_linear_simt_w32(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), _p(bias), M, N, K,
                                      _actf(a.dtype), _stream()), "linear_simt_w32")
    return out


def seq_group_rmsnorm(x, w, groups, eps, out_dtype=torch.float32, rows=None, add_vec=None):
    """RMS norm of fp32 rows in `groups` equal consecutive parts, times w. rows: int32 row numbers to norm (all when
    None). add_vec fp32 [C]: added to x first; then (x + add_vec, norm) is returned."""
    _req(x, torch.float32), _req(w, torch.float32)
    C = x.shape[1]
    n = rows.numel() if rows is not None else x.shape[0]
    out = torch.empty((n, C), device=x.device, dtype=out_dtype)
    x_out = torch.empty_like(x) if add_vec is not None else None
    check(lib().llark_seq_group_rmsnorm(_p(x), _p(rows), _p(add_vec), _p(x_out), _p(w), _p(out), n, C, int(groups),
                                        float(eps), _actf(out_dtype), _stream()), "seq_group_rmsnorm")
    return (x_out, out) if add_vec is not None else out


def seq_residual_combine(x, y, z=None, pos_of=None, wts=None, top=0):
    """x + (y + sum_k wts[t, k] * z[pos_of[t, k]]) fp32 (top = 0: x + y)."""
    _req(x, torch.float32), _req(y, torch.float32)
    out = torch.empty_like(x)
    check(lib().llark_seq_residual_combine(_p(x), _p(y), _p(z), _p(pos_of), _p(wts), int(top), _p(out), x.shape[0],
                                           x.shape[1], _stream()), "seq_residual_combine")
    return out


def seq_conv_act(src, w, carry, st, silu=True, bias=None):
    """src fp32 [n_tok, n_ch] (a column slice of a wider matrix is fine), w fp32 [n_ch, taps], carry fp32
    [slots, taps-1, n_ch] (updated), bias fp32 [n_ch] or None -> fp32 [n_tok, n_ch] = act(causal depthwise conv)."""
    _req(src, torch.float32), _req(w, torch.float32)
    n_ch, taps = w.shape
    out = torch.empty((st.n_tok, n_ch), device=src.device, dtype=torch.float32)
    check(lib().llark_seq_conv_act(_p(src), src.stride(0), _p(w), _p(carry), _p(st.tok_seq), _p(st.cu), _p(st.slot),
                                   _p(out), st.n_tok, st.n_seq, n_ch, taps, int(silu), _p(bias), _stream()), "seq_conv_act")
    return out


DELTA_GATED, DELTA_GENERALIZED, DELTA_GATED_SCALAR, DELTA_STATE_SPACE = 0, 1, 2, 3


def seq_delta_prep(rule, q, k, dec, mix, H, G, D, dec_bias=None, rate_log=None, unit_eps=1e-6):
    """The five vectors [n_tok, H, 5, D] of seq_delta_scan from fp32 projections (column slices are fine).
    DELTA_GATED_SCALAR: dec [n_tok, H], dec_bias [H] (one decay per head). DELTA_STATE_SPACE: q = the read-out vectors,
    k = the write vectors [n_tok, G, D], dec = the step size before its softplus [n_tok, H]; mix is not used."""
    n = q.shape[0]
    if mix is None:
        mix = dec
    vec = torch.empty((n, H, 5, D), device=q.device, dtype=torch.float32)
    check(lib().llark_seq_delta_prep(int(rule), _p(_req(q, torch.float32)), q.stride(0), _p(_req(k, torch.float32)),
                                     k.stride(0), _p(_req(dec, torch.float32)), dec.stride(0), _p(dec_bias),
                                     _p(rate_log), _p(_req(mix, torch.float32)), mix.stride(0), _p(vec), n, H, G, D,
                                     float(unit_eps), _stream()), "seq_delta_prep")
    return vec


def seq_delta_scan(vec, v, state, st, H, D, E, correct=True):
    """vec fp32 [n_tok, H, 5, D], v fp32 [n_tok, H*E] (column slice fine), state fp32 [slots, H, D, E] (updated) ->
    o fp32 [n_tok, H*E]. correct=False: the rule has no correction term (DELTA_STATE_SPACE)."""
    _req(vec, torch.float32), _req(v, torch.float32), _req(state, torch.float32)
    o = torch.empty((st.n_tok, H * E), device=v.device, dtype=torch.float32)
    check(lib().llark_seq_delta_scan(_p(vec), _p(v), v.stride(0), _p(state), _p(o), _p(st.cu), _p(st.slot), st.n_seq,
                                     st.n_tok, H, D, E, int(correct), _stream()), "seq_delta_scan")
    return o


def seq_head_norm_gate(x, w, H, E, eps, act, gate=None, w_per_head=False, gate_silu=False):
    """x fp32 [n_tok, H*E]: per-head RMS norm, times w ([E] or [H*E]), times sigmoid(gate fp32 [n_tok, H*E]) (gate_silu:
    times silu(gate)) -> act."""
    _req(x, torch.float32), _req(w, torch.float32)
    out = torch.empty(x.shape, device=x.device, dtype=act)
    check(lib().llark_seq_head_norm_gate(_p(x), _p(w), int(w_per_head), _p(gate), gate.stride(0) if gate is not None else 0,
                                         _p(out), x.shape[0], H, E, float(eps), int(gate_silu), _actf(act), _stream()),
          "seq_head_norm_gate")
    return out


def seq_skip_gate_group_norm(o, xin, skip, gate, w, H, E, groups, eps, act):
    """(o + skip[h] * xin) * silu(gate) over the H*E channels of a token, RMS norm in `groups` equal parts, times w -> act.
    o fp32 [n_tok, H*E] contiguous; xin, gate fp32 column slices."""
    _req(o, torch.float32), _req(xin, torch.float32), _req(gate, torch.float32), _req(w, torch.float32)
    out = torch.empty(o.shape, device=o.device, dtype=act)
    check(lib().llark_seq_skip_gate_group_norm(_p(o), _p(xin), xin.stride(0), _p(_req(skip, torch.float32)), _p(gate),
                                               gate.stride(0), _p(w), _p(out), o.shape[0], H, E, int(groups), float(eps),
                                               _actf(act), _stream()), "seq_skip_gate_group_norm")
    return out


def seq_post_norm(x, alpha, w, eps, y1=None, w1=None, y2=None, w2=None, branch_scale=1.0, z=None, pos_of=None, wts=None,
                  ids=None, n_real=0, act=None):
    """rmsnorm(alpha * x + f) * w on fp32 rows, f = branch_scale * (b1 + b2) + the chosen experts' weighted outputs:
    b_i = y_i, or rmsnorm(y_i) * w_i when w_i is given; expert entries (z, pos_of, wts [n_tok, top]) whose number in `ids`
    is >= n_real add wts * x instead of a row of z. Returns x_out fp32, or (x_out, copy in `act`) when act is given (for
    act = float32 the copy is x_out itself)."""
    _req(x, torch.float32), _req(w, torch.float32)
    rows, C = x.shape
    out = torch.empty_like(x)
    xa = torch.empty((rows, C), device=x.device, dtype=act) if act == BF16 else None
    top = wts.shape[1] if wts is not None else 0
    check(lib().llark_seq_post_norm(_p(x), float(alpha), _p(y1), _p(w1), _p(y2), _p(w2), float(branch_scale), _p(z),
                                    _p(pos_of), _p(wts), _p(ids), int(top), int(n_real), _p(w), _p(out), _p(xa), rows, C,
                                    float(eps), 0, _stream()), "seq_post_norm")
    if act is None:
        return out
    return out, (xa if xa is not None else out)


def seq_glu_clamped(gu, limit, slope=1.702):
    """gu [rows, 2*ff] = [g | u] -> min(g, limit) * sigmoid(slope * min(g, limit)) * (clamp(u, -limit, limit) + 1)."""
    rows, ff2 = gu.shape
    if not gu.is_contiguous():
        raise ValueError("seq_glu_clamped needs contiguous rows")
    act = torch.empty((rows, ff2 // 2), device=gu.device, dtype=gu.dtype)
    check(lib().llark_seq_glu_clamped(_p(gu), _p(act), rows, ff2 // 2, float(limit), float(slope), _actf(gu.dtype),
                                      _stream()), "seq_glu_clamped")
    return act


def seq_logit_cap_(z, scale, cap):
    """z fp32 <- cap * tanh(z * scale / cap) in place (cap None or <= 0: only the scale)."""
    _req(z, torch.float32)
    if not z.is_contiguous():
        raise ValueError("seq_logit_cap_ needs a contiguous tensor")
    check(lib().llark_seq_logit_cap(_p(z), z.numel(), float(scale), float(cap or 0.0), _stream()), "seq_logit_cap")
    return z


def seq_latent_prep(q, lat, norm_w, freqs, mult, st, H, Dn, P, R, eps, act, ring=None, cap=0, halves=False):
    """q fp32 [n_tok, H*(Dn+P)], lat fp32 [n_tok, R+P] (column slices fine) -> ckr act [n_tok, R+P] (normed latent |
    rotated shared key part) and qf act [n_tok, H, R+P] with columns R.. = rotated query parts (columns < R are left
    for seq_head_linear). With `ring` the ckr rows also go to the ring entries of the tokens' positions. Rotary pairs are
    (2i, 2i + 1), or (i, i + n_rot / 2) with `halves`."""
    n = st.n_tok
    ckr = torch.empty((n, R + P), device=q.device, dtype=act)
    qf = torch.empty((n, H * (R + P)), device=q.device, dtype=act)
    n_rot = 2 * freqs.numel() if freqs is not None else 0
    check(lib().llark_seq_latent_prep(_p(_req(q, torch.float32)), q.stride(0), _p(_req(lat, torch.float32)),
                                      lat.stride(0), _p(norm_w), _p(freqs), n_rot, float(mult), _p(ckr), _p(qf), _p(ring),
                                      _p(st.tok_seq), _p(st.cu), _p(st.pos0), _p(st.slot), n, H, Dn, P, R, int(cap),
                                      float(eps), int(halves), _actf(act), _stream()), "seq_latent_prep")
    return ckr, qf


def seq_head_linear(x, x_hs, w, y, y_hs, N, K, gate=None):
    """y[m, h*y_hs + n] = sum_k x[m, h*x_hs + k] * w[h, n, k] (* sigmoid(gate[m, h*N + n])); x fp32 or the dtype of w;
    y (given, written in place) has the dtype of w."""
    H = w.shape[0]
    check(lib().llark_seq_head_linear(_p(x), int(x.dtype == torch.float32), x.stride(0), x_hs, _p(w), _p(y), y.stride(0),
                                      y_hs, _p(gate), gate.stride(0) if gate is not None else 0, x.shape[0], H, N, K,
                                      _actf(w.dtype), _stream()), "seq_head_linear")
    return y


def seq_moe_route(logits, n_groups, keep, top, scale, softmax_bias=False, correction=None):
    """Expert numbers int32 [n, top] and weights fp32 [n, top]. Default: sigmoid scores, groups ranked by the sum of their
    two best, weights renormalised. softmax_bias: softmax scores, the choice made on score + correction, groups ranked by
    their best choice score, weights = the plain scores."""
    n, n_exp = logits.shape
    ids = torch.empty((n, top), device=logits.device, dtype=torch.int32)
    wts = torch.empty((n, top), device=logits.device, dtype=torch.float32)
    if softmax_bias:
        check(lib().llark_seq_moe_route_bias(_p(_req(logits, torch.float32)), logits.stride(0), _p(correction), _p(ids),
                                             _p(wts), n, n_exp, int(n_groups), int(keep), int(top), float(scale),
                                             _stream()), "seq_moe_route_bias")
        return ids, wts
    check(lib().llark_seq_moe_route(_p(_req(logits, torch.float32)), logits.stride(0), _p(ids), _p(wts), n, n_exp,
                                    int(n_groups), int(keep), int(top), float(scale), _stream()), "seq_moe_route")
    return ids, wts


# entries (tokens x choices) from which a bf16 step runs every expert's rows through the tcgen05 GEMM core; smaller steps,
# and fp32, stay on the grouped SIMT kernels. Neither route reads anything back to the host.
MOE_DENSE_MIN_ENTRIES = 2048


def seq_moe_experts(x, ids, w_gate_up, w_down, n_through=0):
    """x act [n_tok, C]; ids int32 [n_tok, top]; w_gate_up act [n_exp, 2*ff, C] (gate rows, then up rows);
    w_down act [n_exp, C, ff] -> (z fp32 [n_tok*top, C] expert outputs in sorted order, pos_of int32 [n_tok*top]).
    n_through: expert numbers n_exp .. n_exp + n_through - 1 have no weights; their rows of z are not written."""
    L = lib()
    n_tok, top = ids.shape
    n_real, ff2, C = w_gate_up.shape
    n_exp = n_real + int(n_through)
    ff = ff2 // 2
    n_ent = n_tok * top
    dense = (x.dtype == BF16 and n_ent >= MOE_DENSE_MIN_ENTRIES and C % 8 == 0 and ff % 8 == 0 and C >= 64 and ff >= 64
             and L.llark_gemm_get_mode() == 1)
    max_tiles = (n_ent + L.llark_seq_moe_tile_rows() - 1) // L.llark_seq_moe_tile_rows() + n_exp
    max256 = (n_ent + 255) // 256 + n_exp if dense else 0
    ints = torch.empty(2 * n_ent + 3 * max_tiles + 2 + n_exp + 1 + 3 * max256, device=x.device, dtype=torch.int32)
    o = 0

    def take(n):
        nonlocal o
        o += n
        return ints[o - n:o]

    perm, pos_of, tiles, meta, seg_off, tiles256 = (take(n_ent), take(n_ent), take(3 * max_tiles), take(2),
                                                    take(n_exp + 1), take(3 * max256))
    check(L.llark_seq_moe_sort(_p(ids), n_ent, n_exp, n_real, _p(perm), _p(pos_of), _p(tiles), _p(meta), _p(seg_off),
                               _p(tiles256) if dense else None, _stream()), "seq_moe_sort")
    z = torch.empty((n_ent, C), device=x.device, dtype=torch.float32)
    act = torch.empty((n_ent, ff), device=x.device, dtype=x.dtype)
    if dense:
        if not _INITED:
            init()
        count = meta[1:]
        xs = torch.empty((n_ent, C), device=x.device, dtype=x.dtype)
        check(L.llark_seq_moe_gather(_p(x), x.stride(0), _p(perm), top, _p(xs), n_ent, C, 0, _stream()), "seq_moe_gather")
        gu = torch.empty((n_ent, ff2), device=x.device, dtype=x.dtype)
        check(L.llark_gemm_segments(_p(xs), C, _p(w_gate_up), _p(gu), ff2, 0, None, n_real, _p(tiles256), max256, _p(count),
                                    n_ent, ff2, C, _stream()), "gemm_segments(gate|up)")
        check(L.llark_seq_silu_mul(_p(gu), _p(act), n_ent, ff, 0, _stream()), "seq_silu_mul")
        check(L.llark_gemm_segments(_p(act), ff, _p(w_down), _p(z), C, 1, None, n_real, _p(tiles256), max256, _p(count),
                                    n_ent, C, ff, _stream()), "gemm_segments(down)")
        return z, pos_of
    check(L.llark_seq_moe_up(_p(x), x.stride(0), _p(perm), top, _p(w_gate_up), _p(act), _p(tiles), _p(meta), max_tiles,
                             n_ent, ff, C, _actf(x.dtype), _stream()), "seq_moe_up")
    check(L.llark_seq_moe_down(_p(act), _p(w_down), _p(z), _p(tiles), _p(meta), max_tiles, n_ent, C, ff, _actf(x.dtype),
                               _stream()), "seq_moe_down")
    return z, pos_of


def seq_tanh(u, act):
    """tanh of an fp32 tensor -> `act`."""
    _req(u, torch.float32)
    y = torch.empty(u.shape, device=u.device, dtype=act)
    check(lib().llark_seq_tanh(_p(u), _p(y), u.numel(), _actf(act), _stream()), "seq_tanh")
    return y
