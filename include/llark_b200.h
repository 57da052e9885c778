/* llark_b200 C-ABI: the inner boundary of the B200-native LLark hot path.
 *
 * The reference (spotify-research/llark) has no C/FFI layer: its boundary is the Python API of
 * m2t/models/llamav2.py, m2t/data_modules.py and jukebox/main.py, and every FLOP is a PyTorch/cuBLAS/cuDNN
 * call. This header is what those call sites bind to instead: plain device pointers, sizes and a CUDA stream,
 * no torch types. Each entry point cites the reference call site (file:line under the reference root) whose
 * arithmetic it replaces. The Python mirror of the reference API lives in llark_b200/ and calls these through
 * ctypes (INTEGRATION.md shows the binding).
 *
 * Conventions: all pointers are DEVICE pointers owned by the caller unless stated; functions never allocate,
 * never free, never synchronise; they enqueue work on `stream` and return LLARK_OK (0) or a negative LLARK_E*.
 * "bf16" buffers are raw __nv_bfloat16. Row-major everywhere. Thread-safe for distinct streams.
 */
#ifndef LLARK_B200_H
#define LLARK_B200_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLARK_OK 0
#define LLARK_EINVAL (-1)
#define LLARK_ECUDA (-2)
#define LLARK_EDRIVER (-3)
#define LLARK_ENCCL (-4)

/* Last CUDA / driver / NCCL error code seen by the calling thread (for LLARK_ECUDA / EDRIVER / ENCCL). */
int llark_last_cuda_error(void);
/* One-time per-process set-up on the current device (TMA descriptor encoder, tile-counter ring of the GEMM scheduler).
 * The only entry point that allocates or synchronises; every other llark_* call just enqueues on the caller's stream. */
int llark_init(void);

/* ---------------------------------------------------------------------------------------------------------
 * GEMM core (tcgen05 / TMEM / TMA).  C[M,N] = A[M,K] * B[N,K]^T (+ bias[N]) (+ R[M,N]), fp32 accumulate.
 *   a_mn_major = 0: A stored [M][lda] (K contiguous);  1: A stored [K][lda] (M contiguous).
 *   b_mn_major = 0: B stored [N][ldb] (K contiguous);  1: B stored [K][ldb] (N contiguous).
 *   in_fp32 = 0: A,B bf16 (kind::f16);  1: A,B fp32 consumed as TF32 (kind::tf32, K-major operands only).
 *   c_fp32: C (and R) fp32 instead of bf16.  bias: bf16[N] (fp32[N] if bias_fp32) or NULL.  R may alias C.
 *   max_ctas: 0 = one CTA per SM; >0 caps the persistent grid (tests / overlap with a comm stream).
 * Replaces: nn.Linear / addmm at m2t/models/llamav2.py:133 (mm_projector), :224 (LlamaModel q/k/v/o/gate/up/
 * down projections, via transformers), :312 (lm_head), their autograd dgrad/wgrad, and the prior's Conv1D
 * addmm in openai/jukebox reached from jukebox/main.py:108.
 */
int llark_gemm(const void* A, int a_mn_major, long long lda, const void* B, int b_mn_major, long long ldb, void* C,
               long long ldc, int c_fp32, const void* bias, int bias_fp32, const void* R, long long ldr, int M, int N,
               int K, int in_fp32, int max_ctas, cudaStream_t stream);
/* Fused epilogues of the GEMM core (llark_gemm_ex; ep == NULL or kind 0 behaves exactly like llark_gemm):
 *   LLARK_EPI_QUICK_GELU  C = quick_gelu(acc + bias)            -- prior MLP `fc` (openai/jukebox MLP, reached from
 *                                                                  jukebox/main.py:108); replaces llark_quick_gelu (+ cast)
 *   LLARK_EPI_ROPE        columns [0, i1) of C (q | k heads of the fused QKV projection, head_dim 128) are rotated
 *                         with a = cos, b = sin (bf16 [S,128]), position = row % i0 -- transformers
 *                         apply_rotary_pos_emb reached from m2t/models/llamav2.py:224; replaces llark_rope(inverse=0)
 *   LLARK_EPI_SWIGLU_BWD  acc = d(act) of the down projection's dgrad; a = gu bf16 [M, ld] (gate | up, N apart);
 *                         C[:, c] = dgate, C[:, N + c] = dup (C is dgu [M, ldc >= 2N]); replaces llark_swiglu_bwd
 * Results are bit-identical to the unfused sequences (same bf16 rounding points). */
/*   LLARK_EPI_SEGMENTS    not an epilogue: the rows of A / C come in runs that each multiply their own block of B (stacked
 *                         [i1, N, K]); a = device int triples (block, first row, rows <= 256), i0 = their number (an upper
 *                         bound when b points at a device word with the real number). Used by llark_gemm_segments. */
enum { LLARK_EPI_NONE = 0, LLARK_EPI_QUICK_GELU = 1, LLARK_EPI_ROPE = 2, LLARK_EPI_SWIGLU_BWD = 3, LLARK_EPI_SEGMENTS = 4 };
typedef struct LlarkGemmEpilogue {
    int kind;
    const void* a;
    const void* b;
    long long ld;
    int i0, i1;
} LlarkGemmEpilogue;
int llark_gemm_ex(const void* A, int a_mn_major, long long lda, const void* B, int b_mn_major, long long ldb, void* C,
                  long long ldc, int c_fp32, const void* bias, int bias_fp32, const void* R, long long ldr, int M, int N,
                  int K, int in_fp32, int max_ctas, const LlarkGemmEpilogue* ep, cudaStream_t stream);
void llark_gemm_clear_cache(void);
/* Kernel variant: 1 = CTA-pair kernel (cta_group::2, 256x256 tile per 2-CTA cluster; default), 0 = single-CTA
 * kernel (128x256 tile). Default comes from the environment variable LLARK_GEMM_2CTA (unset or != "0" -> 1). */
void llark_gemm_set_mode(int two_cta);
int llark_gemm_get_mode(void);

/* ---------------------------------------------------------------------------------------------------------
 * Embedding gather + audio splice (m2t/models/llamav2.py:124 embed_tokens, :141-222 splice loop).
 * llark_splice_scan finds each sample's <audio_start> position on the device and raises the reference's two
 * ValueError conditions as bits in *flags (1: start/end count mismatch :146-152; 2: end token not at
 * start+frames+1 :169-175; 4: more than one audio segment, unsupported) instead of a host sync per sample.
 *   ids int64 [B,S]; frames int32 [B] (audio frames of sample b); start_pos int32 [B] out (-1 = no audio).
 * llark_embed_splice_fwd: out[b,s,:] = audio[audio_off[b] + s-pos-1, :] inside the audio block else table[ids].
 *   table bf16 [vocab,H]; audio bf16 [sum(frames),H] (projected features); audio_off int64 [B] row offsets.
 * llark_embed_splice_bwd: daudio <- dout audio rows; dtable[ids] += dout for the two marker rows only when
 *   detach_text != 0 (the orig_embeds_params path, :176-198), else for every text row (:199-207).
 */
int llark_splice_scan(const long long* ids, int B, int S, long long start_id, long long end_id, const int* frames,
                      int* start_pos, int* flags, cudaStream_t stream);
int llark_embed_splice_fwd(const long long* ids, const void* table, const void* audio, const long long* audio_off,
                           const int* frames, const int* start_pos, void* out, int B, int S, int H, long long vocab,
                           cudaStream_t stream);
int llark_embed_splice_bwd(const long long* ids, const void* dout, void* daudio, const long long* audio_off,
                           const int* frames, const int* start_pos, void* dtable, int B, int S, int H,
                           long long vocab, int detach_text, cudaStream_t stream);

/* dtype casts (autocast of fp32 audio_encodings to bf16 before mm_projector, llamav2.py:133). */
int llark_cast_f32_to_bf16(const float* in, void* out, long long n, cudaStream_t stream);
int llark_cast_bf16_to_f32(const void* in, float* out, long long n, cudaStream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Llama decoder pieces (transformers LlamaRMSNorm / apply_rotary_pos_emb / LlamaMLP, reached at
 * m2t/models/llamav2.py:224). H must be a multiple of 256 (<= 16384).
 * rmsnorm_fwd: y = w * bf16(x * rsqrt(mean(x^2) + eps)); rstd fp32 [rows] saved for backward (may be NULL).
 * rmsnorm_bwd: dx = (dres ? dres : 0) + norm-path gradient; dw (+)= sum_rows dy * bf16(xhat).
 */
int llark_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int H, float eps,
                      cudaStream_t stream);
long long llark_rmsnorm_bwd_workspace(long long rows, int H);
int llark_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, const void* dres, void* dx,
                      void* dw, int accumulate_dw, long long rows, int H, void* workspace, cudaStream_t stream);
/* RoPE in place on the q and k heads of a packed [rows, row_stride] buffer (q heads | k heads | v heads),
 * cos/sin bf16 [S, D] tables (HF LlamaRotaryEmbedding values rounded to bf16), position = row % S.
 * inverse != 0 applies the transpose (backward). */
int llark_rope(void* qkv, const void* cos_t, const void* sin_t, long long rows, int S, int n_heads, int D,
               long long row_stride, int inverse, cudaStream_t stream);
/* SwiGLU on the fused gate|up projection gu [rows, 2I]: act = bf16(silu(gate)) * up. */
int llark_swiglu_fwd(const void* gu, void* act, long long rows, int I, cudaStream_t stream);
int llark_swiglu_bwd(const void* gu, const void* dact, void* dgu, long long rows, int I, cudaStream_t stream);

/* Causal attention with key-padding mask, head_dim 128. qkv bf16 [B*S, 3*n_heads*128] (RoPE applied),
 * key_mask uint8/bool [B,S] or NULL, out bf16 [B*S, n_heads*128], lse fp32 [B,n_heads,S].
 * Backward writes dq|dk|dv into dqkv (same packing). workspace: llark_attn_bwd_workspace bytes. */
int llark_attn_fwd(const void* qkv, const unsigned char* key_mask, void* out, float* lse, int B, int S, int n_heads,
                   int head_dim, float scale, cudaStream_t stream);
/* ALiBi variant of the causal attention for the CLAP + MPT-1B path (m2t/llava/model/mpt/attention.py:31-83,458-484):
 * scores = q.k * scale + slopes[h] * (key - (S - 1)); packed qkv WITHOUT RoPE; slopes fp32 [n_heads]; otherwise the contract of
 * llark_attn_fwd / llark_attn_bwd (workspace: llark_attn_bwd_workspace bytes). S <= 4096. */
int llark_attn_alibi_fwd(const void* qkv, const unsigned char* key_mask, void* out, float* lse, const float* slopes,
                         int B, int S, int n_heads, int head_dim, float scale, cudaStream_t stream);
int llark_attn_alibi_bwd(const void* qkv, const unsigned char* key_mask, const void* out, const void* dout,
                         const float* lse, void* dqkv, const float* slopes, int B, int S, int n_heads, int head_dim,
                         float scale, void* workspace, cudaStream_t stream);
/* Bias-free LayerNorm over bf16 rows with row strides (elements) ldx / ldy: y = bf16(((x - mean) * rstd) * w), fp32
 * statistics written to mean / rstd (may be NULL). LPLayerNorm (m2t/llava/model/mpt/norm.py:26-52) and the q_ln / k_ln
 * of attention.py:289-292. Backward: dx = [dres +] rstd * (g - mean(g) - xhat * mean(g * xhat)), g = dy * w; dw (bf16
 * [W], may be NULL) receives (or accumulates) sum_rows dy * xhat; dres is a dense [rows, W] tensor or NULL. */
int llark_ln_fwd(const void* x, long long ldx, const void* w, void* y, long long ldy, float* mean, float* rstd,
                 long long rows, int W, float eps, cudaStream_t stream);
long long llark_ln_bwd_workspace(long long rows, int W);
int llark_ln_bwd(const void* x, long long ldx, const void* w, const void* dy, long long lddy, const float* mean,
                 const float* rstd, const void* dres, void* dx, long long lddx, void* dw, int accumulate_dw, long long rows,
                 int W, void* workspace, cudaStream_t stream);
/* Exact GELU (nn.GELU(approximate="none"), m2t/llava/model/mpt/blocks.py:14) and its backward du = dh * (Phi(u) +
 * u * phi(u)); bf16, n a multiple of 8. */
int llark_gelu_fwd(const void* u, void* h, long long n, cudaStream_t stream);
int llark_gelu_bwd(const void* u, const void* dh, void* du, long long n, cudaStream_t stream);
/* Skinny linear layer of the decode step: C[M,N] = A[M,K] . W[N,K]^T (+ bias[N]) (+ R[M,N]), 1 <= M <= 8, bf16, fp32
 * accumulation; K and the leading dimensions (elements) multiples of 8. Streams W once (HBM-bound SIMT kernel; the tcgen05
 * GEMM core would run 128-row tiles of padding). Same arithmetic contract as llark_gemm with these arguments
 * (transformers LlamaDecoderLayer linears reached from m2t/models/llamav2.py:224 during generate, m2t/infer.py:146-152). */
int llark_gemv(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc, const void* bias,
               const void* R, long long ldr, int M, int N, int K, cudaStream_t stream);
/* Single-token decode step against a KV cache (transformers' cached LlamaAttention behind m2t/infer.py's
 * model.generate): q [B, n_heads*128] (RoPE applied), k_cache / v_cache [B, s_max, n_heads*128] bf16, lens int32 [B] =
 * valid cached positions per row including the new token (<= s_max <= 4096), out [B, n_heads*128]. */
int llark_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* lens, void* out, int B,
                      int s_max, int n_heads, int head_dim, float scale, cudaStream_t stream);
long long llark_attn_bwd_workspace(int B, int S, int n_heads);
int llark_attn_bwd(const void* qkv, const unsigned char* key_mask, const void* out, const void* dout, const float* lse,
                   void* dqkv, int B, int S, int n_heads, int head_dim, float scale, void* workspace,
                   cudaStream_t stream);
/* llark_attn_bwd with the inverse rotary embedding of the dq | dk heads fused into the backward kernels' epilogues
 * (rope_cos / rope_sin: bf16 [S, 128], position = row % S): dqkv is then the gradient of the PRE-RoPE QKV projection
 * output, bit-identical to llark_attn_bwd followed by llark_rope(inverse = 1) -- one pass over dqkv less per layer. */
int llark_attn_bwd_rope(const void* qkv, const unsigned char* key_mask, const void* out, const void* dout,
                        const float* lse, void* dqkv, int B, int S, int n_heads, int head_dim, float scale,
                        const void* rope_cos, const void* rope_sin, void* workspace, cudaStream_t stream);

/* Column sum of a bf16 [rows, H] matrix into bf16 [H] (+= if accumulate): the mm_projector bias gradient. */
int llark_colsum(const void* x, void* out, long long rows, int H, int accumulate, cudaStream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Shifted cross-entropy on bf16 logits (m2t/models/llamav2.py:314-325): target of row (b,s) is labels[b,s+1],
 * ignore_index -100, mean over valid targets. logits bf16 [B*S, ldv] (ldv >= V, multiple of 8).
 * fwd: row_loss,row_lse fp32 [B*S]; loss_out fp32[2] = {mean loss, n_valid}.
 * bwd: dlogits = (gscale or *gscale_ptr) / n_valid * (softmax - onehot); rows without target and pad columns 0.
 */
int llark_ce_fwd(const void* logits, long long ldv, int V, const long long* labels, int B, int S, float* row_loss,
                 float* row_lse, float* loss_out, cudaStream_t stream);
int llark_ce_bwd(const void* logits, long long ldv, int V, const long long* labels, int B, int S, const float* row_lse,
                 const float* loss_out, const float* gscale_ptr, float gscale, void* dlogits, cudaStream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Optimizer over the flat bf16 parameter / gradient buckets (HF Trainer: clip_grad_norm_(1.0) + torch AdamW on
 * bf16 tensors, m2t/arguments.py:84, m2t/train.py:101-103). sumsq: fp32[1] device scalar = sum g^2 (before
 * grad_scale). Step applies g*grad_scale, the global-norm clip (max_norm <= 0 disables), then AdamW with a bf16
 * rounding after every elementwise op as torch's foreach implementation does. n % 8 == 0.
 */
long long llark_sumsq_workspace(void);
int llark_grad_sumsq(const void* g, long long n, float* out, int accumulate, void* workspace, cudaStream_t stream);
int llark_adamw_step(void* p, void* g, void* m, void* v, long long n, const float* sumsq, float lr, float beta1,
                     float beta2, float eps, float weight_decay, int step, float grad_scale, float max_norm,
                     int zero_grad, cudaStream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Gradient-bucket all-reduce (DDP, scripts/training/train_llark.sh:20-22,44): one ncclAllReduce(sum, bf16) over
 * the flat gradient bucket. The communicator is created from a 128-byte ncclUniqueId that rank 0 obtains with
 * llark_comm_unique_id and shares out of band (torch.distributed broadcast).
 */
int llark_comm_unique_id(void* id128_host);
int llark_comm_init(void** comm_out, const void* id128_host, int world, int rank);
int llark_comm_destroy(void* comm);
int llark_grad_bucket_allreduce(void* comm, void* grads_bf16, long long n, cudaStream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Jukebox front end (jukebox/main.py:54-68 get_z, :101-110 get_final_activations, :113-130 windowed_average;
 * arithmetic of openai/jukebox@08efbbc). All fp32 activations unless noted.
 */
/* Strided down-conv Conv1d(c_in -> c_out, k=4, s=2, p=1) + bias. x [N, c_in, T] -> y [N, c_out, T/2]. */
int llark_jb_conv_down(const float* x, const float* w, const float* bias, float* y, int N, int c_in, int c_out, int T,
                       cudaStream_t stream);
/* Fused ResConv1DBlock: y = x + W2 * relu(W1 (*dil) relu(x) + b1) + b2, width 32 channels. x,y [N,32,T]. */
int llark_jb_resblock(const float* x, const float* w1, const float* b1, const float* w2, const float* b2, float* y,
                      int N, int T, int dilation, cudaStream_t stream);
/* Conv1d(c_in -> c_out, k=3, s=1, p=1) + bias (block output projection 32 -> 64). */
int llark_jb_conv_k3(const float* x, const float* w, const float* bias, float* y, int N, int c_in, int c_out, int T,
                     cudaStream_t stream);
/* Nearest-code search: x [N,64,T] (channels-first), codebook [n_codes,64]; codes int64 [N,T].
 * dist = |x|^2 - 2 x.k + |k|^2 in fp32, first minimum wins (torch.min semantics). */
int llark_jb_vq_encode(const float* x, const float* codebook, long long* codes, int N, int T, int n_codes,
                       cudaStream_t stream);
/* LayerNorm over the last dim (eps 1e-5, affine), fp32 in, bf16 or fp32 out. */
int llark_layernorm_fwd(const float* x, const float* gamma, const float* beta, void* y, int y_bf16, long long rows,
                        int W, float eps, cudaStream_t stream);
/* x0[t,:] = (t == 0 ? y_cond : emb[codes[t-1]]) + pos_emb[t] + x_cond[t]   (shift-right + conditioning). */
int llark_jb_embed_tokens(const long long* codes, const float* emb, const float* y_cond, const float* pos_emb,
                          const float* x_cond, float* out, int N, int T, int W, cudaStream_t stream);
/* Jukebox factored attention on qkv [N*T, 3*heads*dh] (fp32): pattern 0 = block (causal inside blocks of
 * `block`), 1 = transposed block (causal across blocks at equal offset), 2 = previous block (full, block 0 sees
 * nothing -> zeros). out fp32 [N*T, heads*dh]. */
int llark_jb_sparse_attn(const float* qkv, float* out, int N, int T, int heads, int dh, int block, int pattern,
                         cudaStream_t stream);
/* Same contract on tensor cores (mma.sync m16n8k8: operands rounded to TF32, fp32 accumulate and softmax): groups of
 * 64 or 128 rows, even dh <= 152. out: fp32, or bf16 when out_bf16 != 0 (the bf16 prior's cast fused in). Returns
 * LLARK_EINVAL for a geometry outside that envelope (use llark_jb_sparse_attn then). */
int llark_jb_sparse_attn_tc(const float* qkv, void* out, int out_bf16, int N, int T, int heads, int dh, int block,
                            int pattern, cudaStream_t stream);
/* y = x * sigmoid(1.702 x) in place-safe form. */
int llark_quick_gelu(const float* x, float* y, long long n, cudaStream_t stream);
/* out = a + b + c (c may be NULL). */
int llark_add3(const float* a, const float* b, const float* c, float* out, long long n, cudaStream_t stream);
/* AvgPool1d(frame, stride frame, floor) over time: acts [T, W] -> out [T/frame, W] (jukebox/main.py:113-130). */
int llark_jb_pool(const float* acts, float* out, int T_valid, int W, int frame, cudaStream_t stream);
/* Timing conditioning x_cond of the top-level prior (upstream LabelConditioner's pos_emb, reached from
 * jukebox/main.py:93): out[t,:] = (total_row + abs_table[abs_bins[t],:]) + rel_table[rel_bins[t],:], fp32 [T, W]. */
int llark_jb_label_cond(const float* total_row, const float* abs_table, const float* rel_table, const int* abs_bins,
                        const int* rel_bins, float* out, int T, int W, cudaStream_t stream);
/* the same pool over N clips in one launch: acts [N, clip_stride/W rows, W], out [N, T_valid/frame, W] */
int llark_jb_pool_batched(const float* acts, float* out, int N, long long clip_stride, int T_valid, int W, int frame,
                          cudaStream_t stream);

/* ---- fp32 verification path of the Llama forward (csrc/verify_fp32.cu): what llark_b200/verify.py runs to check
 * north_star's "fp32 logits within 1e-3 relative" against the reference's fp32 run of m2t/models/llamav2.py:259-337
 * (transformers LlamaModel: LlamaRMSNorm, rotate_half RoPE, eager softmax attention, SiLU(gate)*up, shifted mean CE).
 * All tensors fp32. The linears are llark_gemm(in_fp32=1) composed as 3xTF32 from llark_v32_split_tf32's halves. */
int llark_v32_split_tf32(const float* x, float* hi, float* lo, long long n, cudaStream_t stream);
int llark_v32_embed_splice_fwd(const long long* ids, const float* table, const float* audio, const long long* audio_off,
                               const int* frames, const int* start_pos, float* out, int B, int S, int H, long long vocab,
                               cudaStream_t stream);
int llark_v32_rmsnorm_fwd(const float* x, const float* w, float* y, long long rows, int H, float eps, cudaStream_t stream);
int llark_v32_rope(float* qkv, const float* cos_t, const float* sin_t, long long rows, int S, int n_rot_heads, int D,
                   long long ld, cudaStream_t stream);
int llark_v32_swiglu_fwd(const float* gu, float* act, long long rows, int I, cudaStream_t stream);
int llark_v32_attn_fwd(const float* qkv, const unsigned char* key_mask, float* out, int B, int S, int n_heads, int D,
                       float scale, cudaStream_t stream);
int llark_v32_ce_fwd(const float* logits, long long ldv, int V, const long long* labels, int B, int S, float* row_loss,
                     float* loss_out, cudaStream_t stream);

/* ---- generation path of layer-list decoders (csrc/seq_ops.cu, csrc/seq_mixers.cu). The reference generates through
 * transformers' GenerationMixin with a per-layer key / value cache (m2t/infer.py:146-152 -> m2t/models/llamav2.py:339-365);
 * these are the per-step ops of decoders assembled from other parts (sliding-window attention, gated linear recurrence,
 * short convolutions, norm-on-output residual blocks), which the reference does not have. One step is a PACKED batch:
 * the new tokens of all requests concatenated [n_tok, width]; tok_seq[t] = request of token t, cu[b] = first row of
 * request b (cu[n_seq] = n_tok), pos0[b] = position of that row in its sequence, slot[b] = the request's row in every
 * state store. The residual stream, norms, scores, softmax and recurrent state are fp32; `act_fp32` selects the
 * activation / matrix dtype (0: bf16, 1: float = the all-fp32 mode). */
int llark_seq_embed(const int* ids, const int* tok_seq, const int* cu, const int* pos0, const void* table,
                    const void* pos_table, float scale, float* x, int n_tok, int C, int act_fp32, cudaStream_t stream);
/* y = h + conv(h): causal depthwise convolution over time, w fp32 [C, taps], tail fp32 [slots, taps-1, C] = the last
 * taps-1 inputs of each request, oldest first. inline_tail = 1 (every request brings one token) also shifts the tail;
 * otherwise call llark_seq_conv_tail after it. */
int llark_seq_short_conv(const float* h, const float* w, float* tail, const int* tok_seq, const int* cu, const int* slot,
                         void* y, int n_tok, int C, int taps, int inline_tail, int act_fp32, cudaStream_t stream);
int llark_seq_conv_tail(const float* h, float* tail, const int* cu, const int* slot, int n_seq, int C, int taps,
                        cudaStream_t stream);
/* x_out = x + y / sqrt(mean(y^2) + eps) * w (row-wise; x_out may not alias x when other rows of x are still read by the
 * caller); x_act (optional) receives x_out in the activation dtype. */
int llark_seq_add_rmsnorm(const float* x, const float* y, const float* w, float* x_out, void* x_act, long long rows, int C,
                          float eps, int act_fp32, cudaStream_t stream);
/* x_out = x + rmsnorm(y * sigmoid(gate)) * w (gate optional: a column slice with row pitch gate_ld); when x_act != NULL it
 * also receives rmsnorm(x_out) * w_next in the activation dtype (the next sublayer's input norm). All norms over the row. */
int llark_seq_gated_norm_add(const float* x, const float* y, const float* gate, long long gate_ld, const float* w,
                             const float* w_next, float* x_out, void* x_act, long long rows, int C, float eps,
                             int act_fp32, cudaStream_t stream);
/* out[i] = rmsnorm(x[rows[i]]) * w in the activation dtype (rows == NULL: row i). */
int llark_seq_rmsnorm_rows(const float* x, const int* rows, const float* w, void* out, int n_rows, int C, float eps,
                           int act_fp32, cudaStream_t stream);
int llark_seq_relu2(const void* u, void* y, long long n, int act_fp32, cudaStream_t stream);
/* C[M,N] = A[M,K] W[N,K]^T (+ bias fp32[N]), fp32 accumulation, A / W bf16 or (in_fp32) float, C float if c_fp32.
 * _rows: weight-streaming, for a handful of rows (decode). _simt: tiled, any shape, true fp32 when in_fp32. */
int llark_linear_rows(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc, int c_fp32,
                      const float* bias, int M, int N, int K, int in_fp32, cudaStream_t stream);
int llark_linear_simt(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc, int c_fp32,
                      const float* bias, int M, int N, int K, int in_fp32, cudaStream_t stream);
/* Per-head RMS norm of the q (H heads at column q_off) and k (G heads at k_off) parts of src fp32 [n_tok, ld] with
 * weights wq, wk fp32 [D]: qn [n_tok, H, D], kn [n_tok, G, D], vraw = the un-normed k. kring / vring non-NULL: also
 * written to ring entry position % cap of the request's slot (only when every request brings one token). */
int llark_seq_qk_headnorm(const float* src, long long ld, int q_off, int k_off, const float* wq, const float* wk, void* qn,
                          void* kn, void* vraw, void* kring, void* vring, const int* tok_seq, const int* cu,
                          const int* pos0, const int* slot, int n_tok, int H, int G, int D, int cap, float eps,
                          int act_fp32, cudaStream_t stream);
/* The same with values of their own: E columns per key / value head at v_off of src, copied (not normed) to vv
 * [n_tok, G, E] and the value ring. temp_every > 0: the query at position p of its sequence is also multiplied by
 * 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1). */
int llark_seq_qkv_headnorm(const float* src, long long ld, int q_off, int k_off, int v_off, const float* wq,
                           const float* wk, void* qn, void* kn, void* vv, void* kring, void* vring, const int* tok_seq,
                           const int* cu, const int* pos0, const int* slot, int n_tok, int H, int G, int D, int E, int cap,
                           float eps, float temp_coef, int temp_every, int act_fp32, cudaStream_t stream);
/* q / k / v of a fused projection with rotary positions. wq / wk (both or neither): RMS norm over the WHOLE q (H*D) and k
 * (G*D) projection with weights of that size. qk_freq fp32 [n_rot / 2]: the first n_rot entries of every q / k head are
 * rotated by position * qk_freq[i], pairs (i, i + n_rot/2) or, qk_interleaved, (2i, 2i + 1). v_freq fp32 [E / 2] (optional):
 * every value head is rotated the same way over all of E. Results in the activation dtype; with kring / vring the k / v rows
 * also go to ring entry position % cap of the slot. */
int llark_seq_qkv_rotary(const float* src, long long ld, int q_off, int k_off, int v_off, const float* wq, const float* wk,
                         const float* qk_freq, int n_rot, int qk_interleaved, const float* v_freq, int v_interleaved,
                         void* qn, void* kn, void* vv, void* kring, void* vring, const int* tok_seq, const int* cu,
                         const int* pos0, const int* slot, int n_tok, int H, int G, int D, int E, int cap, float eps,
                         int act_fp32, cudaStream_t stream);
/* Sliding-window softmax attention: query at position i sees keys j with 0 <= i - j < window. Keys / values of this
 * step come from kn / vv ([n_tok, G, D] / [n_tok, G, E]), earlier ones from the rings [slots, cap, G, D|E] (entry
 * j % cap); from_ring_only = 1: the step's own token is already in the ring. score = q.k * scale_h[h]; the output is
 * multiplied by sigmoid(gate[t, h*E + e]) when gate != NULL (gate_per_head: by sigmoid(gate[t, h])). sink (optional)
 * fp32 [H]: exp(sink[h]), unscaled, is one more term of head h's softmax denominator; it has no value. A window of at
 * least cap positions with cap >= the longest sequence is plain causal attention. chunk > 0 replaces the window: the query
 * sees j <= i with floor(j / chunk) = floor(i / chunk). softcap > 0: score <- softcap * tanh(score / softcap). vfreq fp32
 * [E / 2] (optional): the values are stored rotated by their own position (llark_seq_qkv_rotary); each head's weighted sum is
 * turned back by the query's position before the gate (v_interleaved: pairs (2m, 2m + 1), else (m, m + E/2)).
 * out [n_tok, H, E]. */
int llark_seq_swa_attn(const void* qn, const void* kn, const void* vv, const void* kring, const void* vring,
                       const float* gate, long long gate_ld, const float* scale_h, void* out, const int* tok_seq,
                       const int* cu, const int* pos0, const int* slot, int n_tok, int H, int G, int D, int E, int window,
                       int cap, int from_ring_only, const float* sink, int gate_per_head, int chunk, float softcap,
                       const float* vfreq, int v_interleaved, int act_fp32, cudaStream_t stream);
/* The same attention for steps that bring many tokens per request (prompts, portions): bf16 only, D = E a multiple of
 * 16 up to 256, 64-query CTAs on mma.sync with fp32 scores / softmax (csrc/seq_swa_mma.cu). max_len = the longest
 * request of the step. Un-rotation in halves needs D = 64, 128 or 256. */
int llark_seq_swa_attn_mma(const void* qn, const void* kn, const void* vv, const void* kring, const void* vring,
                           const float* gate, long long gate_ld, const float* scale_h, void* out, const int* cu,
                           const int* pos0, const int* slot, int n_seq, int max_len, int H, int G, int D, int window,
                           int cap, const float* sink, int gate_per_head, int chunk, float softcap, const float* vfreq,
                           int v_interleaved, cudaStream_t stream);
int llark_seq_kv_ring_write(const void* kn, const void* vv, void* kring, void* vring, const int* tok_seq, const int* cu,
                            const int* pos0, const int* slot, int n_tok, int GD, int GE, int cap, int act_fp32,
                            cudaStream_t stream);
/* Gated linear recurrence over src fp32 [n_tok, ld] (q_pre at q_off, f_pre incl. bias at f_off: H*D columns each; v at
 * v_off: H*E columns): q = silu(q_pre), f = lower + (1 - lower) * sigmoid(f_pre) (lower fp32 [H*D] or NULL = 0),
 * S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t, all fp32, D <= 256. The rows are handed over as work items:
 * item w covers rows item_row0[w] .. + item_n[w] of one request, starts from init_buf[item_init[w]] ([*, H, D, E]; -1:
 * zero) and leaves its last state in final_buf[item_final[w]] (-1: nowhere). decay_buf (optional) [n_items, H, D] gets the
 * product of the item's forget gates; o_raw (optional) fp32 [n_tok, H*E] the outputs. One pass with items = requests and
 * init = final = the slot in the state store is the plain scan. Long prompts: pass 1 over chunks from zero (local states +
 * decays, no outputs), llark_seq_glr_combine turns the local states into each chunk's starting state, pass 2 over the
 * chunks from those writes the outputs and (last chunk) the request's state. */
int llark_seq_glr_scan(const float* src, long long ld, int q_off, int f_off, int v_off, const float* lower,
                       const float* init_buf, float* final_buf, float* decay_buf, float* o_raw, const int* item_row0,
                       const int* item_n, const int* item_init, const int* item_final, int n_items, int H, int D, int E,
                       cudaStream_t stream);
int llark_seq_glr_combine(const float* state, float* chunk_state, const float* chunk_decay, const int* seq_item0,
                          const int* slot, int n_seq, int H, int D, int E, cudaStream_t stream);
int llark_seq_head_rmsnorm(const float* x, const float* w, void* out, long long n_rows, int E, float eps, int act_fp32,
                           cudaStream_t stream);

/* ---- further parts of layer-list decoders: grouped RMS norm, parallel-sublayer residual, delta-rule recurrences
 * (csrc/seq_delta.cu), latent attention (csrc/seq_latent.cu), routed mixture of experts (csrc/seq_moe.cu) ---- */
/* y = A W^T (+ bias) with fp32 weights and bf16 or fp32 activations, fp32 output (router logits) */
int llark_linear_simt_w32(const void* A, long long lda, const float* W, long long ldw, float* C, long long ldc,
                          const float* bias, int M, int N, int K, int in_fp32, cudaStream_t stream);
/* out[r] = norm of x[rows ? rows[r] : r] (+ add_vec) in `groups` equal consecutive parts, each divided by its own
 * sqrt(mean(part^2) + eps), times w; with x_out (rows == NULL) the sum x + add_vec is written too */
int llark_seq_group_rmsnorm(const float* x, const int* rows, const float* add_vec, float* x_out, const float* w, void* out,
                            int n_rows, int C, int groups, float eps, int out_fp32, cudaStream_t stream);
/* x_out = x + (y + sum_k wts[t, k] * z[pos_of[t * top + k]]); top = 0: x + y */
int llark_seq_residual_combine(const float* x, const float* y, const float* z, const int* pos_of, const float* wts,
                               int top, float* x_out, int n_tok, int C, cudaStream_t stream);
/* out[t, c] = act(bias[c] + sum_j w[c, j] * src[t - taps + 1 + j, c]) (bias optional) over n_ch columns of a strided fp32 matrix (src points at the
 * first column); carry fp32 [slots, taps-1, n_ch] holds each request's last inputs and is refreshed */
int llark_seq_conv_act(const float* src, long long ld, const float* w, float* carry, const int* tok_seq, const int* cu,
                       const int* slot, float* out, int n_tok, int n_seq, int n_ch, int taps, int silu, const float* bias,
                       cudaStream_t stream);
/* the five vectors {q, z, d, p1, p2} [n_tok, H, 5, D] of the delta-rule scan; rule 0: gated delta rule, rule 1:
 * generalized delta rule, rule 2: gated delta rule with one decay per head, rule 3: state-space rule S <- a S + dt B x^T,
 * y = S^T C (see csrc/seq_delta.cu) */
int llark_seq_delta_prep(int rule, const float* q, long long q_ld, const float* k, long long k_ld, const float* dec,
                         long long dec_ld, const float* dec_bias, const float* rate_log, const float* mix,
                         long long mix_ld, float* vec, int n_tok, int H, int G, int D, float unit_eps,
                         cudaStream_t stream);
/* S[:, e] = d S[:, e] + p1 (z . S[:, e]) + p2 v[e], o[e] = q . S[:, e] per token; state fp32 [slots, H, D, E];
 * correct = 0: the p1 term is skipped (rules whose p1 is zero) */
int llark_seq_delta_scan(const float* vec, const float* v, long long v_ld, float* state, float* o, const int* cu,
                         const int* slot, int n_seq, int n_tok, int H, int D, int E, int correct, cudaStream_t stream);
/* per-head RMS norm of x fp32 [n_tok, H, E], times w ([E] shared or [H, E]), times sigmoid(gate) (gate_silu: times
 * gate * sigmoid(gate)) -> ACT */
int llark_seq_head_norm_gate(const float* x, const float* w, int w_per_head, const float* gate, long long gate_ld,
                             void* out, long long n_tok, int H, int E, float eps, int gate_silu, int act_fp32,
                             cudaStream_t stream);
/* read-out of a state-space mixer: y = (o + skip[h] * xin) * silu(gate) over the H * E inner channels, RMS norm of each
 * of `groups` equal consecutive parts, times w fp32 [H * E] -> ACT [n_tok, H * E] */
int llark_seq_skip_gate_group_norm(const float* o, const float* xin, long long x_ld, const float* skip, const float* gate,
                                   long long gate_ld, const float* w, void* out, long long n_tok, int H, int E, int groups,
                                   float eps, int act_fp32, cudaStream_t stream);
/* Norm after the residual sum: x_out = rmsnorm(alpha * x + f) * w, f = branch_scale * (b1 + b2) + sum_k wts[t, k] * e_k
 * with b_i = y_i, or rmsnorm(y_i) * w_i when w_i is given (y2 optional), and e_k = row pos_of[t * top + k] of z, or x
 * itself when ids[t * top + k] >= n_real (top = 0: no such terms). x_act (optional) gets x_out in the activation dtype. */
int llark_seq_post_norm(const float* x, float alpha, const float* y1, const float* w1, const float* y2, const float* w2,
                        float branch_scale, const float* z, const int* pos_of, const float* wts, const int* ids, int top,
                        int n_real, const float* w, float* x_out, void* x_act, long long rows, int C, float eps,
                        int act_fp32, cudaStream_t stream);
/* act = g' * sigmoid(slope * g') * (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit); gu = [g | u] rows */
int llark_seq_glu_clamped(const void* gu, void* act, long long rows, int ff, float limit, float slope, int act_fp32,
                          cudaStream_t stream);
/* z <- cap * tanh(z * scale / cap) in place (cap <= 0: z * scale) */
int llark_seq_logit_cap(float* z, long long n, float scale, float cap, cudaStream_t stream);
/* latent attention: normed latent and rotated shared key part -> ckr ACT [n_tok, R + P] (and the ring row of the
 * token's position when ring != NULL), rotated query parts -> qf ACT [n_tok, H, R + P] columns R.. Rotary pairs are
 * (2i, 2i + 1), or with halves = 1 (i, i + n_rot / 2). */
int llark_seq_latent_prep(const float* q, long long q_ld, const float* lat, long long lat_ld, const float* norm_w,
                          const float* freqs, int n_rot, float mult, void* ckr, void* qf, void* ring, const int* tok_seq,
                          const int* cu, const int* pos0, const int* slot, int n_tok, int H, int Dn, int P, int R, int cap,
                          float eps, int halves, int act_fp32, cudaStream_t stream);
/* y[m, h * y_hs + n] = sum_k x[m, h * x_hs + k] * w[h][n][k] (* sigmoid(gate[m, h * N + n])) */
int llark_seq_head_linear(const void* x, int x_fp32, long long ldx, int x_hs, const void* w, void* y, long long ldy,
                          int y_hs, const float* gate, long long gate_ld, int M, int H, int N, int K, int act_fp32,
                          cudaStream_t stream);
/* y = tanh(u), fp32 in, ACT out */
int llark_seq_tanh(const float* u, void* y, long long n, int act_fp32, cudaStream_t stream);
/* C[off[e] .. off[e+1]) = A[same rows] @ B[e]^T, e < n_seg; B bf16 [n_seg, N, K]; seg_off_host on the host */
int llark_gemm_segments(const void* A, long long lda, const void* B, void* C, long long ldc, int c_fp32,
                        const int* seg_off_host, int n_seg, const int* seg_tiles_dev, int n_tiles, const int* seg_count_dev,
                        int m_total, int N, int K, cudaStream_t stream);
/* routed mixture of experts (see csrc/seq_moe.cu) */
int llark_seq_moe_route(const float* logits, long long ld, int* ids, float* wts, int n_tok, int n_exp, int n_groups,
                        int keep, int top, float scale, cudaStream_t stream);
/* softmax scores; choice on score + correction (optional) within the `keep` groups whose best choice score is largest;
 * weights = the chosen experts' plain scores * scale */
int llark_seq_moe_route_bias(const float* logits, long long ld, const float* correction, int* ids, float* wts, int n_tok,
                             int n_exp, int n_groups, int keep, int top, float scale, cudaStream_t stream);
int llark_seq_moe_tile_rows(void);
/* meta[0] = number of 64-row tiles; with tiles256: 256-row tiles for llark_gemm_segments, their number in meta[1];
 * experts >= n_real have no weights and get no tiles */
int llark_seq_moe_sort(const int* ids, int n_ent, int n_exp, int n_real, int* perm, int* pos_of, int* tiles, int* meta,
                       int* seg_off, int* tiles256, cudaStream_t stream);
/* xs[p] = x[perm[p] / top] (rows in sorted order); act = silu(gu[:, :ff]) * gu[:, ff:] */
int llark_seq_moe_gather(const void* x, long long ldx, const int* perm, int top, void* xs, int n_ent, int C, int act_fp32,
                         cudaStream_t stream);
int llark_seq_silu_mul(const void* gu, void* act, long long rows, int ff, int act_fp32, cudaStream_t stream);
int llark_seq_moe_up(const void* x, long long ldx, const int* perm, int top, const void* w_gate_up, void* act,
                     const int* tiles, const int* meta, int max_tiles, int n_ent, int ff, int K, int act_fp32,
                     cudaStream_t stream);
int llark_seq_moe_down(const void* act, const void* w_down, float* z, const int* tiles, const int* meta, int max_tiles,
                       int n_ent, int C, int ff, int act_fp32, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LLARK_B200_H */
