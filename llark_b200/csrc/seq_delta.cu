// Delta-rule recurrences of the generation path (layer-list decoders): a matrix state S [D, E] per head and request that
// every token decays per key channel, corrects along one direction and writes into,
//
//     S_t[:, e] = d_t * S_(t-1)[:, e] + p1_t * (z_t . S_(t-1)[:, e]) + p2_t * v_t[e],      o_t[e] = q_t . S_t[:, e]
//
// with five D-vectors per token and head. Two rules are stated in that form by llark_seq_delta_prep:
//
//   gated delta rule          S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q   (q, k unit vectors, q / sqrt D)
//                             d = g, z = g k, p1 = -beta k, p2 = beta k          g = exp(-exp(A) softplus(a + dt))
//   generalized delta rule    S <- diag(w) S - (a u)(u^T S) + k v^T,  u = k / |k|;  o = S^T r
//                             d = w, z = u, p1 = -(a u), p2 = k                  w = exp(-exp(-1/2) sigmoid(.)), a = sigmoid(.)
//
// Everything here is fp32: the state, the vectors, decays, softplus / exponentials, unit norms and the outputs.
//
//   llark_seq_conv_act        causal depthwise convolution over a column range of a strided fp32 matrix + SiLU, with
//                             carry of the last taps-1 inputs per request (and llark_seq_conv_carry, its refresh)
//   llark_seq_delta_prep      projections -> the five vectors
//   llark_seq_delta_scan      the recurrence; state read and written once per step
//   llark_seq_head_norm_gate  per-head RMS norm of o, weight (shared by the heads or one per head), sigmoid gate -> ACT
#include "common.cuh"

namespace llark {
extern thread_local int g_last_cuda_error;
namespace delta {

static int check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        return LLARK_ECUDA;
    }
    return LLARK_OK;
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// ------------------------------------------------------------------------------------------------ convolution + SiLU
// out[t, c] = act(sum_j w[c, j] * in[t - taps + 1 + j, c]) with in = src[:, col0 + c]; rows before the step's first come
// from carry[slot][k][c], k = 0 .. taps-2 oldest first. inline_carry: one token per request, the reading thread shifts.
__global__ void conv_act_kernel(const float* __restrict__ src, long long ld, const float* __restrict__ w,
                                float* __restrict__ carry, const int* __restrict__ tok_seq, const int* __restrict__ cu,
                                const int* __restrict__ slot, float* __restrict__ out, int n_ch, int taps, int silu,
                                int inline_carry, const float* __restrict__ bias) {
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    const int local = t - cu[b];
    float* cr = carry + (long long)slot[b] * (taps - 1) * n_ch;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n_ch; c += gridDim.y * blockDim.x) {
        const float cur = src[(long long)t * ld + c];
        float acc = bias ? bias[c] : 0.f;
        for (int j = 0; j < taps - 1; ++j) {
            const int s = local - taps + 1 + j;
            const float v = s >= 0 ? src[(long long)(t - local + s) * ld + c] : cr[(long long)(taps - 1 + s) * n_ch + c];
            acc = fmaf(w[c * taps + j], v, acc);
        }
        acc = fmaf(w[c * taps + taps - 1], cur, acc);
        out[(long long)t * n_ch + c] = silu ? acc * sigmoidf_(acc) : acc;
        if (inline_carry) {
            for (int k = 0; k + 1 < taps - 1; ++k) cr[(long long)k * n_ch + c] = cr[(long long)(k + 1) * n_ch + c];
            if (taps > 1) cr[(long long)(taps - 2) * n_ch + c] = cur;
        }
    }
}

// Prompts: a thread walks TB consecutive rows of one channel with the last TAPS-1 inputs in registers, so every input is
// read once (the per-row kernel reads it TAPS times) and the accesses of a warp are adjacent channels of one row. The
// window is rebuilt wherever a request starts inside the run of rows.
template <int TAPS, int TB>
__global__ void conv_act_rows_kernel(const float* __restrict__ src, long long ld, const float* __restrict__ w,
                                     const float* __restrict__ carry, const int* __restrict__ tok_seq,
                                     const int* __restrict__ cu, const int* __restrict__ slot, float* __restrict__ out,
                                     int n_tok, int n_ch, int silu, const float* __restrict__ bias) {
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= n_ch) return;
    const int t0 = blockIdx.x * TB;
    float wr[TAPS], win[TAPS > 1 ? TAPS - 1 : 1];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wr[j] = w[(long long)c * TAPS + j];
    const float b0 = bias ? bias[c] : 0.f;
    for (int i = 0; i < TB && t0 + i < n_tok; ++i) {
        const int t = t0 + i;
        const int b = tok_seq[t];
        const int local = t - cu[b];
        if (i == 0 || local < TAPS - 1) {
            const float* cr = carry + (long long)slot[b] * (TAPS - 1) * n_ch;
#pragma unroll
            for (int j = 0; j < TAPS - 1; ++j) {
                const int s = local - (TAPS - 1) + j;
                win[j] = s >= 0 ? src[(long long)(t - local + s) * ld + c] : cr[(long long)(TAPS - 1 + s) * n_ch + c];
            }
        }
        const float cur = src[(long long)t * ld + c];
        float acc = b0;
#pragma unroll
        for (int j = 0; j < TAPS - 1; ++j) acc = fmaf(wr[j], win[j], acc);
        acc = fmaf(wr[TAPS - 1], cur, acc);
        out[(long long)t * n_ch + c] = silu ? acc * sigmoidf_(acc) : acc;
#pragma unroll
        for (int j = 0; j + 1 < TAPS - 1; ++j) win[j] = win[j + 1];
        if (TAPS > 1) win[TAPS - 2] = cur;
    }
}

// new carry[k] = input at local index n - (taps-1) + k: a row of this step, or an older carry entry when negative
__global__ void conv_carry_kernel(const float* __restrict__ src, long long ld, float* __restrict__ carry,
                                  const int* __restrict__ cu, const int* __restrict__ slot, int n_ch, int taps) {
    const int b = blockIdx.x;
    const int r0 = cu[b], n = cu[b + 1] - r0;
    float* cr = carry + (long long)slot[b] * (taps - 1) * n_ch;
    for (int c = threadIdx.x; c < n_ch; c += blockDim.x)
        for (int k = 0; k < taps - 1; ++k) {  // ascending: entry k + n >= k is read before it is rewritten
            const int s = n - (taps - 1) + k;
            cr[(long long)k * n_ch + c] = s >= 0 ? src[(long long)(r0 + s) * ld + c] : cr[(long long)(taps - 1 + s) * n_ch + c];
        }
}

// ------------------------------------------------------------------------------------------------ the five vectors
// Warp per (token, head). vec[t][h] = { q, z, d, p1, p2 } each [D].
//   rule 0 (gated delta):       q, k [n_tok, G, D] (head h reads h / (H / G)); dec [n_tok, H*D] pre-activation of the
//                               decay, + dec_bias [H*D]; rate_log [H]; mix [n_tok, H] pre-activation of beta
//   rule 1 (generalized delta): q = r, k [n_tok, H, D]; dec [n_tok, H*D] (bias included); mix [n_tok, H*D] pre-activation
//                               of the removal rate
//   rule 2 (gated delta, one decay per head): as rule 0 with dec [n_tok, H], dec_bias [H]
//   rule 3 (state space):       S <- a S + dt B x^T, y = S^T C with a = exp(-exp(rate_log_h) dt), dt = softplus(dec +
//                               dec_bias) per head: q = C, k = B [n_tok, G, D] (D = state size), dec [n_tok, H]; the
//                               vectors are q = C, z = 0, d = a, p1 = 0, p2 = dt B (the scan may skip the correction)
__global__ void delta_prep_kernel(int rule, const float* __restrict__ q, long long q_ld, const float* __restrict__ k,
                                  long long k_ld, const float* __restrict__ dec, long long dec_ld,
                                  const float* __restrict__ dec_bias, const float* __restrict__ rate_log,
                                  const float* __restrict__ mix, long long mix_ld, float* __restrict__ vec, int n_tok,
                                  int H, int G, int D, float unit_eps) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)n_tok * H) return;
    const long long t = item / H;
    const int h = (int)(item % H);
    const int g = h / (H / G);
    const float* qr = q + t * q_ld + (long long)g * D;
    const float* kr = k + t * k_ld + (long long)g * D;
    float* o = vec + item * 5 * D;
    float sk = 0.f, sq = 0.f;
    for (int d = lane; d < D; d += 32) {
        sk = fmaf(kr[d], kr[d], sk);
        sq = fmaf(qr[d], qr[d], sq);
    }
    sk = warp_sum(sk);
    sq = warp_sum(sq);
    const float rk = 1.0f / sqrtf(sk + unit_eps);
    if (rule == 3) {
        const float dt = softplusf_(dec[t * dec_ld + h] + dec_bias[h]);
        const float a = expf(-expf(rate_log[h]) * dt);
        for (int d = lane; d < D; d += 32) {
            o[d] = qr[d];
            o[D + d] = 0.f;
            o[2 * D + d] = a;
            o[3 * D + d] = 0.f;
            o[4 * D + d] = dt * kr[d];
        }
    } else if (rule == 2) {
        const float rq = 1.0f / sqrtf(sq + unit_eps) / sqrtf((float)D);
        const float beta = sigmoidf_(mix[t * mix_ld + h]);
        const float gd = expf(-expf(rate_log[h]) * softplusf_(dec[t * dec_ld + h] + dec_bias[h]));
        for (int d = lane; d < D; d += 32) {
            const float kh = kr[d] * rk;
            o[d] = qr[d] * rq;
            o[D + d] = kh * gd;
            o[2 * D + d] = gd;
            o[3 * D + d] = -beta * kh;
            o[4 * D + d] = beta * kh;
        }
    } else if (rule == 0) {
        const float rq = 1.0f / sqrtf(sq + unit_eps) / sqrtf((float)D);
        const float beta = sigmoidf_(mix[t * mix_ld + h]);
        const float rate = expf(rate_log[h]);
        for (int d = lane; d < D; d += 32) {
            const float kh = kr[d] * rk;
            const float gd = expf(-rate * softplusf_(dec[t * dec_ld + (long long)h * D + d] + dec_bias[h * D + d]));
            o[d] = qr[d] * rq;
            o[D + d] = kh * gd;
            o[2 * D + d] = gd;
            o[3 * D + d] = -beta * kh;
            o[4 * D + d] = beta * kh;
        }
    } else {
        for (int d = lane; d < D; d += 32) {
            const float u = kr[d] * rk;
            const float wd = expf(-0.60653065971263342f * sigmoidf_(dec[t * dec_ld + (long long)h * D + d]));
            const float a = sigmoidf_(mix[t * mix_ld + (long long)h * D + d]);
            o[d] = qr[d];
            o[D + d] = u;
            o[2 * D + d] = wd;
            o[3 * D + d] = -(a * u);
            o[4 * D + d] = kr[d];
        }
    }
}

// ------------------------------------------------------------------------------------------------ the recurrence
// Block per (column slice, head, request). R adjacent lanes share CPT adjacent columns of S; lane r owns the 4-row groups r, r + R,
// r + 2R, ... (rows 4 (r + R i) + c) in registers, so that the R lanes read adjacent 16-byte pieces of a vector (no bank
// conflicts; lanes of other columns get the same words by broadcast), and the partial sums over rows are added by shuffle. The vectors and values of TS tokens are brought to
// shared memory with cp.async while the previous TS are computed. Rows d >= D are zero padding (DPT * R >= D).
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// CORR = false: rules without the correction term (p1 = 0, as the state-space rule) skip the z . S pass.
template <int DPT, int CPT, int R, bool CORR>
__global__ void __launch_bounds__(256, 1)
delta_scan_kernel(const float* __restrict__ vec, const float* __restrict__ v, long long v_ld, float* __restrict__ state,
                  float* __restrict__ o, const int* __restrict__ cu, const int* __restrict__ slot, int H, int D, int E,
                  int cols, int ts) {
    extern __shared__ __align__(16) float sm[];
    constexpr int Dp = DPT * R;
    const int stage_floats = ts * (5 * Dp + cols);
    const int h = blockIdx.y, b = blockIdx.z;
    const int cg = threadIdx.x / R, r = threadIdx.x % R;  // column group (CPT adjacent columns), lane within it
    const int e0 = blockIdx.x * cols;
    const int ec = e0 + cg * CPT;                         // first column of this thread
    const int row0 = cu[b], n = cu[b + 1] - row0;
    float S[CPT][DPT];
    float* sp = state + (((long long)slot[b] * H + h) * D) * E;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = 4 * (r + R * (i >> 2)) + (i & 3);
#pragma unroll
        for (int c = 0; c < CPT; ++c) S[c][i] = (ec + c < E && d < D) ? sp[(long long)d * E + ec + c] : 0.f;
    }
    for (int i = threadIdx.x; i < 2 * stage_floats; i += blockDim.x) sm[i] = 0.f;  // padding rows / columns stay zero
    __syncthreads();
    const bool vec16 = (D % 4) == 0;
    auto issue = [&](int tok0, int st) {
        float* base = sm + st * stage_floats;
        const int cnt = n - tok0 < ts ? n - tok0 : ts;
        if (vec16 && Dp == D) {  // a token's five vectors are one contiguous run on both sides
            const int per = 5 * D / 4;
            for (int tk = 0; tk < cnt; ++tk) {
                const float* src = vec + ((long long)(row0 + tok0 + tk) * H + h) * 5 * D;
                float* dst = base + tk * 5 * Dp;
                for (int i = threadIdx.x; i < per; i += blockDim.x) cp_async16(dst + 4 * i, src + 4 * i);
            }
        } else if (vec16) {
            const int per = 5 * D / 4, dq = D / 4;
            for (int i = threadIdx.x; i < cnt * per; i += blockDim.x) {
                const int tk = i / per, rem = i % per, which = rem / dq, d4 = rem % dq;
                cp_async16(base + (tk * 5 + which) * Dp + d4 * 4,
                           vec + (((long long)(row0 + tok0 + tk) * H + h) * 5 + which) * D + d4 * 4);
            }
        } else {
            const int per = 5 * D;
            for (int i = threadIdx.x; i < cnt * per; i += blockDim.x) {
                const int tk = i / per, rem = i % per, which = rem / D, d = rem % D;
                cp_async4(base + (tk * 5 + which) * Dp + d,
                          vec + (((long long)(row0 + tok0 + tk) * H + h) * 5 + which) * D + d);
            }
        }
        float* sv = base + ts * 5 * Dp;
        for (int i = threadIdx.x; i < cnt * cols; i += blockDim.x) {  // cols is a power of two
            const int tk = i / cols, c = i & (cols - 1);
            if (e0 + c < E) cp_async4(sv + tk * cols + c, v + (long long)(row0 + tok0 + tk) * v_ld + (long long)h * E + e0 + c);
        }
        cp_async_commit();
    };
    issue(0, 0);
    int st = 0;
    for (int tok0 = 0; tok0 < n; tok0 += ts, st ^= 1) {
        if (tok0 + ts < n) {
            issue(tok0 + ts, st ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const float* base = sm + st * stage_floats;
        const float* sv = base + ts * 5 * Dp;
        const int cnt = n - tok0 < ts ? n - tok0 : ts;
        for (int tk = 0; tk < cnt; ++tk) {
            const float4* pq = reinterpret_cast<const float4*>(base + (tk * 5 + 0) * Dp) + r;
            const float4* pz = reinterpret_cast<const float4*>(base + (tk * 5 + 1) * Dp) + r;
            const float4* pd = reinterpret_cast<const float4*>(base + (tk * 5 + 2) * Dp) + r;
            const float4* p1 = reinterpret_cast<const float4*>(base + (tk * 5 + 3) * Dp) + r;
            const float4* p2 = reinterpret_cast<const float4*>(base + (tk * 5 + 4) * Dp) + r;
            // z . S of every column: every vector word loaded once for CPT columns, CPT independent chains (two each when
            // the thread has one column only)
            float zs[CPT], zt[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) zs[c] = zt[c] = 0.f;
            if (CORR) {
#pragma unroll
                for (int i = 0; i < DPT / 4; ++i) {
                    const float4 z = pz[R * i];
#pragma unroll
                    for (int c = 0; c < CPT; ++c) {
                        zs[c] = fmaf(z.x, S[c][4 * i], zs[c]);
                        zt[c] = fmaf(z.y, S[c][4 * i + 1], zt[c]);
                        zs[c] = fmaf(z.z, S[c][4 * i + 2], zs[c]);
                        zt[c] = fmaf(z.w, S[c][4 * i + 3], zt[c]);
                    }
                }
#pragma unroll
                for (int c = 0; c < CPT; ++c) zs[c] += zt[c];
#pragma unroll
                for (int m = 1; m < R; m <<= 1) {
#pragma unroll
                    for (int c = 0; c < CPT; ++c) zs[c] += __shfl_xor_sync(0xffffffffu, zs[c], m);
                }
            }
            float vv[CPT], os[CPT], ot[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                vv[c] = sv[tk * cols + cg * CPT + c];
                os[c] = ot[c] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < DPT / 4; ++i) {
                const float4 dd = pd[R * i], w2 = p2[R * i], qq = pq[R * i];
                const float4 a = CORR ? p1[R * i] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    if (CORR) {
                        S[c][4 * i] = fmaf(w2.x, vv[c], fmaf(a.x, zs[c], dd.x * S[c][4 * i]));
                        S[c][4 * i + 1] = fmaf(w2.y, vv[c], fmaf(a.y, zs[c], dd.y * S[c][4 * i + 1]));
                        S[c][4 * i + 2] = fmaf(w2.z, vv[c], fmaf(a.z, zs[c], dd.z * S[c][4 * i + 2]));
                        S[c][4 * i + 3] = fmaf(w2.w, vv[c], fmaf(a.w, zs[c], dd.w * S[c][4 * i + 3]));
                    } else {
                        S[c][4 * i] = fmaf(w2.x, vv[c], dd.x * S[c][4 * i]);
                        S[c][4 * i + 1] = fmaf(w2.y, vv[c], dd.y * S[c][4 * i + 1]);
                        S[c][4 * i + 2] = fmaf(w2.z, vv[c], dd.z * S[c][4 * i + 2]);
                        S[c][4 * i + 3] = fmaf(w2.w, vv[c], dd.w * S[c][4 * i + 3]);
                    }
                    os[c] = fmaf(qq.x, S[c][4 * i], os[c]);
                    ot[c] = fmaf(qq.y, S[c][4 * i + 1], ot[c]);
                    os[c] = fmaf(qq.z, S[c][4 * i + 2], os[c]);
                    ot[c] = fmaf(qq.w, S[c][4 * i + 3], ot[c]);
                }
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) os[c] += ot[c];
#pragma unroll
            for (int m = 1; m < R; m <<= 1) {
#pragma unroll
                for (int c = 0; c < CPT; ++c) os[c] += __shfl_xor_sync(0xffffffffu, os[c], m);
            }
            if (r == 0) {
                float* orow = o + (long long)(row0 + tok0 + tk) * H * E + (long long)h * E + ec;
#pragma unroll
                for (int c = 0; c < CPT; ++c)
                    if (ec + c < E) orow[c] = os[c];
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = 4 * (r + R * (i >> 2)) + (i & 3);
#pragma unroll
        for (int c = 0; c < CPT; ++c)
            if (ec + c < E && d < D) sp[(long long)d * E + ec + c] = S[c][i];
    }
}

// ------------------------------------------------------------------------------------------------ read-out norm + gate
// Warp per (token, head): y = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate)   (gate_silu: * gate * sigmoid(gate))
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ x, const float* __restrict__ w, int w_per_head,
                                      const float* __restrict__ gate, long long gate_ld, T* __restrict__ out,
                                      long long n_items, int H, int E, float eps, int gate_silu) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= n_items) return;
    const long long t = item / H;
    const int h = (int)(item % H);
    const float* xr = x + item * E;
    float ss = 0.f;
    for (int e = lane; e < E; e += 32) ss = fmaf(xr[e], xr[e], ss);
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)E + eps);
    const float* wr = w + (w_per_head ? (long long)h * E : 0);
    for (int e = lane; e < E; e += 32) {
        float y = xr[e] * r * wr[e];
        if (gate) {
            const float gv = gate[t * gate_ld + (long long)h * E + e];
            y *= gate_silu ? gv * sigmoidf_(gv) : sigmoidf_(gv);
        }
        stf(out + item * E + e, y);
    }
}

// ------------------------------------------------------------------------------------------------ skip, gate, grouped norm
// Read-out of a state-space mixer: y = (o + skip_h * xin) * silu(gate) over the H * E inner channels of a token, then an RMS
// norm of each of `groups` equal consecutive parts by its own root mean square, times w [H * E]. Block per (token, part).
template <typename T>
__global__ void skip_gate_group_norm_kernel(const float* __restrict__ o, const float* __restrict__ xin, long long x_ld,
                                            const float* __restrict__ skip, const float* __restrict__ gate,
                                            long long gate_ld, const float* __restrict__ w, T* __restrict__ out, int H,
                                            int E, int groups, float eps) {
    __shared__ float red[32];
    const long long t = blockIdx.x;
    const int inner = H * E, per = inner / groups, c0 = blockIdx.y * per;
    float ss = 0.f;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const int c = c0 + i;
        const float gv = gate[t * gate_ld + c];
        const float y = (o[t * inner + c] + skip[c / E] * xin[t * x_ld + c]) * (gv * sigmoidf_(gv));
        ss = fmaf(y, y, ss);
    }
    ss = warp_sum(ss);
    const int wi = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (l == 0) red[wi] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < nw; ++i) tot += red[i];
    const float r = 1.0f / sqrtf(tot / (float)per + eps);
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const int c = c0 + i;
        const float gv = gate[t * gate_ld + c];
        const float y = (o[t * inner + c] + skip[c / E] * xin[t * x_ld + c]) * (gv * sigmoidf_(gv));
        stf(out + t * inner + c, y * r * w[c]);
    }
}

// The same with the part's values kept in shared memory between the two passes (one read of every input) and 16-byte
// accesses: per, E, x_ld and gate_ld multiples of 4, every pointer 16-byte aligned.
template <typename T>
__global__ void skip_gate_group_norm4_kernel(const float* __restrict__ o, const float* __restrict__ xin, long long x_ld,
                                             const float* __restrict__ skip, const float* __restrict__ gate,
                                             long long gate_ld, const float* __restrict__ w, T* __restrict__ out, int H,
                                             int E, int groups, float eps) {
    extern __shared__ float4 sy4[];
    __shared__ float red[32];
    const long long t = blockIdx.x;
    const int inner = H * E, per = inner / groups, c0 = blockIdx.y * per, per4 = per >> 2;
    const float4* o4 = reinterpret_cast<const float4*>(o + t * inner + c0);
    const float4* x4 = reinterpret_cast<const float4*>(xin + t * x_ld + c0);
    const float4* g4 = reinterpret_cast<const float4*>(gate + t * gate_ld + c0);
    float ss = 0.f;
    for (int i = threadIdx.x; i < per4; i += blockDim.x) {
        const float4 ov = o4[i], xv = x4[i], gv = g4[i];
        const float sk = skip[(c0 + 4 * i) / E];
        float4 y;
        y.x = fmaf(sk, xv.x, ov.x) * (gv.x * sigmoidf_(gv.x));
        y.y = fmaf(sk, xv.y, ov.y) * (gv.y * sigmoidf_(gv.y));
        y.z = fmaf(sk, xv.z, ov.z) * (gv.z * sigmoidf_(gv.z));
        y.w = fmaf(sk, xv.w, ov.w) * (gv.w * sigmoidf_(gv.w));
        sy4[i] = y;
        ss = fmaf(y.x, y.x, fmaf(y.y, y.y, fmaf(y.z, y.z, fmaf(y.w, y.w, ss))));
    }
    ss = warp_sum(ss);
    const int wi = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (l == 0) red[wi] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < nw; ++i) tot += red[i];
    const float r = 1.0f / sqrtf(tot / (float)per + eps);
    const float4* w4 = reinterpret_cast<const float4*>(w + c0);
    for (int i = threadIdx.x; i < per4; i += blockDim.x) {
        const float4 y = sy4[i], ww = w4[i];
        T* dst = out + t * inner + c0 + 4 * i;
        if constexpr (sizeof(T) == 4) {
            *reinterpret_cast<float4*>(dst) = make_float4(y.x * r * ww.x, y.y * r * ww.y, y.z * r * ww.z, y.w * r * ww.w);
        } else {
            uint2 u;
            u.x = pack_bf16x2(y.x * r * ww.x, y.y * r * ww.y);
            u.y = pack_bf16x2(y.z * r * ww.z, y.w * r * ww.w);
            *reinterpret_cast<uint2*>(dst) = u;
        }
    }
}

}  // namespace delta
}  // namespace llark

using namespace llark;
using namespace llark::delta;

extern "C" int llark_seq_conv_act(const float* src, long long ld, const float* w, float* carry, const int* tok_seq,
                                  const int* cu, const int* slot, float* out, int n_tok, int n_seq, int n_ch, int taps,
                                  int silu, const float* bias, cudaStream_t st) {
    if (n_tok <= 0 || n_seq <= 0 || n_ch <= 0 || taps < 1 || !src || !w || !out || ld < n_ch || (taps > 1 && !carry) ||
        !tok_seq || !cu || !slot)
        return LLARK_EINVAL;
    int th = 32;
    while (th < n_ch && th < 256) th <<= 1;
    const int inline_carry = n_tok == n_seq;  // every request brings one token
    if (!inline_carry && n_tok >= 64 && taps >= 2 && taps <= 4) {
        constexpr int TB = 16;
        dim3 grid((n_tok + TB - 1) / TB, (n_ch + 127) / 128);
        if (taps == 2)
            conv_act_rows_kernel<2, TB><<<grid, 128, 0, st>>>(src, ld, w, carry, tok_seq, cu, slot, out, n_tok, n_ch, silu,
                                                              bias);
        else if (taps == 3)
            conv_act_rows_kernel<3, TB><<<grid, 128, 0, st>>>(src, ld, w, carry, tok_seq, cu, slot, out, n_tok, n_ch, silu,
                                                              bias);
        else
            conv_act_rows_kernel<4, TB><<<grid, 128, 0, st>>>(src, ld, w, carry, tok_seq, cu, slot, out, n_tok, n_ch, silu,
                                                              bias);
    } else {
        // few rows (decode): the channels are spread over blocks too, so that a handful of tokens still fills the GPU
        int gy = (n_ch + th - 1) / th;
        if ((long long)gy * n_tok > 4 * 148) gy = (4 * 148 + n_tok - 1) / n_tok;
        conv_act_kernel<<<dim3(n_tok, gy), th, 0, st>>>(src, ld, w, carry, tok_seq, cu, slot, out, n_ch, taps, silu,
                                                        inline_carry, bias);
    }
    int rc = check_launch();
    if (rc != LLARK_OK || inline_carry || taps == 1) return rc;
    conv_carry_kernel<<<n_seq, th, 0, st>>>(src, ld, carry, cu, slot, n_ch, taps);
    return check_launch();
}

extern "C" int llark_seq_delta_prep(int rule, const float* q, long long q_ld, const float* k, long long k_ld,
                                    const float* dec, long long dec_ld, const float* dec_bias, const float* rate_log,
                                    const float* mix, long long mix_ld, float* vec, int n_tok, int H, int G, int D,
                                    float unit_eps, cudaStream_t st) {
    if (n_tok <= 0 || H <= 0 || G <= 0 || (H % G) || D <= 0 || !q || !k || !dec || (!mix && rule != 3) || !vec)
        return LLARK_EINVAL;
    if (rule < 0 || rule > 3) return LLARK_EINVAL;
    if (rule == 1 ? G != H : (!dec_bias || !rate_log)) return LLARK_EINVAL;
    const long long items = (long long)n_tok * H;
    delta_prep_kernel<<<(unsigned)((items + 3) / 4), 128, 0, st>>>(rule, q, q_ld, k, k_ld, dec, dec_ld, dec_bias, rate_log,
                                                                   mix, mix_ld, vec, n_tok, H, G, D, unit_eps);
    return check_launch();
}

extern "C" int llark_seq_delta_scan(const float* vec, const float* v, long long v_ld, float* state, float* o,
                                    const int* cu, const int* slot, int n_seq, int n_tok, int H, int D, int E,
                                    int correct, cudaStream_t st) {
    if (n_seq <= 0 || n_tok < n_seq || H <= 0 || D <= 0 || E <= 0 || !vec || !v || !state || !o || !cu || !slot)
        return LLARK_EINVAL;
    // 16 rows of a column per thread (short dependent chains) while a column then still fits one warp, 32 rows for the
    // widest heads. Steps with many tokens per request give a thread two adjacent columns: a vector word read from
    // shared memory then serves both (the shared-memory pipe is what bounds the one-column form on prompts);
    // single-token steps keep one column per thread, which reads and writes the state in whole rows.
    const int dpt = D <= 16 * 32 ? 16 : 32;
    if (D > 32 * 32) return LLARK_EINVAL;
    int cpt = (dpt == 16 && n_tok >= 16 * n_seq && E >= 4) ? 2 : 1;
    {
        static int forced = -1;  // LLARK_DELTA_CPT = 1 | 2 | 4: columns per thread on long steps (measurement aid)
        if (forced < 0) {
            const char* e = getenv("LLARK_DELTA_CPT");
            forced = e ? atoi(e) : 0;
        }
        if (cpt == 2 && (forced == 1 || forced == 4)) cpt = forced;
    }
    int R = 1;
    while (R * dpt < D) R <<= 1;
    // columns per block: enough blocks to fill the GPU at small batches, at least two warps, at most 256 threads
    const int floor_cols = cpt * (64 / R > 1 ? 64 / R : 1) > 8 ? cpt * (64 / R > 1 ? 64 / R : 1) : 8;
    int cols = cpt * (256 / R > 1 ? 256 / R : 1);
    if (cols < floor_cols) cols = floor_cols;
    while (cols > floor_cols && (long long)((E + cols - 1) / cols) * H * n_seq < 2 * 148) cols >>= 1;
    while (cols > floor_cols && cols / 2 >= E) cols >>= 1;
    const int threads = cols / cpt * R;
    if (threads % 32 || threads > 256) return LLARK_EINVAL;
    const int ts = D <= 128 ? 8 : (D <= 256 ? 4 : (D <= 512 ? 2 : 1));  // two stages stay under 48 KB
    const size_t smem = sizeof(float) * 2 * (size_t)ts * (5 * dpt * R + cols);
    dim3 grid((E + cols - 1) / cols, H, n_seq);
#define LLARK_DSCAN(DPT_, CPT_, R_)                                                                                   \
    if (correct)                                                                                                      \
        delta_scan_kernel<DPT_, CPT_, R_, true><<<grid, threads, smem, st>>>(vec, v, v_ld, state, o, cu, slot, H, D, E, \
                                                                             cols, ts);                               \
    else                                                                                                              \
        delta_scan_kernel<DPT_, CPT_, R_, false><<<grid, threads, smem, st>>>(vec, v, v_ld, state, o, cu, slot, H, D,   \
                                                                              E, cols, ts)
#define LLARK_DSCAN_R(DPT_, CPT_)                                                                                     \
    switch (R) {                                                                                                      \
        case 1: LLARK_DSCAN(DPT_, CPT_, 1); break;                                                                    \
        case 2: LLARK_DSCAN(DPT_, CPT_, 2); break;                                                                    \
        case 4: LLARK_DSCAN(DPT_, CPT_, 4); break;                                                                    \
        case 8: LLARK_DSCAN(DPT_, CPT_, 8); break;                                                                    \
        case 16: LLARK_DSCAN(DPT_, CPT_, 16); break;                                                                  \
        default: LLARK_DSCAN(DPT_, CPT_, 32); break;                                                                  \
    }
    if (dpt == 32) {
        LLARK_DSCAN(32, 1, 32);  // 512 < D <= 1024
    } else if (cpt == 4) {
        LLARK_DSCAN_R(16, 4)
    } else if (cpt == 2) {
        LLARK_DSCAN_R(16, 2)
    } else {
        LLARK_DSCAN_R(16, 1)
    }
#undef LLARK_DSCAN_R
#undef LLARK_DSCAN
    return check_launch();
}

extern "C" int llark_seq_head_norm_gate(const float* x, const float* w, int w_per_head, const float* gate,
                                        long long gate_ld, void* out, long long n_tok, int H, int E, float eps,
                                        int gate_silu, int act_fp32, cudaStream_t st) {
    if (n_tok <= 0 || H <= 0 || E <= 0 || !x || !w || !out) return LLARK_EINVAL;
    const long long items = n_tok * H;
    const unsigned grid = (unsigned)((items + 3) / 4);
    if (act_fp32)
        head_norm_gate_kernel<float><<<grid, 128, 0, st>>>(x, w, w_per_head, gate, gate_ld, (float*)out, items, H, E, eps,
                                                           gate_silu);
    else
        head_norm_gate_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(x, w, w_per_head, gate, gate_ld, (__nv_bfloat16*)out,
                                                                   items, H, E, eps, gate_silu);
    return check_launch();
}

extern "C" int llark_seq_skip_gate_group_norm(const float* o, const float* xin, long long x_ld, const float* skip,
                                              const float* gate, long long gate_ld, const float* w, void* out,
                                              long long n_tok, int H, int E, int groups, float eps, int act_fp32,
                                              cudaStream_t st) {
    if (n_tok <= 0 || H <= 0 || E <= 0 || groups <= 0 || ((H * E) % groups) || !o || !xin || !skip || !gate || !w || !out)
        return LLARK_EINVAL;
    const int per = H * E / groups;
    int th = 32;
    while (th < per && th < 256) th <<= 1;
    dim3 grid((unsigned)n_tok, groups);
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (per % 4 == 0 && E % 4 == 0 && x_ld % 4 == 0 && gate_ld % 4 == 0 && al(o) && al(xin) && al(gate) && al(w) && al(out) &&
        (size_t)per * sizeof(float) <= 48 * 1024) {
        int t4 = 32;
        while (t4 * 8 < per && t4 < 256) t4 <<= 1;
        const size_t smem = sizeof(float) * (size_t)per;
        if (act_fp32)
            skip_gate_group_norm4_kernel<float><<<grid, t4, smem, st>>>(o, xin, x_ld, skip, gate, gate_ld, w, (float*)out, H,
                                                                        E, groups, eps);
        else
            skip_gate_group_norm4_kernel<__nv_bfloat16><<<grid, t4, smem, st>>>(o, xin, x_ld, skip, gate, gate_ld, w,
                                                                                (__nv_bfloat16*)out, H, E, groups, eps);
        return check_launch();
    }
    if (act_fp32)
        skip_gate_group_norm_kernel<float><<<grid, th, 0, st>>>(o, xin, x_ld, skip, gate, gate_ld, w, (float*)out, H, E,
                                                                groups, eps);
    else
        skip_gate_group_norm_kernel<__nv_bfloat16><<<grid, th, 0, st>>>(o, xin, x_ld, skip, gate, gate_ld, w,
                                                                        (__nv_bfloat16*)out, H, E, groups, eps);
    return check_launch();
}
