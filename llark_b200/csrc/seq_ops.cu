// Token-major ops of the generation path for layer-list decoders (Kelutar and whatever else is assembled from the
// same parts). One step of the engine is a PACKED batch: the new tokens of all requests concatenated, [Ttot, width],
// no padding; `tok_seq[t]` names the request of token t, `cu[b]` its first row, `pos0[b]` the position of that row in
// its sequence and `slot[b]` the request's row in every state store. A request that starts, goes on by a portion of
// its prompt, or decodes one token is the same launch with other numbers.
//
// Precision: the residual stream, every norm and the convolution state are fp32. `ACT` is the activation / matrix
// dtype: bf16 when serving, float in the all-fp32 mode (act_fp32 = 1), where the linears run on the SIMT kernels below
// in true fp32 (no TF32).
//
//   llark_seq_embed         x = table[id] * scale + pos_table[position]
//   llark_seq_short_conv    y = h + causal depthwise conv(h) with carry-in of the last taps-1 inputs per request
//   llark_seq_conv_tail     refresh of that carry after a step of more than one token per request
//   llark_seq_add_rmsnorm   x_out = x + rmsnorm(y) * w   (norm on the sublayer's output), optional ACT copy of x_out
//   llark_seq_gated_norm_add  x_out = x + rmsnorm(y * sigmoid(gate)) * w, optional ACT copy of rmsnorm(x_out) * w_next
//   llark_seq_rmsnorm_rows  y[i] = rmsnorm(x[rows[i]]) * w -> ACT (final norm of the rows whose logits are wanted)
//   llark_seq_relu2         y = relu(u)^2
//   llark_linear_rows       C = A W^T (+ bias) for a handful of rows: weight-streaming, one or two output columns per warp
//   llark_linear_simt       C = A W^T (+ bias), any shape, tiled SIMT with fp32 accumulation (the fp32 mode's GEMM and the
//                           fallback for shapes the TMA descriptors of the tcgen05 core cannot take)
#include "common.cuh"

namespace llark {
extern thread_local int g_last_cuda_error;
namespace seq {

static int check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        return LLARK_ECUDA;
    }
    return LLARK_OK;
}

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (l == 0) red[w] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nw; ++i) s += red[i];
    return s;
}

// ------------------------------------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ tok_seq, const int* __restrict__ cu,
                             const int* __restrict__ pos0, const T* __restrict__ table, const T* __restrict__ pos_table,
                             float scale, float* __restrict__ x, int C) {
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    const long long p = pos0[b] + (t - cu[b]);
    const T* e = table + (long long)ids[t] * C;
    const T* pe = pos_table ? pos_table + p * C : nullptr;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float v = ldf(e + c) * scale;
        if (pe) v += ldf(pe + c);
        x[(long long)t * C + c] = v;
    }
}

// ------------------------------------------------------------------------------------------------ short convolution
// y[t, c] = h[t, c] + sum_j w[c, j] * h[t - taps + 1 + j, c]; inputs before this step's first row come from
// tail[slot][k][c], k = 0 .. taps-2 oldest first (zeros for a fresh request). inline_tail: every request brings exactly
// one token and the thread that read the carry also shifts it.
template <typename T>
__global__ void short_conv_kernel(const float* __restrict__ h, const float* __restrict__ w, float* __restrict__ tail,
                                  const int* __restrict__ tok_seq, const int* __restrict__ cu,
                                  const int* __restrict__ slot, T* __restrict__ y, int C, int taps, int inline_tail) {
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    const int local = t - cu[b];
    float* tl = tail + (long long)slot[b] * (taps - 1) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float cur = h[(long long)t * C + c];
        float acc = w[c * taps + taps - 1] * cur;
        for (int j = 0; j < taps - 1; ++j) {
            const int s = local - taps + 1 + j;
            const float v = s >= 0 ? h[(long long)(t - local + s) * C + c] : tl[(long long)(taps - 1 + s) * C + c];
            acc = fmaf(w[c * taps + j], v, acc);
        }
        stf(y + (long long)t * C + c, cur + acc);
        if (inline_tail) {
            for (int k = 0; k + 1 < taps - 1; ++k) tl[(long long)k * C + c] = tl[(long long)(k + 1) * C + c];
            if (taps > 1) tl[(long long)(taps - 2) * C + c] = cur;
        }
    }
}

// The same with four channels per thread (C % 4 == 0): 16-byte loads of h and of the four channels' taps.
template <typename T>
__global__ void short_conv4_kernel(const float* __restrict__ h, const float* __restrict__ w, float* __restrict__ tail,
                                   const int* __restrict__ tok_seq, const int* __restrict__ cu,
                                   const int* __restrict__ slot, T* __restrict__ y, int C, int taps, int inline_tail) {
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    const int local = t - cu[b];
    float* tl = tail + (long long)slot[b] * (taps - 1) * C;
    for (int c = threadIdx.x * 4; c < C; c += blockDim.x * 4) {
        const float4 cur = *reinterpret_cast<const float4*>(h + (long long)t * C + c);
        const float* wc = w + (long long)c * taps;  // taps of channel c, then of c + 1, ...
        float4 acc = make_float4(wc[taps - 1] * cur.x, wc[2 * taps - 1] * cur.y, wc[3 * taps - 1] * cur.z,
                                 wc[4 * taps - 1] * cur.w);
        for (int j = 0; j < taps - 1; ++j) {
            const int s = local - taps + 1 + j;
            const float4 v = *reinterpret_cast<const float4*>(
                s >= 0 ? h + (long long)(t - local + s) * C + c : tl + (long long)(taps - 1 + s) * C + c);
            acc.x = fmaf(wc[j], v.x, acc.x);
            acc.y = fmaf(wc[taps + j], v.y, acc.y);
            acc.z = fmaf(wc[2 * taps + j], v.z, acc.z);
            acc.w = fmaf(wc[3 * taps + j], v.w, acc.w);
        }
        T* yo = y + (long long)t * C + c;
        stf(yo, cur.x + acc.x);
        stf(yo + 1, cur.y + acc.y);
        stf(yo + 2, cur.z + acc.z);
        stf(yo + 3, cur.w + acc.w);
        if (inline_tail) {
            for (int k = 0; k + 1 < taps - 1; ++k)
                *reinterpret_cast<float4*>(tl + (long long)k * C + c) =
                    *reinterpret_cast<const float4*>(tl + (long long)(k + 1) * C + c);
            if (taps > 1) *reinterpret_cast<float4*>(tl + (long long)(taps - 2) * C + c) = cur;
        }
    }
}

// Prompts: a CTA walks TB consecutive rows with the last TAPS-1 inputs of each 4-channel group in registers, so a row of
// h and the taps are read once per CTA instead of once per output row (the per-row kernels above are bound by the number
// of L1 requests, not by bytes). The window is rebuilt from h / the tail wherever a request starts inside the group.
template <typename T> __device__ __forceinline__ void st4(T* p, float4 v);
template <> __device__ __forceinline__ void st4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void st4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
}

template <typename T, int TAPS, int TB>
__global__ void short_conv4t_kernel(const float* __restrict__ h, const float* __restrict__ w,
                                    const float* __restrict__ tail, const int* __restrict__ tok_seq,
                                    const int* __restrict__ cu, const int* __restrict__ slot, T* __restrict__ y, int C,
                                    int n_tok) {
    const int t0 = blockIdx.x * TB;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= C) return;
    float wr[4][TAPS];
#pragma unroll
    for (int ch = 0; ch < 4; ++ch)
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wr[ch][j] = w[(long long)(c + ch) * TAPS + j];
    float4 win[TAPS > 1 ? TAPS - 1 : 1];
    for (int i = 0; i < TB && t0 + i < n_tok; ++i) {
        const int t = t0 + i;
        const int b = tok_seq[t];
        const int local = t - cu[b];
        if (i == 0 || local < TAPS - 1) {
            const float* tl = tail + (long long)slot[b] * (TAPS - 1) * C;
#pragma unroll
            for (int j = 0; j < TAPS - 1; ++j) {
                const int s = local - (TAPS - 1) + j;
                win[j] = *reinterpret_cast<const float4*>(s >= 0 ? h + (long long)(t - local + s) * C + c
                                                                 : tl + (long long)(TAPS - 1 + s) * C + c);
            }
        }
        const float4 cur = *reinterpret_cast<const float4*>(h + (long long)t * C + c);
        float4 acc = make_float4(wr[0][TAPS - 1] * cur.x, wr[1][TAPS - 1] * cur.y, wr[2][TAPS - 1] * cur.z,
                                 wr[3][TAPS - 1] * cur.w);
#pragma unroll
        for (int j = 0; j < TAPS - 1; ++j) {
            acc.x = fmaf(wr[0][j], win[j].x, acc.x);
            acc.y = fmaf(wr[1][j], win[j].y, acc.y);
            acc.z = fmaf(wr[2][j], win[j].z, acc.z);
            acc.w = fmaf(wr[3][j], win[j].w, acc.w);
        }
        st4(y + (long long)t * C + c, make_float4(cur.x + acc.x, cur.y + acc.y, cur.z + acc.z, cur.w + acc.w));
#pragma unroll
        for (int j = 0; j + 1 < TAPS - 1; ++j) win[j] = win[j + 1];
        if (TAPS > 1) win[TAPS - 2] = cur;
    }
}

template <typename T, int TAPS>
static void launch_conv4t(const float* h, const float* w, const float* tail, const int* tok_seq, const int* cu,
                          const int* slot, void* y, int n_tok, int C, cudaStream_t st) {
    constexpr int TB = 16;
    const int th = C / 4 < 128 ? ((C / 4 + 31) / 32) * 32 : 128;
    dim3 grid((n_tok + TB - 1) / TB, (C / 4 + th - 1) / th);
    short_conv4t_kernel<T, TAPS, TB><<<grid, th, 0, st>>>(h, w, tail, tok_seq, cu, slot, (T*)y, C, n_tok);
}

// new tail[k] = input at local index n - (taps-1) + k (from this step's rows, or from the old tail when negative)
__global__ void conv_tail_kernel(const float* __restrict__ h, float* __restrict__ tail, const int* __restrict__ cu,
                                 const int* __restrict__ slot, int C, int taps) {
    const int b = blockIdx.x;
    const int r0 = cu[b], n = cu[b + 1] - r0;
    float* tl = tail + (long long)slot[b] * (taps - 1) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x)
        for (int k = 0; k < taps - 1; ++k) {  // ascending k: an old entry is read at index k + n >= k before it is rewritten
            const int s = n - (taps - 1) + k;
            tl[(long long)k * C + c] = s >= 0 ? h[(long long)(r0 + s) * C + c] : tl[(long long)(taps - 1 + s) * C + c];
        }
}

// ------------------------------------------------------------------------------------------------ norms
// C % 4 == 0: 16-byte loads, the row of y stays in registers between the two passes (up to 4 vectors per thread).
template <typename T>
__global__ void add_rmsnorm4_kernel(const float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w,
                                    float* __restrict__ x_out, T* __restrict__ x_act, int C, float eps) {
    __shared__ float red[32];
    const long long row = blockIdx.x;
    const float4* yr = reinterpret_cast<const float4*>(y + row * C);
    const int nv = C >> 2;
    float4 keep[4];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nv) {
            keep[i] = yr[v];
            ss += keep[i].x * keep[i].x + keep[i].y * keep[i].y + keep[i].z * keep[i].z + keep[i].w * keep[i].w;
        }
    }
    for (int v = threadIdx.x + 4 * blockDim.x; v < nv; v += blockDim.x) {
        const float4 a = yr[v];
        ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)C + eps);
    const float4* xr = reinterpret_cast<const float4*>(x + row * C);
    const float4* wr = reinterpret_cast<const float4*>(w);
    float4* outr = reinterpret_cast<float4*>(x_out + row * C);
    auto emit = [&](int v, const float4& a) {
        const float4 xv = xr[v], wv = wr[v];
        float4 o;
        o.x = xv.x + a.x * r * wv.x;
        o.y = xv.y + a.y * r * wv.y;
        o.z = xv.z + a.z * r * wv.z;
        o.w = xv.w + a.w * r * wv.w;
        outr[v] = o;
        if (x_act) {
            T* xa = x_act + row * C + 4 * v;
            stf(xa, o.x);
            stf(xa + 1, o.y);
            stf(xa + 2, o.z);
            stf(xa + 3, o.w);
        }
    };
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nv) emit(v, keep[i]);
    }
    for (int v = threadIdx.x + 4 * blockDim.x; v < nv; v += blockDim.x) emit(v, yr[v]);
}

template <typename T>
__global__ void add_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w,
                                   float* __restrict__ x_out, T* __restrict__ x_act, int C, float eps) {
    __shared__ float red[32];
    const long long row = blockIdx.x;
    const float* yr = y + row * C;
    float ss = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) ss = fmaf(yr[c], yr[c], ss);
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)C + eps);
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float v = x[row * C + c] + yr[c] * r * w[c];
        x_out[row * C + c] = v;
        if (x_act) stf(x_act + row * C + c, v);
    }
}

// x_out = x + rmsnorm(y * sigmoid(gate)) * w, and optionally the NEXT sublayer's input norm in the same pass:
// x_act = rmsnorm(x_out) * w_next -> T. gate (optional) is a column slice [rows, gate_ld] of a fused projection. The gated
// row stays in shared memory between its reduction and its use, and is replaced there by the new stream for the second
// norm.
__device__ __forceinline__ float sigmoid_(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename T> __device__ __forceinline__ void st4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void st4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void st4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
    uint2 v;
    v.x = pack_bf16x2(a, b);
    v.y = pack_bf16x2(c, d);
    *reinterpret_cast<uint2*>(p) = v;
}

// C % 4 == 0, rows 16-byte aligned, C <= 4 * NV * blockDim.x: the row lives in registers (NV float4 per thread) from the
// first read to the last write; 16-byte loads, 16- / 8-byte stores.
template <typename T, int NV>
__global__ void gated_norm_add4_kernel(const float* __restrict__ x, const float* __restrict__ y,
                                       const float* __restrict__ gate, long long gate_ld, const float* __restrict__ w,
                                       const float* __restrict__ w_next, float* __restrict__ x_out, T* __restrict__ x_act,
                                       int C, float eps) {
    __shared__ float red[32];
    const long long row = blockIdx.x;
    const int nv = C >> 2;
    const float4* yr = reinterpret_cast<const float4*>(y + row * C);
    const float4* gr = gate ? reinterpret_cast<const float4*>(gate + row * gate_ld) : nullptr;
    const float4* xr = reinterpret_cast<const float4*>(x + row * C);
    float4 keep[NV], xv[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nv) {
            float4 a = yr[v];
            xv[i] = xr[v];
            if (gr) {
                const float4 g = gr[v];
                a.x *= sigmoid_(g.x), a.y *= sigmoid_(g.y), a.z *= sigmoid_(g.z), a.w *= sigmoid_(g.w);
            }
            keep[i] = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)C + eps);
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nv) {
            const float4 a = keep[i], wv = reinterpret_cast<const float4*>(w)[v];
            float4 o;
            o.x = xv[i].x + a.x * r * wv.x, o.y = xv[i].y + a.y * r * wv.y;
            o.z = xv[i].z + a.z * r * wv.z, o.w = xv[i].w + a.w * r * wv.w;
            reinterpret_cast<float4*>(x_out + row * C)[v] = o;
            keep[i] = o;
            s2 += o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w;
        }
    }
    if (!x_act) return;
    s2 = block_sum(s2, red);
    const float r2 = 1.0f / sqrtf(s2 / (float)C + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nv) {
            const float4 o = keep[i], wn = reinterpret_cast<const float4*>(w_next)[v];
            st4(x_act + row * C + 4 * v, o.x * r2 * wn.x, o.y * r2 * wn.y, o.z * r2 * wn.z, o.w * r2 * wn.w);
        }
    }
}

// Any C: the gated row stays in shared memory between its reduction and its use, and is replaced there by the new stream
// for the second norm.
template <typename T>
__global__ void gated_norm_add_kernel(const float* __restrict__ x, const float* __restrict__ y,
                                      const float* __restrict__ gate, long long gate_ld, const float* __restrict__ w,
                                      const float* __restrict__ w_next, float* __restrict__ x_out, T* __restrict__ x_act,
                                      int C, float eps) {
    extern __shared__ __align__(16) float rowbuf[];
    __shared__ float red[32];
    const long long row = blockIdx.x;
    const float* yr = y + row * C;
    const float* gr = gate ? gate + row * gate_ld : nullptr;
    const float* xr = x + row * C;
    float* xo = x_out + row * C;
    float ss = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float a = yr[c];
        if (gr) a *= sigmoid_(gr[c]);
        rowbuf[c] = a;
        ss = fmaf(a, a, ss);
    }
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)C + eps);
    float s2 = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float o = xr[c] + rowbuf[c] * r * w[c];
        xo[c] = o;
        rowbuf[c] = o;
        s2 = fmaf(o, o, s2);
    }
    if (!x_act) return;
    s2 = block_sum(s2, red);
    const float r2 = 1.0f / sqrtf(s2 / (float)C + eps);
    T* xa = x_act + row * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) stf(xa + c, rowbuf[c] * r2 * w_next[c]);  // each thread reads its own
}

template <typename T>
__global__ void rmsnorm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                                    T* __restrict__ out, int C, float eps) {
    __shared__ float red[32];
    const long long src = rows ? rows[blockIdx.x] : blockIdx.x;
    const float* xr = x + src * C;
    float ss = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)C + eps);
    for (int c = threadIdx.x; c < C; c += blockDim.x) stf(out + (long long)blockIdx.x * C + c, xr[c] * r * w[c]);
}

template <typename T>
__global__ void relu2_kernel(const T* __restrict__ u, T* __restrict__ y, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = fmaxf(ldf(u + i), 0.f);
        stf(y + i, v * v);
    }
}

template <typename T>
__global__ void tanh_kernel(const float* __restrict__ u, T* __restrict__ y, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        stf(y + i, tanhf(u[i]));
}

// ------------------------------------------------------------------------------------------------ linears
// Few rows (decode): a warp owns NC adjacent output columns, its lanes stride over K in 16-byte pieces (streamed,
// evict-first), the rows of A come from L1 / L2 and are read once per NC weight pieces.
template <typename T, typename TC, int MB, int NC>
__global__ void __launch_bounds__(256)
linear_rows_kernel(const T* __restrict__ A, long long lda, const T* __restrict__ W, long long ldw, TC* __restrict__ Cm,
                   long long ldc, const float* __restrict__ bias, int M, int N, int K, int vec_ok) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long n0 = ((long long)blockIdx.x * (blockDim.x >> 5) + warp) * NC;
    const int m0 = blockIdx.y * MB;
    if (n0 >= N) return;
    float acc[MB][NC];
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[m][c] = 0.f;
    const T* wr[NC];
#pragma unroll
    for (int c = 0; c < NC; ++c) wr[c] = W + (n0 + c < N ? n0 + c : (long long)N - 1) * ldw;  // tail: re-read, never stored
    constexpr int VEC = 16 / (int)sizeof(T);
    int k0 = 0;
    if (vec_ok) {
        const int kv = K / VEC;
        for (int v = lane; v < kv; v += 32) {
            uint4 wv[NC];
#pragma unroll
            for (int c = 0; c < NC; ++c) wv[c] = __ldcs(reinterpret_cast<const uint4*>(wr[c]) + v);
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                if (m0 + m < M) {
                    const uint4 av = __ldg(reinterpret_cast<const uint4*>(A + (long long)(m0 + m) * lda) + v);
                    const T* ap = reinterpret_cast<const T*>(&av);
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        const T* wp = reinterpret_cast<const T*>(&wv[c]);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) acc[m][c] = fmaf(ldf(ap + e), ldf(wp + e), acc[m][c]);
                    }
                }
            }
        }
        k0 = kv * VEC;
    }
    for (int k = k0 + lane; k < K; k += 32) {
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const float wv = ldf(wr[c] + k);
#pragma unroll
            for (int m = 0; m < MB; ++m)
                if (m0 + m < M) acc[m][c] = fmaf(ldf(A + (long long)(m0 + m) * lda + k), wv, acc[m][c]);
        }
    }
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const float s = warp_sum(acc[m][c]);
            if (lane == 0 && m0 + m < M && n0 + c < N)
                stf(Cm + (long long)(m0 + m) * ldc + n0 + c, s + (bias ? bias[n0 + c] : 0.f));
        }
}

// Any shape: 64 x 64 tile, 16-deep k slices through shared memory, 4 x 4 outputs per thread, fp32 FMA.
template <typename T, typename TC, typename TW = T>
__global__ void __launch_bounds__(256)
linear_simt_kernel(const T* __restrict__ A, long long lda, const TW* __restrict__ W, long long ldw, TC* __restrict__ Cm,
                   long long ldc, const float* __restrict__ bias, int M, int N, int K) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            const int r = i / BK, k = i % BK;
            As[k][r] = (m0 + r < M && k0 + k < K) ? ldf(A + (long long)(m0 + r) * lda + k0 + k) : 0.f;
            Ws[k][r] = (n0 + r < N && k0 + k < K) ? ldf(W + (long long)(n0 + r) * ldw + k0 + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) stf(Cm + (long long)m * ldc + n, acc[i][j] + (bias ? bias[n] : 0.f));
        }
}

// ------------------------------------------------------------------------------------------------ grouped RMS norm
// Row r of the output is the norm of x[rows ? rows[r] : r] (+ add_vec): the row is cut into `groups` equal consecutive
// parts, each divided by its own sqrt(mean(part^2) + eps), the whole times w. With x_out the sum x + add_vec is also
// written (a vector added to the residual stream right before a norm).
template <typename T>
__global__ void group_rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                     const float* __restrict__ add_vec, float* __restrict__ x_out,
                                     const float* __restrict__ w, T* __restrict__ out, int C, int groups, float eps) {
    __shared__ float red[32];
    const long long src = rows ? rows[blockIdx.x] : blockIdx.x;
    const float* xr = x + src * C;
    const int per = C / groups;
    for (int g = 0; g < groups; ++g) {
        const int c0 = g * per;
        float ss = 0.f;
        for (int c = threadIdx.x; c < per; c += blockDim.x) {
            const float v = xr[c0 + c] + (add_vec ? add_vec[c0 + c] : 0.f);
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, red);
        const float r = 1.0f / sqrtf(ss / (float)per + eps);
        for (int c = threadIdx.x; c < per; c += blockDim.x) {
            const float v = xr[c0 + c] + (add_vec ? add_vec[c0 + c] : 0.f);
            if (x_out) x_out[src * C + c0 + c] = v;
            stf(out + (long long)blockIdx.x * C + c0 + c, v * r * w[c0 + c]);
        }
    }
}

// The same with a warp per (row, part) when a part is a whole number of 16-byte pieces: the part stays in registers
// between the sum of squares and the scaling (up to 1024 elements; longer parts are read twice), no block barrier.
template <typename T>
__global__ void group_rmsnorm_warp_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                          const float* __restrict__ add_vec, float* __restrict__ x_out,
                                          const float* __restrict__ w, T* __restrict__ out, int n_rows, int C, int groups,
                                          float eps) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)n_rows * groups) return;
    const long long r = item / groups;
    const int g = (int)(item % groups);
    const long long src = rows ? rows[r] : r;
    const int per = C / groups, nv = per >> 2;
    const float4* xr = reinterpret_cast<const float4*>(x + src * C + (long long)g * per);
    const float4* av = add_vec ? reinterpret_cast<const float4*>(add_vec + (long long)g * per) : nullptr;
    float4 keep[8];
    float ss = 0.f;
    auto load = [&](int v) {
        float4 a = xr[v];
        if (av) {
            const float4 b = av[v];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        return a;
    };
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int v = lane + 32 * i;
        if (v < nv) {
            keep[i] = load(v);
            ss += keep[i].x * keep[i].x + keep[i].y * keep[i].y + keep[i].z * keep[i].z + keep[i].w * keep[i].w;
        }
    }
    for (int v = lane + 256; v < nv; v += 32) {
        const float4 a = load(v);
        ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
    ss = warp_sum(ss);
    const float rn = 1.0f / sqrtf(ss / (float)per + eps);
    const float4* wr = reinterpret_cast<const float4*>(w + (long long)g * per);
    float4* xo = x_out ? reinterpret_cast<float4*>(x_out + src * C + (long long)g * per) : nullptr;
    T* orow = out + r * C + (long long)g * per;
    auto emit = [&](int v, const float4& a) {
        if (xo) xo[v] = a;
        const float4 wv = wr[v];
        st4(orow + 4 * v, make_float4(a.x * rn * wv.x, a.y * rn * wv.y, a.z * rn * wv.z, a.w * rn * wv.w));
    };
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int v = lane + 32 * i;
        if (v < nv) emit(v, keep[i]);
    }
    for (int v = lane + 256; v < nv; v += 32) emit(v, load(v));
}

// x_out = x + (y + sum_k wts[t, k] * z[pos_of[t * top + k]]): the residual sum of a layer whose sublayers run side by
// side, the second one a mixture whose chosen experts' outputs sit in rows pos_of[...] of z (top = 0: no second one).
__global__ void residual_combine_kernel(const float* __restrict__ x, const float* __restrict__ y,
                                        const float* __restrict__ z, const int* __restrict__ pos_of,
                                        const float* __restrict__ wts, int top, float* __restrict__ x_out, int C) {
    const long long t = blockIdx.x;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float m = 0.f;
        for (int k = 0; k < top; ++k)
            m = fmaf(wts[t * top + k], z[(long long)pos_of[t * top + k] * C + c], m);
        x_out[t * C + c] = x[t * C + c] + (y[t * C + c] + m);
    }
}

// ------------------------------------------------------------------------------------------------ norm after the sum
// x_out = rmsnorm(alpha * x + f) * w for blocks whose norm sits on the residual SUM. f is made of up to two sublayer
// outputs y1, y2 (each first RMS-normed over the width with its own weight when w1 / w2 is given; with two of them
// branch_scale weighs their sum) and, optionally, of a mixture's chosen experts: entry k of token t adds wts[t, k] times
// row pos_of[t * top + k] of z, or times x itself when its expert number ids[t * top + k] >= n_real (an expert that hands
// its input through). The sum is kept in shared memory between the reduction and the scaling. Block per row.
template <typename T>
__global__ void post_norm_kernel(const float* __restrict__ x, float alpha, const float* __restrict__ y1,
                                 const float* __restrict__ w1, const float* __restrict__ y2, const float* __restrict__ w2,
                                 float branch_scale, const float* __restrict__ z, const int* __restrict__ pos_of,
                                 const float* __restrict__ wts, const int* __restrict__ ids, int top, int n_real,
                                 const float* __restrict__ w, float* __restrict__ x_out, T* __restrict__ x_act, int C,
                                 float eps) {
    extern __shared__ float srow[];
    __shared__ float red[32];
    const long long t = blockIdx.x;
    const float* xr = x + t * C;
    float r1 = 1.f, r2 = 1.f;
    if (y1 && w1) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < C; c += blockDim.x) ss = fmaf(y1[t * C + c], y1[t * C + c], ss);
        r1 = 1.0f / sqrtf(block_sum(ss, red) / (float)C + eps);
    }
    if (y2 && w2) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < C; c += blockDim.x) ss = fmaf(y2[t * C + c], y2[t * C + c], ss);
        r2 = 1.0f / sqrtf(block_sum(ss, red) / (float)C + eps);
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float xv = xr[c];
        float f = 0.f;
        if (y1) f = w1 ? y1[t * C + c] * r1 * w1[c] : y1[t * C + c];
        if (y2) f += w2 ? y2[t * C + c] * r2 * w2[c] : y2[t * C + c];
        f *= branch_scale;
        for (int k = 0; k < top; ++k) {
            const bool through = ids && ids[t * top + k] >= n_real;
            f = fmaf(wts[t * top + k], through ? xv : z[(long long)pos_of[t * top + k] * C + c], f);
        }
        const float s = fmaf(alpha, xv, f);
        srow[c] = s;
        ss = fmaf(s, s, ss);
    }
    const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)C + eps);
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float v = srow[c] * r * w[c];
        x_out[t * C + c] = v;
        if (x_act) stf(x_act + t * C + c, v);
    }
}

__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    uint2 u;
    u.x = pack_bf16x2(v.x, v.y);
    u.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = u;
}

// The same with 16-byte accesses (C a multiple of 4, every pointer 16-byte aligned).
template <typename T>
__global__ void post_norm4_kernel(const float* __restrict__ x, float alpha, const float* __restrict__ y1,
                                  const float* __restrict__ w1, const float* __restrict__ y2, const float* __restrict__ w2,
                                  float branch_scale, const float* __restrict__ z, const int* __restrict__ pos_of,
                                  const float* __restrict__ wts, const int* __restrict__ ids, int top, int n_real,
                                  const float* __restrict__ w, float* __restrict__ x_out, T* __restrict__ x_act, int C,
                                  float eps) {
    extern __shared__ float4 srow4[];
    __shared__ float red[32];
    const long long t = blockIdx.x;
    const int C4 = C >> 2;
    const float4* xr = reinterpret_cast<const float4*>(x + t * C);
    const float4* a1 = y1 ? reinterpret_cast<const float4*>(y1 + t * C) : nullptr;
    const float4* a2 = y2 ? reinterpret_cast<const float4*>(y2 + t * C) : nullptr;
    float r1 = 1.f, r2 = 1.f;
    if (a1 && w1) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < C4; c += blockDim.x) {
            const float4 v = a1[c];
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
        r1 = 1.0f / sqrtf(block_sum(ss, red) / (float)C + eps);
    }
    if (a2 && w2) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < C4; c += blockDim.x) {
            const float4 v = a2[c];
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
        r2 = 1.0f / sqrtf(block_sum(ss, red) / (float)C + eps);
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < C4; c += blockDim.x) {
        const float4 xv = xr[c];
        float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
        if (a1) {
            f = a1[c];
            if (w1) {
                const float4 ww = reinterpret_cast<const float4*>(w1)[c];
                f = make_float4(f.x * r1 * ww.x, f.y * r1 * ww.y, f.z * r1 * ww.z, f.w * r1 * ww.w);
            }
        }
        if (a2) {
            float4 g = a2[c];
            if (w2) {
                const float4 ww = reinterpret_cast<const float4*>(w2)[c];
                g = make_float4(g.x * r2 * ww.x, g.y * r2 * ww.y, g.z * r2 * ww.z, g.w * r2 * ww.w);
            }
            f = make_float4(f.x + g.x, f.y + g.y, f.z + g.z, f.w + g.w);
        }
        f = make_float4(f.x * branch_scale, f.y * branch_scale, f.z * branch_scale, f.w * branch_scale);
        for (int k = 0; k < top; ++k) {
            const bool through = ids && ids[t * top + k] >= n_real;
            const float wt = wts[t * top + k];
            const float4 e = through ? xv : reinterpret_cast<const float4*>(z + (long long)pos_of[t * top + k] * C)[c];
            f = make_float4(fmaf(wt, e.x, f.x), fmaf(wt, e.y, f.y), fmaf(wt, e.z, f.z), fmaf(wt, e.w, f.w));
        }
        const float4 sv = make_float4(fmaf(alpha, xv.x, f.x), fmaf(alpha, xv.y, f.y), fmaf(alpha, xv.z, f.z),
                                      fmaf(alpha, xv.w, f.w));
        srow4[c] = sv;
        ss = fmaf(sv.x, sv.x, fmaf(sv.y, sv.y, fmaf(sv.z, sv.z, fmaf(sv.w, sv.w, ss))));
    }
    const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)C + eps);
    for (int c = threadIdx.x; c < C4; c += blockDim.x) {
        const float4 sv = srow4[c], ww = reinterpret_cast<const float4*>(w)[c];
        const float4 v = make_float4(sv.x * r * ww.x, sv.y * r * ww.y, sv.z * r * ww.z, sv.w * r * ww.w);
        st4(x_out + t * C + 4 * c, v);
        if (x_act) st4(x_act + t * C + 4 * c, v);
    }
}

// act = g' * sigmoid(slope * g') * (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit); gu = [gate | up] rows
template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gu, T* __restrict__ act, long long rows, int ff, float limit,
                                   float slope) {
    const long long n = rows * ff;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / ff;
        const int c = (int)(i % ff);
        const float g = fminf(ldf(gu + r * 2 * ff + c), limit);
        const float u = fminf(fmaxf(ldf(gu + r * 2 * ff + ff + c), -limit), limit);
        stf(act + i, g / (1.0f + expf(-slope * g)) * (u + 1.0f));
    }
}

// logits <- cap * tanh(logits * scale / cap) in place (cap <= 0: only the scale)
__global__ void logit_cap_kernel(float* __restrict__ z, long long n, float scale, float cap) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = z[i] * scale;
        z[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
    }
}

// Few rows, 32-bit weights (router logits while decoding): block per row, the row in shared memory as floats, a warp per
// output column at a time.
template <typename TA>
__global__ void linear_rows_w32_kernel(const TA* __restrict__ A, long long lda, const float* __restrict__ W,
                                       long long ldw, float* __restrict__ Cm, long long ldc,
                                       const float* __restrict__ bias, int N, int K) {
    extern __shared__ float xrow[];
    const long long m = blockIdx.x;
    for (int k = threadIdx.x; k < K; k += blockDim.x) xrow[k] = ldf(A + m * lda + k);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int n = warp; n < N; n += nw) {
        const float* wr = W + (long long)n * ldw;
        float acc = 0.f;
        for (int k = lane; k < K; k += 32) acc = fmaf(xrow[k], wr[k], acc);
        acc = warp_sum(acc);
        if (lane == 0) Cm[m * ldc + n] = acc + (bias ? bias[n] : 0.f);
    }
}

static int norm_threads(int C) {
    int t = 32;
    while (t < C / 4 && t < 512) t <<= 1;
    return t;
}

}  // namespace seq
}  // namespace llark

using namespace llark;
using namespace llark::seq;
typedef __nv_bfloat16 bf16_t;

extern "C" int llark_seq_embed(const int* ids, const int* tok_seq, const int* cu, const int* pos0, const void* table,
                               const void* pos_table, float scale, float* x, int n_tok, int C, int act_fp32,
                               cudaStream_t st) {
    if (n_tok <= 0 || C <= 0 || !ids || !tok_seq || !cu || !pos0 || !table || !x) return LLARK_EINVAL;
    const int th = norm_threads(C);
    if (act_fp32)
        embed_kernel<float><<<n_tok, th, 0, st>>>(ids, tok_seq, cu, pos0, (const float*)table, (const float*)pos_table,
                                                  scale, x, C);
    else
        embed_kernel<bf16_t><<<n_tok, th, 0, st>>>(ids, tok_seq, cu, pos0, (const bf16_t*)table,
                                                   (const bf16_t*)pos_table, scale, x, C);
    return check_launch();
}

extern "C" int llark_seq_short_conv(const float* h, const float* w, float* tail, const int* tok_seq, const int* cu,
                                    const int* slot, void* y, int n_tok, int C, int taps, int inline_tail, int act_fp32,
                                    cudaStream_t st) {
    if (n_tok <= 0 || C <= 0 || taps < 1 || !h || !w || !y || (taps > 1 && !tail)) return LLARK_EINVAL;
    const int th = norm_threads(C);
    const bool v4 = (C % 4 == 0) && (((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(tail)) & 15) == 0);
    if (v4 && !inline_tail && taps >= 2 && taps <= 4 && n_tok >= 64) {
        if (act_fp32) {
            if (taps == 2) launch_conv4t<float, 2>(h, w, tail, tok_seq, cu, slot, y, n_tok, C, st);
            else if (taps == 3) launch_conv4t<float, 3>(h, w, tail, tok_seq, cu, slot, y, n_tok, C, st);
            else launch_conv4t<float, 4>(h, w, tail, tok_seq, cu, slot, y, n_tok, C, st);
        } else {
            if (taps == 2) launch_conv4t<bf16_t, 2>(h, w, tail, tok_seq, cu, slot, y, n_tok, C, st);
            else if (taps == 3) launch_conv4t<bf16_t, 3>(h, w, tail, tok_seq, cu, slot, y, n_tok, C, st);
            else launch_conv4t<bf16_t, 4>(h, w, tail, tok_seq, cu, slot, y, n_tok, C, st);
        }
    } else if (v4) {
        int t4 = 32;
        while (t4 * 4 < C && t4 < 256) t4 <<= 1;
        if (act_fp32)
            short_conv4_kernel<float><<<n_tok, t4, 0, st>>>(h, w, tail, tok_seq, cu, slot, (float*)y, C, taps, inline_tail);
        else
            short_conv4_kernel<bf16_t><<<n_tok, t4, 0, st>>>(h, w, tail, tok_seq, cu, slot, (bf16_t*)y, C, taps,
                                                            inline_tail);
    } else if (act_fp32)
        short_conv_kernel<float><<<n_tok, th, 0, st>>>(h, w, tail, tok_seq, cu, slot, (float*)y, C, taps, inline_tail);
    else
        short_conv_kernel<bf16_t><<<n_tok, th, 0, st>>>(h, w, tail, tok_seq, cu, slot, (bf16_t*)y, C, taps, inline_tail);
    return check_launch();
}

extern "C" int llark_seq_conv_tail(const float* h, float* tail, const int* cu, const int* slot, int n_seq, int C,
                                   int taps, cudaStream_t st) {
    if (n_seq <= 0 || C <= 0 || taps < 1 || !h) return LLARK_EINVAL;
    if (taps == 1) return LLARK_OK;
    conv_tail_kernel<<<n_seq, norm_threads(C), 0, st>>>(h, tail, cu, slot, C, taps);
    return check_launch();
}

extern "C" int llark_seq_add_rmsnorm(const float* x, const float* y, const float* w, float* x_out, void* x_act,
                                     long long rows, int C, float eps, int act_fp32, cudaStream_t st) {
    if (rows <= 0 || C <= 0 || !x || !y || !w || !x_out) return LLARK_EINVAL;
    const int th = norm_threads(C);
    const bool v4 = (C % 4 == 0) && (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                                       reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x_out)) & 15) == 0);
    if (v4) {
        int t4 = 32;
        while (t4 * 8 < C && t4 < 256) t4 <<= 1;  // two vectors per thread at the usual widths
        if (act_fp32)
            add_rmsnorm4_kernel<float><<<(unsigned)rows, t4, 0, st>>>(x, y, w, x_out, (float*)x_act, C, eps);
        else
            add_rmsnorm4_kernel<bf16_t><<<(unsigned)rows, t4, 0, st>>>(x, y, w, x_out, (bf16_t*)x_act, C, eps);
    } else if (act_fp32)
        add_rmsnorm_kernel<float><<<(unsigned)rows, th, 0, st>>>(x, y, w, x_out, (float*)x_act, C, eps);
    else
        add_rmsnorm_kernel<bf16_t><<<(unsigned)rows, th, 0, st>>>(x, y, w, x_out, (bf16_t*)x_act, C, eps);
    return check_launch();
}

extern "C" int llark_seq_gated_norm_add(const float* x, const float* y, const float* gate, long long gate_ld,
                                        const float* w, const float* w_next, float* x_out, void* x_act, long long rows,
                                        int C, float eps, int act_fp32, cudaStream_t st) {
    if (rows <= 0 || C <= 0 || !x || !y || !w || !x_out || (x_act && !w_next)) return LLARK_EINVAL;
    const bool vec = (C % 4 == 0) && C <= 4 * 4 * 512 && (!gate || gate_ld % 4 == 0) && ((uintptr_t)x % 16 == 0) &&
                     ((uintptr_t)y % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)x_out % 16 == 0) &&
                     (!gate || (uintptr_t)gate % 16 == 0) && (!x_act || ((uintptr_t)x_act % 16 == 0 && (uintptr_t)w_next % 16 == 0));
    if (vec) {
        const int nv = C / 4;
        const int per = nv <= 256 ? 1 : (nv <= 1024 ? 2 : 4);  // float4 per thread: 256 .. 512 threads on wide rows
        int threads = ((nv + per - 1) / per + 31) / 32 * 32;
#define LLARK_GNA4(T, NV) \
    gated_norm_add4_kernel<T, NV><<<(unsigned)rows, threads, 0, st>>>(x, y, gate, gate_ld, w, w_next, x_out, (T*)x_act, C, eps)
        if (act_fp32) {
            if (per == 1) LLARK_GNA4(float, 1);
            else if (per == 2) LLARK_GNA4(float, 2);
            else LLARK_GNA4(float, 4);
        } else {
            if (per == 1) LLARK_GNA4(bf16_t, 1);
            else if (per == 2) LLARK_GNA4(bf16_t, 2);
            else LLARK_GNA4(bf16_t, 4);
        }
#undef LLARK_GNA4
        return check_launch();
    }
    const size_t smem = sizeof(float) * (size_t)C;
    if (smem > 200 * 1024) return LLARK_EINVAL;
    int threads = C < 64 ? 64 : (C > 512 ? 512 : (C + 31) / 32 * 32);
#define LLARK_GNA(T)                                                                                                 \
    do {                                                                                                              \
        if (smem > 48 * 1024) {                                                                                       \
            cudaError_t e = cudaFuncSetAttribute(gated_norm_add_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                 (int)smem);                                                          \
            if (e != cudaSuccess) {                                                                                   \
                g_last_cuda_error = (int)e;                                                                           \
                return LLARK_ECUDA;                                                                                   \
            }                                                                                                         \
        }                                                                                                             \
        gated_norm_add_kernel<T><<<(unsigned)rows, threads, smem, st>>>(x, y, gate, gate_ld, w, w_next, x_out,        \
                                                                        (T*)x_act, C, eps);                          \
    } while (0)
    if (act_fp32) LLARK_GNA(float);
    else LLARK_GNA(bf16_t);
#undef LLARK_GNA
    return check_launch();
}

extern "C" int llark_seq_rmsnorm_rows(const float* x, const int* rows, const float* w, void* out, int n_rows, int C,
                                      float eps, int act_fp32, cudaStream_t st) {
    if (n_rows <= 0 || C <= 0 || !x || !w || !out) return LLARK_EINVAL;
    const int th = norm_threads(C);
    if (act_fp32)
        rmsnorm_rows_kernel<float><<<n_rows, th, 0, st>>>(x, rows, w, (float*)out, C, eps);
    else
        rmsnorm_rows_kernel<bf16_t><<<n_rows, th, 0, st>>>(x, rows, w, (bf16_t*)out, C, eps);
    return check_launch();
}

extern "C" int llark_seq_relu2(const void* u, void* y, long long n, int act_fp32, cudaStream_t st) {
    if (n <= 0 || !u || !y) return LLARK_EINVAL;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (act_fp32)
        relu2_kernel<float><<<grid, 256, 0, st>>>((const float*)u, (float*)y, n);
    else
        relu2_kernel<bf16_t><<<grid, 256, 0, st>>>((const bf16_t*)u, (bf16_t*)y, n);
    return check_launch();
}

template <typename T, typename TC>
static void launch_rows(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc,
                        const float* bias, int M, int N, int K, cudaStream_t st) {
    const int vec = 16 / (int)sizeof(T);
    const int vec_ok = (K % vec == 0) && (lda % vec == 0) && (ldw % vec == 0) &&
                       (((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) == 0);
    const int warps = 8;
    // two columns per warp once that still leaves several warps per SM (148 SMs); one for narrow outputs
    const bool two = (long long)N >= 2LL * warps * 148 * 2;
    const int nc = two ? 2 : 1;
    const unsigned gx = (unsigned)((N + warps * nc - 1) / (warps * nc));
#define LLARK_ROWS(MB_, NC_)                                                                                            \
    linear_rows_kernel<T, TC, MB_, NC_><<<dim3(gx, (M + MB_ - 1) / MB_), warps * 32, 0, st>>>(                          \
        (const T*)A, lda, (const T*)W, ldw, (TC*)C, ldc, bias, M, N, K, vec_ok)
    if (M <= 2) {
        if (two) LLARK_ROWS(2, 2);
        else LLARK_ROWS(2, 1);
    } else {
        if (two) LLARK_ROWS(8, 2);
        else LLARK_ROWS(8, 1);
    }
#undef LLARK_ROWS
}

extern "C" int llark_linear_rows(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc,
                                 int c_fp32, const float* bias, int M, int N, int K, int in_fp32, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0 || !A || !W || !C || lda < K || ldw < K || ldc < N) return LLARK_EINVAL;
    if (in_fp32 && !c_fp32) return LLARK_EINVAL;
    if (in_fp32)
        launch_rows<float, float>(A, lda, W, ldw, C, ldc, bias, M, N, K, st);
    else if (c_fp32)
        launch_rows<bf16_t, float>(A, lda, W, ldw, C, ldc, bias, M, N, K, st);
    else
        launch_rows<bf16_t, bf16_t>(A, lda, W, ldw, C, ldc, bias, M, N, K, st);
    return check_launch();
}

extern "C" int llark_linear_simt(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc,
                                 int c_fp32, const float* bias, int M, int N, int K, int in_fp32, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0 || !A || !W || !C || lda < K || ldw < K || ldc < N) return LLARK_EINVAL;
    if (in_fp32 && !c_fp32) return LLARK_EINVAL;
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    if (in_fp32)
        linear_simt_kernel<float, float><<<grid, 256, 0, st>>>((const float*)A, lda, (const float*)W, ldw, (float*)C, ldc,
                                                               bias, M, N, K);
    else if (c_fp32)
        linear_simt_kernel<bf16_t, float><<<grid, 256, 0, st>>>((const bf16_t*)A, lda, (const bf16_t*)W, ldw, (float*)C,
                                                                ldc, bias, M, N, K);
    else
        linear_simt_kernel<bf16_t, bf16_t><<<grid, 256, 0, st>>>((const bf16_t*)A, lda, (const bf16_t*)W, ldw, (bf16_t*)C,
                                                                 ldc, bias, M, N, K);
    return check_launch();
}

extern "C" int llark_linear_simt_w32(const void* A, long long lda, const float* W, long long ldw, float* C,
                                     long long ldc, const float* bias, int M, int N, int K, int in_fp32,
                                     cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0 || !A || !W || !C || lda < K || ldw < K || ldc < N) return LLARK_EINVAL;
    if (M <= 128 && (size_t)K * sizeof(float) <= 48 * 1024) {
        if (in_fp32)
            linear_rows_w32_kernel<float><<<M, 256, K * sizeof(float), st>>>((const float*)A, lda, W, ldw, C, ldc, bias, N, K);
        else
            linear_rows_w32_kernel<bf16_t><<<M, 256, K * sizeof(float), st>>>((const bf16_t*)A, lda, W, ldw, C, ldc, bias, N,
                                                                            K);
        return check_launch();
    }
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    if (in_fp32)
        linear_simt_kernel<float, float, float><<<grid, 256, 0, st>>>((const float*)A, lda, W, ldw, C, ldc, bias, M, N, K);
    else
        linear_simt_kernel<bf16_t, float, float><<<grid, 256, 0, st>>>((const bf16_t*)A, lda, W, ldw, C, ldc, bias, M, N,
                                                                      K);
    return check_launch();
}

extern "C" int llark_seq_group_rmsnorm(const float* x, const int* rows, const float* add_vec, float* x_out,
                                       const float* w, void* out, int n_rows, int C, int groups, float eps, int out_fp32,
                                       cudaStream_t st) {
    if (n_rows <= 0 || C <= 0 || groups <= 0 || (C % groups) || !x || !w || !out) return LLARK_EINVAL;
    if (x_out && rows) return LLARK_EINVAL;
    const int per = C / groups;
    const bool al = (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out) |
                       reinterpret_cast<uintptr_t>(add_vec) | reinterpret_cast<uintptr_t>(x_out)) & 15) == 0);
    if (per % 4 == 0 && al) {
        const long long items = (long long)n_rows * groups;
        const unsigned grid = (unsigned)((items + 3) / 4);
        if (out_fp32)
            group_rmsnorm_warp_kernel<float><<<grid, 128, 0, st>>>(x, rows, add_vec, x_out, w, (float*)out, n_rows, C,
                                                                   groups, eps);
        else
            group_rmsnorm_warp_kernel<bf16_t><<<grid, 128, 0, st>>>(x, rows, add_vec, x_out, w, (bf16_t*)out, n_rows, C,
                                                                    groups, eps);
        return check_launch();
    }
    const int th = norm_threads(C / groups * 4);
    if (out_fp32)
        group_rmsnorm_kernel<float><<<n_rows, th, 0, st>>>(x, rows, add_vec, x_out, w, (float*)out, C, groups, eps);
    else
        group_rmsnorm_kernel<bf16_t><<<n_rows, th, 0, st>>>(x, rows, add_vec, x_out, w, (bf16_t*)out, C, groups, eps);
    return check_launch();
}

extern "C" int llark_seq_residual_combine(const float* x, const float* y, const float* z, const int* pos_of,
                                          const float* wts, int top, float* x_out, int n_tok, int C, cudaStream_t st) {
    if (n_tok <= 0 || C <= 0 || top < 0 || !x || !y || !x_out || (top > 0 && (!z || !pos_of || !wts)))
        return LLARK_EINVAL;
    residual_combine_kernel<<<n_tok, norm_threads(C * 4), 0, st>>>(x, y, z, pos_of, wts, top, x_out, C);
    return check_launch();
}

extern "C" int llark_seq_post_norm(const float* x, float alpha, const float* y1, const float* w1, const float* y2,
                                   const float* w2, float branch_scale, const float* z, const int* pos_of,
                                   const float* wts, const int* ids, int top, int n_real, const float* w, float* x_out,
                                   void* x_act, long long rows, int C, float eps, int act_fp32, cudaStream_t st) {
    if (rows <= 0 || C <= 0 || top < 0 || !x || !w || !x_out || (top > 0 && (!z || !pos_of || !wts)) || (y2 && !y1) ||
        (w1 && !y1) || (w2 && !y2))
        return LLARK_EINVAL;
    const size_t smem = sizeof(float) * (size_t)C;
    if (smem > 48 * 1024) return LLARK_EINVAL;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (C % 4 == 0 && al(x) && al(y1) && al(w1) && al(y2) && al(w2) && al(z) && al(w) && al(x_out) && al(x_act)) {
        int t4 = 32;
        while (t4 * 8 < C && t4 < 256) t4 <<= 1;  // two vectors per thread at the usual widths
        if (act_fp32)
            post_norm4_kernel<float><<<(unsigned)rows, t4, smem, st>>>(x, alpha, y1, w1, y2, w2, branch_scale, z, pos_of,
                                                                       wts, ids, top, n_real, w, x_out, (float*)x_act, C,
                                                                       eps);
        else
            post_norm4_kernel<bf16_t><<<(unsigned)rows, t4, smem, st>>>(x, alpha, y1, w1, y2, w2, branch_scale, z, pos_of,
                                                                        wts, ids, top, n_real, w, x_out, (bf16_t*)x_act,
                                                                        C, eps);
        return check_launch();
    }
    const int th = norm_threads(C);
    if (act_fp32)
        post_norm_kernel<float><<<(unsigned)rows, th, smem, st>>>(x, alpha, y1, w1, y2, w2, branch_scale, z, pos_of, wts,
                                                                  ids, top, n_real, w, x_out, (float*)x_act, C, eps);
    else
        post_norm_kernel<bf16_t><<<(unsigned)rows, th, smem, st>>>(x, alpha, y1, w1, y2, w2, branch_scale, z, pos_of, wts,
                                                                   ids, top, n_real, w, x_out, (bf16_t*)x_act, C, eps);
    return check_launch();
}

extern "C" int llark_seq_glu_clamped(const void* gu, void* act, long long rows, int ff, float limit, float slope,
                                     int act_fp32, cudaStream_t st) {
    if (rows <= 0 || ff <= 0 || !gu || !act || !(limit > 0.f)) return LLARK_EINVAL;
    const long long n = rows * ff;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (act_fp32)
        glu_clamped_kernel<float><<<grid, 256, 0, st>>>((const float*)gu, (float*)act, rows, ff, limit, slope);
    else
        glu_clamped_kernel<bf16_t><<<grid, 256, 0, st>>>((const bf16_t*)gu, (bf16_t*)act, rows, ff, limit, slope);
    return check_launch();
}

extern "C" int llark_seq_logit_cap(float* z, long long n, float scale, float cap, cudaStream_t st) {
    if (n <= 0 || !z) return LLARK_EINVAL;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    logit_cap_kernel<<<grid, 256, 0, st>>>(z, n, scale, cap);
    return check_launch();
}

extern "C" int llark_seq_tanh(const float* u, void* y, long long n, int act_fp32, cudaStream_t st) {
    if (n <= 0 || !u || !y) return LLARK_EINVAL;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (act_fp32)
        tanh_kernel<float><<<grid, 256, 0, st>>>(u, (float*)y, n);
    else
        tanh_kernel<bf16_t><<<grid, 256, 0, st>>>(u, (bf16_t*)y, n);
    return check_launch();
}
