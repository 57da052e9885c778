// Latent attention on the generation path: keys and values of all heads are expansions W_uk c, W_uv c of one low-rank
// latent c per token, plus one rotated key part shared by the heads. Only [c | rotated part] (R + P numbers per token) is
// cached. The expansions are folded into the query and the output instead of being applied to every cached key:
//
//     score_h(i, j) = (W_uk,h^T q_h,i) . c_j + rot(q'_h,i) . rot(k'_j)        o_h,i = W_uv,h (sum_j p_h(i, j) c_j)
//
// so attention runs as H query heads of size R + P over ONE shared key head whose rows are also the values (the last P
// output channels are not used), through the window-attention kernels of seq_mixers.cu / seq_swa_mma.cu.
//
//   llark_seq_latent_prep   RMS norm of the latent, rotation (interleaved pairs or halves, given frequency table and magnitude
//                           factor) of the shared key part and of every head's rotated query part at the token's
//                           position (fp32 angles); writes [c | rot k] (also straight into the ring on single-token
//                           steps) and the rotated query parts into the folded-query buffer
//   llark_seq_head_linear   y[t, h, :] = W[h] x[t, h, :] for all heads in one launch (the two foldings), optional
//                           sigmoid gate on the output
#include "common.cuh"

namespace llark {
extern thread_local int g_last_cuda_error;
namespace latent {

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
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// Block per token. src row: q at q (H heads of Dn + P, the rotated part last), latent at lat (R, then P).
template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ q, long long q_ld, const float* __restrict__ lat,
                                   long long lat_ld, const float* __restrict__ norm_w, const float* __restrict__ freqs,
                                   int n_rot, float mult, T* __restrict__ ckr, T* __restrict__ qf, T* __restrict__ ring,
                                   const int* __restrict__ tok_seq, const int* __restrict__ cu,
                                   const int* __restrict__ pos0, const int* __restrict__ slot, int H, int Dn, int P, int R,
                                   int cap, float eps, int halves) {
    __shared__ float red[32];
    __shared__ float cs[2 * 128];  // cos / sin of up to 128 pairs; more are recomputed
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    const long long p = pos0[b] + (t - cu[b]);
    const int half = n_rot / 2;
    for (int i = threadIdx.x; i < half && i < 128; i += blockDim.x) {
        const float ang = (float)p * freqs[i];
        cs[2 * i] = cosf(ang) * mult;
        cs[2 * i + 1] = sinf(ang) * mult;
    }
    const float* lr = lat + (long long)t * lat_ld;
    float ss = 0.f;
    for (int c = threadIdx.x; c < R; c += blockDim.x) ss = fmaf(lr[c], lr[c], ss);
    ss = warp_sum(ss);
    {
        const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
        if (l == 0) red[w] = ss;
        __syncthreads();  // also publishes cs
        ss = 0.f;
        for (int i = 0; i < nw; ++i) ss += red[i];
    }
    const float rn = 1.0f / sqrtf(ss / (float)R + eps);
    const int W = R + P;
    T* row = ckr + (long long)t * W;
    T* rrow = ring ? ring + ((long long)slot[b] * cap + (p % cap)) * W : nullptr;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        const float v = lr[c] * rn * norm_w[c];
        stf(row + c, v);
        if (rrow) stf(rrow + c, v);
    }
    // pair i of a rotated part: entries (2i, 2i + 1), or (i, i + half) in the halves layout
    const int pu = halves ? 1 : 2, pv0 = halves ? half : 1;
    auto turn = [&](const float* in, int i, float& a, float& bb) {
        float co, si;
        if (i < 128) {
            co = cs[2 * i];
            si = cs[2 * i + 1];
        } else {
            const float ang = (float)p * freqs[i];
            co = cosf(ang) * mult;
            si = sinf(ang) * mult;
        }
        const float u = in[pu * i], v = in[pu * i + pv0];
        a = u * co - v * si;
        bb = v * co + u * si;
    };
    // shared key part
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float a, bb;
        turn(lr + R, i, a, bb);
        stf(row + R + pu * i, a);
        stf(row + R + pu * i + pv0, bb);
        if (rrow) {
            stf(rrow + R + pu * i, a);
            stf(rrow + R + pu * i + pv0, bb);
        }
    }
    for (int c = 2 * half + threadIdx.x; c < P; c += blockDim.x) {  // entries past the rotated ones pass
        stf(row + R + c, lr[R + c]);
        if (rrow) stf(rrow + R + c, lr[R + c]);
    }
    // every head's rotated query part -> columns R .. R + P of its folded query
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        const int h = i / half, j = i % half;
        float a, bb;
        turn(q + (long long)t * q_ld + (long long)h * (Dn + P) + Dn, j, a, bb);
        T* o = qf + ((long long)t * H + h) * W + R;
        stf(o + pu * j, a);
        stf(o + pu * j + pv0, bb);
    }
    const int rest = P - 2 * half;
    for (int i = threadIdx.x; i < H * rest; i += blockDim.x) {
        const int h = i / rest, c = 2 * half + i % rest;
        stf(qf + ((long long)t * H + h) * W + R + c, q[(long long)t * q_ld + (long long)h * (Dn + P) + Dn + c]);
    }
}

// y[m, h * y_hs + n] = sum_k x[m, h * x_hs + k] * W[h][n][k] (* sigmoid(gate[m, h * N + n])): 64 x 64 tile per block,
// 16-deep slices through shared memory, 4 x 4 outputs per thread, fp32 FMA.
template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256)
head_linear_kernel(const TX* __restrict__ X, long long ldx, int x_hs, const TW* __restrict__ W, TY* __restrict__ Y,
                   long long ldy, int y_hs, const float* __restrict__ gate, long long gate_ld, int M, int N, int K) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int h = blockIdx.z;
    const TX* A = X + (long long)h * x_hs;
    const TW* Wh = W + (long long)h * N * K;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            const int r = i / BK, k = i % BK;
            As[k][r] = (m0 + r < M && k0 + k < K) ? ldf(A + (long long)(m0 + r) * ldx + k0 + k) : 0.f;
            Ws[k][r] = (n0 + r < N && k0 + k < K) ? ldf(Wh + (long long)(n0 + r) * K + k0 + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], bq[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bq[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bq[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) {
                float y = acc[i][j];
                if (gate) y *= sigmoidf_(gate[(long long)m * gate_ld + (long long)h * N + n]);
                stf(Y + (long long)m * ldy + (long long)h * y_hs + n, y);
            }
        }
}

}  // namespace latent
}  // namespace llark

using namespace llark;
using namespace llark::latent;
typedef __nv_bfloat16 bf16_t;

extern "C" int llark_seq_latent_prep(const float* q, long long q_ld, const float* lat, long long lat_ld,
                                     const float* norm_w, const float* freqs, int n_rot, float mult, void* ckr, void* qf,
                                     void* ring, const int* tok_seq, const int* cu, const int* pos0, const int* slot,
                                     int n_tok, int H, int Dn, int P, int R, int cap, float eps, int halves, int act_fp32,
                                     cudaStream_t st) {
    if (n_tok <= 0 || H <= 0 || Dn < 0 || P < 0 || R <= 0 || n_rot < 0 || (n_rot % 2) || n_rot > P || !q || !lat ||
        !norm_w || (n_rot && !freqs) || !ckr || !qf || !tok_seq || !cu || !pos0 || !slot || (ring && cap <= 0))
        return LLARK_EINVAL;
    if (act_fp32)
        latent_prep_kernel<float><<<n_tok, 128, 0, st>>>(q, q_ld, lat, lat_ld, norm_w, freqs, n_rot, mult, (float*)ckr,
                                                         (float*)qf, (float*)ring, tok_seq, cu, pos0, slot, H, Dn, P, R,
                                                         cap, eps, halves);
    else
        latent_prep_kernel<bf16_t><<<n_tok, 128, 0, st>>>(q, q_ld, lat, lat_ld, norm_w, freqs, n_rot, mult, (bf16_t*)ckr,
                                                          (bf16_t*)qf, (bf16_t*)ring, tok_seq, cu, pos0, slot, H, Dn, P, R,
                                                          cap, eps, halves);
    return check_launch();
}

extern "C" int llark_seq_head_linear(const void* x, int x_fp32, long long ldx, int x_hs, const void* w, void* y,
                                     long long ldy, int y_hs, const float* gate, long long gate_ld, int M, int H, int N,
                                     int K, int act_fp32, cudaStream_t st) {
    if (M <= 0 || H <= 0 || N <= 0 || K <= 0 || !x || !w || !y) return LLARK_EINVAL;
    if (act_fp32 && !x_fp32) return LLARK_EINVAL;
    dim3 grid((N + 63) / 64, (M + 63) / 64, H);
    if (act_fp32)
        head_linear_kernel<float, float, float><<<grid, 256, 0, st>>>((const float*)x, ldx, x_hs, (const float*)w,
                                                                      (float*)y, ldy, y_hs, gate, gate_ld, M, N, K);
    else if (x_fp32)
        head_linear_kernel<float, bf16_t, bf16_t><<<grid, 256, 0, st>>>((const float*)x, ldx, x_hs, (const bf16_t*)w,
                                                                        (bf16_t*)y, ldy, y_hs, gate, gate_ld, M, N, K);
    else
        head_linear_kernel<bf16_t, bf16_t, bf16_t><<<grid, 256, 0, st>>>((const bf16_t*)x, ldx, x_hs, (const bf16_t*)w,
                                                                         (bf16_t*)y, ldy, y_hs, gate, gate_ld, M, N, K);
    return check_launch();
}
