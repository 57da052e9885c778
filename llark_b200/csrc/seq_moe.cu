// Routed mixture of experts on the generation path: every token uses `top` of n small gated feed-forwards
// down(silu(gate x) * (up x)). The router picks experts on the device, one kernel sorts the (token, choice) entries by
// expert and cuts each expert's run into row tiles, and two grouped GEMM launches walk that tile list (rows gathered
// through the sort permutation). Large bf16 steps instead run every expert's rows through the tcgen05 GEMM core in its
// rows-in-runs mode (llark_seq_moe_gather, llark_gemm_segments with the sort kernel's list of 256-row tiles and its
// device-side count, llark_seq_silu_mul). Neither route returns to the host. The
// weighted sum over a token's choices is taken in the order of the choices when the residual is assembled
// (llark_seq_residual_combine), so a token's result does not depend on what else is in the batch.
//
//   llark_seq_moe_route     scores = sigmoid(logits) fp32; experts form `n_groups` groups of neighbours, a group's score
//                           is the sum of its two best, only experts of the best `keep` groups can be chosen; the `top`
//                           best of those; weights = their scores / (sum + 1e-20) * scale
//   llark_seq_moe_route_bias  scores = softmax(logits) fp32 over all router outputs; the CHOICE is made on score +
//                           correction (which may be negative), a group's score is its best choice score, experts outside
//                           the best `keep` groups cannot be chosen; weights = the chosen experts' plain scores * scale,
//                           not renormalised. Router outputs >= n_real are experts without weights that hand their input
//                           through: the sort leaves them out of the tile lists, the residual kernel adds the input.
//   llark_seq_moe_sort      entries -> perm (sorted by expert), pos_of (inverse), tiles (expert, first row, rows)
//   llark_seq_moe_up        act[pos] = silu(W_gate,e x) * (W_up,e x)     x = the entry's token row
//   llark_seq_moe_down      z[pos]   = W_down,e act[pos]                 fp32
#include "common.cuh"

namespace llark {
extern thread_local int g_last_cuda_error;
namespace moe {

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

constexpr int kTileRows = 64;
constexpr int kRowsRouteMaxEntries = 512;  // steps up to this many (token, choice) entries take the weight-streaming kernel

// ------------------------------------------------------------------------------------------------ router
// Warp per token; scores in shared memory. Ties go to the lower expert / group number.
__global__ void route_kernel(const float* __restrict__ logits, long long ld, int* __restrict__ ids,
                             float* __restrict__ wts, int n_tok, int n_exp, int n_groups, int keep, int top,
                             float scale) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const long long t = (long long)blockIdx.x * nw + warp;
    if (t >= n_tok) return;
    float* s = sm + (long long)warp * (n_exp + n_groups);   // scores; -1 once taken or shut out
    float* gs = s + n_exp;                                  // group scores
    const int per = n_exp / n_groups;
    for (int e = lane; e < n_exp; e += 32) s[e] = sigmoidf_(logits[t * ld + e]);
    __syncwarp();
    for (int g = lane; g < n_groups; g += 32) {
        float a = -1.f, b = -1.f;  // the two largest (scores are positive)
        for (int i = 0; i < per; ++i) {
            const float v = s[g * per + i];
            if (v > a) {
                b = a;
                a = v;
            } else if (v > b) {
                b = v;
            }
        }
        gs[g] = a + (b > 0.f ? b : 0.f);
    }
    __syncwarp();
    if (keep < n_groups) {
        if (lane == 0) {
            for (int r = 0; r < keep; ++r) {  // mark the best `keep` groups with a negative score - 2 (still ordered)
                int best = -1;
                float bv = -1.f;
                for (int g = 0; g < n_groups; ++g)
                    if (gs[g] >= 0.f && gs[g] > bv) {
                        bv = gs[g];
                        best = g;
                    }
                gs[best] = -2.f;
            }
        }
        __syncwarp();
        for (int e = lane; e < n_exp; e += 32)
            if (gs[e / per] != -2.f) s[e] = -1.f;
        __syncwarp();
    }
    float chosen_w = 0.f;  // lane k keeps choice k (top <= 32)
    int chosen_e = 0;
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -1.f;
        int be = 0x7fffffff;
        for (int e = lane; e < n_exp; e += 32)
            if (s[e] > bv) {
                bv = s[e];
                be = e;
            }
        for (int m = 16; m > 0; m >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
            const int oe = __shfl_xor_sync(0xffffffffu, be, m);
            if (ov > bv || (ov == bv && oe < be)) {
                bv = ov;
                be = oe;
            }
        }
        if (lane == k) {
            chosen_w = bv;
            chosen_e = be;
        }
        sum += bv;
        if (lane == 0) s[be] = -1.f;
        __syncwarp();
    }
    if (lane < top) {
        ids[t * top + lane] = chosen_e;
        wts[t * top + lane] = chosen_w / (sum + 1e-20f) * scale;
    }
}

// Warp per token. s = plain scores, c = choice scores (-inf once taken or shut out). Ties go to the lower number.
__global__ void route_bias_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ correction,
                                  int* __restrict__ ids, float* __restrict__ wts, int n_tok, int n_exp, int n_groups,
                                  int keep, int top, float scale) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const long long t = (long long)blockIdx.x * nw + warp;
    if (t >= n_tok) return;
    float* s = sm + (long long)warp * (2 * n_exp + n_groups);
    float* c = s + n_exp;
    float* gs = c + n_exp;
    const int per = n_exp / n_groups;
    float mx = -INFINITY;
    for (int e = lane; e < n_exp; e += 32) mx = fmaxf(mx, logits[t * ld + e]);
    mx = warp_max(mx);
    float den = 0.f;
    for (int e = lane; e < n_exp; e += 32) {
        const float v = expf(logits[t * ld + e] - mx);
        s[e] = v;
        den += v;
    }
    den = warp_sum(den);
    for (int e = lane; e < n_exp; e += 32) {
        s[e] = s[e] / den;
        c[e] = s[e] + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    if (keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY;
            for (int i = 0; i < per; ++i) a = fmaxf(a, c[g * per + i]);
            gs[g] = a;
        }
        __syncwarp();
        if (lane == 0) {
            for (int r = 0; r < keep; ++r) {  // the best `keep` groups are marked with +inf
                int best = -1;
                float bv = -INFINITY;
                for (int g = 0; g < n_groups; ++g)
                    if (gs[g] != INFINITY && (best < 0 || gs[g] > bv)) {
                        bv = gs[g];
                        best = g;
                    }
                gs[best] = INFINITY;
            }
        }
        __syncwarp();
        for (int e = lane; e < n_exp; e += 32)
            if (gs[e / per] != INFINITY) c[e] = -INFINITY;
        __syncwarp();
    }
    float chosen_w = 0.f;  // lane k keeps choice k (top <= 32)
    int chosen_e = 0;
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY;
        int be = 0x7fffffff;
        for (int e = lane; e < n_exp; e += 32)
            if (c[e] > bv) {
                bv = c[e];
                be = e;
            }
        for (int m = 16; m > 0; m >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
            const int oe = __shfl_xor_sync(0xffffffffu, be, m);
            if (ov > bv || (ov == bv && oe < be)) {
                bv = ov;
                be = oe;
            }
        }
        if (lane == k) {
            chosen_e = be;
            chosen_w = s[be];
        }
        __syncwarp();
        if (lane == 0) c[be] = -INFINITY;
        __syncwarp();
    }
    if (lane < top) {
        ids[t * top + lane] = chosen_e;
        wts[t * top + lane] = chosen_w * scale;
    }
}

// ------------------------------------------------------------------------------------------------ sort by expert
// One block. meta[0] = number of tiles; tiles[i] = (expert, first sorted row, rows). Experts >= n_real (no weights) keep
// their place in the sorted order but get no tiles.
__global__ void sort_kernel(const int* __restrict__ ids, int n_ent, int n_exp, int n_real, int* __restrict__ perm,
                            int* __restrict__ pos_of, int* __restrict__ tiles, int* __restrict__ meta,
                            int* __restrict__ seg_off, int* __restrict__ tiles256) {
    extern __shared__ int si[];
    int* cnt = si;               // [n_exp]
    int* off = cnt + n_exp;      // [n_exp + 1]
    int* cur = off + n_exp + 1;  // [n_exp]
    for (int e = threadIdx.x; e < n_exp; e += blockDim.x) cnt[e] = cur[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_ent; i += blockDim.x) atomicAdd(&cnt[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 32 && tiles256) {  // the GEMM core's tile list (256-row m-blocks), by another warp
        int o = 0, nt = 0;
        for (int e = 0; e < n_real; ++e) {
            for (int r = 0; r < cnt[e]; r += 256) {
                tiles256[3 * nt] = e;
                tiles256[3 * nt + 1] = o + r;
                tiles256[3 * nt + 2] = cnt[e] - r < 256 ? cnt[e] - r : 256;
                ++nt;
            }
            o += cnt[e];
        }
        meta[1] = nt;
    }
    if (threadIdx.x == 0) {
        int o = 0, nt = 0;
        for (int e = 0; e < n_exp; ++e) {
            off[e] = o;
            for (int r = 0; e < n_real && r < cnt[e]; r += kTileRows) {
                tiles[3 * nt] = e;
                tiles[3 * nt + 1] = o + r;
                tiles[3 * nt + 2] = cnt[e] - r < kTileRows ? cnt[e] - r : kTileRows;
                ++nt;
            }
            o += cnt[e];
        }
        off[n_exp] = o;
        meta[0] = nt;
    }
    __syncthreads();
    if (seg_off)
        for (int e = threadIdx.x; e <= n_exp; e += blockDim.x) seg_off[e] = off[e];
    for (int i = threadIdx.x; i < n_ent; i += blockDim.x) {
        const int e = ids[i];
        const int p = off[e] + atomicAdd(&cur[e], 1);
        perm[p] = i;
        pos_of[i] = p;
    }
}

// ------------------------------------------------------------------------------------------------ grouped GEMMs
// Block = one row tile of one expert x 64 output columns. DUAL: two weight matrices (gate rows, then up rows, of the
// expert's [2 * N, K] block) and out = silu(a) * b; otherwise out = the product. Rows of A: gather ? perm[pos] / top : pos.
template <typename T, typename TC, bool DUAL>
__global__ void __launch_bounds__(256)
grouped_linear_kernel(const T* __restrict__ A, long long lda, const int* __restrict__ perm, int top,
                      const T* __restrict__ W, TC* __restrict__ Cm, long long ldc, const int* __restrict__ tiles,
                      const int* __restrict__ meta, int N, int K) {
    constexpr int BM = kTileRows, BN = 64, BK = 16;
    if ((int)blockIdx.y >= meta[0]) return;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[DUAL ? 2 : 1][BK][BN + 4];
    __shared__ int rows[BM];
    const int ex = tiles[3 * blockIdx.y], r0 = tiles[3 * blockIdx.y + 1], nr = tiles[3 * blockIdx.y + 2];
    const T* We = W + (long long)ex * (DUAL ? 2 : 1) * N * K;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int n0 = blockIdx.x * BN;
    for (int i = threadIdx.x; i < BM; i += 256) rows[i] = i < nr ? (perm ? perm[r0 + i] / top : r0 + i) : -1;
    __syncthreads();
    float acc[4][4] = {}, acc2[DUAL ? 4 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            const int r = i / BK, k = i % BK;
            As[k][r] = (rows[r] >= 0 && k0 + k < K) ? ldf(A + (long long)rows[r] * lda + k0 + k) : 0.f;
            const bool in = n0 + r < N && k0 + k < K;
            Ws[0][k][r] = in ? ldf(We + (long long)(n0 + r) * K + k0 + k) : 0.f;
            if (DUAL) Ws[1][k][r] = in ? ldf(We + (long long)(N + n0 + r) * K + k0 + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], b[4], b2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                b[j] = Ws[0][k][tx * 4 + j];
                if (DUAL) b2[j] = Ws[1][k][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (DUAL) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < nr && n < N) {
                float y = acc[i][j];
                if (DUAL) y = y * sigmoidf_(y) * acc2[i][j];
                stf(Cm + (long long)(r0 + m) * ldc + n, y);
            }
        }
}

// Few rows per expert (decode): a warp owns one output column of one row tile and streams its weight row (DUAL: the gate
// and the up row) once in 16-byte pieces; the tile's rows come from L1 / L2, eight at a time.
template <typename T, typename TC, bool DUAL>
__global__ void __launch_bounds__(256)
grouped_rows_kernel(const T* __restrict__ A, long long lda, const int* __restrict__ perm, int top,
                    const T* __restrict__ W, TC* __restrict__ Cm, long long ldc, const int* __restrict__ tiles,
                    const int* __restrict__ meta, int N, int K, int vec_ok) {
    constexpr int MB = 8, VEC = 16 / (int)sizeof(T);
    if ((int)blockIdx.y >= meta[0]) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + warp;
    if (n >= N) return;
    const int ex = tiles[3 * blockIdx.y], r0 = tiles[3 * blockIdx.y + 1], nr = tiles[3 * blockIdx.y + 2];
    const T* w1 = W + ((long long)ex * (DUAL ? 2 : 1) * N + n) * K;
    const T* w2 = w1 + (long long)N * K;
    for (int m0 = 0; m0 < nr; m0 += MB) {
        const T* ar[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const int p = r0 + (m0 + m < nr ? m0 + m : nr - 1);
            ar[m] = A + (long long)(perm ? perm[p] / top : p) * lda;
        }
        float acc[MB], acc2[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[m] = acc2[m] = 0.f;
        int k0 = 0;
        if (vec_ok) {
            const int kv = K / VEC;
            for (int v = lane; v < kv; v += 32) {
                const uint4 wa = __ldcs(reinterpret_cast<const uint4*>(w1) + v);
                uint4 wb = wa;
                if (DUAL) wb = __ldcs(reinterpret_cast<const uint4*>(w2) + v);
                const T* pa = reinterpret_cast<const T*>(&wa);
                const T* pb = reinterpret_cast<const T*>(&wb);
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    if (m0 + m < nr) {
                        const uint4 av = __ldg(reinterpret_cast<const uint4*>(ar[m]) + v);
                        const T* px = reinterpret_cast<const T*>(&av);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) {
                            const float xv = ldf(px + e);
                            acc[m] = fmaf(xv, ldf(pa + e), acc[m]);
                            if (DUAL) acc2[m] = fmaf(xv, ldf(pb + e), acc2[m]);
                        }
                    }
                }
            }
            k0 = kv * VEC;
        }
        for (int k = k0 + lane; k < K; k += 32) {
            const float wa = ldf(w1 + k), wb = DUAL ? ldf(w2 + k) : 0.f;
#pragma unroll
            for (int m = 0; m < MB; ++m)
                if (m0 + m < nr) {
                    const float xv = ldf(ar[m] + k);
                    acc[m] = fmaf(xv, wa, acc[m]);
                    if (DUAL) acc2[m] = fmaf(xv, wb, acc2[m]);
                }
        }
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            float y = warp_sum(acc[m]);
            if (DUAL) {
                const float u = warp_sum(acc2[m]);
                y = y * sigmoidf_(y) * u;
            }
            if (lane == 0 && m0 + m < nr) stf(Cm + (long long)(r0 + m0 + m) * ldc + n, y);
        }
    }
}

// ------------------------------------------------------------------------------------------------ dense-GEMM route
// Large steps run each expert's rows through the framework's GEMM core instead: rows gathered into sorted order first,
// silu(gate) * up afterwards.
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, long long ldx, const int* __restrict__ perm, int top,
                                   T* __restrict__ xs, int C) {
    const long long p = blockIdx.x;
    const T* src = x + (long long)(perm[p] / top) * ldx;
    T* dst = xs + p * C;
    if ((C * (int)sizeof(T)) % 16 == 0 && (ldx * (long long)sizeof(T)) % 16 == 0) {
        const int nv = C * (int)sizeof(T) / 16;
        for (int i = threadIdx.x; i < nv; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = src[i];
    }
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ act, long long rows, int ff) {
    const long long n = rows * ff;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / ff;
        const int c = (int)(i % ff);
        const float g = ldf(gu + r * 2 * ff + c), u = ldf(gu + r * 2 * ff + ff + c);
        stf(act + i, g * sigmoidf_(g) * u);
    }
}

}  // namespace moe
}  // namespace llark

using namespace llark;
using namespace llark::moe;
typedef __nv_bfloat16 bf16_t;

extern "C" int llark_seq_moe_route(const float* logits, long long ld, int* ids, float* wts, int n_tok, int n_exp,
                                   int n_groups, int keep, int top, float scale, cudaStream_t st) {
    if (n_tok <= 0 || n_exp <= 0 || n_groups <= 0 || (n_exp % n_groups) || keep <= 0 || keep > n_groups || top <= 0 ||
        top > 32 || top > keep * (n_exp / n_groups) || !logits || !ids || !wts)
        return LLARK_EINVAL;
    const int nw = 4;
    const size_t smem = sizeof(float) * nw * (size_t)(n_exp + n_groups);
    if (smem > 48 * 1024) return LLARK_EINVAL;
    route_kernel<<<(n_tok + nw - 1) / nw, nw * 32, smem, st>>>(logits, ld, ids, wts, n_tok, n_exp, n_groups, keep, top,
                                                              scale);
    return check_launch();
}

extern "C" int llark_seq_moe_route_bias(const float* logits, long long ld, const float* correction, int* ids, float* wts,
                                        int n_tok, int n_exp, int n_groups, int keep, int top, float scale,
                                        cudaStream_t st) {
    if (n_tok <= 0 || n_exp <= 0 || n_groups <= 0 || (n_exp % n_groups) || keep <= 0 || keep > n_groups || top <= 0 ||
        top > 32 || top > keep * (n_exp / n_groups) || !logits || !ids || !wts)
        return LLARK_EINVAL;
    const int nw = 4;
    const size_t smem = sizeof(float) * nw * (size_t)(2 * n_exp + n_groups);
    if (smem > 48 * 1024) return LLARK_EINVAL;
    route_bias_kernel<<<(n_tok + nw - 1) / nw, nw * 32, smem, st>>>(logits, ld, correction, ids, wts, n_tok, n_exp,
                                                                   n_groups, keep, top, scale);
    return check_launch();
}

extern "C" int llark_seq_moe_tile_rows(void) { return kTileRows; }

extern "C" int llark_seq_moe_sort(const int* ids, int n_ent, int n_exp, int n_real, int* perm, int* pos_of, int* tiles,
                                  int* meta, int* seg_off, int* tiles256, cudaStream_t st) {
    if (n_ent <= 0 || n_exp <= 0 || n_real < 0 || n_real > n_exp || !ids || !perm || !pos_of || !tiles || !meta)
        return LLARK_EINVAL;
    const size_t smem = sizeof(int) * (3 * (size_t)n_exp + 1);
    if (smem > 48 * 1024) return LLARK_EINVAL;
    sort_kernel<<<1, 1024, smem, st>>>(ids, n_ent, n_exp, n_real, perm, pos_of, tiles, meta, seg_off, tiles256);
    return check_launch();
}

extern "C" int llark_seq_moe_up(const void* x, long long ldx, const int* perm, int top, const void* w_gate_up, void* act,
                                const int* tiles, const int* meta, int max_tiles, int n_ent, int ff, int K, int act_fp32,
                                cudaStream_t st) {
    if (max_tiles <= 0 || ff <= 0 || K <= 0 || top <= 0 || !x || !perm || !w_gate_up || !act || !tiles || !meta)
        return LLARK_EINVAL;
    if (n_ent <= kRowsRouteMaxEntries) {  // a handful of rows per expert: stream the weights once
        dim3 g2((ff + 7) / 8, max_tiles);
        const int esz = act_fp32 ? 4 : 2, vec = 16 / esz;
        const int vec_ok = (K % vec == 0) && (ldx % vec == 0) &&
                           (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_gate_up)) & 15) == 0);
        if (act_fp32)
            grouped_rows_kernel<float, float, true><<<g2, 256, 0, st>>>((const float*)x, ldx, perm, top,
                                                                        (const float*)w_gate_up, (float*)act, ff, tiles,
                                                                        meta, ff, K, vec_ok);
        else
            grouped_rows_kernel<bf16_t, bf16_t, true><<<g2, 256, 0, st>>>((const bf16_t*)x, ldx, perm, top,
                                                                          (const bf16_t*)w_gate_up, (bf16_t*)act, ff,
                                                                          tiles, meta, ff, K, vec_ok);
        return check_launch();
    }
    dim3 grid((ff + 63) / 64, max_tiles);
    if (act_fp32)
        grouped_linear_kernel<float, float, true><<<grid, 256, 0, st>>>((const float*)x, ldx, perm, top,
                                                                        (const float*)w_gate_up, (float*)act, ff, tiles,
                                                                        meta, ff, K);
    else
        grouped_linear_kernel<bf16_t, bf16_t, true><<<grid, 256, 0, st>>>((const bf16_t*)x, ldx, perm, top,
                                                                          (const bf16_t*)w_gate_up, (bf16_t*)act, ff,
                                                                          tiles, meta, ff, K);
    return check_launch();
}

extern "C" int llark_seq_moe_down(const void* act, const void* w_down, float* z, const int* tiles, const int* meta,
                                  int max_tiles, int n_ent, int C, int ff, int act_fp32, cudaStream_t st) {
    if (max_tiles <= 0 || ff <= 0 || C <= 0 || !act || !w_down || !z || !tiles || !meta) return LLARK_EINVAL;
    if (n_ent <= kRowsRouteMaxEntries) {
        dim3 g2((C + 7) / 8, max_tiles);
        const int esz = act_fp32 ? 4 : 2, vec = 16 / esz;
        const int vec_ok = (ff % vec == 0) &&
                           (((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(w_down)) & 15) == 0);
        if (act_fp32)
            grouped_rows_kernel<float, float, false><<<g2, 256, 0, st>>>((const float*)act, ff, nullptr, 1,
                                                                         (const float*)w_down, z, C, tiles, meta, C, ff,
                                                                         vec_ok);
        else
            grouped_rows_kernel<bf16_t, float, false><<<g2, 256, 0, st>>>((const bf16_t*)act, ff, nullptr, 1,
                                                                          (const bf16_t*)w_down, z, C, tiles, meta, C, ff,
                                                                          vec_ok);
        return check_launch();
    }
    dim3 grid((C + 63) / 64, max_tiles);
    if (act_fp32)
        grouped_linear_kernel<float, float, false><<<grid, 256, 0, st>>>((const float*)act, ff, nullptr, 1,
                                                                         (const float*)w_down, z, C, tiles, meta, C, ff);
    else
        grouped_linear_kernel<bf16_t, float, false><<<grid, 256, 0, st>>>((const bf16_t*)act, ff, nullptr, 1,
                                                                          (const bf16_t*)w_down, z, C, tiles, meta, C, ff);
    return check_launch();
}

extern "C" int llark_seq_moe_gather(const void* x, long long ldx, const int* perm, int top, void* xs, int n_ent, int C,
                                    int act_fp32, cudaStream_t st) {
    if (n_ent <= 0 || C <= 0 || top <= 0 || !x || !perm || !xs) return LLARK_EINVAL;
    if (act_fp32)
        gather_rows_kernel<float><<<n_ent, 128, 0, st>>>((const float*)x, ldx, perm, top, (float*)xs, C);
    else
        gather_rows_kernel<bf16_t><<<n_ent, 128, 0, st>>>((const bf16_t*)x, ldx, perm, top, (bf16_t*)xs, C);
    return check_launch();
}

extern "C" int llark_seq_silu_mul(const void* gu, void* act, long long rows, int ff, int act_fp32, cudaStream_t st) {
    if (rows <= 0 || ff <= 0 || !gu || !act) return LLARK_EINVAL;
    const long long n = rows * ff;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (act_fp32)
        silu_mul_kernel<float><<<grid, 256, 0, st>>>((const float*)gu, (float*)act, rows, ff);
    else
        silu_mul_kernel<bf16_t><<<grid, 256, 0, st>>>((const bf16_t*)gu, (bf16_t*)act, rows, ff);
    return check_launch();
}
