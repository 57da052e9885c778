// Sequence mixers of the generation path for layer-list decoders, on the packed-step layout of seq_ops.cu (tok_seq, cu,
// pos0, slot). Every mixer keeps its per-request memory in a store indexed by slot, reads what earlier steps left there
// and leaves what later steps need, so a whole prompt, a portion of one and a single decoded token are the same launch.
//
//   llark_seq_qk_headnorm   per-head RMS norm of the q and k columns of a fused projection; the raw k is kept as well
//                           (designs whose values are the un-normed keys); optionally writes the ring directly (decode)
//   llark_seq_qkv_rotary    optional whole-projection RMS norm of q and k, rotary positions on q / k (halves or interleaved
//                           pairs, partial head) and optionally on the values; optionally writes the rings (decode)
//   llark_seq_swa_attn      softmax attention over a sliding window (or the query's block of `chunk` positions; scores
//                           optionally squashed by cap * tanh(s / cap); weighted value sums optionally turned back by the
//                           query's position): keys of this step from the step's buffers, older
//                           ones from the per-slot ring of the last `cap` positions; per-head score scale; optional
//                           sigmoid output gate; scores, softmax and accumulation in fp32
//   llark_seq_kv_ring_write stores the step's keys / values into the ring (after attention has read the old entries)
//   llark_seq_glr_scan      gated linear recurrence S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t with
//                           f = low + (1 - low) * sigmoid(f_pre), q = silu(q_pre); fp32 state [slot, H, D, E]; long
//                           prompts run as chunks in three passes (local states, llark_seq_glr_combine, outputs)
//   llark_seq_head_rmsnorm  per-head RMS norm of the recurrence's output
#include "common.cuh"

namespace llark {
extern thread_local int g_last_cuda_error;
namespace seqmix {

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

// ------------------------------------------------------------------------------------------------ q / k head norm
// src [n_tok, ld] fp32 with q heads at column q_off, k heads at k_off and the values' source at v_off (E per key / value
// head; v_off = k_off with E = D makes the un-normed keys the values). Warp per (token, head). temp_every > 0: the query
// is also multiplied by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) at position p of its sequence.
template <typename T>
__global__ void qk_headnorm_kernel(const float* __restrict__ src, long long ld, int q_off, int k_off, int v_off,
                                   const float* __restrict__ wq, const float* __restrict__ wk, T* __restrict__ qn,
                                   T* __restrict__ kn, T* __restrict__ vraw, T* __restrict__ kring, T* __restrict__ vring,
                                   const int* __restrict__ tok_seq, const int* __restrict__ cu,
                                   const int* __restrict__ pos0, const int* __restrict__ slot, int H, int G, int D, int E,
                                   int cap, float eps, float temp_coef, int temp_every) {
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int hh = warp; hh < H + G; hh += nw) {
        const bool is_q = hh < H;
        const int head = is_q ? hh : hh - H;
        const float* s = src + (long long)t * ld + (is_q ? q_off : k_off) + head * D;
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) ss = fmaf(s[d], s[d], ss);
        ss = warp_sum(ss);
        float r = 1.0f / sqrtf(ss / (float)D + eps);
        const float* w = is_q ? wq : wk;
        if (is_q) {
            if (temp_every > 0) {
                const int b = tok_seq[t];
                const long long p = pos0[b] + (t - cu[b]);
                r *= 1.0f + temp_coef * logf((float)((p + 1) / temp_every) + 1.0f);
            }
            T* o = qn + ((long long)t * H + head) * D;
            for (int d = lane; d < D; d += 32) stf(o + d, s[d] * r * w[d]);
        } else {
            const float* sv = src + (long long)t * ld + v_off + head * E;
            T* o = kn + ((long long)t * G + head) * D;
            T* ov = vraw + ((long long)t * G + head) * E;
            T *rk = nullptr, *rv = nullptr;
            if (kring) {  // one token per request: the entry it replaces is already outside the window
                const int b = tok_seq[t];
                const long long p = pos0[b] + (t - cu[b]);
                const long long e = ((long long)slot[b] * cap + (p % cap)) * G + head;
                rk = kring + e * D;
                rv = vring + e * E;
            }
            for (int d = lane; d < D; d += 32) {
                const float kv = s[d] * r * w[d];
                stf(o + d, kv);
                if (rk) stf(rk + d, kv);
            }
            for (int d = lane; d < E; d += 32) {
                stf(ov + d, sv[d]);
                if (rv) stf(rv + d, sv[d]);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ q / k / v with rotary positions
// src [n_tok, ld] fp32 with q heads (H x D) at q_off, k heads (G x D) at k_off, v heads (G x E) at v_off. Block per token.
//   wq / wk (optional): RMS norm over the WHOLE q (H*D numbers) and the whole k (G*D) projection, weights of that size
//   qk_freq [n_rot / 2] (optional): the first n_rot entries of every q and k head are rotated by position * qk_freq[i];
//            pair i = (i, i + n_rot/2) ("halves") or (2i, 2i+1) (qk_interleaved); the rest of the head passes
//   v_freq [E / 2] (optional): every value head is rotated by its position the same way over all of E (v_interleaved);
//            the attention kernels turn their weighted sums back by the query's position
// Angles are float(position) * frequency, cos / sin in fp32. Results in T; with kring / vring the k / v rows also go to
// ring entry position % cap of the token's slot (steps of one token per request).
template <typename T>
__global__ void qkv_rotary_kernel(const float* __restrict__ src, long long ld, int q_off, int k_off, int v_off,
                                  const float* __restrict__ wq, const float* __restrict__ wk,
                                  const float* __restrict__ qk_freq, int n_rot, int qk_interleaved,
                                  const float* __restrict__ v_freq, int v_interleaved, T* __restrict__ qn,
                                  T* __restrict__ kn, T* __restrict__ vv, T* __restrict__ kring, T* __restrict__ vring,
                                  const int* __restrict__ tok_seq, const int* __restrict__ cu,
                                  const int* __restrict__ pos0, const int* __restrict__ slot, int H, int G, int D, int E,
                                  int cap, float eps) {
    extern __shared__ float cs[];  // cos | sin of the q / k pairs [2 * (n_rot / 2)], then of the value pairs [2 * (E / 2)]
    __shared__ float red[2][32];
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    const long long p = pos0[b] + (t - cu[b]);
    const int hq = n_rot >> 1, hv = v_freq ? (E >> 1) : 0;
    float* csv = cs + 2 * hq;
    for (int i = threadIdx.x; i < hq; i += blockDim.x) sincosf((float)p * qk_freq[i], &cs[2 * i + 1], &cs[2 * i]);
    for (int i = threadIdx.x; i < hv; i += blockDim.x) sincosf((float)p * v_freq[i], &csv[2 * i + 1], &csv[2 * i]);
    const float* row = src + (long long)t * ld;
    float rq = 1.f, rk = 1.f;
    if (wq) {  // wk comes with it
        float sq = 0.f, sk = 0.f;
        for (int c = threadIdx.x; c < H * D; c += blockDim.x) sq = fmaf(row[q_off + c], row[q_off + c], sq);
        for (int c = threadIdx.x; c < G * D; c += blockDim.x) sk = fmaf(row[k_off + c], row[k_off + c], sk);
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
        if (l == 0) {
            red[0][w] = sq;
            red[1][w] = sk;
        }
        __syncthreads();
        sq = sk = 0.f;
        for (int i = 0; i < nw; ++i) {
            sq += red[0][i];
            sk += red[1][i];
        }
        rq = 1.0f / sqrtf(sq / (float)(H * D) + eps);
        rk = 1.0f / sqrtf(sk / (float)(G * D) + eps);
    } else {
        __syncthreads();
    }
    T *rk_row = nullptr, *rv_row = nullptr;
    if (kring) {
        const long long e = (long long)slot[b] * cap + (p % cap);
        rk_row = kring + e * G * D;
        rv_row = vring + e * G * E;
    }
    // q and k heads: hh < H is a query head, the others key heads
    const int per_head = hq + (D - 2 * hq);  // work items of a head: its pairs, then the entries that pass
    for (int i = threadIdx.x; i < (H + G) * per_head; i += blockDim.x) {
        const int hh = i / per_head, j = i % per_head;
        const bool is_q = hh < H;
        const int head = is_q ? hh : hh - H;
        const int c0 = head * D;
        const float* s = row + (is_q ? q_off : k_off) + c0;
        const float* w = is_q ? wq : wk;
        const float r = is_q ? rq : rk;
        T* o = is_q ? qn + (long long)t * H * D + c0 : kn + (long long)t * G * D + c0;
        T* o2 = (!is_q && rk_row) ? rk_row + c0 : nullptr;
        if (j < hq) {
            const int iu = qk_interleaved ? 2 * j : j, iv = qk_interleaved ? 2 * j + 1 : j + hq;
            float u = s[iu] * r, v = s[iv] * r;
            if (w) {
                u *= w[c0 + iu];
                v *= w[c0 + iv];
            }
            const float co = cs[2 * j], si = cs[2 * j + 1];
            const float a = u * co - v * si, bb = v * co + u * si;
            stf(o + iu, a);
            stf(o + iv, bb);
            if (o2) {
                stf(o2 + iu, a);
                stf(o2 + iv, bb);
            }
        } else {
            const int c = 2 * hq + (j - hq);
            float u = s[c] * r;
            if (w) u *= w[c0 + c];
            stf(o + c, u);
            if (o2) stf(o2 + c, u);
        }
    }
    // value heads
    const int per_v = v_freq ? hv + (E - 2 * hv) : E;
    for (int i = threadIdx.x; i < G * per_v; i += blockDim.x) {
        const int head = i / per_v, j = i % per_v;
        const int c0 = head * E;
        const float* s = row + v_off + c0;
        T* o = vv + (long long)t * G * E + c0;
        T* o2 = rv_row ? rv_row + c0 : nullptr;
        if (j < hv) {
            const int iu = v_interleaved ? 2 * j : j, iv = v_interleaved ? 2 * j + 1 : j + hv;
            const float u = s[iu], v = s[iv];
            const float co = csv[2 * j], si = csv[2 * j + 1];
            const float a = u * co - v * si, bb = v * co + u * si;
            stf(o + iu, a);
            stf(o + iv, bb);
            if (o2) {
                stf(o2 + iu, a);
                stf(o2 + iv, bb);
            }
        } else {
            const int c = v_freq ? 2 * hv + (j - hv) : j;
            stf(o + c, s[c]);
            if (o2) stf(o2 + c, s[c]);
        }
    }
}

template <typename T> __device__ __forceinline__ void st_quad(T* p, const float (&v)[4]);
template <> __device__ __forceinline__ void st_quad<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void st_quad<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
    uint2 u;
    u.x = pack_bf16x2(v[0], v[1]);
    u.y = pack_bf16x2(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = u;
}

// One head of n entries of which the first r are rotated, four entries at a time (16-byte loads, 16- / 8-byte stores).
// Work item j of the head: interleaved pairs -> entries 4j .. 4j+3 (two pairs when inside the rotated zone); halves ->
// entries 4j .. 4j+3 of the first half together with their partners r/2 + 4j .., then the entries behind the zone.
// s: source row of the head; scale r_; w: norm weights of the head or NULL; cs: cos | sin per pair; o / o2: destinations.
template <typename T>
__device__ __forceinline__ void rotate_quads(const float* __restrict__ s, float r_, const float* __restrict__ w,
                                             const float* __restrict__ cs, int r, int interleaved, int j,
                                             T* __restrict__ o, T* __restrict__ o2) {
    auto load = [&](int c, float (&v)[4]) {
        const float4 a = *reinterpret_cast<const float4*>(s + c);
        v[0] = a.x * r_, v[1] = a.y * r_, v[2] = a.z * r_, v[3] = a.w * r_;
        if (w) {
            const float4 b = *reinterpret_cast<const float4*>(w + c);
            v[0] *= b.x, v[1] *= b.y, v[2] *= b.z, v[3] *= b.w;
        }
    };
    auto store = [&](int c, const float (&v)[4]) {
        st_quad(o + c, v);
        if (o2) st_quad(o2 + c, v);
    };
    float a[4], b[4];
    if (interleaved) {
        const int c = 4 * j;
        load(c, a);
        if (c < r) {
            const int p0 = c >> 1;
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const float co = cs[2 * (p0 + k)], si = cs[2 * (p0 + k) + 1];
                const float u = a[2 * k], v = a[2 * k + 1];
                a[2 * k] = u * co - v * si;
                a[2 * k + 1] = v * co + u * si;
            }
        }
        store(c, a);
        return;
    }
    const int hq = r >> 1, nq = hq >> 2;  // quads in the first half of the zone
    if (j < nq) {
        load(4 * j, a);
        load(hq + 4 * j, b);
        float ua[4], vb[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float co = cs[2 * (4 * j + k)], si = cs[2 * (4 * j + k) + 1];
            ua[k] = a[k] * co - b[k] * si;
            vb[k] = b[k] * co + a[k] * si;
        }
        store(4 * j, ua);
        store(hq + 4 * j, vb);
    } else {
        const int c = r + 4 * (j - nq);
        load(c, a);
        store(c, a);
    }
}

// The same as qkv_rotary_kernel for sizes and addresses that allow four entries per access (checked by the launcher).
template <typename T>
__global__ void qkv_rotary4_kernel(const float* __restrict__ src, long long ld, int q_off, int k_off, int v_off,
                                   const float* __restrict__ wq, const float* __restrict__ wk,
                                   const float* __restrict__ qk_freq, int n_rot, int qk_interleaved,
                                   const float* __restrict__ v_freq, int v_interleaved, T* __restrict__ qn,
                                   T* __restrict__ kn, T* __restrict__ vv, T* __restrict__ kring, T* __restrict__ vring,
                                   const int* __restrict__ tok_seq, const int* __restrict__ cu,
                                   const int* __restrict__ pos0, const int* __restrict__ slot, int H, int G, int D, int E,
                                   int cap, float eps) {
    extern __shared__ float cs[];
    __shared__ float red[2][32];
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    const long long p = pos0[b] + (t - cu[b]);
    const int hq = n_rot >> 1, hv = v_freq ? (E >> 1) : 0;
    float* csv = cs + 2 * hq;
    for (int i = threadIdx.x; i < hq; i += blockDim.x) sincosf((float)p * qk_freq[i], &cs[2 * i + 1], &cs[2 * i]);
    for (int i = threadIdx.x; i < hv; i += blockDim.x) sincosf((float)p * v_freq[i], &csv[2 * i + 1], &csv[2 * i]);
    const float* row = src + (long long)t * ld;
    float rq = 1.f, rk = 1.f;
    if (wq) {
        float sq = 0.f, sk = 0.f;
        for (int c = threadIdx.x; c < (H * D) >> 2; c += blockDim.x) {
            const float4 a = reinterpret_cast<const float4*>(row + q_off)[c];
            sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
        for (int c = threadIdx.x; c < (G * D) >> 2; c += blockDim.x) {
            const float4 a = reinterpret_cast<const float4*>(row + k_off)[c];
            sk += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
        if (l == 0) {
            red[0][w] = sq;
            red[1][w] = sk;
        }
        __syncthreads();
        sq = sk = 0.f;
        for (int i = 0; i < nw; ++i) {
            sq += red[0][i];
            sk += red[1][i];
        }
        rq = 1.0f / sqrtf(sq / (float)(H * D) + eps);
        rk = 1.0f / sqrtf(sk / (float)(G * D) + eps);
    } else {
        __syncthreads();
    }
    T *rk_row = nullptr, *rv_row = nullptr;
    if (kring) {
        const long long e = (long long)slot[b] * cap + (p % cap);
        rk_row = kring + e * G * D;
        rv_row = vring + e * G * E;
    }
    const int iq = qk_interleaved ? D >> 2 : (hq >> 2) + ((D - n_rot) >> 2);  // work items of a q / k head
    const int rv = v_freq ? E : 0;
    const int iv = (v_interleaved || !v_freq) ? E >> 2 : (E >> 3);             // of a value head (halves: all of E rotates)
    const int n_qk = (H + G) * iq;
    for (int i = threadIdx.x; i < n_qk + G * iv; i += blockDim.x) {
        if (i < n_qk) {
            const int hh = i / iq, j = i - hh * iq;
            const bool is_q = hh < H;
            const int c0 = (is_q ? hh : hh - H) * D;
            const float* w = is_q ? wq : wk;
            rotate_quads<T>(row + (is_q ? q_off : k_off) + c0, is_q ? rq : rk, w ? w + c0 : nullptr, cs, n_rot,
                            qk_interleaved, j, is_q ? qn + (long long)t * H * D + c0 : kn + (long long)t * G * D + c0,
                            (!is_q && rk_row) ? rk_row + c0 : (T*)nullptr);
        } else {
            const int head = (i - n_qk) / iv, j = (i - n_qk) - head * iv;
            const int c0 = head * E;
            rotate_quads<T>(row + v_off + c0, 1.f, nullptr, csv, rv, v_interleaved, j, vv + (long long)t * G * E + c0,
                            rv_row ? rv_row + c0 : (T*)nullptr);
        }
    }
}

// N consecutive elements -> float, with one 4 / 8 / 16-byte load per piece when `vec` (the address is then aligned to
// the piece); scalar loads otherwise.
template <typename T, int N>
__device__ __forceinline__ void load_run(const T* p, float (&out)[N], bool vec) {
    constexpr int BYTES = N * (int)sizeof(T);
    if (vec && BYTES >= 4) {
        constexpr int PIECE = BYTES >= 16 ? 16 : BYTES;  // N is a power of two here
        constexpr int PER = PIECE / (int)sizeof(T);
#pragma unroll
        for (int i = 0; i < N; i += PER) {
            if constexpr (PIECE == 16) {
                const uint4 v = *reinterpret_cast<const uint4*>(p + i);
                const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
                for (int j = 0; j < PER; ++j) out[i + j] = ldf(e + j);
            } else if constexpr (PIECE == 8) {
                const uint2 v = *reinterpret_cast<const uint2*>(p + i);
                const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
                for (int j = 0; j < PER; ++j) out[i + j] = ldf(e + j);
            } else {
                const uint32_t v = *reinterpret_cast<const uint32_t*>(p + i);
                const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
                for (int j = 0; j < PER; ++j) out[i + j] = ldf(e + j);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = ldf(p + i);
    }
}

// ------------------------------------------------------------------------------------------------ windowed attention
// Block per (token, head); its warps take the 32-key tiles of the window round-robin, each with its own online softmax,
// and are merged at the end. Lane = key while scoring (the key row is read in 16-byte pieces when it is aligned),
// lane = DPL adjacent output channels while accumulating (one load of DPL elements per key when E = 32 * DPL; channels
// lane + 32 i otherwise). DPL = ceil(E / 32) rounded up to a power of two.
template <typename T, int DPL>
__global__ void swa_attn_kernel(const T* __restrict__ qn, const T* __restrict__ kn, const T* __restrict__ vv,
                                const T* __restrict__ kring, const T* __restrict__ vring, const float* __restrict__ gate,
                                long long gate_ld, const float* __restrict__ scale_h, T* __restrict__ out,
                                const int* __restrict__ tok_seq, const int* __restrict__ cu,
                                const int* __restrict__ pos0, const int* __restrict__ slot, int H, int G, int D, int E,
                                int window, int cap, int from_ring_only, const float* __restrict__ sink,
                                int gate_per_head, int chunk, float softcap, const float* __restrict__ vfreq,
                                int v_interleaved) {
    extern __shared__ float sm[];
    const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* sq = sm;                      // [D]
    float* sp = sq + D;                  // [nw][32]
    float* sm_m = sp + nw * 32;          // [nw]
    float* sm_l = sm_m + nw;             // [nw]
    float* sacc = sm_l + nw;             // [nw][E]
    const int t = blockIdx.x, h = blockIdx.y;
    const int g = h / (H / G);
    const int b = tok_seq[t];
    const long long p0 = pos0[b];
    const long long p = p0 + (t - cu[b]);
    // first visible key: the start of the query's block of `chunk` positions (blocks counted from position 0), or the
    // start of the sliding window
    const long long lo = chunk > 0 ? (p / chunk) * chunk : (p - window + 1 > 0 ? p - window + 1 : 0);
    const int nkeys = (int)(p - lo + 1);
    const float sc = scale_h[h];
    for (int d = threadIdx.x; d < D; d += blockDim.x) sq[d] = ldf(qn + ((long long)t * H + h) * D + d);
    __syncthreads();
    const long long ring_base = (long long)slot[b] * cap;
    const int row_b = cu[b];
    const int ring0 = (int)(lo % cap);  // ring entry of the window's first key; key jj sits at ring0 + jj (- cap), as
                                        // the keys of a window never outnumber the ring's entries
    const long long first_here = from_ring_only ? p + 1 : p0;  // positions >= first_here are rows of this step
    constexpr int KV = 16 / (int)sizeof(T);  // elements of a 16-byte piece of a key row
    const bool kvec = (D % KV) == 0;         // rows then start on 16-byte boundaries (torch allocations are 256-byte aligned)
    const bool vvec = DPL > 1 && E == 32 * DPL;
    float m = -INFINITY, l = 0.f, acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
    for (int tile = warp; tile * 32 < nkeys; tile += nw) {
        const int jj = tile * 32 + lane;
        const long long j = lo + jj;
        float s = -INFINITY;
        if (jj < nkeys) {
            int ridx = ring0 + jj;
            if (ridx >= cap) ridx -= cap;
            const T* kr = j >= first_here ? kn + ((long long)(row_b + (j - p0)) * G + g) * D
                                          : kring + ((ring_base + ridx) * G + g) * D;
            float dot = 0.f;
            if (kvec) {
                // eight 16-byte pieces of the key row in flight at a time: every lane reads a row of its own, so a piece
                // is a trip to L2 and the loop is bound by how many of them overlap. The raw pieces wait in registers.
                int d = 0;
                for (; d + 8 * KV <= D; d += 8 * KV) {
                    uint4 raw[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) raw[u] = *reinterpret_cast<const uint4*>(kr + d + u * KV);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
                        for (int x = 0; x < KV; ++x) dot = fmaf(sq[d + u * KV + x], ldf(e + x), dot);
                    }
                }
                for (; d < D; d += KV) {
                    float kk[KV];
                    load_run<T, KV>(kr + d, kk, true);
#pragma unroll
                    for (int x = 0; x < KV; ++x) dot = fmaf(sq[d + x], kk[x], dot);
                }
            } else {
                for (int d = 0; d < D; ++d) dot = fmaf(sq[d], ldf(kr + d), dot);
            }
            s = dot * sc;
            if (softcap > 0.f) s = softcap * tanhf(s / softcap);
        }
        const float mt = warp_max(s);
        const float mn = fmaxf(m, mt);
        const float corr = expf(m - mn);  // m = -inf on the first tile: exp(-inf) = 0
        const float pj = jj < nkeys ? expf(s - mn) : 0.f;
        l = l * corr + warp_sum(pj);
        m = mn;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] *= corr;
        sp[warp * 32 + lane] = pj;
        __syncwarp();
        const int cnt = nkeys - tile * 32 < 32 ? nkeys - tile * 32 : 32;
        auto value_row = [&](int k) -> const T* {
            const long long j2 = lo + tile * 32 + k;
            int ridx = ring0 + tile * 32 + k;
            if (ridx >= cap) ridx -= cap;
            return j2 >= first_here ? vv + ((long long)(row_b + (j2 - p0)) * G + g) * E
                                    : vring + ((ring_base + ridx) * G + g) * E;
        };
        int k = 0;
        if (vvec) {
            // the rows of eight keys are requested before the first is used: one trip to L2 per batch, not per key
            constexpr int VB = DPL <= 4 ? 8 : 4;
            for (; k + VB <= cnt; k += VB) {
                float vx[VB][DPL];
#pragma unroll
                for (int u = 0; u < VB; ++u) load_run<T, DPL>(value_row(k + u) + lane * DPL, vx[u], true);
#pragma unroll
                for (int u = 0; u < VB; ++u) {
                    const float pk = sp[warp * 32 + k + u];
#pragma unroll
                    for (int i = 0; i < DPL; ++i) acc[i] = fmaf(pk, vx[u][i], acc[i]);
                }
            }
        }
        for (; k < cnt; ++k) {
            const T* vr = value_row(k);
            const float pk = sp[warp * 32 + k];
            if (vvec) {
                float vx[DPL];
                load_run<T, DPL>(vr + lane * DPL, vx, true);
#pragma unroll
                for (int i = 0; i < DPL; ++i) acc[i] = fmaf(pk, vx[i], acc[i]);
            } else {
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const int e = lane + 32 * i;
                    if (e < E) acc[i] = fmaf(pk, ldf(vr + e), acc[i]);
                }
            }
        }
        __syncwarp();
    }
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int e = vvec ? lane * DPL + i : lane + 32 * i;
        if (e < E) sacc[warp * E + e] = acc[i];
    }
    __syncthreads();
    float mm = sink ? sink[h] : -INFINITY;  // a sink is one more term exp(sink_h) of the denominator, with no value
    for (int w = 0; w < nw; ++w) mm = fmaxf(mm, sm_m[w]);
    float lt = sink ? expf(sink[h] - mm) : 0.f;
    for (int w = 0; w < nw; ++w) lt += sm_m[w] == -INFINITY ? 0.f : sm_l[w] * expf(sm_m[w] - mm);
    if (!vfreq) {
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            float o = 0.f;
            for (int w = 0; w < nw; ++w)
                if (sm_m[w] != -INFINITY) o = fmaf(sacc[w * E + e], expf(sm_m[w] - mm), o);
            o /= lt;
            if (gate) o *= sigmoidf_(gate[(long long)t * gate_ld + (gate_per_head ? h : h * E + e)]);
            stf(out + ((long long)t * H + h) * E + e, o);
        }
        return;
    }
    // Values were stored rotated by their own position: the weighted sum is turned back by the query's position, pair m
    // by -p * vfreq[m], before the gate. The normalised row passes through shared memory (E more floats behind sacc).
    float* so = sacc + nw * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < nw; ++w)
            if (sm_m[w] != -INFINITY) o = fmaf(sacc[w * E + e], expf(sm_m[w] - mm), o);
        so[e] = o / lt;
    }
    __syncthreads();
    const int half = E >> 1;
    for (int mpair = threadIdx.x; mpair < half; mpair += blockDim.x) {
        const int iu = v_interleaved ? 2 * mpair : mpair, iv = v_interleaved ? 2 * mpair + 1 : mpair + half;
        float si, co;
        sincosf((float)p * vfreq[mpair], &si, &co);
        const float u = so[iu], v = so[iv];
        float a = u * co + v * si, bb = v * co - u * si;  // rotation by the negative angle
        if (gate) {
            a *= sigmoidf_(gate[(long long)t * gate_ld + (gate_per_head ? h : h * E + iu)]);
            bb *= sigmoidf_(gate[(long long)t * gate_ld + (gate_per_head ? h : h * E + iv)]);
        }
        stf(out + ((long long)t * H + h) * E + iu, a);
        stf(out + ((long long)t * H + h) * E + iv, bb);
    }
    if ((E & 1) && threadIdx.x == 0) {  // an odd last channel has no partner and passes
        float o = so[E - 1];
        if (gate) o *= sigmoidf_(gate[(long long)t * gate_ld + (gate_per_head ? h : h * E + E - 1)]);
        stf(out + ((long long)t * H + h) * E + E - 1, o);
    }
}

template <typename T>
__global__ void kv_ring_write_kernel(const T* __restrict__ kn, const T* __restrict__ vv, T* __restrict__ kring,
                                     T* __restrict__ vring, const int* __restrict__ tok_seq,
                                     const int* __restrict__ cu, const int* __restrict__ pos0,
                                     const int* __restrict__ slot, int GD, int GE, int cap) {
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    const int local = t - cu[b], n = cu[b + 1] - cu[b];
    if (n - 1 - local >= cap) return;  // an older row of this step that a later one replaces
    const long long p = pos0[b] + local;
    const long long e = (long long)slot[b] * cap + (p % cap);
    for (int d = threadIdx.x; d < GD; d += blockDim.x) kring[e * GD + d] = kn[(long long)t * GD + d];
    if (vring)  // keys that are their own values keep one ring
        for (int d = threadIdx.x; d < GE; d += blockDim.x) vring[e * GE + d] = vv[(long long)t * GE + d];
}

// ------------------------------------------------------------------------------------------------ gated linear recurrence
// Block per (E-slice, head, request). Thread (ec, r) owns rows d = r * DPT .. r * DPT + DPT - 1 of column e of S in
// registers; R threads (adjacent lanes) share a column and add their partial outputs by shuffle. The inputs of TS steps
// are brought to shared memory with cp.async while the previous TS steps are computed, and the gate arithmetic is done
// once per element there.
constexpr int kTS = 8;  // steps per stage: two stages of a 128-wide head stay under 32 KB, six CTAs per SM

__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// A work item is a run of consecutive rows of one request: the whole step of the request (one pass: init = final = its
// slot of the state store), or one chunk of a long prompt (three passes, see llark_seq_glr_scan). item_init / item_final
// index init_buf / final_buf ([*, H, D, E]); -1 = start from zero / keep nothing. decay_buf (optional) [items, H, D]
// receives the product of the item's forget gates per channel; o_raw may be NULL (no outputs wanted).
template <int DPT, int EC, bool OUT>
__global__ void glr_scan_kernel(const float* __restrict__ src, long long ld, int q_off, int f_off, int v_off,
                                const float* __restrict__ lower, const float* __restrict__ init_buf,
                                float* __restrict__ final_buf, float* __restrict__ decay_buf, float* __restrict__ o_raw,
                                const int* __restrict__ item_row0, const int* __restrict__ item_n,
                                const int* __restrict__ item_init, const int* __restrict__ item_final, int H, int D,
                                int E, int R, int ecols) {
    extern __shared__ __align__(16) float sm[];
    constexpr int DPS = DPT + 4;  // padded row-group stride: 16-byte reads of the R groups of a column hit different banks
    const int DP = R * DPS;
    const int stage_floats = kTS * (3 * DP + ecols);
    const int h = blockIdx.y, b = blockIdx.z;
    const int r = threadIdx.x % R, ec = threadIdx.x / R;
    const int e0 = blockIdx.x * ecols + ec * EC;  // this thread's EC adjacent columns: a DPT x EC tile of S in registers
    const int row0 = item_row0[b], n = item_n[b];
    const int i_init = item_init[b], i_final = item_final[b];
    const float* st_in = i_init >= 0 ? init_buf + ((long long)i_init * H + h) * (long long)D * E : nullptr;
    float S[DPT][EC];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = r * DPT + i;
#pragma unroll
        for (int c = 0; c < EC; ++c) S[i][c] = (st_in && d < D && e0 + c < E) ? st_in[(long long)d * E + e0 + c] : 0.f;
    }
    const bool want_decay = decay_buf != nullptr && blockIdx.x == 0;
    float decay[8];  // rows threadIdx.x + k * blockDim.x (8 * 32 >= the widest padded head)
#pragma unroll
    for (int k = 0; k < 8; ++k) decay[k] = 1.f;
    const int nstage = (n + kTS - 1) / kTS;
    // stage layout: q[kTS][DP] | f[kTS][DP] | g[kTS][DP] | v[kTS][ecols]; raw q_pre / f_pre land in q / f
    auto issue = [&](int s, float* buf) {
        const int steps = n - s * kTS < kTS ? n - s * kTS : kTS;
        for (int ts = 0; ts < steps; ++ts) {
            const float* rowp = src + (long long)(row0 + s * kTS + ts) * ld;
            for (int d = threadIdx.x; d < D; d += blockDim.x) {
                const int at = ts * DP + (d / DPT) * DPS + (d % DPT);
                cp_async4(buf + at, rowp + q_off + h * D + d);
                cp_async4(buf + kTS * DP + at, rowp + f_off + h * D + d);
            }
            for (int c = threadIdx.x; c < ecols; c += blockDim.x) {
                const int ee = blockIdx.x * ecols + c;
                if (ee < E) cp_async4(buf + 3 * kTS * DP + ts * ecols + c, rowp + v_off + h * E + ee);
            }
        }
        cp_async_commit();
    };
    if (nstage > 0) issue(0, sm);
    for (int s = 0; s < nstage; ++s) {
        float* buf = sm + (s & 1) * stage_floats;
        const int steps = n - s * kTS < kTS ? n - s * kTS : kTS;
        cp_async_wait_all();
        __syncthreads();  // stage s has landed; everybody is done computing stage s - 1 (the other buffer)
        if (s + 1 < nstage) issue(s + 1, sm + ((s + 1) & 1) * stage_floats);
        for (int d = threadIdx.x; d < R * DPT; d += blockDim.x) {
            const float lowv = (lower && d < D) ? lower[h * D + d] : 0.f;
            for (int ts = 0; ts < steps; ++ts) {
                const int at = ts * DP + (d / DPT) * DPS + (d % DPT);
                float q = 0.f, f = 0.f, g = 0.f;  // padded rows: nothing kept, nothing written, nothing read out
                if (d < D) {
                    const float qp = buf[at], fp = buf[kTS * DP + at];
                    q = qp * sigmoidf_(qp);
                    f = lowv + (1.0f - lowv) * sigmoidf_(fp);
                    g = 1.0f - f;
                }
                buf[at] = q;
                buf[kTS * DP + at] = f;
                buf[2 * kTS * DP + at] = g;
            }
        }
        __syncthreads();
        if (want_decay) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int d = threadIdx.x + k * blockDim.x;
                if (d < D)
                    for (int ts = 0; ts < steps; ++ts) decay[k] *= buf[kTS * DP + ts * DP + (d / DPT) * DPS + (d % DPT)];
            }
        }
        for (int ts = 0; ts < steps; ++ts) {
            float vt[EC], part[EC];
#pragma unroll
            for (int c = 0; c < EC; ++c) {
                vt[c] = e0 + c < E ? buf[3 * kTS * DP + ts * ecols + ec * EC + c] : 0.f;
                part[c] = 0.f;
            }
            const float4* q4 = reinterpret_cast<const float4*>(buf + ts * DP + r * DPS);
            const float4* f4 = reinterpret_cast<const float4*>(buf + kTS * DP + ts * DP + r * DPS);
            const float4* g4 = reinterpret_cast<const float4*>(buf + 2 * kTS * DP + ts * DP + r * DPS);
#pragma unroll
            for (int i4 = 0; i4 < DPT / 4; ++i4) {
                const float4 fv = f4[i4], gv = g4[i4];  // read once, used for all EC columns
                float4 qv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (OUT) qv = q4[i4];
                const float fa[4] = {fv.x, fv.y, fv.z, fv.w}, ga[4] = {gv.x, gv.y, gv.z, gv.w},
                            qa[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int c = 0; c < EC; ++c) {
                        S[i4 * 4 + j][c] = fmaf(fa[j], S[i4 * 4 + j][c], ga[j] * vt[c]);
                        if (OUT) part[c] = fmaf(S[i4 * 4 + j][c], qa[j], part[c]);
                    }
            }
            if (OUT) {
#pragma unroll
                for (int c = 0; c < EC; ++c) {
                    for (int o = R >> 1; o > 0; o >>= 1) part[c] += __shfl_xor_sync(0xffffffffu, part[c], o);
                    if (r == 0 && e0 + c < E)
                        o_raw[(long long)(row0 + s * kTS + ts) * ((long long)H * E) + h * E + e0 + c] = part[c];
                }
            }
        }
    }
    if (i_final >= 0) {
        float* st_out = final_buf + ((long long)i_final * H + h) * (long long)D * E;
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = r * DPT + i;
#pragma unroll
            for (int c = 0; c < EC; ++c)
                if (d < D && e0 + c < E) st_out[(long long)d * E + e0 + c] = S[i][c];
        }
    }
    if (want_decay) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int d = threadIdx.x + k * blockDim.x;
            if (d < D) decay_buf[((long long)b * H + h) * D + d] = decay[k];
        }
    }
}

// Between the two chunk passes: walks the chunks of each request in order. On entry chunk_state[w] is the state chunk w
// builds from zero and chunk_decay[w] the product of its forget gates; on exit chunk_state[w] is the state chunk w
// STARTS from: S_in(first) = the request's stored state, S_in(w + 1) = diag(decay_w) S_in(w) + S_local(w).
__global__ void glr_combine_kernel(const float* __restrict__ state, float* __restrict__ chunk_state,
                                   const float* __restrict__ chunk_decay, const int* __restrict__ seq_item0,
                                   const int* __restrict__ slot, int H, int D, int E) {
    const int h = blockIdx.y, b = blockIdx.z;
    const long long de = (long long)D * E;
    const int w0 = seq_item0[b], w1 = seq_item0[b + 1];
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < de; i += (long long)gridDim.x * blockDim.x) {
        const int d = (int)(i / E);
        float S = state[((long long)slot[b] * H + h) * de + i];
        for (int w = w0; w < w1; ++w) {
            float* cs = chunk_state + ((long long)w * H + h) * de + i;
            const float loc = *cs;
            *cs = S;
            S = fmaf(chunk_decay[((long long)w * H + h) * D + d], S, loc);
        }
    }
}

template <typename T>
__global__ void head_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ out,
                                    long long n_rows, int E, float eps) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const float* xr = x + row * E;
    float ss = 0.f;
    for (int e = lane; e < E; e += 32) ss = fmaf(xr[e], xr[e], ss);
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)E + eps);
    for (int e = lane; e < E; e += 32) stf(out + row * E + e, xr[e] * r * w[e]);
}

}  // namespace seqmix
}  // namespace llark

using namespace llark;
using namespace llark::seqmix;
typedef __nv_bfloat16 bf16_t;

static int launch_headnorm(const float* src, long long ld, int q_off, int k_off, int v_off, const float* wq,
                           const float* wk, void* qn, void* kn, void* vv, void* kring, void* vring, const int* tok_seq,
                           const int* cu, const int* pos0, const int* slot, int n_tok, int H, int G, int D, int E, int cap,
                           float eps, float temp_coef, int temp_every, int act_fp32, cudaStream_t st) {
    if (n_tok <= 0 || H <= 0 || G <= 0 || D <= 0 || E <= 0 || !src || !wq || !wk || !qn || !kn || !vv) return LLARK_EINVAL;
    if (kring && (!vring || cap <= 0 || !tok_seq || !cu || !pos0 || !slot)) return LLARK_EINVAL;
    if (temp_every > 0 && (!tok_seq || !cu || !pos0)) return LLARK_EINVAL;
    int warps = H + G < 8 ? H + G : 8;
    if (act_fp32)
        qk_headnorm_kernel<float><<<n_tok, warps * 32, 0, st>>>(src, ld, q_off, k_off, v_off, wq, wk, (float*)qn,
                                                                (float*)kn, (float*)vv, (float*)kring, (float*)vring,
                                                                tok_seq, cu, pos0, slot, H, G, D, E, cap, eps, temp_coef,
                                                                temp_every);
    else
        qk_headnorm_kernel<bf16_t><<<n_tok, warps * 32, 0, st>>>(src, ld, q_off, k_off, v_off, wq, wk, (bf16_t*)qn,
                                                                 (bf16_t*)kn, (bf16_t*)vv, (bf16_t*)kring, (bf16_t*)vring,
                                                                 tok_seq, cu, pos0, slot, H, G, D, E, cap, eps, temp_coef,
                                                                 temp_every);
    return check_launch();
}

extern "C" int llark_seq_qk_headnorm(const float* src, long long ld, int q_off, int k_off, const float* wq,
                                     const float* wk, void* qn, void* kn, void* vraw, void* kring, void* vring,
                                     const int* tok_seq, const int* cu, const int* pos0, const int* slot, int n_tok, int H,
                                     int G, int D, int cap, float eps, int act_fp32, cudaStream_t st) {
    return launch_headnorm(src, ld, q_off, k_off, k_off, wq, wk, qn, kn, vraw, kring, vring, tok_seq, cu, pos0, slot, n_tok,
                           H, G, D, D, cap, eps, 0.f, 0, act_fp32, st);
}

extern "C" int llark_seq_qkv_headnorm(const float* src, long long ld, int q_off, int k_off, int v_off, const float* wq,
                                      const float* wk, void* qn, void* kn, void* vv, void* kring, void* vring,
                                      const int* tok_seq, const int* cu, const int* pos0, const int* slot, int n_tok,
                                      int H, int G, int D, int E, int cap, float eps, float temp_coef, int temp_every,
                                      int act_fp32, cudaStream_t st) {
    if (temp_every < 0) return LLARK_EINVAL;
    return launch_headnorm(src, ld, q_off, k_off, v_off, wq, wk, qn, kn, vv, kring, vring, tok_seq, cu, pos0, slot, n_tok,
                           H, G, D, E, cap, eps, temp_coef, temp_every, act_fp32, st);
}

extern "C" int llark_seq_qkv_rotary(const float* src, long long ld, int q_off, int k_off, int v_off, const float* wq,
                                    const float* wk, const float* qk_freq, int n_rot, int qk_interleaved,
                                    const float* v_freq, int v_interleaved, void* qn, void* kn, void* vv, void* kring,
                                    void* vring, const int* tok_seq, const int* cu, const int* pos0, const int* slot,
                                    int n_tok, int H, int G, int D, int E, int cap, float eps, int act_fp32,
                                    cudaStream_t st) {
    if (n_tok <= 0 || H <= 0 || G <= 0 || D <= 0 || E <= 0 || !src || !qn || !kn || !vv || !tok_seq || !cu || !pos0 ||
        !slot || n_rot < 0 || (n_rot % 2) || n_rot > D || (n_rot && !qk_freq) || (!wq != !wk))
        return LLARK_EINVAL;
    if (kring && (!vring || cap <= 0)) return LLARK_EINVAL;
    const size_t smem = sizeof(float) * (size_t)(n_rot + (v_freq ? 2 * (E / 2) : 0));
    if (smem > 48 * 1024) return LLARK_EINVAL;
    // Four entries per access when every head, zone and offset is a multiple of four entries (of eight for zones in halves)
    // and the rows start on 16-byte boundaries.
    const bool quads = D % 4 == 0 && E % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0 && ld % 4 == 0 &&
                       n_rot % (qk_interleaved ? 4 : 8) == 0 && (!v_freq || E % (v_interleaved ? 4 : 8) == 0) &&
                       (((uintptr_t)src | (uintptr_t)qn | (uintptr_t)kn | (uintptr_t)vv | (uintptr_t)kring | (uintptr_t)vring |
                         (uintptr_t)wq | (uintptr_t)wk) & 15) == 0;
    // work items of a token: few tokens (decoding): as many threads as items, so that no thread walks a chain of dependent
    // loads; many tokens: 256 threads, the grid fills the GPU anyway.
    int items = (H + G) * (D - n_rot / 2) + G * (v_freq ? E - E / 2 : E);
    if (quads) items /= 4;
    int threads = n_tok >= 1024 ? 256 : (items + 31) / 32 * 32;
    threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
#define LLARK_ROTARY(KERNEL, T)                                                                                      \
    KERNEL<T><<<n_tok, threads, smem, st>>>(src, ld, q_off, k_off, v_off, wq, wk, qk_freq, n_rot, qk_interleaved, v_freq, \
                                            v_interleaved, (T*)qn, (T*)kn, (T*)vv, (T*)kring, (T*)vring, tok_seq, cu, pos0, \
                                            slot, H, G, D, E, cap, eps)
    if (quads) {
        if (act_fp32) LLARK_ROTARY(qkv_rotary4_kernel, float);
        else LLARK_ROTARY(qkv_rotary4_kernel, bf16_t);
    } else {
        if (act_fp32) LLARK_ROTARY(qkv_rotary_kernel, float);
        else LLARK_ROTARY(qkv_rotary_kernel, bf16_t);
    }
#undef LLARK_ROTARY
    return check_launch();
}

template <typename T>
static int launch_swa(const void* qn, const void* kn, const void* vv, const void* kring, const void* vring,
                      const float* gate, long long gate_ld, const float* scale_h, void* out, const int* tok_seq,
                      const int* cu, const int* pos0, const int* slot, int n_tok, int H, int G, int D, int E, int window,
                      int cap, int from_ring_only, const float* sink, int gate_per_head, int chunk, float softcap,
                      const float* vfreq, int v_interleaved, cudaStream_t st) {
    const int span = chunk > 0 ? chunk : window;  // most keys a query sees
    int nw = 1;
    while (nw < 8 && nw * 64 < span) nw <<= 1;  // two tiles per warp before another warp pays off
    const size_t smem = sizeof(float) * (size_t)(D + nw * 32 + 2 * nw + nw * E + (vfreq ? E : 0));
    dim3 grid(n_tok, H);
    const int dpl = (E + 31) / 32;
#define LLARK_SWA(DPL)                                                                                              \
    swa_attn_kernel<T, DPL><<<grid, nw * 32, smem, st>>>((const T*)qn, (const T*)kn, (const T*)vv, (const T*)kring, \
                                                         (const T*)vring, gate, gate_ld, scale_h, (T*)out, tok_seq, \
                                                         cu, pos0, slot, H, G, D, E, window, cap, from_ring_only, \
                                                         sink, gate_per_head, chunk, softcap, vfreq, v_interleaved)
    if (dpl <= 1) LLARK_SWA(1);
    else if (dpl <= 2) LLARK_SWA(2);
    else if (dpl <= 4) LLARK_SWA(4);
    else if (dpl <= 8) LLARK_SWA(8);
    else if (dpl <= 16) LLARK_SWA(16);
    else if (dpl <= 32) LLARK_SWA(32);
    else return LLARK_EINVAL;
#undef LLARK_SWA
    return check_launch();
}

extern "C" int llark_seq_swa_attn(const void* qn, const void* kn, const void* vv, const void* kring, const void* vring,
                                  const float* gate, long long gate_ld, const float* scale_h, void* out,
                                  const int* tok_seq, const int* cu, const int* pos0, const int* slot, int n_tok, int H,
                                  int G, int D, int E, int window, int cap, int from_ring_only, const float* sink,
                                  int gate_per_head, int chunk, float softcap, const float* vfreq, int v_interleaved,
                                  int act_fp32, cudaStream_t st) {
    if (n_tok <= 0 || H <= 0 || G <= 0 || (H % G) || D <= 0 || E <= 0 || window <= 0 || cap <= 0 || !qn || !kring ||
        !vring || !scale_h || !out || !tok_seq || !cu || !pos0 || !slot || chunk < 0 || softcap < 0.f)
        return LLARK_EINVAL;
    if (!from_ring_only && (!kn || !vv)) return LLARK_EINVAL;
    if ((size_t)(D + 8 * 32 + 16 + 9 * E) * sizeof(float) > 48 * 1024) return LLARK_EINVAL;
    return act_fp32 ? launch_swa<float>(qn, kn, vv, kring, vring, gate, gate_ld, scale_h, out, tok_seq, cu, pos0, slot,
                                        n_tok, H, G, D, E, window, cap, from_ring_only, sink, gate_per_head, chunk,
                                        softcap, vfreq, v_interleaved, st)
                    : launch_swa<bf16_t>(qn, kn, vv, kring, vring, gate, gate_ld, scale_h, out, tok_seq, cu, pos0, slot,
                                         n_tok, H, G, D, E, window, cap, from_ring_only, sink, gate_per_head, chunk,
                                         softcap, vfreq, v_interleaved, st);
}

extern "C" int llark_seq_kv_ring_write(const void* kn, const void* vv, void* kring, void* vring, const int* tok_seq,
                                       const int* cu, const int* pos0, const int* slot, int n_tok, int GD, int GE, int cap,
                                       int act_fp32, cudaStream_t st) {
    if (n_tok <= 0 || GD <= 0 || GE <= 0 || cap <= 0 || !kn || !kring || (vring && !vv)) return LLARK_EINVAL;
    if (act_fp32)
        kv_ring_write_kernel<float><<<n_tok, 128, 0, st>>>((const float*)kn, (const float*)vv, (float*)kring,
                                                           (float*)vring, tok_seq, cu, pos0, slot, GD, GE, cap);
    else
        kv_ring_write_kernel<bf16_t><<<n_tok, 128, 0, st>>>((const bf16_t*)kn, (const bf16_t*)vv, (bf16_t*)kring,
                                                            (bf16_t*)vring, tok_seq, cu, pos0, slot, GD, GE, cap);
    return check_launch();
}

extern "C" int llark_seq_glr_scan(const float* src, long long ld, int q_off, int f_off, int v_off, const float* lower,
                                  const float* init_buf, float* final_buf, float* decay_buf, float* o_raw,
                                  const int* item_row0, const int* item_n, const int* item_init, const int* item_final,
                                  int n_items, int H, int D, int E, cudaStream_t st) {
    if (n_items <= 0 || H <= 0 || D <= 0 || E <= 0 || !src || !item_row0 || !item_n || !item_init || !item_final)
        return LLARK_EINVAL;
    if (D > 256) return LLARK_EINVAL;
    const int dpt = D <= 128 ? 16 : 32;
    int R = 1;
    while (R * dpt < D) R <<= 1;  // 1, 2, 4 or 8 row groups: a power of two for the shuffle tree
    // each thread keeps a dpt x EC tile of S: the gates and q of a row are read from shared memory once per EC columns,
    // which is what keeps the scan off the shared-memory bandwidth limit; narrow heads take fewer columns per thread
    const int ec = (dpt == 16 && E >= 64) ? 4 : (E >= 32 ? 2 : 1);
    int threads = 128;
    int ecols = threads / R * ec;
    while (ecols / 2 >= E && threads > 32) {  // do not carry idle columns
        threads >>= 1;
        ecols >>= 1;
    }
    const int DP = R * (dpt + 4);
    const size_t smem = sizeof(float) * 2 * (size_t)kTS * (3 * DP + ecols);
    dim3 grid((E + ecols - 1) / ecols, H, n_items);
#define LLARK_GLR2(DPT_, EC_, OUT_)                                                                                        \
    do {                                                                                                                   \
        if (smem > 48 * 1024)                                                                                              \
            cudaFuncSetAttribute(glr_scan_kernel<DPT_, EC_, OUT_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        glr_scan_kernel<DPT_, EC_, OUT_><<<grid, threads, smem, st>>>(src, ld, q_off, f_off, v_off, lower, init_buf,        \
                                                                      final_buf, decay_buf, o_raw, item_row0, item_n,       \
                                                                      item_init, item_final, H, D, E, R, ecols);            \
    } while (0)
#define LLARK_GLR(DPT_, EC_)                   \
    do {                                       \
        if (o_raw) LLARK_GLR2(DPT_, EC_, true); \
        else LLARK_GLR2(DPT_, EC_, false);     \
    } while (0)
    if (dpt == 16 && ec == 4) LLARK_GLR(16, 4);
    else if (dpt == 16 && ec == 2) LLARK_GLR(16, 2);
    else if (dpt == 16) LLARK_GLR(16, 1);
    else if (ec == 2) LLARK_GLR(32, 2);
    else LLARK_GLR(32, 1);
#undef LLARK_GLR2
#undef LLARK_GLR
    return check_launch();
}

extern "C" int llark_seq_glr_combine(const float* state, float* chunk_state, const float* chunk_decay,
                                     const int* seq_item0, const int* slot, int n_seq, int H, int D, int E,
                                     cudaStream_t st) {
    if (n_seq <= 0 || H <= 0 || D <= 0 || E <= 0 || !state || !chunk_state || !chunk_decay || !seq_item0 || !slot)
        return LLARK_EINVAL;
    const long long de = (long long)D * E;
    dim3 grid((unsigned)((de + 255) / 256), H, n_seq);
    glr_combine_kernel<<<grid, 256, 0, st>>>(state, chunk_state, chunk_decay, seq_item0, slot, H, D, E);
    return check_launch();
}

extern "C" int llark_seq_head_rmsnorm(const float* x, const float* w, void* out, long long n_rows, int E, float eps,
                                      int act_fp32, cudaStream_t st) {
    if (n_rows <= 0 || E <= 0 || !x || !w || !out) return LLARK_EINVAL;
    const unsigned grid = (unsigned)((n_rows + 3) / 4);
    if (act_fp32)
        head_rmsnorm_kernel<float><<<grid, 128, 0, st>>>(x, w, (float*)out, n_rows, E, eps);
    else
        head_rmsnorm_kernel<bf16_t><<<grid, 128, 0, st>>>(x, w, (bf16_t*)out, n_rows, E, eps);
    return check_launch();
}
