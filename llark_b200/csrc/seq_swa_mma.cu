// Sliding-window attention for prompts and portions of prompts on the packed-step layout (see seq_mixers.cu), bf16
// operands on the warp-level tensor-core path (mma.sync m16n8k16, fp32 accumulation): scores, mask, softmax and the
// running maximum / sum are fp32, the probabilities are rounded to bf16 only as the A operand of P.V.
//
// CTA = 4 warps = 64 queries of one (request, head); it walks the 64-key tiles that intersect the window of any of its
// queries. A key at position j of the sequence comes from the step's own buffers when j >= pos0 (it arrived with this
// step) and from ring entry j % cap of the request's slot otherwise. Q, K and V tiles sit in shared memory row-major and
// reach the registers through ldmatrix (V through ldmatrix.trans); the row pitch (+8 elements) keeps those
// conflict-free. K / V tiles are double-buffered: the next tile is in flight (cp.async) while this one is multiplied. Per-head score scale (softmax scale x temperature) and the optional sigmoid output gate are applied
// in registers. The SIMT kernel of seq_mixers.cu remains the path for single-token steps, fp32 and head
// sizes that are not multiples of 16.
#include "common.cuh"

namespace llark {
extern thread_local int g_last_cuda_error;
namespace swamma {

typedef __nv_bfloat16 bf16_t;
constexpr int BQ = 64, BK = 64;

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}

template <int DMAX>
__global__ void __launch_bounds__(128)
swa_mma_kernel(const bf16_t* __restrict__ qn, const bf16_t* __restrict__ kn, const bf16_t* __restrict__ vv,
               const bf16_t* __restrict__ kring, const bf16_t* __restrict__ vring, const float* __restrict__ gate,
               long long gate_ld, const float* __restrict__ scale_h, bf16_t* __restrict__ out,
               const int* __restrict__ cu, const int* __restrict__ pos0, const int* __restrict__ slot, int H, int G,
               int D, int window, int cap, const float* __restrict__ sink, int gate_per_head, int chunk, float softcap,
               const float* __restrict__ vfreq, int v_interleaved) {
    const int b = blockIdx.z, h = blockIdx.y;
    const int g = h / (H / G);
    const int row0 = cu[b], n = cu[b + 1] - row0;
    const int qt0 = blockIdx.x * BQ;
    if (qt0 >= n) return;
    const long long p0 = pos0[b];
    extern __shared__ __align__(16) unsigned char smraw[];
    const int DS = D + 8;                           // row pitch: 16 bytes more than the row, so that the eight
    bf16_t* sQ = reinterpret_cast<bf16_t*>(smraw);  // [BQ][DS]   rows of an ldmatrix fall into different banks
    bf16_t* sK0 = sQ + BQ * DS;                     // [2][BK][DS]  two stages: the next tile arrives by cp.async
    bf16_t* sV0 = sK0 + 2 * BK * DS;                // [2][BK][DS]  while this one is multiplied; row-major, P.V reads
                                                    //              it through ldmatrix.trans
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
    const int dv = D >> 3;  // 16-byte vectors per row

    for (int i = threadIdx.x; i < BQ * dv; i += blockDim.x) {
        const int r = i / dv, c = (i % dv) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (qt0 + r < n) v = *reinterpret_cast<const uint4*>(qn + ((long long)(row0 + qt0 + r) * H + h) * D + c);
        *reinterpret_cast<uint4*>(sQ + r * DS + c) = v;
    }
    const int q_last = (qt0 + BQ - 1 < n - 1) ? qt0 + BQ - 1 : n - 1;
    const long long pq_lo = p0 + qt0, pq_hi = p0 + q_last;
    // first key any query of the tile sees: the start of the first query's block of `chunk` positions (blocks counted
    // from position 0 of the sequence), or of its sliding window
    const long long k_lo = chunk > 0 ? (pq_lo / chunk) * chunk : (pq_lo - window + 1 > 0 ? pq_lo - window + 1 : 0);
    const long long ring_base = (long long)slot[b] * cap;
    constexpr float kLog2e = 1.4426950408889634f;
    // scores in units of log2: softmax through exp2. With a soft cap the score is squashed first: cap tanh(s scale / cap)
    const float sc = softcap > 0.f ? scale_h[h] / softcap : scale_h[h] * kLog2e;
    const float cap2 = softcap * kLog2e;

    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int qrow = warp * 16 + gq;  // this thread's rows: qrow and qrow + 8

    // A key before this step sits in ring entry (position % cap). Those keys are fewer than cap positions past k_lo, so
    // their entry is ring0 + (position - k_lo), minus cap once if it runs over: no division in the loop. The walk over
    // (row, 16-byte piece) advances by the CTA's 128 threads without dividing either.
    const int ring0 = (int)(k_lo % cap);
    const int step_r = (int)blockDim.x / dv, step_c = (int)blockDim.x % dv;
    const int my_r0 = (int)threadIdx.x / dv, my_c0 = (int)threadIdx.x % dv;
    auto load_tile = [&](long long kt, int stage) {
        bf16_t* dk = sK0 + stage * BK * DS;
        bf16_t* dvp = sV0 + stage * BK * DS;
        int r = my_r0, cp = my_c0;
        while (r < BK) {
            const int c = cp * 8;
            const long long j = kt + r;
            if (j <= pq_hi) {
                if (j >= p0) {
                    const long long e = (long long)(row0 + (int)(j - p0)) * G + g;
                    cp_async16(dk + r * DS + c, kn + e * D + c);
                    cp_async16(dvp + r * DS + c, vv + e * D + c);
                } else {
                    int idx = ring0 + (int)(j - k_lo);
                    if (idx >= cap) idx -= cap;
                    const long long e = (ring_base + idx) * G + g;
                    cp_async16(dk + r * DS + c, kring + e * D + c);
                    cp_async16(dvp + r * DS + c, vring + e * D + c);
                }
            } else {
                *reinterpret_cast<uint4*>(dk + r * DS + c) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(dvp + r * DS + c) = make_uint4(0, 0, 0, 0);
            }
            r += step_r;
            cp += step_c;
            if (cp >= dv) {
                cp -= dv;
                ++r;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int n_tiles = (int)((pq_hi - k_lo) / BK) + 1;
    load_tile(k_lo, 0);
    for (int it = 0; it < n_tiles; ++it) {
        const long long kt = k_lo + (long long)it * BK;
        if (it + 1 < n_tiles) {
            load_tile(kt + BK, (it + 1) & 1);  // that stage was released by the barrier at the end of the last pass
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // tile `it` (and, on the first pass, sQ) is in shared memory for everybody
        const bf16_t* sK = sK0 + (it & 1) * BK * DS;
        const bf16_t* sV = sV0 + (it & 1) * BK * DS;
        // ---- S = Q K^T for this warp's 16 rows x 64 keys
        float s[BK / 8][4];
#pragma unroll
        for (int nt = 0; nt < BK / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int kb = 0; kb < DMAX / 16; ++kb) {
            if (kb * 16 < D) {
                // A fragment: rows (lane & 7) + 8 * bit 3 of the warp's 16, columns + 8 for lanes 16..31
                uint32_t a[4];
                ldsm_x4(a, sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DS + kb * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int nt = 0; nt < BK / 8; nt += 2) {
                    // B fragments of two key groups: (nt, k lo), (nt, k hi), (nt + 1, k lo), (nt + 1, k hi)
                    uint32_t kf[4];
                    ldsm_x4(kf, sK + ((nt + (lane >> 4)) * 8 + (lane & 7)) * DS + kb * 16 + ((lane >> 3) & 1) * 8);
                    mma_bf16(s[nt], a[0], a[1], a[2], a[3], kf[0], kf[1]);
                    mma_bf16(s[nt + 1], a[0], a[1], a[2], a[3], kf[2], kf[3]);
                }
            }
        }
        // ---- scale, mask (causal and window), online softmax in fp32
        float mt[2] = {-INFINITY, -INFINITY};
        // rel = query position - first key of the tile: key column c is visible iff lob <= c <= rel, where lob is the
        // row's first visible position minus the tile's first key (window: rel - window + 1; chunk: start of the row's
        // block). A tile whose 64 keys are visible to all 16 rows of the warp (the usual case inside a wide window)
        // skips the test: the largest lob of the warp's rows is that of its last row.
        const long long rel_lo = pq_lo + warp * 16 - kt;  // rel of the warp's first row; its rows are consecutive
        const bool rows_ok = qt0 + warp * 16 + 15 < n;
        const long long p_last = pq_lo + warp * 16 + 15;
        const long long lob_last = chunk > 0 ? (p_last / chunk) * chunk - kt : rel_lo + 15 - window + 1;
        const bool interior = rows_ok && rel_lo >= BK - 1 && lob_last <= 0;
        if (softcap > 0.f) {
#pragma unroll
            for (int nt = 0; nt < BK / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] = cap2 * tanhf(s[nt][e] * sc);
        } else {
#pragma unroll
            for (int nt = 0; nt < BK / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] *= sc;
        }
        if (interior) {
#pragma unroll
            for (int nt = 0; nt < BK / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) mt[e >> 1] = fmaxf(mt[e >> 1], s[nt][e]);
        } else {
            // clamp so that the 32-bit arithmetic below cannot overflow: beyond +-2^30 the answer is the same
            auto clamp30 = [](long long v) { return (int)(v > (1LL << 30) ? (1LL << 30) : (v < -(1LL << 30) ? -(1LL << 30) : v)); };
            int rel_x[2], lob_x[2];
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const long long rl = rel_lo + gq + x * 8;
                rel_x[x] = clamp30(rl);
                lob_x[x] = clamp30(chunk > 0 ? ((rl + kt) / chunk) * chunk - kt : rl - window + 1);
            }
#pragma unroll
            for (int nt = 0; nt < BK / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int x = e >> 1;
                    const int c = nt * 8 + 2 * tq + (e & 1);
                    const bool ok = (qt0 + qrow + x * 8 < n) && c <= rel_x[x] && c >= lob_x[x];
                    if (!ok) s[nt][e] = -INFINITY;
                    mt[x] = fmaxf(mt[x], s[nt][e]);
                }
        }
        float alpha[2], mn[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            mt[x] = fmaxf(mt[x], __shfl_xor_sync(0xffffffffu, mt[x], 1));
            mt[x] = fmaxf(mt[x], __shfl_xor_sync(0xffffffffu, mt[x], 2));
            mn[x] = fmaxf(m[x], mt[x]);
            alpha[x] = mn[x] == -INFINITY ? 1.f : exp2f(m[x] - mn[x]);
            m[x] = mn[x];
            l[x] *= alpha[x];
        }
#pragma unroll
        for (int nt = 0; nt < BK / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int x = e >> 1;
                const float p = mn[x] == -INFINITY ? 0.f : exp2f(s[nt][e] - mn[x]);
                s[nt][e] = p;
                l[x] += p;
            }
#pragma unroll
        for (int i = 0; i < DMAX / 8; ++i) {
            o[i][0] *= alpha[0];
            o[i][1] *= alpha[0];
            o[i][2] *= alpha[1];
            o[i][3] *= alpha[1];
        }
        // ---- O += P V
#pragma unroll
        for (int kb = 0; kb < BK / 16; ++kb) {
            const uint32_t a0 = pack_bf16x2(s[2 * kb][0], s[2 * kb][1]);
            const uint32_t a1 = pack_bf16x2(s[2 * kb][2], s[2 * kb][3]);
            const uint32_t a2 = pack_bf16x2(s[2 * kb + 1][0], s[2 * kb + 1][1]);
            const uint32_t a3 = pack_bf16x2(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
            for (int nt = 0; nt < DMAX / 8; nt += 2) {
                if (nt * 8 < D) {
                    // transposed 8x8 blocks of V: (keys lo, nt), (keys hi, nt), (keys lo, nt + 1), (keys hi, nt + 1)
                    uint32_t vf[4];
                    ldsm_x4_trans(vf, sV + (kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DS + nt * 8 + (lane >> 4) * 8);
                    mma_bf16(o[nt], a0, a1, a2, a3, vf[0], vf[1]);
                    mma_bf16(o[nt + 1], a0, a1, a2, a3, vf[2], vf[3]);
                }
            }
        }
        __syncthreads();  // everybody is done with this stage before the pass after next refills it
    }
    // ---- normalise, gate, store
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        l[x] += __shfl_xor_sync(0xffffffffu, l[x], 1);
        l[x] += __shfl_xor_sync(0xffffffffu, l[x], 2);
    }
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int r = qrow + x * 8;
        if (qt0 + r >= n) continue;
        const long long trow = row0 + qt0 + r;
        // a sink adds exp(sink_h) to the denominator (m is in units of log2; every row has seen its own key, so m is finite)
        const float inv = 1.0f / (sink ? l[x] + exp2f(sink[h] * kLog2e - m[x]) : l[x]);
        const float gh = (gate && gate_per_head) ? 1.0f / (1.0f + expf(-gate[trow * gate_ld + h])) : 1.0f;
        if (vfreq) {
            // Values were stored rotated by their own position: the row's weighted sum is turned back by the query's
            // position, pair mp by -p * vfreq[mp], before the gate. Interleaved pairs (2 mp, 2 mp + 1) are the two
            // adjacent columns of one accumulator fragment; halves (mp, mp + D / 2) sit D / 16 fragments apart in the
            // same thread (the launcher takes halves only when D = DMAX, so that the fragment index is a constant).
            const float pf = (float)(p0 + qt0 + r);
            if (v_interleaved) {
#pragma unroll
                for (int nt = 0; nt < DMAX / 8; ++nt)
                    if (nt * 8 < D) {
                        float si, co;
                        sincosf(pf * vfreq[nt * 4 + tq], &si, &co);
                        const float u = o[nt][2 * x], v = o[nt][2 * x + 1];
                        o[nt][2 * x] = u * co + v * si;
                        o[nt][2 * x + 1] = v * co - u * si;
                    }
            } else {
                constexpr int hn = DMAX / 16;  // fragments per half
#pragma unroll
                for (int nt = 0; nt < hn; ++nt) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            float si, co;
                            sincosf(pf * vfreq[nt * 8 + 2 * tq + e], &si, &co);
                            const float u = o[nt][2 * x + e], v = o[nt + hn][2 * x + e];
                            o[nt][2 * x + e] = u * co + v * si;
                            o[nt + hn][2 * x + e] = v * co - u * si;
                        }
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < DMAX / 8; ++nt) {
            if (nt * 8 < D) {
                const int c = nt * 8 + 2 * tq;
                float v0 = o[nt][2 * x] * inv * gh, v1 = o[nt][2 * x + 1] * inv * gh;
                if (gate && !gate_per_head) {
                    const float* gp = gate + trow * gate_ld + h * D + c;
                    v0 *= 1.0f / (1.0f + expf(-gp[0]));
                    v1 *= 1.0f / (1.0f + expf(-gp[1]));
                }
                *reinterpret_cast<uint32_t*>(out + (trow * H + h) * D + c) = pack_bf16x2(v0, v1);
            }
        }
    }
}

template <int DMAX>
static int launch(const void* qn, const void* kn, const void* vv, const void* kring, const void* vring,
                  const float* gate, long long gate_ld, const float* scale_h, void* out, const int* cu, const int* pos0,
                  const int* slot, int n_seq, int max_len, int H, int G, int D, int window, int cap, const float* sink,
                  int gate_per_head, int chunk, float softcap, const float* vfreq, int v_interleaved, cudaStream_t st) {
    const size_t smem = sizeof(bf16_t) * (size_t)(BQ + 4 * BK) * (D + 8);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(swa_mma_kernel<DMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            g_last_cuda_error = (int)e;
            return LLARK_ECUDA;
        }
    }
    dim3 grid((max_len + BQ - 1) / BQ, H, n_seq);
    swa_mma_kernel<DMAX><<<grid, 128, smem, st>>>((const bf16_t*)qn, (const bf16_t*)kn, (const bf16_t*)vv,
                                                  (const bf16_t*)kring, (const bf16_t*)vring, gate, gate_ld, scale_h,
                                                  (bf16_t*)out, cu, pos0, slot, H, G, D, window, cap, sink, gate_per_head,
                                                  chunk, softcap, vfreq, v_interleaved);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        return LLARK_ECUDA;
    }
    return LLARK_OK;
}

}  // namespace swamma
}  // namespace llark

using namespace llark;

extern "C" int llark_seq_swa_attn_mma(const void* qn, const void* kn, const void* vv, const void* kring, const void* vring,
                                      const float* gate, long long gate_ld, const float* scale_h, void* out,
                                      const int* cu, const int* pos0, const int* slot, int n_seq, int max_len, int H,
                                      int G, int D, int window, int cap, const float* sink, int gate_per_head,
                                      int chunk, float softcap, const float* vfreq, int v_interleaved, cudaStream_t st) {
    if (n_seq <= 0 || max_len <= 0 || H <= 0 || G <= 0 || (H % G) || D <= 0 || (D % 16) || D > 256 || window <= 0 ||
        cap <= 0 || !qn || !kn || !vv || !kring || !vring || !scale_h || !out || !cu || !pos0 || !slot || chunk < 0 ||
        softcap < 0.f)
        return LLARK_EINVAL;
    if (gate && !gate_per_head && (gate_ld % 2)) return LLARK_EINVAL;
    if (vfreq && !v_interleaved && D != 64 && D != 128 && D != 256) return LLARK_EINVAL;
    if (D <= 64)
        return swamma::launch<64>(qn, kn, vv, kring, vring, gate, gate_ld, scale_h, out, cu, pos0, slot, n_seq, max_len, H,
                                  G, D, window, cap, sink, gate_per_head, chunk, softcap, vfreq, v_interleaved, st);
    if (D <= 128)
        return swamma::launch<128>(qn, kn, vv, kring, vring, gate, gate_ld, scale_h, out, cu, pos0, slot, n_seq, max_len,
                                   H, G, D, window, cap, sink, gate_per_head, chunk, softcap, vfreq, v_interleaved, st);
    return swamma::launch<256>(qn, kn, vv, kring, vring, gate, gate_ld, scale_h, out, cu, pos0, slot, n_seq, max_len, H, G,
                               D, window, cap, sink, gate_per_head, chunk, softcap, vfreq, v_interleaved, st);
}
