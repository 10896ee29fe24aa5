// Attention over the packed cache for the early scales of a schedule: tens of queries over at most a few hundred cached
// tokens per (sample, head).  There the work is a few MFLOP per (sample, head) and the tcgen05 kernel spends its time on
// what surrounds its tile loop (TMEM allocation, barrier set-up, a 128-row tile for 25 queries, one CTA per SM), while the
// CUDA-core streaming kernel pays queries x keys x head_dim on the FMA pipe.  This kernel sits between them: warp-level
// tensor-core instructions (mma.sync m16n8k16, fp16 operands, fp32 accumulators in registers), no asynchronous machinery,
// 18 KB of shared memory, so several thread blocks share an SM and hide each other's latencies.
//
// One CTA = one (sample, head) x 32 or 64 queries, two or four warps of 16 query rows.  Keys go through shared memory 64 at a time:
// the packed rows are turned into exact fp16 integer codes (byte permutes), S = Q K^T on codes, the per-key K scale and
// zero-point are applied to S in fp32 (s_k * (acc - z_k * sum q)), online softmax in registers (base 2), the per-key V scale is
// folded into P through the exponent before it is rounded to fp16 (and divided out of the normaliser), O += P V on codes, and the V zero-point term sum_k P_k z_k is subtracted at the
// end.  An fp32 query is split into fp16 hi + lo operands (two MMAs), like in the tcgen05 kernel.  Only groupings with one
// scale / zero-point per key (per token, per token and head, per appended step) and head_dim 64 are taken.
#include <cfloat>

#include "varq_attn.cuh"

namespace varq {

namespace {

constexpr int MID_KEYS = 64;        // keys per shared-memory chunk

__device__ __forceinline__ uint32_t mid_h2_sub(uint32_t a, uint32_t b) {
    __half2 r = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
// one packed word -> 32 / BITS fp16 codes (exact integers), in field order: 0x6400 | u is the fp16 number 1024 + u
template <int BITS> struct MidCodes;
template <> struct MidCodes<8> {
    static __device__ __forceinline__ void cvt(uint32_t w, uint32_t* h) {
        const uint32_t u = w ^ 0x80808080u;
        h[0] = mid_h2_sub(__byte_perm(u, 0x64646464u, 0x4140), 0x64806480u);
        h[1] = mid_h2_sub(__byte_perm(u, 0x64646464u, 0x4342), 0x64806480u);
    }
};
template <> struct MidCodes<4> {
    static __device__ __forceinline__ void cvt(uint32_t w, uint32_t* h) {
        const uint32_t x = w ^ 0x88888888u;
        const uint32_t lo = x & 0x0F0F0F0Fu, hi = (x >> 4) & 0x0F0F0F0Fu;      // fields 0,2,4,6 / 1,3,5,7
        const uint32_t a = __byte_perm(lo, hi, 0x5140), b = __byte_perm(lo, hi, 0x7362);   // bytes = fields 0,1,2,3 / 4,5,6,7
        h[0] = mid_h2_sub(__byte_perm(a, 0x64646464u, 0x4140), 0x64086408u);
        h[1] = mid_h2_sub(__byte_perm(a, 0x64646464u, 0x4342), 0x64086408u);
        h[2] = mid_h2_sub(__byte_perm(b, 0x64646464u, 0x4140), 0x64086408u);
        h[3] = mid_h2_sub(__byte_perm(b, 0x64646464u, 0x4342), 0x64086408u);
    }
};
template <> struct MidCodes<2> {
    static __device__ __forceinline__ void cvt(uint32_t w, uint32_t* h) {
        const uint32_t x = w ^ 0xAAAAAAAAu;
#pragma unroll
        for (int b = 0; b < 4; ++b) {             // byte b holds fields 4b .. 4b + 3
            const uint32_t y = x >> (8 * b);
            const uint32_t f01 = (y & 3u) | (((y >> 2) & 3u) << 16), f23 = ((y >> 4) & 3u) | (((y >> 6) & 3u) << 16);
            h[2 * b] = mid_h2_sub(f01 | 0x64006400u, 0x64026402u);
            h[2 * b + 1] = mid_h2_sub(f23 | 0x64006400u, 0x64026402u);
        }
    }
};

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ float mid_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// WARPS = 2 (32 queries per CTA; up to 32 queries measured fastest with many small blocks per SM) or 4 (64 queries)
template <int KB, int VB, bool QSPLIT, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, (QSPLIT ? 12 : 16) / WARPS) attn_mid_kernel(AttnArgs a) {
    constexpr int MID_ROWS = WARPS * 16, MID_THREADS = WARPS * 32;
    constexpr int D = 64, PITCH = D + 8;                 // halves per shared-memory row: 144 bytes, conflict-free for ldmatrix
    constexpr int KW = D * KB / 32, VW = D * VB / 32;    // packed words per row
    constexpr int NQ = QSPLIT ? 2 : 1;
    __shared__ __align__(16) __half sK[MID_KEYS * PITCH];
    __shared__ __align__(16) __half sV[MID_KEYS * PITCH];
    __shared__ float sKs[MID_KEYS], sKz[MID_KEYS], sVs[MID_KEYS], sVr[MID_KEYS], sVz[MID_KEYS];    // sVs = log2 (V scale), sVr = 1 / (V scale)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int qt = (int)(blockIdx.x % (unsigned)a.n_qtiles), bh = (int)(blockIdx.x / (unsigned)a.n_qtiles), b = bh / a.H, h = bh - b * a.H;
    const int q0 = qt * MID_ROWS + warp * 16;            // first query row of this warp
    const int r0 = q0 + (lane >> 2), r1 = r0 + 8;         // the two rows this thread holds in every fragment
    const int cq = (lane & 3) * 2;                       // its column pair inside an 8-wide tile
    const bool warp_live = q0 < a.Lq;                    // warps past the last query only help with the conversion

    // ---- Q fragments (A operand, 16 x 64 per warp: four k-steps), straight from global memory
    uint32_t qf[NQ][4][4];
    float qsum0 = 0.f, qsum1 = 0.f;
#pragma unroll
    for (int qi = 0; qi < NQ; ++qi)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
#pragma unroll
            for (int e = 0; e < 4; ++e) qf[qi][kk][e] = 0u;
    if (warp_live) {
        const int es = a.q_dtype == VARQ_F32 ? 4 : 2;
        const long long base_bh = b * a.qs_b + h * a.qs_h;
        const uintptr_t row_addr[2] = {reinterpret_cast<uintptr_t>(a.q) + (unsigned long long)(base_bh + (long long)r0 * a.qs_l) * es,
                                       reinterpret_cast<uintptr_t>(a.q) + (unsigned long long)(base_bh + (long long)r1 * a.qs_l) * es};
        auto load2 = [&](int which, int row, int col, float& x, float& y) {
            x = 0.f; y = 0.f;
            if (row < a.Lq) {
                const uintptr_t addr = row_addr[which] + (unsigned)col * es;
                const long long off = base_bh + (long long)row * a.qs_l + col;
                if (addr & (2 * es - 1)) {                       // the pair is not naturally aligned: two loads
                    x = load_q_elem(a.q, a.q_dtype, off);
                    y = load_q_elem(a.q, a.q_dtype, off + 1);
                } else if (a.q_dtype == VARQ_F32) {
                    const float2 v = __ldg(reinterpret_cast<const float2*>(addr));
                    x = v.x; y = v.y;
                } else {
                    const uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(addr));
                    if (a.q_dtype == VARQ_F16) { const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v)); x = f.x; y = f.y; }
                    else { x = __uint_as_float(v << 16); y = __uint_as_float(v & 0xffff0000u); }
                }
                x = fminf(fmaxf(x, -65504.f), 65504.f);          // the operand is fp16: saturate instead of overflowing
                y = fminf(fmaxf(y, -65504.f), 65504.f);
            }
        };
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {                 // a0: (r0, k), a1: (r1, k), a2: (r0, k + 8), a3: (r1, k + 8)
                const int row = (e & 1) ? r1 : r0, col = kk * 16 + cq + ((e & 2) ? 8 : 0);
                float x, y;
                load2(e & 1, row, col, x, y);
                const __half2 hh = __floats2half2_rn(x, y);
                qf[0][kk][e] = *reinterpret_cast<const uint32_t*>(&hh);
                float sx = x, sy = y;
                if (QSPLIT) {
                    const float2 hf = __half22float2(hh);
                    qf[NQ - 1][kk][e] = pack_h2(x - hf.x, y - hf.y);
                } else {
                    const float2 hf = __half22float2(hh);     // the sum has to match the operand the MMA sees
                    sx = hf.x; sy = hf.y;
                }
                if (e & 1) qsum1 += sx + sy; else qsum0 += sx + sy;
            }
        }
        qsum0 += __shfl_xor_sync(0xffffffffu, qsum0, 1); qsum0 += __shfl_xor_sync(0xffffffffu, qsum0, 2);
        qsum1 += __shfl_xor_sync(0xffffffffu, qsum1, 1); qsum1 += __shfl_xor_sync(0xffffffffu, qsum1, 2);
    }

    float o[8][4];                   // 16 x 64 output accumulator: eight 8-wide tiles
#pragma unroll
    for (int j = 0; j < 8; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }
    float m0 = -1e30f, m1 = -1e30f, l0 = 0.f, l1 = 0.f, cz0 = 0.f, cz1 = 0.f;

    const int32_t* kbase = a.kc + b * a.ks_b + h * a.ks_h;
    const int32_t* vbase = a.vc + b * a.vs_b + h * a.vs_h;
    const bool kz_on = a.kp.zp != nullptr, vz_on = a.vp.zp != nullptr;

    for (int k0 = 0; k0 < a.Lk; k0 += MID_KEYS) {
        __syncthreads();                                   // the previous chunk's tiles are no longer read
        // ---- packed rows -> fp16 codes in shared memory (rows past the cache: zeros), per-key parameters.
        // All global loads of a thread are issued before the first conversion, so their latencies overlap.
        {
            constexpr int KIT = MID_KEYS * KW / MID_THREADS, VIT = MID_KEYS * VW / MID_THREADS;
            uint32_t kwd[KIT], vwd[VIT];
#pragma unroll
            for (int i = 0; i < KIT; ++i) {
                const int idx = tid + i * MID_THREADS, key = idx / KW, w = idx - key * KW;
                kwd[i] = (k0 + key < a.Lk) ? (uint32_t)__ldg(kbase + (long long)(k0 + key) * a.ks_l + w) : 0u;
            }
#pragma unroll
            for (int i = 0; i < VIT; ++i) {
                const int idx = tid + i * MID_THREADS, key = idx / VW, w = idx - key * VW;
                vwd[i] = (k0 + key < a.Lk) ? (uint32_t)__ldg(vbase + (long long)(k0 + key) * a.vs_l + w) : 0u;
            }
#pragma unroll
            for (int i = 0; i < KIT; ++i) {
                const int idx = tid + i * MID_THREADS, key = idx / KW, w = idx - key * KW;
                uint32_t hh[32 / KB / 2];
                MidCodes<KB>::cvt(kwd[i], hh);
                uint32_t* dst = reinterpret_cast<uint32_t*>(sK + key * PITCH + w * (32 / KB));
#pragma unroll
                for (int e = 0; e < 32 / KB / 2; ++e) dst[e] = (k0 + key < a.Lk) ? hh[e] : 0u;
            }
#pragma unroll
            for (int i = 0; i < VIT; ++i) {
                const int idx = tid + i * MID_THREADS, key = idx / VW, w = idx - key * VW;
                uint32_t hh[32 / VB / 2];
                MidCodes<VB>::cvt(vwd[i], hh);
                uint32_t* dst = reinterpret_cast<uint32_t*>(sV + key * PITCH + w * (32 / VB));
#pragma unroll
                for (int e = 0; e < 32 / VB / 2; ++e) dst[e] = (k0 + key < a.Lk) ? hh[e] : 0u;
            }
        }
        if (tid < MID_KEYS) {
            const int key = k0 + tid;
            float ks = 0.f, kz = 0.f, vs = 0.f, vz = 0.f;
            if (key < a.Lk) {
                const long long pk = a.kp.index(b, a.kp.row(key), h, 0), pv = a.vp.index(b, a.vp.row(key), h, 0);
                ks = __ldg(a.kp.scale + pk) * a.scale_log2;
                if (kz_on) kz = __ldg(a.kp.zp + pk) * ks;
                vs = fmaxf(__ldg(a.vp.scale + pv), 9.5367431640625e-07f);      // a V scale below 2^-20 is folded as 2^-20
                if (vz_on) vz = __ldg(a.vp.zp + pv);
            }
            // the V scale enters the exponent (P stays normalised in fp16 whatever its magnitude) and leaves the normaliser again
            sKs[tid] = ks; sKz[tid] = kz; sVs[tid] = key < a.Lk ? __log2f(vs) : 0.f; sVr[tid] = key < a.Lk ? __frcp_rn(vs) : 0.f; sVz[tid] = vz;
        }
        __syncthreads();
        if (!warp_live) continue;
        const int nkt = (min(MID_KEYS, a.Lk - k0) + 7) >> 3;        // 8-key tiles of this chunk that hold a key

        // ---- S = Q K^T on codes: eight 8-key tiles
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) { s[j][0] = 0.f; s[j][1] = 0.f; s[j][2] = 0.f; s[j][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {               // two key tiles per ldmatrix.x4
                if (2 * jp >= nkt) break;
                uint32_t bf[4];
                // matrices: (keys 16 jp + 0..7, k 0..7), (same keys, k 8..15), (keys + 8, k 0..7), (keys + 8, k 8..15)
                const int mrow = jp * 16 + (lane & 7) + ((lane >> 4) << 3), mcol = kk * 16 + ((lane >> 3) & 1) * 8;
                ldsm_x4(bf, sK + mrow * PITCH + mcol);
#pragma unroll
                for (int qi = 0; qi < NQ; ++qi) {
                    mma16816(s[2 * jp], qf[qi][kk], bf[0], bf[1]);
                    mma16816(s[2 * jp + 1], qf[qi][kk], bf[2], bf[3]);
                }
            }
        }
        // ---- scores in the log2 domain, maxima of the two rows
        float mx0 = -1e30f, mx1 = -1e30f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int kc = j * 8 + cq;                     // key (inside the chunk) of c0 / c2; c1 / c3 are the next key
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const bool live = k0 + kc + e < a.Lk;
                const float ks = sKs[kc + e], kz = sKz[kc + e], lv = sVs[kc + e];
                s[j][e] = live ? fmaf(s[j][e], ks, fmaf(-kz, qsum0, lv)) : -1e30f;
                s[j][2 + e] = live ? fmaf(s[j][2 + e], ks, fmaf(-kz, qsum1, lv)) : -1e30f;
                mx0 = fmaxf(mx0, s[j][e]);
                mx1 = fmaxf(mx1, s[j][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float al0 = mid_ex2(m0 - n0), al1 = mid_ex2(m1 - n1);
        m0 = n0; m1 = n1;
        l0 *= al0; l1 *= al1; cz0 *= al0; cz1 *= al1;
#pragma unroll
        for (int j = 0; j < 8; ++j) { o[j][0] *= al0; o[j][1] *= al0; o[j][2] *= al1; o[j][3] *= al1; }
        // ---- P (with the V scale folded in, rounded to fp16) as A fragments; normaliser and zero-point sums in fp32
        uint32_t pf[4][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int kc = j * 8 + cq;
            const float vr_a = sVr[kc], vr_b = sVr[kc + 1], vz_a = sVz[kc], vz_b = sVz[kc + 1];
            const float p00 = mid_ex2(s[j][0] - m0), p01 = mid_ex2(s[j][1] - m0);      // = softmax weight x V scale, at most 1
            const float p10 = mid_ex2(s[j][2] - m1), p11 = mid_ex2(s[j][3] - m1);
            l0 = fmaf(p00, vr_a, fmaf(p01, vr_b, l0));
            l1 = fmaf(p10, vr_a, fmaf(p11, vr_b, l1));
            const __half2 h0 = __floats2half2_rn(p00, p01), h1 = __floats2half2_rn(p10, p11);
            const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);     // the zero-point term uses the rounded P
            cz0 = fmaf(f0.x, vz_a, fmaf(f0.y, vz_b, cz0));
            cz1 = fmaf(f1.x, vz_a, fmaf(f1.y, vz_b, cz1));
            // key tiles 2t and 2t + 1 are the two k halves of MMA step t: a0 (r0, k), a1 (r1, k), a2 (r0, k + 8), a3 (r1, k + 8)
            pf[j >> 1][(j & 1) * 2] = *reinterpret_cast<const uint32_t*>(&h0);
            pf[j >> 1][(j & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&h1);
        }
        // ---- O += P V on codes: V is the B operand read transposed (rows = keys)
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            if (2 * t >= nkt) break;                         // P is zero from here on
#pragma unroll
            for (int np = 0; np < 4; ++np) {               // two 8-wide output tiles per ldmatrix.x4
                uint32_t bf[4];
                // matrices: (keys 16 t + 0..7, d 16 np + 0..7), (keys + 8, same d), (keys 0..7, d + 8), (keys + 8, d + 8)
                const int mrow = t * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, mcol = np * 16 + (lane >> 4) * 8;
                ldsm_x4_trans(bf, sV + mrow * PITCH + mcol);
                mma16816(o[2 * np], pf[t], bf[0], bf[1]);
                mma16816(o[2 * np + 1], pf[t], bf[2], bf[3]);
            }
        }
    }
    if (!warp_live) return;
    // ---- out = (O - sum_k P_k z_k) / sum_k p_k
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    cz0 += __shfl_xor_sync(0xffffffffu, cz0, 1); cz0 += __shfl_xor_sync(0xffffffffu, cz0, 2);
    cz1 += __shfl_xor_sync(0xffffffffu, cz1, 1); cz1 += __shfl_xor_sync(0xffffffffu, cz1, 2);
    const float i0 = 1.f / l0, i1 = 1.f / l1;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int col = j * 8 + cq;
        if (r0 < a.Lq) {
            const long long off = b * a.os_b + (long long)r0 * a.os_l + h * a.os_h + col;
            store_o_elem(a.out, a.o_dtype, off, (o[j][0] - cz0) * i0);
            store_o_elem(a.out, a.o_dtype, off + 1, (o[j][1] - cz0) * i0);
        }
        if (r1 < a.Lq) {
            const long long off = b * a.os_b + (long long)r1 * a.os_l + h * a.os_h + col;
            store_o_elem(a.out, a.o_dtype, off, (o[j][2] - cz1) * i1);
            store_o_elem(a.out, a.o_dtype, off + 1, (o[j][3] - cz1) * i1);
        }
    }
}

}  // namespace

bool attn_mid_eligible(const AttnArgs& a, int kb, int vb) {
    (void)kb; (void)vb;
    return a.D == 64 && a.kp.group == a.D && a.vp.group == a.D;      // one scale / zero-point per key
}

template <int KB, int VB, int WARPS>
static int launch_mid(AttnArgs& a, cudaStream_t st) {
    constexpr int MID_ROWS = WARPS * 16, MID_THREADS = WARPS * 32;
    const int nqt = (a.Lq + MID_ROWS - 1) / MID_ROWS;
    const long long blocks = (long long)a.B * a.H * nqt;
    if (blocks > 0x7fffffffLL) return fail(VARQ_ERR_UNSUPPORTED, "varq_attn_fwd: more than 2^31 thread blocks");
    a.n_qtiles = nqt;
    if (a.q_dtype == VARQ_F32) attn_mid_kernel<KB, VB, true, WARPS><<<(unsigned)blocks, MID_THREADS, 0, st>>>(a);
    else attn_mid_kernel<KB, VB, false, WARPS><<<(unsigned)blocks, MID_THREADS, 0, st>>>(a);
    VARQ_CUDA_TRY(cudaGetLastError());
    count_launches(1);
    return VARQ_OK;
}

int attn_mid_run(AttnArgs& a, int kb, int vb, cudaStream_t st) {
#define GO(K_, V_) if (kb == K_ && vb == V_) return a.Lq <= 32 ? launch_mid<K_, V_, 2>(a, st) : launch_mid<K_, V_, 4>(a, st);
    GO(8, 8) GO(8, 4) GO(8, 2) GO(4, 8) GO(4, 4) GO(4, 2) GO(2, 8) GO(2, 4) GO(2, 2)
#undef GO
    return fail(VARQ_ERR_ARG, "varq_attn_fwd: store bits must be 2, 4 or 8");
}

}  // namespace varq
