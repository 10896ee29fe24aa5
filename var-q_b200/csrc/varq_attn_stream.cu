// Attention over the packed cache for a handful of queries (four per CTA): a pure streaming kernel on CUDA cores.
//
// The packed K and V rows of a (sample, head) are contiguous, so a warp reads them straight from
// global memory, fully coalesced, with no shared-memory staging: every lane owns 16 consecutive
// head_dim values of one key (16 / 8 / 4 bytes at 8 / 4 / 2 bits), i.e. c/16 lanes per key and
// 32/(c/16) keys per warp step, the same mapping for K and V whatever their bit widths.  The 16
// codes become exact fp16 integers by byte permutes (no conversion instructions), are widened to
// fp32 and meet the lane's slice of the queries kept in registers.  A key's score is completed by
// c/16 - 1 shuffles; after that every lane runs its own online softmax over the keys it sees
// (no cross-lane traffic in the loop) and accumulates P V for its 16 head_dim values.  Lanes,
// warps and CTAs (key ranges) are merged at the end with the usual log-sum-exp rule; partial
// results of a split go to the caller's workspace in the layout of the small-query kernel.
// Applies when a lane's 16 head_dim values share one scale / zero-point, for K and for V: per-token-per-head,
// per-token and per-step groupings, and groups of 16, 32 or 64 along head_dim (every lane then applies its own
// group's parameters before the lanes of a key are summed).  Per-dim groupings stay on attn_small_kernel.
#include <cfloat>

#include "varq_attn.cuh"

namespace varq {

constexpr int ST_WARPS = 4;        // warps per CTA for caches that keep four warps busy ...
constexpr int ST_SHORT_KEYS = 64;  // ... and one-warp CTAs below this many keys (the first scales: a CTA's fixed cost dominates there)
constexpr int ST_QT = 4;          // query slots (matches the merge kernel's record layout)
constexpr int ST_UNROLL = 4;      // warp steps in flight

// ---- packed codes -> fp32 without conversion instructions.  A byte u placed in the low byte of 0x4B000000 is the float
// 2^23 + u; codes are biased to unsigned bytes first, so one byte permute per value builds 2^23 + BIAS + code and one packed
// fp32 add per two values removes 2^23 + BIAS.  Arithmetic then runs on packed fp32 pairs (two FMAs per instruction).
__device__ __forceinline__ void st_fma2(float& d0, float& d1, float a0, float a1, float b0, float b1) {      // d += a * b, pairwise
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rd, {%0, %1};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rd;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "+f"(d0), "+f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void st_add2(float& d0, float& d1, float b) {                                     // d += b, pairwise
    asm("{\n\t.reg .b64 rb, rd;\n\tmov.b64 rb, {%2, %2};\n\tmov.b64 rd, {%0, %1};\n\t"
        "add.rn.f32x2 rd, rd, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "+f"(d0), "+f"(d1) : "f"(b));
}
__device__ __forceinline__ float st_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// byte `B` of u -> 2^23 + that byte, as a float
template <int B> __device__ __forceinline__ float st_byte_f(uint32_t u) { return __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540 + B)); }
__device__ __forceinline__ void st_bytes_f4(uint32_t u, float* f) {
    f[0] = st_byte_f<0>(u); f[1] = st_byte_f<1>(u); f[2] = st_byte_f<2>(u); f[3] = st_byte_f<3>(u);
}

// 16 codes of `BITS` bits (little-endian fields) -> 16 floats holding the signed integers, in field order
template <int BITS> struct StCodes;
template <> struct StCodes<8> {
    using Raw = uint4;
    static __device__ __forceinline__ Raw load(const int32_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
    static __device__ __forceinline__ void cvt(const Raw& r, float* f) {
        st_bytes_f4(r.x ^ 0x80808080u, f);
        st_bytes_f4(r.y ^ 0x80808080u, f + 4);
        st_bytes_f4(r.z ^ 0x80808080u, f + 8);
        st_bytes_f4(r.w ^ 0x80808080u, f + 12);
#pragma unroll
        for (int j = 0; j < 16; j += 2) st_add2(f[j], f[j + 1], -(8388608.f + 128.f));
    }
};
template <> struct StCodes<4> {
    using Raw = uint2;
    static __device__ __forceinline__ Raw load(const int32_t* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }
    static __device__ __forceinline__ void word(uint32_t w, float* f) {
        const uint32_t x = w ^ 0x88888888u;
        const uint32_t lo = x & 0x0F0F0F0Fu, hi = (x >> 4) & 0x0F0F0F0Fu;      // fields 0,2,4,6 / 1,3,5,7
        f[0] = st_byte_f<0>(lo); f[1] = st_byte_f<0>(hi); f[2] = st_byte_f<1>(lo); f[3] = st_byte_f<1>(hi);
        f[4] = st_byte_f<2>(lo); f[5] = st_byte_f<2>(hi); f[6] = st_byte_f<3>(lo); f[7] = st_byte_f<3>(hi);
    }
    static __device__ __forceinline__ void cvt(const Raw& r, float* f) {
        word(r.x, f); word(r.y, f + 8);
#pragma unroll
        for (int j = 0; j < 16; j += 2) st_add2(f[j], f[j + 1], -(8388608.f + 8.f));
    }
};
template <> struct StCodes<2> {
    using Raw = uint32_t;
    static __device__ __forceinline__ Raw load(const int32_t* p) { return (uint32_t)__ldg(p); }
    static __device__ __forceinline__ void cvt(const Raw& w, float* f) {
        const uint32_t x = w ^ 0xAAAAAAAAu;
        const uint32_t t0 = x & 0x03030303u, t1 = (x >> 2) & 0x03030303u;       // fields 0,4,8,12 / 1,5,9,13
        const uint32_t t2 = (x >> 4) & 0x03030303u, t3 = (x >> 6) & 0x03030303u; // fields 2,6,10,14 / 3,7,11,15
        f[0] = st_byte_f<0>(t0); f[1] = st_byte_f<0>(t1); f[2] = st_byte_f<0>(t2); f[3] = st_byte_f<0>(t3);
        f[4] = st_byte_f<1>(t0); f[5] = st_byte_f<1>(t1); f[6] = st_byte_f<1>(t2); f[7] = st_byte_f<1>(t3);
        f[8] = st_byte_f<2>(t0); f[9] = st_byte_f<2>(t1); f[10] = st_byte_f<2>(t2); f[11] = st_byte_f<2>(t3);
        f[12] = st_byte_f<3>(t0); f[13] = st_byte_f<3>(t1); f[14] = st_byte_f<3>(t2); f[15] = st_byte_f<3>(t3);
#pragma unroll
        for (int j = 0; j < 16; j += 2) st_add2(f[j], f[j + 1], -(8388608.f + 2.f));
    }
};

template <int KB, int VB, int D, int QT, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) attn_stream_kernel(AttnArgs a, int keys_per_split) {
    constexpr int LPK = D / 16;               // lanes per key
    constexpr int KPS = 32 / LPK;             // keys per warp step
    constexpr int KW = 16 * KB / 32, VW = 16 * VB / 32;   // packed words per lane and step
    __shared__ float s_part[WARPS][QT][D + 2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned blk = blockIdx.x;            // query tile fastest (tiles of one key range run together and share it in L2)
    const int qtile = (int)(blk % (unsigned)a.n_qtiles);
    const int split = (int)((blk / (unsigned)a.n_qtiles) % (unsigned)a.splits);
    const int bh = (int)(blk / ((unsigned)a.splits * (unsigned)a.n_qtiles)), b = bh / a.H, h = bh - b * a.H;
    const int q0 = qtile * ST_QT;
    const int nq = min(QT, a.Lq - q0);
    const int chunk = lane % LPK, kin = lane / LPK;      // head_dim slice and key slot of this lane
    const int d0 = chunk * 16;

    // the lane's slice of the queries, pre-scaled by softmax_scale * log2(e), and its sum (zero-point term of the lane's group)
    float q[QT][16], qsum[QT];
#pragma unroll
    for (int qi = 0; qi < QT; ++qi) {
        float part = 0.f;
        float lo8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, hi8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (qi < nq) {
            const long long off = b * a.qs_b + (long long)(q0 + qi) * a.qs_l + h * a.qs_h + d0;
            load_q8(a.q, a.q_dtype, off, lo8);
            load_q8(a.q, a.q_dtype, off + 8, hi8);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            q[qi][j] = lo8[j] * a.scale_log2;
            q[qi][j + 8] = hi8[j] * a.scale_log2;
            part += q[qi][j] + q[qi][j + 8];
        }
        qsum[qi] = part;
    }

    float m_run[QT], l_run[QT], corr[QT], acc[QT][16];
#pragma unroll
    for (int qi = 0; qi < QT; ++qi) {
        m_run[qi] = -FLT_MAX; l_run[qi] = 0.f; corr[qi] = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[qi][j] = 0.f;
    }

    // key range of this warp inside the CTA's split
    const int split_begin = split * keys_per_split;
    const int split_end = min(a.Lk, split_begin + keys_per_split);
    const int per_warp = ((split_end - split_begin + WARPS * KPS - 1) / (WARPS * KPS)) * KPS;
    const int w_begin = split_begin + warp * per_warp;
    const int w_end = min(split_end, w_begin + per_warp);

    const int32_t* kbase = a.kc + b * a.ks_b + h * a.ks_h + chunk * KW;
    const int32_t* vbase = a.vc + b * a.vs_b + h * a.vs_h + chunk * VW;
    const bool kz_on = a.kp.zp != nullptr, vz_on = a.vp.zp != nullptr;

    for (int k0 = w_begin; k0 < w_end; k0 += KPS * ST_UNROLL) {
        typename StCodes<KB>::Raw kr[ST_UNROLL];
        typename StCodes<VB>::Raw vr[ST_UNROLL];
        float ksc[ST_UNROLL], kzp[ST_UNROLL], vsc[ST_UNROLL], vzp[ST_UNROLL];
        bool ok[ST_UNROLL];
#pragma unroll
        for (int u = 0; u < ST_UNROLL; ++u) {
            const int key = k0 + u * KPS + kin;
            ok[u] = key < w_end;
            ksc[u] = 0.f; kzp[u] = 0.f; vsc[u] = 0.f; vzp[u] = 0.f;
            if (ok[u]) {
                kr[u] = StCodes<KB>::load(kbase + (long long)key * a.ks_l);
                vr[u] = StCodes<VB>::load(vbase + (long long)key * a.vs_l);
                const long long pk = a.kp.index(b, a.kp.row(key), h, d0), pv = a.vp.index(b, a.vp.row(key), h, d0);
                ksc[u] = __ldg(a.kp.scale + pk);
                vsc[u] = __ldg(a.vp.scale + pv);
                if (kz_on) kzp[u] = __ldg(a.kp.zp + pk);
                if (vz_on) vzp[u] = __ldg(a.vp.zp + pv);
            } else {
                kr[u] = typename StCodes<KB>::Raw();
                vr[u] = typename StCodes<VB>::Raw();
            }
        }
#pragma unroll
        for (int u = 0; u < ST_UNROLL; ++u) {
            if (k0 + u * KPS >= w_end) break;          // warp-uniform: no key of this step exists
            float kf[16];
            StCodes<KB>::cvt(kr[u], kf);
            float s[QT];
#pragma unroll
            for (int qi = 0; qi < QT; ++qi) {
                float da = 0.f, db = 0.f;
#pragma unroll
                for (int j = 0; j < 16; j += 2) st_fma2(da, db, q[qi][j], q[qi][j + 1], kf[j], kf[j + 1]);
                // this lane's group: scale_k * (q . code - zp_k * sum q) over its 16 values, already in log2 units
                s[qi] = ksc[u] * ((da + db) - kzp[u] * qsum[qi]);
            }
#pragma unroll
            for (int m = 1; m < LPK; m <<= 1)
#pragma unroll
                for (int qi = 0; qi < QT; ++qi) s[qi] += __shfl_xor_sync(0xffffffffu, s[qi], m);
            float vf[16];
            StCodes<VB>::cvt(vr[u], vf);
#pragma unroll
            for (int qi = 0; qi < QT; ++qi) {
                const float x = ok[u] ? s[qi] : -FLT_MAX;
                if (x > m_run[qi] + 8.f) {           // lazy rescale: p stays below 2^8
                    const float alpha = st_ex2(m_run[qi] - x);
                    m_run[qi] = x;
                    l_run[qi] *= alpha;
                    corr[qi] *= alpha;
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[qi][j] *= alpha;
                }
                const float p = ok[u] ? st_ex2(x - m_run[qi]) : 0.f;
                l_run[qi] += p;
                const float pv = p * vsc[u];
                corr[qi] = fmaf(pv, vzp[u], corr[qi]);
#pragma unroll
                for (int j = 0; j < 16; j += 2) st_fma2(acc[qi][j], acc[qi][j + 1], pv, pv, vf[j], vf[j + 1]);
            }
        }
    }

    // ---- merge the key slots of the warp (lanes that share a head_dim slice)
#pragma unroll
    for (int qi = 0; qi < QT; ++qi) {
#pragma unroll
        for (int off = LPK; off < 32; off <<= 1) {
            const float m_o = __shfl_xor_sync(0xffffffffu, m_run[qi], off);
            const float M = fmaxf(m_run[qi], m_o);
            const float wa = exp2f(m_run[qi] - M), wb = exp2f(m_o - M);
            l_run[qi] = l_run[qi] * wa + __shfl_xor_sync(0xffffffffu, l_run[qi], off) * wb;
            corr[qi] = corr[qi] * wa + __shfl_xor_sync(0xffffffffu, corr[qi], off) * wb;
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[qi][j] = acc[qi][j] * wa + __shfl_xor_sync(0xffffffffu, acc[qi][j], off) * wb;
            m_run[qi] = M;
        }
        if (kin == 0) {
#pragma unroll
            for (int j = 0; j < 16; ++j) s_part[warp][qi][d0 + j] = acc[qi][j] - corr[qi];
            if (chunk == 0) { s_part[warp][qi][D] = m_run[qi]; s_part[warp][qi][D + 1] = l_run[qi]; }
        }
    }
    __syncthreads();
    // ---- merge the warps, then write the output or this split's partial record
    for (int i = tid; i < QT * D; i += WARPS * 32) {
        const int qi = i / D, d = i - qi * D;
        if (qi >= nq) continue;
        float M = -FLT_MAX;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, s_part[w][qi][D]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float wt = exp2f(s_part[w][qi][D] - M);
            num = fmaf(wt, s_part[w][qi][d], num);
            den = fmaf(wt, s_part[w][qi][D + 1], den);
        }
        if (a.splits == 1) {
            store_o_elem(a.out, a.o_dtype, b * a.os_b + (long long)(q0 + qi) * a.os_l + h * a.os_h + d, num / den);
        } else {
            float* rec = a.ws + (((long long)bh * a.n_qtiles + qtile) * a.splits + split) * (ST_QT * (2 + D));
            rec[ST_QT * 2 + qi * D + d] = num;
            if (d == 0) { rec[qi] = M; rec[ST_QT + qi] = den; }
        }
    }
}

// ---------------------------------------------------------------- host side
bool attn_stream_eligible(const AttnArgs& a, int kb, int vb) {
    if (a.D != 64 && a.D != 128) return false;
    if (a.kp.group % 16 || a.vp.group % 16) return false;           // a lane's 16 values share their parameters
    const int kw = 16 * kb / 32, vw = 16 * vb / 32;                   // words per lane: loads must be naturally aligned
    auto aligned = [](const void* p, long long sb, long long sl, long long sh, int words) {
        return (reinterpret_cast<uintptr_t>(p) % (words * 4) == 0) && sb % words == 0 && sl % words == 0 && sh % words == 0;
    };
    return aligned(a.kc, a.ks_b, a.ks_l, a.ks_h, kw) && aligned(a.vc, a.vs_b, a.vs_l, a.vs_h, vw);
}

static int stream_splits(const AttnArgs& a, int& keys_per_split) {
    if (a.Lk <= ST_SHORT_KEYS) { keys_per_split = ST_SHORT_KEYS; return 1; }     // one warp walks the whole cache
    const int kps = 32 / (a.D / 16);
    const int unit = ST_WARPS * kps * ST_UNROLL;                       // keys one CTA consumes per loop trip
    const long long base = (long long)a.B * a.H * ((a.Lq + ST_QT - 1) / ST_QT);
    const long long target = (long long)sm_count() * 8;
    long long s = (target + base - 1) / base;
    const long long max_s = (a.Lk + unit - 1) / unit;
    if (s > max_s) s = max_s;
    if (s < 1) s = 1;
    keys_per_split = (int)(((a.Lk + s - 1) / s + unit - 1) / unit) * unit;
    return (a.Lk + keys_per_split - 1) / keys_per_split;
}

size_t attn_stream_workspace_bytes(int B, int H, int Lq, int Lk, int D) {
    AttnArgs a;
    a.B = B; a.H = H; a.Lq = Lq; a.Lk = Lk; a.D = D;
    int kps;
    const int splits = stream_splits(a, kps);
    if (splits <= 1) return 0;
    return (size_t)B * H * ((Lq + ST_QT - 1) / ST_QT) * splits * (ST_QT * (2 + D)) * sizeof(float);
}

void attn_small_merge_launch(const AttnArgs& a, int n_qtiles, cudaStream_t st);

template <int KB, int VB, int D>
static int launch_stream(AttnArgs& a, int keys_per_split, cudaStream_t st) {
    const int nqt = (a.Lq + ST_QT - 1) / ST_QT;
    const long long blocks_1d = (long long)a.B * a.H * nqt * a.splits;
    if (blocks_1d > 0x7fffffffLL) return fail(VARQ_ERR_UNSUPPORTED, "varq_attn_fwd: more than 2^31 thread blocks");
    a.n_qtiles = nqt;
    const unsigned grid = (unsigned)blocks_1d;
    const int qmax = a.Lq < ST_QT ? a.Lq : ST_QT;
    if (a.Lk <= ST_SHORT_KEYS) {
        if (qmax == 1) attn_stream_kernel<KB, VB, D, 1, 1><<<grid, 32, 0, st>>>(a, keys_per_split);
        else if (qmax == 2) attn_stream_kernel<KB, VB, D, 2, 1><<<grid, 32, 0, st>>>(a, keys_per_split);
        else attn_stream_kernel<KB, VB, D, 4, 1><<<grid, 32, 0, st>>>(a, keys_per_split);
    } else {
        if (qmax == 1) attn_stream_kernel<KB, VB, D, 1, ST_WARPS><<<grid, ST_WARPS * 32, 0, st>>>(a, keys_per_split);
        else if (qmax == 2) attn_stream_kernel<KB, VB, D, 2, ST_WARPS><<<grid, ST_WARPS * 32, 0, st>>>(a, keys_per_split);
        else attn_stream_kernel<KB, VB, D, 4, ST_WARPS><<<grid, ST_WARPS * 32, 0, st>>>(a, keys_per_split);
    }
    VARQ_CUDA_TRY(cudaGetLastError());
    count_launches(1);
    if (a.splits > 1) {
        attn_small_merge_launch(a, nqt, st);
        VARQ_CUDA_TRY(cudaGetLastError());
        count_launches(1);
    }
    return VARQ_OK;
}

int attn_stream_run(AttnArgs& a, int kb, int vb, void* ws, size_t ws_bytes, cudaStream_t st) {
    int keys_per_split = 0;
    a.splits = stream_splits(a, keys_per_split);
    if (a.splits > 1) {
        const size_t need = attn_stream_workspace_bytes(a.B, a.H, a.Lq, a.Lk, a.D);
        if (!ws || ws_bytes < need)
            return fail(VARQ_ERR_WORKSPACE, "varq_attn_fwd: workspace of %zu bytes needed, %zu given", need, ws_bytes);
        a.ws = reinterpret_cast<float*>(ws);
    }
#define GO(K_, V_)                                                              \
    if (kb == K_ && vb == V_) {                                                 \
        if (a.D == 64) return launch_stream<K_, V_, 64>(a, keys_per_split, st); \
        return launch_stream<K_, V_, 128>(a, keys_per_split, st);               \
    }
    GO(8, 8) GO(8, 4) GO(8, 2) GO(4, 8) GO(4, 4) GO(4, 2) GO(2, 8) GO(2, 4) GO(2, 2)
#undef GO
    return fail(VARQ_ERR_ARG, "varq_attn_fwd: store bits must be 2, 4 or 8");
}

}  // namespace varq
