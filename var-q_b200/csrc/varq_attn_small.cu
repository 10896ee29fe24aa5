// Attention over the packed cache for small query counts (the early scales): CUDA cores only.
//
// A CTA of 128 threads owns one (batch, head), a tile of QT queries and a contiguous range of
// keys.  Packed K and V tiles of 128 keys are staged into shared memory with cp.async (double
// buffered); the scores are computed with one key per thread on the integer codes, the scale and
// zero-point of a group are applied once per group:
//     s = sum_g scale_g * ( sum_{d in g} q_d * code_d  -  zp_g * sum_{d in g} q_d )
// and the PV product with one packed V word per thread.  Key ranges are split across CTAs when
// (batch x heads x query tiles) cannot fill the machine; partial (max, sum, numerator) triples go
// to the caller's workspace and a second kernel merges them.
#include <cfloat>

#include "varq_attn.cuh"

namespace varq {

constexpr int A1_THREADS = 128;
constexpr int A1_TILE = 128;   // keys per tile
constexpr int A1_QT = 4;       // queries per CTA

// 32-bit words of the float section of shared memory, rounded to 16 bytes
__host__ __device__ inline int a1_float_words(int D, int gk) {
    return (A1_QT * D + A1_QT * gk + A1_QT * A1_TILE + 8 * A1_QT + 3) & ~3;
}


__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// stage `n` rows of `words` int32 each (row r at src + r*src_pitch) into dst rows of dst_pitch words
__device__ __forceinline__ void stage_tile(uint32_t* dst, int dst_pitch, const int32_t* src, long long src_pitch,
                                           int n, int words, bool use16) {
    if (use16) {
        const int cpr = words >> 2;
        for (int i = threadIdx.x; i < n * cpr; i += A1_THREADS) {
            const int r = i / cpr, c = i - r * cpr;
            cp_async16(dst + r * dst_pitch + c * 4, src + r * src_pitch + c * 4);
        }
    } else {
        for (int i = threadIdx.x; i < n * words; i += A1_THREADS) {
            const int r = i / words, c = i - r * words;
            cp_async4(dst + r * dst_pitch + c, src + r * src_pitch + c);
        }
    }
}

template <int KB, int VB>
__global__ void __launch_bounds__(A1_THREADS) attn_small_kernel(AttnArgs a) {
    constexpr int KV = 32 / KB, VV = 32 / VB;   // codes per K / V word
    constexpr int QT = A1_QT;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int D = a.D;
    const int gk = D / a.kp.group;              // K groups per row (group >= 1)
    // shared memory carve-up
    float* sQ = reinterpret_cast<float*>(smem_raw);                 // [QT][D]   (scaled by softmax_scale*log2e)
    float* sQsum = sQ + QT * D;                                      // [QT][gk]
    float* sP = sQsum + QT * gk;                                     // [QT][TILE]
    float* sRed = sP + QT * A1_TILE;                                 // [2][4 warps][QT]
    uint32_t* sK = reinterpret_cast<uint32_t*>(smem_raw) + a1_float_words(D, gk);   // [2][TILE][kpitch]
    uint32_t* sV = sK + 2 * A1_TILE * a.kpitch;                      // [2][TILE][wv]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned blk = blockIdx.x;            // split fastest, then query tile, then (sample, head)
    const int split = (int)(blk % (unsigned)a.splits);
    const int qtile = (int)((blk / (unsigned)a.splits) % (unsigned)a.n_qtiles);
    const int bh = (int)(blk / ((unsigned)a.splits * (unsigned)a.n_qtiles)), b = bh / a.H, h = bh - b * a.H;
    const int q0 = qtile * QT;
    const int nq = min(QT, a.Lq - q0);

    // ---- queries -> shared (scaled), per-group sums
    for (int i = tid; i < QT * D; i += A1_THREADS) {
        const int qi = i / D, d = i - qi * D;
        float v = 0.f;
        if (qi < nq) v = load_q_elem(a.q, a.q_dtype, b * a.qs_b + (long long)(q0 + qi) * a.qs_l + h * a.qs_h + d) * a.scale_log2;
        sQ[i] = v;
    }
    __syncthreads();
    for (int i = tid; i < QT * gk; i += A1_THREADS) {
        const int qi = i / gk, g = i - qi * gk;
        float s = 0.f;
        for (int d = g * a.kp.group; d < (g + 1) * a.kp.group; ++d) s += sQ[qi * D + d];
        sQsum[i] = s;
    }

    const int n_tiles_total = (a.Lk + A1_TILE - 1) / A1_TILE;
    const int t_begin = split * a.tiles_per_split;
    const int t_end = min(n_tiles_total, t_begin + a.tiles_per_split);

    const int32_t* kbase = a.kc + b * a.ks_b + h * a.ks_h;
    const int32_t* vbase = a.vc + b * a.vs_b + h * a.vs_h;

    auto issue = [&](int t, int buf) {
        const int k0 = t * A1_TILE;
        const int n = min(A1_TILE, a.Lk - k0);
        stage_tile(sK + buf * A1_TILE * a.kpitch, a.kpitch, kbase + (long long)k0 * a.ks_l, a.ks_l, n, a.wk, a.k16);
        stage_tile(sV + buf * A1_TILE * a.wv, a.wv, vbase + (long long)k0 * a.vs_l, a.vs_l, n, a.wv, a.v16);
        cp_async_commit();
    };

    // PV ownership: thread -> (key subset ks, V word wv_i)
    const int wv_i = tid % a.wv;
    const int ks = tid / a.wv;
    const int ks_count = A1_THREADS / a.wv;       // host guarantees wv divides 128
    float acc[QT][VV];
#pragma unroll
    for (int qi = 0; qi < QT; ++qi)
#pragma unroll
        for (int j = 0; j < VV; ++j) acc[qi][j] = 0.f;
    float m_run[QT], l_run[QT];
#pragma unroll
    for (int qi = 0; qi < QT; ++qi) { m_run[qi] = -FLT_MAX; l_run[qi] = 0.f; }

    if (t_begin < t_end) issue(t_begin, 0);
    const bool k_uniform = (a.kp.group % KV) == 0;
    const bool v_uniform = (a.vp.group % VV) == 0;

    for (int t = t_begin; t < t_end; ++t) {
        const int buf = (t - t_begin) & 1;
        if (t + 1 < t_end) { issue(t + 1, buf ^ 1); cp_async_wait<1>(); }
        else               { cp_async_wait<0>(); }
        __syncthreads();

        const int k0 = t * A1_TILE;
        const int n = min(A1_TILE, a.Lk - k0);

        // ---- scores: thread tid <-> key k0 + tid
        float s[QT];
#pragma unroll
        for (int qi = 0; qi < QT; ++qi) s[qi] = -FLT_MAX;
        if (tid < n) {
            const uint32_t* krow = sK + (buf * A1_TILE + tid) * a.kpitch;
            const int row = a.kp.row(k0 + tid);
#pragma unroll
            for (int qi = 0; qi < QT; ++qi) s[qi] = 0.f;
            if (k_uniform) {
                const int wpg = a.kp.group / KV;     // words per group
                const bool wide = (a.wk & 3) == 0;
                float part[QT];
#pragma unroll
                for (int qi = 0; qi < QT; ++qi) part[qi] = 0.f;
                for (int w0 = 0; w0 < a.wk; w0 += 4) {
                    uint32_t wd[4];
                    if (wide) {
                        *reinterpret_cast<uint4*>(wd) = *reinterpret_cast<const uint4*>(krow + w0);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) wd[i] = (w0 + i < a.wk) ? krow[w0 + i] : 0u;
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int wi = w0 + i;
                        if (wi < a.wk) {
                            const uint32_t word = wd[i];
                            const float* qd = sQ + wi * KV;
#pragma unroll
                            for (int j = 0; j < KV; j += 4) {
                                const float c0 = (float)field<KB>(word, j), c1 = (float)field<KB>(word, j + 1),
                                            c2 = (float)field<KB>(word, j + 2), c3 = (float)field<KB>(word, j + 3);
#pragma unroll
                                for (int qi = 0; qi < QT; ++qi) {
                                    const float4 qq = *reinterpret_cast<const float4*>(qd + qi * D + j);
                                    part[qi] = fmaf(qq.x, c0, fmaf(qq.y, c1, fmaf(qq.z, c2, fmaf(qq.w, c3, part[qi]))));
                                }
                            }
                            if (((wi + 1) % wpg) == 0) {   // group complete: apply its scale and zero-point
                                const int g = wi / wpg;
                                const long long pi = a.kp.index(b, row, h, g * a.kp.group);
                                const float sc = __ldg(a.kp.scale + pi);
                                const float z = a.kp.zp ? __ldg(a.kp.zp + pi) : 0.f;
#pragma unroll
                                for (int qi = 0; qi < QT; ++qi) {
                                    s[qi] = fmaf(sc, part[qi] - z * sQsum[qi * gk + g], s[qi]);
                                    part[qi] = 0.f;
                                }
                            }
                        }
                    }
                }
            } else {
                for (int wi = 0; wi < a.wk; ++wi) {
                    const uint32_t word = krow[wi];
#pragma unroll
                    for (int j = 0; j < KV; ++j) {
                        const int d = wi * KV + j;
                        const long long pi = a.kp.index(b, row, h, d);
                        const float sc = __ldg(a.kp.scale + pi);
                        const float z = a.kp.zp ? __ldg(a.kp.zp + pi) : 0.f;
                        const float kd = ((float)field<KB>(word, j) - z) * sc;
#pragma unroll
                        for (int qi = 0; qi < QT; ++qi) s[qi] = fmaf(sQ[qi * D + d], kd, s[qi]);
                    }
                }
            }
        }
        // ---- tile max
        float mt[QT];
#pragma unroll
        for (int qi = 0; qi < QT; ++qi) {
            float v = s[qi];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
            mt[qi] = v;
        }
        if (lane == 0) {
#pragma unroll
            for (int qi = 0; qi < QT; ++qi) sRed[warp * QT + qi] = mt[qi];
        }
        __syncthreads();
        float p[QT], alpha[QT];
#pragma unroll
        for (int qi = 0; qi < QT; ++qi) {
            const float m_tile = fmaxf(fmaxf(sRed[qi], sRed[QT + qi]), fmaxf(sRed[2 * QT + qi], sRed[3 * QT + qi]));
            const float m_new = fmaxf(m_run[qi], m_tile);
            alpha[qi] = exp2f(m_run[qi] - m_new);
            m_run[qi] = m_new;
            p[qi] = (tid < n) ? exp2f(s[qi] - m_new) : 0.f;
            sP[qi * A1_TILE + tid] = p[qi];
            float v = p[qi];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) sRed[4 * QT + warp * QT + qi] = v;
        }
        __syncthreads();
#pragma unroll
        for (int qi = 0; qi < QT; ++qi) {
            const float sum = sRed[4 * QT + qi] + sRed[5 * QT + qi] + sRed[6 * QT + qi] + sRed[7 * QT + qi];
            l_run[qi] = l_run[qi] * alpha[qi] + sum;
        }

        // ---- PV: thread owns V word wv_i of keys ks, ks + ks_count, ...
#pragma unroll
        for (int qi = 0; qi < QT; ++qi)
#pragma unroll
            for (int j = 0; j < VV; ++j) acc[qi][j] *= alpha[qi];
        const uint32_t* vt = sV + buf * A1_TILE * a.wv;
        for (int key = ks; key < n; key += ks_count) {
            const uint32_t word = vt[key * a.wv + wv_i];
            const int row = a.vp.row(k0 + key);
            float vv[VV];
            if (v_uniform) {
                const long long pi = a.vp.index(b, row, h, wv_i * VV);
                const float sc = __ldg(a.vp.scale + pi);
                const float z = a.vp.zp ? __ldg(a.vp.zp + pi) : 0.f;
#pragma unroll
                for (int j = 0; j < VV; ++j) vv[j] = ((float)field<VB>(word, j) - z) * sc;
            } else {
#pragma unroll
                for (int j = 0; j < VV; ++j) {
                    const long long pi = a.vp.index(b, row, h, wv_i * VV + j);
                    const float sc = __ldg(a.vp.scale + pi);
                    const float z = a.vp.zp ? __ldg(a.vp.zp + pi) : 0.f;
                    vv[j] = ((float)field<VB>(word, j) - z) * sc;
                }
            }
#pragma unroll
            for (int qi = 0; qi < QT; ++qi) {
                const float pq = sP[qi * A1_TILE + key];
#pragma unroll
                for (int j = 0; j < VV; ++j) acc[qi][j] = fmaf(pq, vv[j], acc[qi][j]);
            }
        }
        __syncthreads();   // sP, sRed and the tile buffers are reused by the next iteration
    }

    // ---- fold the key subsets: reuse the K/V staging area as [ks_count][QT][D] floats
    float* sO = reinterpret_cast<float*>(sK);
#pragma unroll
    for (int qi = 0; qi < QT; ++qi)
#pragma unroll
        for (int j = 0; j < VV; ++j) sO[(ks * QT + qi) * D + wv_i * VV + j] = acc[qi][j];
    __syncthreads();
    for (int i = tid; i < QT * D; i += A1_THREADS) {
        const int qi = i / D, d = i - qi * D;
        if (qi >= nq) continue;
        float o = 0.f;
        for (int k = 0; k < ks_count; ++k) o += sO[(k * QT + qi) * D + d];
        // m_run / l_run are identical in every thread
        float m = 0.f, l = 0.f;
#pragma unroll
        for (int x = 0; x < QT; ++x) if (x == qi) { m = m_run[x]; l = l_run[x]; }
        if (a.splits == 1) {
            store_o_elem(a.out, a.o_dtype, b * a.os_b + (long long)(q0 + qi) * a.os_l + h * a.os_h + d, o / l);
        } else {
            float* rec = a.ws + (((long long)bh * a.n_qtiles + qtile) * a.splits + split) * (QT * (2 + D));
            rec[QT * 2 + qi * D + d] = o;
            if (d == 0) { rec[qi] = m; rec[QT + qi] = l; }
        }
    }
}

// merge the per-split partials: one thread per output element
__global__ void attn_small_merge_kernel(AttnArgs a, int n_qtiles) {
    constexpr int QT = A1_QT;
    const long long total = (long long)a.B * a.H * a.Lq * a.D;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int d = (int)(i % a.D);
        long long r = i / a.D;
        const int qg = (int)(r % a.Lq); r /= a.Lq;
        const int bh = (int)r, b = bh / a.H, h = bh - b * a.H;
        const int qtile = qg / QT, qi = qg - qtile * QT;
        const float* rec0 = a.ws + ((long long)bh * n_qtiles + qtile) * a.splits * (QT * (2 + a.D));
        float M = -FLT_MAX;
        for (int s = 0; s < a.splits; ++s) M = fmaxf(M, rec0[s * (QT * (2 + a.D)) + qi]);
        float num = 0.f, den = 0.f;
        for (int s = 0; s < a.splits; ++s) {
            const float* rec = rec0 + s * (QT * (2 + a.D));
            const float w = exp2f(rec[qi] - M);
            num = fmaf(w, rec[QT * 2 + qi * a.D + d], num);
            den = fmaf(w, rec[QT + qi], den);
        }
        store_o_elem(a.out, a.o_dtype, b * a.os_b + (long long)qg * a.os_l + h * a.os_h + d, num / den);
    }
}

void attn_small_merge_launch(const AttnArgs& a, int n_qtiles, cudaStream_t st) {
    const long long total = (long long)a.B * a.H * a.Lq * a.D;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    attn_small_merge_kernel<<<(unsigned)blocks, 256, 0, st>>>(a, n_qtiles);
}

static int pick_splits(int B, int H, int Lq, int Lk, int& tiles_per_split) {
    const int n_tiles = (Lk + A1_TILE - 1) / A1_TILE;
    const long long base = (long long)B * H * ((Lq + A1_QT - 1) / A1_QT);
    const long long target = (long long)sm_count() * 6;
    long long s = (target + base - 1) / base;
    if (s > n_tiles) s = n_tiles;
    if (s < 1) s = 1;
    tiles_per_split = (int)((n_tiles + s - 1) / s);
    return (n_tiles + tiles_per_split - 1) / tiles_per_split;
}

size_t attn_small_workspace_bytes(int B, int H, int Lq, int Lk, int D) {
    int tps;
    const int splits = pick_splits(B, H, Lq, Lk, tps);
    if (splits <= 1) return 0;
    const long long nqt = (Lq + A1_QT - 1) / A1_QT;
    return (size_t)B * H * nqt * splits * (A1_QT * (2 + D)) * sizeof(float);
}

static size_t attn_small_smem(const AttnArgs& a) {
    const int gk = a.D / a.kp.group;
    const size_t floats = (size_t)a1_float_words(a.D, gk);
    size_t words = (size_t)2 * A1_TILE * a.kpitch + (size_t)2 * A1_TILE * a.wv;
    const size_t fold = (size_t)(A1_THREADS / a.wv) * A1_QT * a.D;   // floats, aliased on the staging area
    if (words < fold) words = fold;
    return (floats + words) * 4;
}

template <int KB, int VB>
static int launch_small(AttnArgs& a, cudaStream_t st) {
    const size_t smem = attn_small_smem(a);
    if (smem > 200 * 1024) return fail(VARQ_ERR_UNSUPPORTED, "varq_attn_fwd: head_dim %d needs %zu bytes of shared memory", a.D, smem);
    static bool configured[64] = {false};    // per device; the attribute is sticky, set it outside any stream capture
    int dev = 0;
    VARQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        VARQ_CUDA_TRY(cudaFuncSetAttribute(attn_small_kernel<KB, VB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int nqt = (a.Lq + A1_QT - 1) / A1_QT;
    const long long blocks_1d = (long long)a.B * a.H * nqt * a.splits;
    if (blocks_1d > 0x7fffffffLL) return fail(VARQ_ERR_UNSUPPORTED, "varq_attn_fwd: more than 2^31 thread blocks");
    a.n_qtiles = nqt;
    attn_small_kernel<KB, VB><<<(unsigned)blocks_1d, A1_THREADS, smem, st>>>(a);
    VARQ_CUDA_TRY(cudaGetLastError());
    count_launches(1);
    if (a.splits > 1) {
        const long long total = (long long)a.B * a.H * a.Lq * a.D;
        long long blocks = (total + 255) / 256;
        const long long cap = (long long)sm_count() * 8;
        if (blocks > cap) blocks = cap;
        attn_small_merge_kernel<<<(unsigned)blocks, 256, 0, st>>>(a, nqt);
        VARQ_CUDA_TRY(cudaGetLastError());
        count_launches(1);
    }
    return VARQ_OK;
}

int attn_small_run(AttnArgs& a, int kb, int vb, void* ws, size_t ws_bytes, cudaStream_t st) {
    a.splits = pick_splits(a.B, a.H, a.Lq, a.Lk, a.tiles_per_split);
    if (a.splits > 1) {
        const size_t need = attn_small_workspace_bytes(a.B, a.H, a.Lq, a.Lk, a.D);
        if (!ws || ws_bytes < need)
            return fail(VARQ_ERR_WORKSPACE, "varq_attn_fwd: workspace of %zu bytes needed, %zu given", need, ws_bytes);
        a.ws = reinterpret_cast<float*>(ws);
    }
    a.kpitch = ((a.wk / 4) & 1) || (a.wk % 4) ? a.wk : a.wk + 4;
    if (a.wk % 4) a.kpitch = a.wk | 1;   // odd pitch: conflict-free 32-bit reads
#define GO(K_, V_) if (kb == K_ && vb == V_) return launch_small<K_, V_>(a, st)
    GO(8, 8); GO(8, 4); GO(8, 2); GO(4, 8); GO(4, 4); GO(4, 2); GO(2, 8); GO(2, 4); GO(2, 2);
#undef GO
    return fail(VARQ_ERR_ARG, "varq_attn_fwd: store bits must be 2, 4 or 8");
}

}  // namespace varq
