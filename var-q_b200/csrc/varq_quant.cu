// Fused quantize + pack of fresh K/V.
//
// Two device paths, both with one thread per packed int32 word (4 / 8 / 16 inputs):
//   * rows path   - groups that keep (token, head) [per-token-per-head, optionally split
//                   along head_dim and/or shared over the batch]: a CTA holds every member
//                   of its groups in registers, so the input is read once;
//   * tables path - any other grouping (per-dim, per-token, per-tensor ...): a statistics
//                   kernel folds min/max into a small table with integer atomics on an
//                   order-preserving encoding, a second kernel quantizes.
// Arithmetic is fp32 with true division and round-half-even, the clamp after the round.
#include "varq_common.cuh"

namespace varq {

struct QuantArgs {
    const void* x;
    long long xs_b, xs_l, xs_h;
    int B, L, H, D;
    int bits, symmetric, words;
    float eps;
    int32_t* codes;
    long long cs_b, cs_l, cs_h;
    float* scale;
    float* zp;
    long long ps_b, ps_r, ps_h, ps_g;   // strides of shared dims already zeroed
    int share_b, share_l, share_h, group;
    int nL, nH, nG;                     // statistics table dims ([nB, nL, nH, nG], 1 where shared)
    uint32_t* stats;                    // [groups][2]: ord(max), ~ord(min)  (zero-initialised)
    int l_fixed;                        // tables path: the row stride is a multiple of L, so a thread keeps its token index
};

struct Range { uint32_t hi, lo; };      // hi = max f2ord(x or |x|), lo = max ~f2ord(x)

__device__ __forceinline__ void range_init(Range& r) { r.hi = 0u; r.lo = 0u; }
__device__ __forceinline__ void range_add(Range& r, float v, bool symmetric) {
    if (symmetric) {
        r.hi = max(r.hi, f2ord(fabsf(v)));
    } else {
        const uint32_t o = f2ord(v);
        r.hi = max(r.hi, o);
        r.lo = max(r.lo, ~o);
    }
}
__device__ __forceinline__ void range_merge(Range& r, const Range& o) { r.hi = max(r.hi, o.hi); r.lo = max(r.lo, o.lo); }

// scale / zero-point of a group from its range
__device__ __forceinline__ void params_from_range(const Range& r, int bits, bool symmetric, float eps, float& scale,
                                                  float& zp) {
    if (symmetric) {
        const float amax = ord2f(r.hi);
        scale = fmaxf(__fdiv_rn(amax, (float)((1 << (bits - 1)) - 1)), eps);
        zp = 0.0f;
    } else {
        const float mx = ord2f(r.hi), mn = ord2f(~r.lo);
        scale = fmaxf(__fdiv_rn(__fsub_rn(mx, mn), (float)((1 << bits) - 1)), eps);
        zp = __fadd_rn(rintf(__fsub_rn(-(float)(1 << (bits - 1)), __fdiv_rn(mn, scale))), 0.0f);
    }
}

// Per-group constants of the division-free quantizer.  RN(x / scale) lies strictly between
// x * rcp_lo and x * rcp_hi (rcp_lo/hi = RN(1/scale) * (1 -/+ 2^-21)), and rint is monotonic, so
// when both ends round to the same integer that integer is the reference's code; otherwise (about
// once in 10^4 elements) the exact division decides.  Rounding is done by adding 1.5 * 2^23, which
// also leaves the two's-complement code in the low mantissa bits.
struct GroupQ {
    float scale, zp, rcp_lo, rcp_hi;
};
constexpr float Q_MAGIC = 12582912.0f;
__device__ __forceinline__ GroupQ make_group_q(float scale, float zp) {
    GroupQ g;
    const float rcp = __frcp_rn(scale);
    g.scale = scale; g.zp = zp;
    g.rcp_lo = rcp * (1.0f - 4.76837158e-7f);
    g.rcp_hi = rcp * (1.0f + 4.76837158e-7f);
    return g;
}
// The code range depends on the bit width only: Q_MAGIC + bound_min / bound_max, one pair per thread.
struct CodeRange { float y_min, y_max; };
__device__ __forceinline__ CodeRange make_code_range(int bits) {
    CodeRange r;
    r.y_min = Q_MAGIC - (float)(1 << (bits - 1));
    r.y_max = Q_MAGIC + (float)((1 << (bits - 1)) - 1);
    return r;
}
template <bool SYM>
__device__ __forceinline__ uint32_t quant_code(float x, const GroupQ& g, const CodeRange& cr) {
    float y = fmaf(x, g.rcp_hi, Q_MAGIC);
    const float y2 = fmaf(x, g.rcp_lo, Q_MAGIC);
    bool slow = y != y2;
    if (!SYM) slow = slow || !(fabsf(y - Q_MAGIC) < 2097152.0f);      // offset data: quotient too large for the trick
    if (slow) {
        float k = rintf(__fdiv_rn(x, g.scale));
        if (!SYM) k = __fadd_rn(k, g.zp);
        y = fminf(fmaxf(k, cr.y_min - Q_MAGIC), cr.y_max - Q_MAGIC) + Q_MAGIC;
    } else if (!SYM) {
        y = ((y - Q_MAGIC) + g.zp) + Q_MAGIC;                           // integers below 2^23: exact
    }
    y = fminf(fmaxf(y, cr.y_min), cr.y_max);
    return __float_as_uint(y);
}

__device__ __forceinline__ uint32_t quant_code_rt(float x, const GroupQ& g, const CodeRange& cr, bool sym) {
    return sym ? quant_code<true>(x, g, cr) : quant_code<false>(x, g, cr);
}

// =====================================================================================
// rows path
// =====================================================================================
struct RowPlan {
    int tpr;        // threads per (b, l, h) row = words per row
    int bp;         // batch lanes per CTA (1 when the batch is not shared)
    int ngr;        // group rows per pass
    int nv;         // vectors per thread
    int lpg;        // lanes per group = group / VPW
    long long n_gr; // group rows in total: L*H (shared batch) or B*L*H
    int h_fast;     // group-row enumeration: 1 = head index fastest
    int d_in, d_mid, d_out;   // ngr decomposed in the (inner, middle, batch) radices of that enumeration
};

template <typename T, int STORE_BITS>
__global__ void __launch_bounds__(256) quant_rows_kernel(QuantArgs a, RowPlan pl) {
    constexpr int VPW = 32 / STORE_BITS;
    constexpr int NVMAX = 32 / VPW;
    extern __shared__ uint32_t s_stats[];   // [ngr * groups_per_row][2], only when bp > 1

    const int tid = threadIdx.x;
    const int w = tid % pl.tpr;
    const int rest = tid / pl.tpr;
    const int g_local = rest % pl.ngr;
    const int bl = rest / pl.ngr;
    const bool sym = a.symmetric != 0;
    const int d0 = w * VPW;
    const int gpr = a.D / a.group;          // groups per row

    if (pl.bp > 1) {
        for (int i = tid; i < pl.ngr * gpr * 2; i += blockDim.x) s_stats[i] = 0u;
        __syncthreads();
    }

    float v[NVMAX][VPW];
    long long xoff[NVMAX];                   // element offset of the vector, -1 = not present
    int vb[NVMAX], vl[NVMAX], vh[NVMAX];

    // (b, l, h) of the thread's first vector; the others follow by constant steps (no per-vector division)
    const unsigned n_gr = (unsigned)pl.n_gr;                 // host guarantees < 2^31
    unsigned gr0 = a.share_b ? blockIdx.x * (unsigned)pl.ngr + g_local
                             : blockIdx.x * (unsigned)(pl.nv * pl.ngr) + g_local;
    int b0, l0, h0;
    {
        unsigned g = gr0;
        if (pl.h_fast) { h0 = (int)(g % (unsigned)a.H); g /= (unsigned)a.H; l0 = (int)(g % (unsigned)a.L); g /= (unsigned)a.L; }
        else           { l0 = (int)(g % (unsigned)a.L); g /= (unsigned)a.L; h0 = (int)(g % (unsigned)a.H); g /= (unsigned)a.H; }
        b0 = a.share_b ? bl : (int)g;
    }
    int cb = b0, cl = l0, ch = h0;           // running coordinates when the batch is not shared
#pragma unroll
    for (int k = 0; k < NVMAX; ++k) {
        xoff[k] = -1;
        if (k < pl.nv) {
            bool ok_k;
            if (a.share_b) {
                cb = bl + k * pl.bp;
                ok_k = gr0 < n_gr && cb < a.B;
            } else {
                if (k > 0) {   // advance the mixed-radix counter by ngr group rows (steps precomputed on the host)
                    if (pl.h_fast) {
                        ch += pl.d_in;  if (ch >= a.H) { ch -= a.H; ++cl; }
                        cl += pl.d_mid; if (cl >= a.L) { cl -= a.L; ++cb; }
                    } else {
                        cl += pl.d_in;  if (cl >= a.L) { cl -= a.L; ++ch; }
                        ch += pl.d_mid; if (ch >= a.H) { ch -= a.H; ++cb; }
                    }
                    cb += pl.d_out;
                }
                ok_k = gr0 + (unsigned)k * (unsigned)pl.ngr < n_gr;
            }
            if (ok_k) {
                vb[k] = cb; vl[k] = cl; vh[k] = ch;
                xoff[k] = cb * a.xs_b + cl * a.xs_l + ch * a.xs_h + d0;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < NVMAX; ++k)
        if (xoff[k] >= 0) load_vals<T, VPW, true>(reinterpret_cast<const T*>(a.x) + xoff[k], v[k], VPW);

    // ---- statistics
    Range rg[NVMAX];
#pragma unroll
    for (int k = 0; k < NVMAX; ++k) {
        range_init(rg[k]);
        if (xoff[k] >= 0) {
#pragma unroll
            for (int j = 0; j < VPW; ++j) range_add(rg[k], v[k][j], sym);
        }
    }
    if (a.share_b) {
        // all vectors of a thread belong to one group: fold them, then across lanes, then across batch lanes
#pragma unroll
        for (int k = 1; k < NVMAX; ++k) range_merge(rg[0], rg[k]);
        for (int m = 1; m < pl.lpg; m <<= 1) {
            Range o;
            o.hi = __shfl_xor_sync(0xffffffffu, rg[0].hi, m);
            o.lo = __shfl_xor_sync(0xffffffffu, rg[0].lo, m);
            range_merge(rg[0], o);
        }
        if (pl.bp > 1) {
            const int slot = (g_local * gpr + d0 / a.group) * 2;
            if ((w % pl.lpg) == 0) {
                atomicMax(&s_stats[slot], rg[0].hi);
                if (!sym) atomicMax(&s_stats[slot + 1], rg[0].lo);
            }
            __syncthreads();
            rg[0].hi = s_stats[slot];
            rg[0].lo = s_stats[slot + 1];
        }
#pragma unroll
        for (int k = 1; k < NVMAX; ++k) rg[k] = rg[0];
    } else {
#pragma unroll
        for (int k = 0; k < NVMAX; ++k) {
            for (int m = 1; m < pl.lpg; m <<= 1) {
                Range o;
                o.hi = __shfl_xor_sync(0xffffffffu, rg[k].hi, m);
                o.lo = __shfl_xor_sync(0xffffffffu, rg[k].lo, m);
                range_merge(rg[k], o);
            }
        }
    }

    // ---- quantize, pack, store
    float scale = 0.f, zp = 0.f;
    const CodeRange cr = make_code_range(a.bits);
    GroupQ gq = make_group_q(1.f, 0.f);
    if (a.share_b) { params_from_range(rg[0], a.bits, sym, a.eps, scale, zp); gq = make_group_q(scale, zp); }
#pragma unroll
    for (int k = 0; k < NVMAX; ++k) {
        if (xoff[k] < 0) continue;
        if (!a.share_b) { params_from_range(rg[k], a.bits, sym, a.eps, scale, zp); gq = make_group_q(scale, zp); }
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < VPW; ++j) {
            word |= (quant_code_rt(v[k][j], gq, cr, sym) & ((1u << STORE_BITS) - 1u)) << (j * STORE_BITS);
        }
        a.codes[vb[k] * a.cs_b + vl[k] * a.cs_l + vh[k] * a.cs_h + w] = (int32_t)word;
        const bool writer = (d0 % a.group) == 0 && (a.share_b ? (vb[k] == 0) : true);
        if (writer) {
            const long long pi = vb[k] * a.ps_b + vl[k] * a.ps_r + vh[k] * a.ps_h + (long long)(d0 / a.group) * a.ps_g;
            a.scale[pi] = scale;
            if (!sym) a.zp[pi] = zp;
        }
    }
}


// =====================================================================================
// lean rows path: groups shared over the batch, every thread holds a full set of vectors
// =====================================================================================
struct LeanPlan {
    int tpr, bp, ngr, lpg, h_fast;
    int xs_row_in, xs_row_out;     // element strides of the inner / outer coordinate of a group row
    int cs_row_in, cs_row_out, ps_row_in, ps_row_out;
    int n_in;                      // size of the inner coordinate (H if h_fast else L)
    int xs_bstep, cs_bstep;        // bp * batch stride (elements / words)
};

template <typename T, int STORE_BITS, bool SYM>
__global__ void __launch_bounds__(256) quant_rows_lean_kernel(QuantArgs a, LeanPlan pl) {
    constexpr int VPW = 32 / STORE_BITS;
    constexpr int NV = 32 / VPW;
    __shared__ uint32_t s_stats[256];          // [ngr * groups per row][2]
    const int tid = threadIdx.x;
    const int w = tid % pl.tpr;
    const int rest = tid / pl.tpr;
    const int g_local = rest % pl.ngr;
    const int bl = rest / pl.ngr;
    const int d0 = w * VPW;
    const int gpr = a.D / a.group;
    const unsigned gr = blockIdx.x * (unsigned)pl.ngr + g_local;
    const int r_in = (int)(gr % (unsigned)pl.n_in), r_out = (int)(gr / (unsigned)pl.n_in);
    const int x0 = bl * (int)a.xs_b + r_in * pl.xs_row_in + r_out * pl.xs_row_out + d0;
    const int c0 = bl * (int)a.cs_b + r_in * pl.cs_row_in + r_out * pl.cs_row_out + w;

    if (pl.bp > 1) {
        if (tid < pl.ngr * gpr * 2) s_stats[tid] = 0u;
        __syncthreads();
    }
    float v[NV][VPW];
    const T* xp = reinterpret_cast<const T*>(a.x) + x0;
#pragma unroll
    for (int k = 0; k < NV; ++k) load_vals<T, VPW, true>(xp + k * pl.xs_bstep, v[k], VPW);

    // statistics in float registers; the order-preserving integer form is only needed for the shared atomics
    float hi = SYM ? 0.f : v[0][0], lo = v[0][0];
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
        for (int j = 0; j < VPW; ++j) {
            if (SYM) hi = fmaxf(hi, fabsf(v[k][j]));
            else { hi = fmaxf(hi, v[k][j]); lo = fminf(lo, v[k][j]); }
        }
    for (int m = 1; m < pl.lpg; m <<= 1) {
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, m));
        if (!SYM) lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, m));
    }
    Range rg;
    rg.hi = f2ord(hi);
    rg.lo = SYM ? 0u : ~f2ord(lo);
    if (pl.bp > 1) {
        const int slot = (g_local * gpr + d0 / a.group) * 2;
        if ((w % pl.lpg) == 0) {
            atomicMax(&s_stats[slot], rg.hi);
            if (!SYM) atomicMax(&s_stats[slot + 1], rg.lo);
        }
        __syncthreads();
        rg.hi = s_stats[slot];
        rg.lo = s_stats[slot + 1];
    }
    float scale, zp;
    params_from_range(rg, a.bits, SYM, a.eps, scale, zp);
    const GroupQ gq = make_group_q(scale, zp);
    const CodeRange cr = make_code_range(a.bits);
    int32_t* cp = a.codes + c0;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < VPW; ++j)
            word |= (quant_code<SYM>(v[k][j], gq, cr) & ((1u << STORE_BITS) - 1u)) << (j * STORE_BITS);
        cp[k * pl.cs_bstep] = (int32_t)word;
    }
    if (bl == 0 && (d0 % a.group) == 0) {
        const long long pi = (long long)r_in * pl.ps_row_in + (long long)r_out * pl.ps_row_out + (long long)(d0 / a.group) * a.ps_g;
        a.scale[pi] = scale;
        if (!SYM) a.zp[pi] = zp;
    }
}

// =====================================================================================
// tables path: blockDim = (TX column slots, TY rows); a column slot is one word of one head
// =====================================================================================
__device__ __forceinline__ long long group_id(const QuantArgs& a, int b, int l, int h, int d) {
    const int bb = a.share_b ? 0 : b, ll = a.share_l ? 0 : l, hh = a.share_h ? 0 : h;
    return (((long long)bb * a.nL + ll) * a.nH + hh) * a.nG + d / a.group;
}

__device__ __forceinline__ void stats_flush(uint32_t* stats, long long gid, const Range& r, bool sym) {
    atomicMax(&stats[gid * 2], r.hi);
    if (!sym) atomicMax(&stats[gid * 2 + 1], r.lo);
}

// Rows r, r + step, r + 2 step, ... of the (batch, token) plane without a division per row: (b, l) and the
// element / word offsets of the row advance incrementally, with one carry when l wraps.
struct RowIter {
    unsigned r, b, l, L, step, step_b, step_l;
    long long xoff, coff, x_step, c_step, x_carry, c_carry;
    __device__ __forceinline__ void init(const QuantArgs& a, unsigned r0, unsigned r_step) {
        L = (unsigned)a.L; step = r_step; r = r0;
        b = r0 / L; l = r0 - b * L;
        step_b = r_step / L; step_l = r_step - step_b * L;
        xoff = b * a.xs_b + l * a.xs_l; coff = b * a.cs_b + l * a.cs_l;
        x_step = step_b * a.xs_b + step_l * a.xs_l; c_step = step_b * a.cs_b + step_l * a.cs_l;
        x_carry = a.xs_b - (long long)L * a.xs_l; c_carry = a.cs_b - (long long)L * a.cs_l;
    }
    __device__ __forceinline__ void next() {
        r += step; b += step_b; l += step_l; xoff += x_step; coff += c_step;
        if (l >= L) { l -= L; ++b; xoff += x_carry; coff += c_carry; }
    }
};

// min / max of a group member set in float registers; the order-preserving integer form is produced once
struct FRange { float hi, lo; };
template <bool SYM> __device__ __forceinline__ void frange_init(FRange& r) { r.hi = SYM ? 0.f : -INFINITY; r.lo = INFINITY; }
template <bool SYM> __device__ __forceinline__ void frange_add(FRange& r, float v) {
    if (SYM) r.hi = fmaxf(r.hi, fabsf(v));
    else { r.hi = fmaxf(r.hi, v); r.lo = fminf(r.lo, v); }
}
template <bool SYM> __device__ __forceinline__ Range frange_ord(const FRange& r) {
    Range o;
    o.hi = f2ord(r.hi);
    o.lo = SYM ? 0u : ~f2ord(r.lo);
    return o;
}

// independent row loads in flight per thread: 32 values whatever the word width (8 rows of 4, 4 of 8, 2 of 16), the
// budget that keeps the single-pass kernel at four CTAs per SM
constexpr int tab_unroll(int vpw) { return 32 / vpw < 2 ? 2 : 32 / vpw; }

template <typename T, int STORE_BITS, bool VEC, bool SYM>
__device__ __forceinline__ void quant_stats_body(const QuantArgs& a, int iters, uint32_t* s_fold) {
    constexpr int VPW = 32 / STORE_BITS;
    const int cs = blockIdx.x * blockDim.x + threadIdx.x;
    const bool col_ok = cs < a.H * a.words;
    const int h = col_ok ? cs / a.words : 0, w = col_ok ? cs % a.words : 0;
    const int d0 = w * VPW;
    const int n_valid = min(VPW, a.D - d0);
    const bool uniform = (a.group % VPW) == 0;      // one group per thread-vector
    // the group depends on the (b, l) row, unless l is shared or every row of this thread has the same l
    const bool row_dep = !(a.share_b && (a.share_l || a.l_fixed));
    const unsigned R = (unsigned)a.B * (unsigned)a.L;       // host guarantees < 2^31
    const T* xcol = reinterpret_cast<const T*>(a.x) + h * a.xs_h + d0;

    FRange acc[VPW];
#pragma unroll
    for (int j = 0; j < VPW; ++j) frange_init<SYM>(acc[j]);

    RowIter ri;
    ri.init(a, blockIdx.y * blockDim.y + threadIdx.y, gridDim.y * blockDim.y);
    const int l0 = (int)ri.l;                       // this thread's token index when it is fixed
    if (!row_dep) {
        // ---- statistics do not depend on the row: accumulate in registers, several loads in flight
        constexpr int TAB_UNROLL = tab_unroll(VPW);
        for (int it = 0; it < iters; it += TAB_UNROLL) {
            float v[TAB_UNROLL][VPW];
            bool ok[TAB_UNROLL];
#pragma unroll
            for (int u = 0; u < TAB_UNROLL; ++u) {
                ok[u] = col_ok && it + u < iters && ri.r < R;
                if (ok[u]) load_vals<T, VPW, VEC>(xcol + ri.xoff, v[u], n_valid);
                ri.next();
            }
#pragma unroll
            for (int u = 0; u < TAB_UNROLL; ++u) {
                if (!ok[u]) continue;
#pragma unroll
                for (int j = 0; j < VPW; ++j)
                    if (j < n_valid) frange_add<SYM>(acc[j], v[u][j]);
            }
        }
        if (uniform) {      // the thread's values share one group: fold them once, here
#pragma unroll
            for (int j = 1; j < VPW; ++j) {
                acc[0].hi = fmaxf(acc[0].hi, acc[j].hi);
                acc[0].lo = fminf(acc[0].lo, acc[j].lo);
            }
        }
        Range ord[VPW];
#pragma unroll
        for (int j = 0; j < VPW; ++j) ord[j] = frange_ord<SYM>(acc[j]);
        // fold the block's rows in shared memory, then one global atomic per column and block
        const int np = uniform ? 1 : VPW;
        if (blockDim.y > 1) {
            for (int i = threadIdx.y * blockDim.x + threadIdx.x; i < (int)blockDim.x * VPW * 2; i += blockDim.x * blockDim.y) s_fold[i] = 0u;
            __syncthreads();
#pragma unroll
            for (int j = 0; j < VPW; ++j) {
                if (j >= np) break;
                atomicMax(&s_fold[(threadIdx.x * VPW + j) * 2], ord[j].hi);
                if (!SYM) atomicMax(&s_fold[(threadIdx.x * VPW + j) * 2 + 1], ord[j].lo);
            }
            __syncthreads();
            if (threadIdx.y != 0) return;
#pragma unroll
            for (int j = 0; j < VPW; ++j) {
                if (j >= np) break;
                ord[j].hi = s_fold[(threadIdx.x * VPW + j) * 2]; ord[j].lo = s_fold[(threadIdx.x * VPW + j) * 2 + 1];
            }
        }
        if (uniform) {
            const long long gid = col_ok ? group_id(a, 0, l0, h, d0) : -1;
            int same;
            __match_all_sync(__activemask(), gid, &same);
            if (same && __activemask() == 0xffffffffu) {
                if (gid >= 0) {
                    Range t;
                    t.hi = __reduce_max_sync(0xffffffffu, ord[0].hi);
                    t.lo = __reduce_max_sync(0xffffffffu, ord[0].lo);
                    if ((threadIdx.x & 31) == 0) stats_flush(a.stats, gid, t, SYM);
                }
            } else if (col_ok) {
                stats_flush(a.stats, gid, ord[0], SYM);
            }
        } else if (col_ok) {
#pragma unroll
            for (int j = 0; j < VPW; ++j)
                if (j < n_valid) stats_flush(a.stats, group_id(a, 0, l0, h, d0 + j), ord[j], SYM);
        }
        return;
    }
    // ---- statistics depend on the row: flush after every row, warp-aggregated when a warp sits in one group
    for (int it = 0; it < iters; ++it, ri.next()) {
        const bool ok = col_ok && ri.r < R;
        const int b = (int)ri.b, l = (int)ri.l;
        if (ok) {
            float v[VPW];
            load_vals<T, VPW, VEC>(xcol + ri.xoff, v, n_valid);
#pragma unroll
            for (int j = 0; j < VPW; ++j)
                if (j < n_valid) frange_add<SYM>(acc[j], v[j]);
        }
        if (uniform) {
#pragma unroll
            for (int j = 1; j < VPW; ++j) {
                acc[0].hi = fmaxf(acc[0].hi, acc[j].hi);
                acc[0].lo = fminf(acc[0].lo, acc[j].lo);
                frange_init<SYM>(acc[j]);
            }
            const long long gid = ok ? group_id(a, b, l, h, d0) : -1;
            const Range mine = frange_ord<SYM>(acc[0]);
            int same;
            __match_all_sync(0xffffffffu, gid, &same);
            if (same) {
                if (gid >= 0) {
                    Range t;
                    t.hi = __reduce_max_sync(0xffffffffu, mine.hi);
                    t.lo = __reduce_max_sync(0xffffffffu, mine.lo);
                    if ((threadIdx.x & 31) == 0) stats_flush(a.stats, gid, t, SYM);
                }
            } else if (ok) {
                stats_flush(a.stats, gid, mine, SYM);
            }
            frange_init<SYM>(acc[0]);
        } else if (ok) {
#pragma unroll
            for (int j = 0; j < VPW; ++j) {
                if (j < n_valid) stats_flush(a.stats, group_id(a, b, l, h, d0 + j), frange_ord<SYM>(acc[j]), SYM);
                frange_init<SYM>(acc[j]);
            }
        }
    }
}

template <typename T, int STORE_BITS, bool VEC, bool SYM>
__global__ void __launch_bounds__(256) quant_stats_kernel(QuantArgs a, int iters) {
    extern __shared__ uint32_t s_fold[];            // [blockDim.x * VPW][2] when rows are folded in the block
    quant_stats_body<T, STORE_BITS, VEC, SYM>(a, iters, s_fold);
}

// Between the two passes: one thread per group turns its (max, min) entry into the scale and zero-point that
// the caller gets back; the apply pass reads them from there instead of redoing the divisions per row.
__global__ void __launch_bounds__(256) quant_finalize_kernel(QuantArgs a, long long groups) {
    const long long gid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (gid >= groups) return;
    long long r = gid;
    const int g = (int)(r % a.nG); r /= a.nG;
    const int hh = (int)(r % a.nH); r /= a.nH;
    const int ll = (int)(r % a.nL);
    const int bb = (int)(r / a.nL);
    Range rg;
    rg.hi = a.stats[gid * 2];
    rg.lo = a.stats[gid * 2 + 1];
    float scale, zp;
    params_from_range(rg, a.bits, a.symmetric != 0, a.eps, scale, zp);
    const long long pi = bb * a.ps_b + ll * a.ps_r + hh * a.ps_h + (long long)g * a.ps_g;
    a.scale[pi] = scale;
    if (!a.symmetric) a.zp[pi] = zp;
}

template <typename T, int STORE_BITS, bool VEC, bool SYM, bool ROWDEP>
__device__ __forceinline__ void quant_apply_body(const QuantArgs& a, int iters) {
    constexpr int VPW = 32 / STORE_BITS;
    constexpr int UN = VPW == 4 ? 4 : tab_unroll(VPW);     // 8-bit words: four rows keep the kernel at three CTAs per SM
    constexpr bool REPL = VPW <= 4;      // replicating shared parameters costs 4 registers per value: only for short words
    const int cs = blockIdx.x * blockDim.x + threadIdx.x;
    if (cs >= a.H * a.words) return;
    const int h = cs / a.words, w = cs % a.words;
    const int d0 = w * VPW;
    const int n_valid = min(VPW, a.D - d0);
    const bool uniform = (a.group % VPW) == 0;
    constexpr bool row_dep = ROWDEP;      // parameters change with the (sample, token) row; otherwise they are fetched once
    const unsigned R = (unsigned)a.B * (unsigned)a.L;
    const int np = uniform ? 1 : VPW;
    const T* xcol = reinterpret_cast<const T*>(a.x) + h * a.xs_h + d0;
    int32_t* ccol = a.codes + h * a.cs_h + w;

    GroupQ gq[VPW];
    const CodeRange cr = make_code_range(a.bits);
    const long long p_h = h * a.ps_h;
    auto fetch = [&](int b, int l) {
        const long long p_row = (a.share_b ? 0 : b) * a.ps_b + (a.share_l ? 0 : l) * a.ps_r + (a.share_h ? 0 : p_h);
#pragma unroll
        for (int j = 0; j < VPW; ++j) {      // compile-time trip count keeps the per-value parameters in registers
            if (j >= np) break;
            const int d = min(d0 + j, a.D - 1);
            const long long pi = p_row + (long long)(d / a.group) * a.ps_g;
            gq[j] = make_group_q(a.scale[pi], SYM ? 0.0f : a.zp[pi]);
        }
        if (REPL && uniform) {   // one group for all of the thread's values: replicate, so the inner loop never selects
#pragma unroll
            for (int j = 1; j < VPW; ++j) gq[j] = gq[0];
        }
    };
    RowIter ri;
    ri.init(a, blockIdx.y * blockDim.y + threadIdx.y, gridDim.y * blockDim.y);
    if (!row_dep) fetch(0, (int)ri.l);

    for (int it = 0; it < iters; it += UN) {
        float v[UN][VPW];
        unsigned rb[UN], rl[UN];
        long long co[UN];
        bool ok[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            ok[u] = it + u < iters && ri.r < R;
            if (ROWDEP) { rb[u] = ri.b; rl[u] = ri.l; }
            co[u] = ri.coff;
            if (ok[u]) load_vals<T, VPW, VEC>(xcol + ri.xoff, v[u], n_valid);
            ri.next();
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            if (!ok[u]) continue;
            if (ROWDEP) fetch((int)rb[u], (int)rl[u]);
            uint32_t word = 0;
#pragma unroll
            for (int j = 0; j < VPW; ++j) {
                if (j < n_valid) {
                    const GroupQ g = (REPL || !uniform) ? gq[j] : gq[0];
                    word |= (quant_code<SYM>(v[u][j], g, cr) & ((1u << STORE_BITS) - 1u)) << (j * STORE_BITS);
                }
            }
            ccol[co[u]] = (int32_t)word;
        }
    }
}

template <typename T, int STORE_BITS, bool VEC, bool SYM, bool ROWDEP>
__global__ void __launch_bounds__(256) quant_apply_kernel(QuantArgs a, int iters) {
    quant_apply_body<T, STORE_BITS, VEC, SYM, ROWDEP>(a, iters);
}

// ---------------------------------------------------------------- host side
static bool vec_ok(const varq_tensor_t* x, int D, int vpw) {
    const int es = dtype_size(x->dtype);
    const int chunk = (vpw * es) < 16 ? (vpw * es) : 16;
    auto m = [&](long long s) { return ((s * es) % chunk) == 0; };
    return (D % vpw == 0) && ((reinterpret_cast<uintptr_t>(x->ptr) % chunk) == 0) && m(x->stride_b) &&
           m(x->stride_l) && m(x->stride_h);
}

static bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

static bool plan_rows(const QuantArgs& a, int vpw, bool vec, RowPlan& pl, int& threads, size_t& smem) {
    if (!vec || a.share_l || a.share_h) return false;
    if (a.group % vpw != 0 || a.D % a.group != 0) return false;
    pl.tpr = a.D / vpw;
    pl.lpg = a.group / vpw;
    if (!is_pow2(pl.tpr) || pl.tpr > 256 || !is_pow2(pl.lpg) || pl.lpg > 32) return false;
    const int nvmax = 32 / vpw;
    pl.h_fast = a.xs_h <= a.xs_l;
    if (a.share_b) {
        int bp = 1;
        while (bp * nvmax < a.B) bp <<= 1;
        if (pl.tpr * bp > 256) return false;
        pl.bp = bp;
        pl.nv = (a.B + bp - 1) / bp;
        pl.ngr = 256 / (pl.tpr * bp);
        if (pl.ngr < 1) pl.ngr = 1;
        pl.n_gr = (long long)a.L * a.H;
        threads = pl.tpr * pl.bp * pl.ngr;
        smem = pl.bp > 1 ? (size_t)pl.ngr * (a.D / a.group) * 2 * sizeof(uint32_t) : 0;
    } else {
        pl.bp = 1;
        pl.ngr = 256 / pl.tpr;
        pl.nv = nvmax;
        pl.n_gr = (long long)a.B * a.L * a.H;
        threads = 256;
        smem = 0;
    }
    if (pl.n_gr >= 0x7fffffffLL) return false;
    {
        const int inner = pl.h_fast ? a.H : a.L, mid = pl.h_fast ? a.L : a.H;
        pl.d_in = pl.ngr % inner;
        pl.d_mid = (pl.ngr / inner) % mid;
        pl.d_out = pl.ngr / (inner * mid);
    }
    return threads % 32 == 0 && threads <= 256;
}

// The lean kernel applies when the batch is shared, fills every register slot (B = bp * NV) and
// all offsets fit 32 bits.
static bool plan_lean(const QuantArgs& a, int vpw, bool vec, const RowPlan& rp, LeanPlan& lp, long long x_extent) {
    if (!vec || !a.share_b || a.share_l || a.share_h) return false;
    const int nv = 32 / vpw;
    if (rp.bp * nv != a.B || rp.nv != nv) return false;
    if (rp.n_gr % rp.ngr != 0) return false;
    if (rp.ngr * (a.D / a.group) * 2 > 256) return false;
    const long long c_extent = (long long)a.B * a.cs_b;
    if (x_extent >= 0x7fffffffLL || c_extent >= 0x7fffffffLL || x_extent < 0) return false;
    lp.tpr = rp.tpr; lp.bp = rp.bp; lp.ngr = rp.ngr; lp.lpg = rp.lpg; lp.h_fast = rp.h_fast;
    if (rp.h_fast) {
        lp.n_in = a.H;
        lp.xs_row_in = (int)a.xs_h; lp.xs_row_out = (int)a.xs_l;
        lp.cs_row_in = (int)a.cs_h; lp.cs_row_out = (int)a.cs_l;
        lp.ps_row_in = (int)a.ps_h; lp.ps_row_out = (int)a.ps_r;
    } else {
        lp.n_in = a.L;
        lp.xs_row_in = (int)a.xs_l; lp.xs_row_out = (int)a.xs_h;
        lp.cs_row_in = (int)a.cs_l; lp.cs_row_out = (int)a.cs_h;
        lp.ps_row_in = (int)a.ps_r; lp.ps_row_out = (int)a.ps_h;
    }
    lp.xs_bstep = rp.bp * (int)a.xs_b;
    lp.cs_bstep = rp.bp * (int)a.cs_b;
    return true;
}

// `have_stats`: the statistics table in `ws` is already filled (by varq_qk_norm_stats); only finalize + apply run.
template <typename T, int SB>
static int launch_quant(const QuantArgs& a0, bool vec, void* ws, size_t ws_bytes, cudaStream_t st, bool have_stats = false) {
    QuantArgs a = a0;
    constexpr int VPW = 32 / SB;
    RowPlan pl;
    int threads = 0;
    size_t smem = 0;
    if (!have_stats && plan_rows(a, VPW, vec, pl, threads, smem) && threads >= 32) {
        const long long per_cta = a.share_b ? pl.ngr : (long long)pl.ngr * pl.nv;
        const long long blocks = (pl.n_gr + per_cta - 1) / per_cta;
        if (blocks > 0x7fffffffLL) return fail(VARQ_ERR_UNSUPPORTED, "varq_quant_pack: tensor too large");
        LeanPlan lp;
        const long long x_extent = (long long)(a.B - 1) * a.xs_b + (long long)(a.L - 1) * a.xs_l + (long long)(a.H - 1) * a.xs_h + a.D;
        if (plan_lean(a, VPW, vec, pl, lp, x_extent)) {
            if (a.symmetric) quant_rows_lean_kernel<T, SB, true><<<(unsigned)blocks, threads, 0, st>>>(a, lp);
            else             quant_rows_lean_kernel<T, SB, false><<<(unsigned)blocks, threads, 0, st>>>(a, lp);
            VARQ_CUDA_TRY(cudaGetLastError());
            count_launches(1);
            return VARQ_OK;
        }
        quant_rows_kernel<T, SB><<<(unsigned)blocks, threads, smem, st>>>(a, pl);
        VARQ_CUDA_TRY(cudaGetLastError());
        count_launches(1);
        return VARQ_OK;
    }
    // tables path
    const long long groups = (long long)(a.share_b ? 1 : a.B) * a.nL * a.nH * a.nG;
    const size_t need = (size_t)groups * 2 * sizeof(uint32_t);
    if (!ws || ws_bytes < need)
        return fail(VARQ_ERR_WORKSPACE, "varq_quant_pack: workspace of %zu bytes needed, %zu given", need, ws_bytes);
    a.stats = reinterpret_cast<uint32_t*>(ws);
    if (!have_stats) VARQ_CUDA_TRY(cudaMemsetAsync(a.stats, 0, need, st));
    const int cols = a.H * a.words;
    int tx = 32;
    while (tx < cols && tx < 256) tx <<= 1;
    // per-token groups shared over the batch keep one row per thread block row (see l_fixed below)
    const bool per_token = a.share_b && !a.share_l && a.L <= 65535;
    const int ty = per_token ? 1 : 256 / tx;
    const long long R = (long long)a.B * a.L;
    const int gx = (cols + tx - 1) / tx;
    if (R >= 0x7fffffffLL) return fail(VARQ_ERR_UNSUPPORTED, "varq_quant_pack: batch x tokens exceeds 2^31");
    // the two kernels of this call, by vector width, symmetry and whether parameters change with the (sample, token) row
    using KernelFn = void (*)(QuantArgs, int);
    const bool row_dep = !(a.share_b && (a.share_l || per_token));
    KernelFn stats_fn, apply_fn;
#define VARQ_PICK(VEC_, SYM_)                                                                           \
    do {                                                                                                 \
        stats_fn = quant_stats_kernel<T, SB, VEC_, SYM_>;                                                \
        apply_fn = row_dep ? (KernelFn)quant_apply_kernel<T, SB, VEC_, SYM_, true> : (KernelFn)quant_apply_kernel<T, SB, VEC_, SYM_, false>; \
    } while (0)
    if (vec) { if (a.symmetric) VARQ_PICK(true, true); else VARQ_PICK(true, false); }
    else     { if (a.symmetric) VARQ_PICK(false, true); else VARQ_PICK(false, false); }
#undef VARQ_PICK
    // the grid is one wave of the heavier (apply) kernel: as many CTAs per SM as its registers allow, no tail wave
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, apply_fn, 256, 0) != cudaSuccess || per_sm < 1) per_sm = 2;
    long long gy = (R + ty - 1) / ty;
    const long long cap = ((long long)sm_count() * per_sm + gx - 1) / gx;
    if (gy > cap) gy = cap;
    if (gy < 1) gy = 1;
    if (gy > 65535) gy = 65535;
    // Parameters that depend on the token but not on the sample (per-token groups shared over the batch): with a
    // row stride of k * L every thread stays on one token, accumulates over the batch in registers and flushes once.
    a.l_fixed = 0;
    if (per_token) {
        long long k = cap * (256 / tx) / a.L;          // thread blocks are tx x 1 here
        if (k > 65535 / a.L) k = 65535 / a.L;
        if (k > a.B) k = a.B;
        if (k < 1) k = 1;
        gy = (long long)a.L * k;
        a.l_fixed = 1;
    }
    const int iters = (int)((R + gy * ty - 1) / (gy * ty));
    dim3 block(tx, ty), grid(gx, (unsigned)gy);
    const size_t fold = ty > 1 ? (size_t)tx * VPW * 2 * sizeof(uint32_t) : 0;
    const unsigned fin_blocks = (unsigned)((groups + 255) / 256);
    if (!have_stats) stats_fn<<<grid, block, fold, st>>>(a, iters);
    quant_finalize_kernel<<<fin_blocks, 256, 0, st>>>(a, groups);
    apply_fn<<<grid, block, 0, st>>>(a, iters);
    VARQ_CUDA_TRY(cudaGetLastError());
    count_launches(have_stats ? 2 : 3);
    return VARQ_OK;
}

template <int SB>
static int dispatch_quant(const QuantArgs& a, int dtype, bool vec, void* ws, size_t wsb, cudaStream_t st, bool have_stats = false) {
    switch (dtype) {
        case VARQ_F32: return launch_quant<float, SB>(a, vec, ws, wsb, st, have_stats);
        case VARQ_F16: return launch_quant<__half, SB>(a, vec, ws, wsb, st, have_stats);
        default:       return launch_quant<__nv_bfloat16, SB>(a, vec, ws, wsb, st, have_stats);
    }
}

static int check_grouping(const char* fn, const varq_qparams_t* p, int D) {
    if (!p) return fail(VARQ_ERR_ARG, "%s: null grouping", fn);
    if (p->group < 1 || p->group > D) return fail(VARQ_ERR_ARG, "%s: group must be in [1, D] (got %d, D=%d)", fn, p->group, D);
    if (D % p->group != 0) return fail(VARQ_ERR_ARG, "%s: head_dim %d is not a multiple of group %d", fn, D, p->group);
    return VARQ_OK;
}

}  // namespace varq

using namespace varq;

extern "C" size_t varq_quant_workspace_bytes(int32_t B, int32_t L, int32_t H, int32_t D, int32_t x_dtype,
                                             int32_t store_bits, const varq_qparams_t* g) {
    (void)x_dtype; (void)store_bits;
    if (!g || B <= 0 || L <= 0 || H <= 0 || D <= 0 || g->group < 1 || g->group > D) return 0;
    // upper bound: the tables path may be taken for any grouping (unaligned input, large batch)
    const long long groups = (long long)(g->share_b ? 1 : B) * (g->share_l ? 1 : L) * (g->share_h ? 1 : H) *
                             ((D + g->group - 1) / g->group);
    return (size_t)groups * 2 * sizeof(uint32_t);
}

static int quant_pack_impl(const char* fn, const varq_tensor_t* x, int32_t B, int32_t L, int32_t H, int32_t D, int32_t bits,
                           int32_t store_bits, float eps, const varq_tensor_t* codes, const varq_qparams_t* p, void* workspace,
                           size_t workspace_bytes, void* stream, bool have_stats) {
    if (!x || !codes || !p) return fail(VARQ_ERR_ARG, "%s: null descriptor", fn);
    if (bits < 2 || bits > 8) return fail(VARQ_ERR_ARG, "%s: bits must be in [2, 8] (got %d)", fn, bits);
    if (store_bits != 2 && store_bits != 4 && store_bits != 8)
        return fail(VARQ_ERR_ARG, "%s: store_bits must be 2, 4 or 8 (got %d)", fn, store_bits);
    if (store_bits < bits) return fail(VARQ_ERR_ARG, "%s: store_bits %d cannot hold %d-bit codes", fn, store_bits, bits);
    if (B < 0 || L < 0 || H < 0 || D <= 0) return fail(VARQ_ERR_ARG, "%s: bad shape (%d,%d,%d,%d)", fn, B, L, H, D);
    if (!dtype_ok(x->dtype)) return fail(VARQ_ERR_ARG, "%s: bad input dtype %d", fn, x->dtype);
    if (int rc = check_grouping(fn, p, D)) return rc;
    if (have_stats && !(p->share_b && p->share_l))
        return fail(VARQ_ERR_UNSUPPORTED, "%s: ready-made statistics exist for groupings shared over batch and tokens only", fn);
    if ((long long)B * L * H == 0) return VARQ_OK;
    if (!x->ptr || !codes->ptr || !p->scale) return fail(VARQ_ERR_ARG, "%s: null pointer", fn);

    const int vpw = 32 / store_bits;
    QuantArgs a;
    a.x = x->ptr; a.xs_b = x->stride_b; a.xs_l = x->stride_l; a.xs_h = x->stride_h;
    a.B = B; a.L = L; a.H = H; a.D = D; a.l_fixed = 0;
    a.bits = bits; a.symmetric = p->zp == nullptr; a.words = (D + vpw - 1) / vpw; a.eps = eps;
    a.codes = (int32_t*)codes->ptr; a.cs_b = codes->stride_b; a.cs_l = codes->stride_l; a.cs_h = codes->stride_h;
    a.scale = p->scale; a.zp = p->zp;
    a.share_b = p->share_b != 0; a.share_l = p->share_l != 0; a.share_h = p->share_h != 0; a.group = p->group;
    a.ps_b = a.share_b ? 0 : p->stride_b; a.ps_r = a.share_l ? 0 : p->stride_r;
    a.ps_h = a.share_h ? 0 : p->stride_h; a.ps_g = p->stride_g;
    a.nL = a.share_l ? 1 : L; a.nH = a.share_h ? 1 : H; a.nG = D / p->group;
    a.stats = nullptr;
    const bool vec = vec_ok(x, D, vpw);
    cudaStream_t st = (cudaStream_t)stream;
    if (store_bits == 8) return dispatch_quant<8>(a, x->dtype, vec, workspace, workspace_bytes, st, have_stats);
    if (store_bits == 4) return dispatch_quant<4>(a, x->dtype, vec, workspace, workspace_bytes, st, have_stats);
    return dispatch_quant<2>(a, x->dtype, vec, workspace, workspace_bytes, st, have_stats);
}

extern "C" int varq_quant_pack(const varq_tensor_t* x, int32_t B, int32_t L, int32_t H, int32_t D, int32_t bits,
                               int32_t store_bits, float eps, const varq_tensor_t* codes, const varq_qparams_t* p,
                               void* workspace, size_t workspace_bytes, void* stream) {
    return quant_pack_impl("varq_quant_pack", x, B, L, H, D, bits, store_bits, eps, codes, p, workspace, workspace_bytes, stream, false);
}

extern "C" int varq_quant_pack_prestats(const varq_tensor_t* x, int32_t B, int32_t L, int32_t H, int32_t D, int32_t bits,
                                        int32_t store_bits, float eps, const varq_tensor_t* codes, const varq_qparams_t* p,
                                        void* stats, size_t stats_bytes, void* stream) {
    return quant_pack_impl("varq_quant_pack_prestats", x, B, L, H, D, bits, store_bits, eps, codes, p, stats, stats_bytes, stream, true);
}

// =====================================================================================
// Quantize + pack without any allocation by the caller or by this library
// =====================================================================================
// Scratch for the statistics table of the tables path, resident in every GPU that loads the
// library until the process exits.  Host code must not hand this name to a kernel: on the host
// it is only a handle; the device address is looked up once per device below.
#define VARQ_STATIC_SCRATCH_GROUPS 65536
static __device__ __align__(256) uint32_t g_static_stats[VARQ_STATIC_SCRATCH_GROUPS * 2];

namespace varq {
static uint32_t* g_static_stats_addr[64] = {nullptr};   // per device ordinal, filled on first use

// Device address of g_static_stats on the current device (looked up with that device current).
static int static_scratch(uint32_t** out) {
    int dev = -1;
    VARQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(VARQ_ERR_UNSUPPORTED, "varq_quant_pack_static: device ordinal %d out of range", dev);
    uint32_t* p = __atomic_load_n(&g_static_stats_addr[dev], __ATOMIC_ACQUIRE);
    if (!p) {
        void* sym = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&sym, g_static_stats);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_static_stats)");
        if (!sym) return fail(VARQ_ERR_CUDA, "varq_quant_pack_static: no device address for the built-in scratch");
        p = reinterpret_cast<uint32_t*>(sym);
        __atomic_store_n(&g_static_stats_addr[dev], p, __ATOMIC_RELEASE);   // same value from any thread
    }
    *out = p;
    return VARQ_OK;
}
}  // namespace varq

extern "C" size_t varq_quant_static_scratch_bytes(void) {
    return (size_t)VARQ_STATIC_SCRATCH_GROUPS * 2 * sizeof(uint32_t);
}

extern "C" int varq_quant_pack_static(const varq_tensor_t* x, int32_t B, int32_t L, int32_t H, int32_t D,
                                      int32_t bits, int32_t store_bits, float eps, const varq_tensor_t* codes,
                                      const varq_qparams_t* p, void* stream) {
    if (!p) return fail(VARQ_ERR_ARG, "varq_quant_pack_static: null grouping");
    const size_t have = varq_quant_static_scratch_bytes();
    const size_t need = varq_quant_workspace_bytes(B, L, H, D, x ? x->dtype : VARQ_F32, store_bits, p);
    if (need > have)
        return fail(VARQ_ERR_WORKSPACE,
                    "varq_quant_pack_static: this grouping has %zu groups but the built-in scratch holds %d; "
                    "use varq_quant_pack with a caller-provided workspace",
                    need / (2 * sizeof(uint32_t)), VARQ_STATIC_SCRATCH_GROUPS);
    uint32_t* scratch = nullptr;
    if (int rc = static_scratch(&scratch)) return rc;
    // the tables path clears the part of the table it uses on `stream` (a memset node) before accumulating into it;
    // groupings that run in the single-pass kernels never touch the scratch
    return varq_quant_pack(x, B, L, H, D, bits, store_bits, eps, codes, p, scratch, have, stream);
}
