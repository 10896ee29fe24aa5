// Producer side of the attention hook, fused: L2-normalisation of q and k and, in the same read, the column statistics
// that the per-dim / per-step / per-tensor quantizers need, so that their statistics pass over K and V disappears.
//
// A warp owns one head and walks over the (sample, token) rows with the grid's row stride: lane i holds head_dim elements
// i, i + 32, ... of a row, the row's sum of squares is a five-step shuffle reduction, and the min / max of the emitted k
// (the very fp32 values the quantizer will read) and of v stay in registers until the warp has seen all its rows; then one
// integer atomic per (head, element) folds them into the statistics table in the format of the two-pass quantizer.
#include "varq_common.cuh"

namespace varq {

struct PrepArgs {
    const void* q; const void* k; const void* v;
    int q_dt, k_dt, v_dt;
    long long qs_b, qs_l, qs_h, ks_b, ks_l, ks_h, vs_b, vs_l, vs_h;
    float* q_out; float* k_out;
    long long qo_b, qo_l, qo_h, ko_b, ko_l, ko_h;
    const float* scale_mul;       // [H] or null
    float eps;
    int B, L, H, D;
    uint32_t* k_stats; uint32_t* v_stats;     // [groups][2] or null
    int k_sym, v_sym, k_share_h, v_share_h, k_group, v_group, k_ng, v_ng;
};

__device__ __forceinline__ float load_any(const void* p, int dt, long long off) {
    if (dt == VARQ_F32) return __ldg(reinterpret_cast<const float*>(p) + off);
    if (dt == VARQ_F16) return __half2float(__ldg(reinterpret_cast<const __half*>(p) + off));
    return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(p) + off));
}

constexpr int PREP_EPL = 4;        // head_dim elements per lane (head_dim <= 128)
constexpr int PREP_WARPS = 8;

__global__ void __launch_bounds__(PREP_WARPS * 32) qk_norm_stats_kernel(PrepArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.x * PREP_WARPS + warp;
    if (h >= a.H) return;
    const unsigned R = (unsigned)a.B * (unsigned)a.L;
    const float mul = a.scale_mul ? __ldg(a.scale_mul + h) : 1.f;
    float k_hi[PREP_EPL], k_lo[PREP_EPL], v_hi[PREP_EPL], v_lo[PREP_EPL];
#pragma unroll
    for (int e = 0; e < PREP_EPL; ++e) {
        k_hi[e] = a.k_sym ? 0.f : -INFINITY; k_lo[e] = INFINITY;
        v_hi[e] = a.v_sym ? 0.f : -INFINITY; v_lo[e] = INFINITY;
    }
    for (unsigned r = blockIdx.y; r < R; r += gridDim.y) {
        const unsigned b = r / (unsigned)a.L, l = r - b * (unsigned)a.L;
        const long long qo = b * a.qs_b + l * a.qs_l + h * a.qs_h, ko = b * a.ks_b + l * a.ks_l + h * a.ks_h;
        const long long vo = b * a.vs_b + l * a.vs_l + h * a.vs_h;
        float qv[PREP_EPL], kv[PREP_EPL], vv[PREP_EPL];
        float qs = 0.f, ks = 0.f;
#pragma unroll
        for (int e = 0; e < PREP_EPL; ++e) {
            const int d = lane + 32 * e;
            qv[e] = kv[e] = vv[e] = 0.f;
            if (d < a.D) {
                qv[e] = load_any(a.q, a.q_dt, qo + d);
                kv[e] = load_any(a.k, a.k_dt, ko + d);
                if (a.v_stats) vv[e] = load_any(a.v, a.v_dt, vo + d);
            }
            qs = fmaf(qv[e], qv[e], qs);
            ks = fmaf(kv[e], kv[e], ks);
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            qs += __shfl_xor_sync(0xffffffffu, qs, m);
            ks += __shfl_xor_sync(0xffffffffu, ks, m);
        }
        // x / max(||x||, eps), as torch.nn.functional.normalize does it (true division)
        const float qd = fmaxf(sqrtf(qs), a.eps), kd = fmaxf(sqrtf(ks), a.eps);
        const long long qoo = b * a.qo_b + l * a.qo_l + h * a.qo_h, koo = b * a.ko_b + l * a.ko_l + h * a.ko_h;
#pragma unroll
        for (int e = 0; e < PREP_EPL; ++e) {
            const int d = lane + 32 * e;
            if (d >= a.D) continue;
            const float qn = __fmul_rn(__fdiv_rn(qv[e], qd), mul), kn = __fdiv_rn(kv[e], kd);
            a.q_out[qoo + d] = qn;
            a.k_out[koo + d] = kn;
            if (a.k_sym) k_hi[e] = fmaxf(k_hi[e], fabsf(kn));
            else { k_hi[e] = fmaxf(k_hi[e], kn); k_lo[e] = fminf(k_lo[e], kn); }
            if (a.v_sym) v_hi[e] = fmaxf(v_hi[e], fabsf(vv[e]));
            else { v_hi[e] = fmaxf(v_hi[e], vv[e]); v_lo[e] = fminf(v_lo[e], vv[e]); }
        }
    }
    if (blockIdx.y >= R) return;       // this warp saw no row
#pragma unroll
    for (int e = 0; e < PREP_EPL; ++e) {
        const int d = lane + 32 * e;
        if (d >= a.D) continue;
        if (a.k_stats) {
            const long long g = ((long long)(a.k_share_h ? 0 : h) * a.k_ng + d / a.k_group) * 2;
            atomicMax(&a.k_stats[g], f2ord(k_hi[e]));
            if (!a.k_sym) atomicMax(&a.k_stats[g + 1], ~f2ord(k_lo[e]));
        }
        if (a.v_stats) {
            const long long g = ((long long)(a.v_share_h ? 0 : h) * a.v_ng + d / a.v_group) * 2;
            atomicMax(&a.v_stats[g], f2ord(v_hi[e]));
            if (!a.v_sym) atomicMax(&a.v_stats[g + 1], ~f2ord(v_lo[e]));
        }
    }
}

static bool column_grouping(const varq_qparams_t* g, int D) {
    return g && g->share_b && g->share_l && g->group >= 1 && g->group <= D && D % g->group == 0;
}

}  // namespace varq

using namespace varq;

extern "C" int varq_qk_norm_stats(const varq_tensor_t* q_in, const varq_tensor_t* k_in, const varq_tensor_t* v_in, int32_t B, int32_t L,
                                  int32_t H, int32_t D, const float* scale_mul, float eps, const varq_tensor_t* q_out,
                                  const varq_tensor_t* k_out, const varq_qparams_t* k_grouping, void* k_stats,
                                  const varq_qparams_t* v_grouping, void* v_stats, void* stream) {
    if (!q_in || !k_in || !q_out || !k_out) return fail(VARQ_ERR_ARG, "varq_qk_norm_stats: null descriptor");
    if (B < 0 || L < 0 || H < 0 || D <= 0) return fail(VARQ_ERR_ARG, "varq_qk_norm_stats: bad shape (%d,%d,%d,%d)", B, L, H, D);
    if (D > 32 * PREP_EPL) return fail(VARQ_ERR_UNSUPPORTED, "varq_qk_norm_stats: head_dim %d > %d", D, 32 * PREP_EPL);
    if (!dtype_ok(q_in->dtype) || !dtype_ok(k_in->dtype) || (v_stats && (!v_in || !dtype_ok(v_in->dtype))))
        return fail(VARQ_ERR_ARG, "varq_qk_norm_stats: bad input dtype");
    if (q_out->dtype != VARQ_F32 || k_out->dtype != VARQ_F32) return fail(VARQ_ERR_ARG, "varq_qk_norm_stats: outputs are fp32");
    if ((k_stats && !column_grouping(k_grouping, D)) || (v_stats && !column_grouping(v_grouping, D)))
        return fail(VARQ_ERR_UNSUPPORTED, "varq_qk_norm_stats: statistics are folded for groupings shared over batch and tokens only");
    if ((long long)B * L * H == 0) return VARQ_OK;
    if ((long long)B * L >= 0x7fffffffLL) return fail(VARQ_ERR_UNSUPPORTED, "varq_qk_norm_stats: batch x tokens exceeds 2^31");
    if (!q_in->ptr || !k_in->ptr || !q_out->ptr || !k_out->ptr) return fail(VARQ_ERR_ARG, "varq_qk_norm_stats: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    PrepArgs a;
    a.q = q_in->ptr; a.k = k_in->ptr; a.v = v_in ? v_in->ptr : nullptr;
    a.q_dt = q_in->dtype; a.k_dt = k_in->dtype; a.v_dt = v_in ? v_in->dtype : VARQ_F32;
    a.qs_b = q_in->stride_b; a.qs_l = q_in->stride_l; a.qs_h = q_in->stride_h;
    a.ks_b = k_in->stride_b; a.ks_l = k_in->stride_l; a.ks_h = k_in->stride_h;
    a.vs_b = v_in ? v_in->stride_b : 0; a.vs_l = v_in ? v_in->stride_l : 0; a.vs_h = v_in ? v_in->stride_h : 0;
    a.q_out = (float*)q_out->ptr; a.k_out = (float*)k_out->ptr;
    a.qo_b = q_out->stride_b; a.qo_l = q_out->stride_l; a.qo_h = q_out->stride_h;
    a.ko_b = k_out->stride_b; a.ko_l = k_out->stride_l; a.ko_h = k_out->stride_h;
    a.scale_mul = scale_mul; a.eps = eps; a.B = B; a.L = L; a.H = H; a.D = D;
    a.k_stats = (uint32_t*)k_stats; a.v_stats = (uint32_t*)v_stats;
    a.k_sym = a.v_sym = 1; a.k_share_h = a.v_share_h = 0; a.k_group = a.v_group = 1; a.k_ng = a.v_ng = D;
    if (k_stats) {
        a.k_sym = k_grouping->zp == nullptr; a.k_share_h = k_grouping->share_h != 0; a.k_group = k_grouping->group; a.k_ng = D / k_grouping->group;
        VARQ_CUDA_TRY(cudaMemsetAsync(k_stats, 0, (size_t)(a.k_share_h ? 1 : H) * a.k_ng * 2 * sizeof(uint32_t), st));
    }
    if (v_stats) {
        a.v_sym = v_grouping->zp == nullptr; a.v_share_h = v_grouping->share_h != 0; a.v_group = v_grouping->group; a.v_ng = D / v_grouping->group;
        VARQ_CUDA_TRY(cudaMemsetAsync(v_stats, 0, (size_t)(a.v_share_h ? 1 : H) * a.v_ng * 2 * sizeof(uint32_t), st));
    }
    const int gx = (H + PREP_WARPS - 1) / PREP_WARPS;
    long long gy = ((long long)sm_count() * 8 + gx - 1) / gx;      // about eight CTAs of 256 threads per SM
    const long long R = (long long)B * L;
    if (gy > R) gy = R;
    if (gy > 65535) gy = 65535;
    if (gy < 1) gy = 1;
    qk_norm_stats_kernel<<<dim3(gx, (unsigned)gy), PREP_WARPS * 32, 0, st>>>(a);
    VARQ_CUDA_TRY(cudaGetLastError());
    count_launches(1);
    return VARQ_OK;
}
