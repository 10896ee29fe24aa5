// Argument block shared by the attention kernels of the varq_b200 library.
#pragma once
#include "varq_common.cuh"

namespace varq {

struct AttnArgs {
    const void* q; int q_dtype; long long qs_b, qs_l, qs_h;
    void* out; int o_dtype; long long os_b, os_l, os_h;
    const int32_t* kc; long long ks_b, ks_l, ks_h;
    const int32_t* vc; long long vs_b, vs_l, vs_h;
    ParamView kp, vp;
    int B, H, Lq, Lk, D;
    int wk, wv, kpitch;         // words per K / V row, padded K pitch in shared memory
    int k16, v16;               // 16-byte cp.async usable
    float scale_log2;           // softmax_scale * log2(e)
    int splits, tiles_per_split;
    int n_qtiles;               // query tiles per (sample, head); grids are 1-D: ((b*H + h) * n_qtiles + qtile) * splits + split
    float* ws;                  // partials: [(b,h,qtile,split)][QT*(2+D)]
    // Tensor-core kernel: per-tile parameter streams written by its preparation kernel, one block per (sample, head, key tile):
    // softmax tables, normaliser records, then (when the packed-half converters apply) the (key, group) records of K and of V,
    // each followed by a 16-byte trailer whose first word says that the tile needs the fp32 converter.
    unsigned char* prep = nullptr;
    long long prep_bh_stride = 0;
    int prep_tile_stride = 0, prep_off_vn = 0, prep_off_krec = 0, prep_off_vrec = 0;
    int prep_krec_bytes = 0, prep_vrec_bytes = 0;       // 0 = no records
    // Per-dim parameters that the tokens of an appended step share: per (sample, head) a table [steps][3][D] of fp16
    // (scale hi, scale lo, 1024 + bias + zero-point), and the records of a tile are then the step index of every key (uint16).
    const unsigned char* prep_ktab = nullptr;
    const unsigned char* prep_vtab = nullptr;
    long long prep_tab_bh_stride = 0;               // bytes between the tables of two (sample, head) pairs
    int tc_k_perdim = 0, tc_v_perdim = 0;
};

__device__ __forceinline__ float load_q_elem(const void* q, int dtype, long long off) {
    if (dtype == VARQ_F32) return __ldg(reinterpret_cast<const float*>(q) + off);
    if (dtype == VARQ_F16) return __half2float(__ldg(reinterpret_cast<const __half*>(q) + off));
    return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(q) + off));
}
// eight consecutive elements starting at element `off`; 16-byte loads when the address allows
__device__ __forceinline__ void load_q8(const void* q, int dtype, long long off, float (&v)[8]) {
    const int es = dtype == VARQ_F32 ? 4 : 2;
    const uintptr_t addr = reinterpret_cast<uintptr_t>(q) + (unsigned long long)off * es;
    if (addr & 15u) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = load_q_elem(q, dtype, off + j);
    } else if (dtype == VARQ_F32) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(addr)), b = __ldg(reinterpret_cast<const float4*>(addr) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(addr));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (dtype == VARQ_F16) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                v[2 * j] = f.x; v[2 * j + 1] = f.y;
            } else {                         // a bf16 is the upper half of an fp32
                v[2 * j] = __uint_as_float(w[j] << 16);
                v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
            }
        }
    }
}
__device__ __forceinline__ void store_o_elem(void* o, int dtype, long long off, float v) {
    if (dtype == VARQ_F32) reinterpret_cast<float*>(o)[off] = v;
    else if (dtype == VARQ_F16) reinterpret_cast<__half*>(o)[off] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16*>(o)[off] = __float2bfloat16_rn(v);
}
// 32 consecutive outputs starting at element `off`; 16-byte stores when the address allows
__device__ __forceinline__ void store_o_row32(void* o, int dtype, long long off, const float (&v)[32]) {
    const int es = dtype == VARQ_F32 ? 4 : 2;
    const bool wide = (((reinterpret_cast<uintptr_t>(o) + (unsigned long long)off * es) & 15u) == 0);
    if (!wide) {
#pragma unroll
        for (int c = 0; c < 32; ++c) store_o_elem(o, dtype, off + c, v[c]);
    } else if (dtype == VARQ_F32) {
        float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + off);
#pragma unroll
        for (int c = 0; c < 8; ++c) p[c] = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
    } else {
        uint4* p = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(o) + off);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (dtype == VARQ_F16) {
                    const __half2 h = __floats2half2_rn(v[8 * c + 2 * j], v[8 * c + 2 * j + 1]);
                    w[j] = *reinterpret_cast<const uint32_t*>(&h);
                } else {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * c + 2 * j], v[8 * c + 2 * j + 1]);
                    w[j] = *reinterpret_cast<const uint32_t*>(&h);
                }
            }
            p[c] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

size_t attn_small_workspace_bytes(int B, int H, int Lq, int Lk, int D);
int attn_small_run(AttnArgs& a, int kb, int vb, void* ws, size_t ws_bytes, cudaStream_t st);
bool attn_stream_eligible(const AttnArgs& a, int kb, int vb);
size_t attn_stream_workspace_bytes(int B, int H, int Lq, int Lk, int D);
int attn_stream_run(AttnArgs& a, int kb, int vb, void* ws, size_t ws_bytes, cudaStream_t st);
bool attn_tc_eligible(const AttnArgs& a, int kb, int vb);
int attn_tc_run(const AttnArgs& a, int kb, int vb, void* ws, size_t ws_bytes, cudaStream_t st);
size_t attn_tc_workspace_bytes(int B, int H, int Lk, int D);
int attn_tc_status(int* out);
bool attn_mid_eligible(const AttnArgs& a, int kb, int vb);
int attn_mid_run(AttnArgs& a, int kb, int vb, cudaStream_t st);

}  // namespace varq
