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
    float* ws;                  // partials: [(b,h,qtile,split)][QT*(2+D)]
};

size_t attn_small_workspace_bytes(int B, int H, int Lq, int Lk, int D);
int attn_small_run(AttnArgs& a, int kb, int vb, void* ws, size_t ws_bytes, cudaStream_t st);

}  // namespace varq
