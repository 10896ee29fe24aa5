// C entry points of attention over the packed cache: argument checks and kernel selection.
#include "varq_attn.cuh"

using namespace varq;

// Kernel choice pinned by varq_attn_force_path (0 = automatic).  A test hook, not a fallback switch: a pinned
// kernel that cannot take the call still yields to the general CUDA-core kernel.
static int g_forced_path = 0;

static bool words_aligned16(const varq_tensor_t* t, int words) {
    return (words % 4 == 0) && aligned16(t->ptr) && (t->stride_b % 4 == 0) && (t->stride_l % 4 == 0) &&
           (t->stride_h % 4 == 0);
}

extern "C" size_t varq_attn_workspace_bytes(int32_t B, int32_t H, int32_t Lq, int32_t Lk, int32_t D,
                                            int32_t k_store_bits, int32_t v_store_bits) {
    (void)k_store_bits; (void)v_store_bits;
    if (B <= 0 || H <= 0 || Lq <= 0 || Lk <= 0 || D <= 0) return 0;
    const size_t s1 = attn_small_workspace_bytes(B, H, Lq, Lk, D), s2 = attn_stream_workspace_bytes(B, H, Lq, Lk, D);
    const size_t s3 = attn_tc_workspace_bytes(B, H, Lk, D);
    const size_t s12 = s1 > s2 ? s1 : s2;
    return s12 > s3 ? s12 : s3;
}

extern "C" int varq_attn_fwd(const varq_tensor_t* q, const varq_tensor_t* k_codes, const varq_tensor_t* v_codes,
                             const varq_qparams_t* kp, const varq_qparams_t* vp, int32_t B, int32_t H, int32_t Lq,
                             int32_t Lk, int32_t D, int32_t kb, int32_t vb, float softmax_scale,
                             const varq_tensor_t* out, void* workspace, size_t workspace_bytes, void* stream) {
    if (!q || !k_codes || !v_codes || !kp || !vp || !out) return fail(VARQ_ERR_ARG, "varq_attn_fwd: null descriptor");
    if ((kb != 2 && kb != 4 && kb != 8) || (vb != 2 && vb != 4 && vb != 8))
        return fail(VARQ_ERR_ARG, "varq_attn_fwd: store bits must be 2, 4 or 8 (got %d, %d)", kb, vb);
    if (B < 0 || H < 0 || Lq < 0 || Lk < 0 || D <= 0) return fail(VARQ_ERR_ARG, "varq_attn_fwd: bad shape");
    if (!dtype_ok(q->dtype) || !dtype_ok(out->dtype)) return fail(VARQ_ERR_ARG, "varq_attn_fwd: bad q/out dtype");
    if ((long long)B * H * Lq == 0) return VARQ_OK;
    if (Lk == 0) return fail(VARQ_ERR_ARG, "varq_attn_fwd: empty cache (Lk = 0)");
    if (!q->ptr || !out->ptr || !k_codes->ptr || !v_codes->ptr || !kp->scale || !vp->scale)
        return fail(VARQ_ERR_ARG, "varq_attn_fwd: null pointer");
    if (kp->group < 1 || kp->group > D || D % kp->group || vp->group < 1 || vp->group > D || D % vp->group)
        return fail(VARQ_ERR_ARG, "varq_attn_fwd: group must divide head_dim");
    const int kvw = 32 / kb, vvw = 32 / vb;
    if (D % kvw || D % vvw || D % 4) return fail(VARQ_ERR_UNSUPPORTED, "varq_attn_fwd: head_dim %d must be a multiple of the codes per word (%d, %d)", D, kvw, vvw);
    const int wk = D / kvw, wv = D / vvw;
    if (wv > 128 || (128 % wv) != 0)
        return fail(VARQ_ERR_UNSUPPORTED, "varq_attn_fwd: V words per row (%d) must divide 128", wv);
    if (D > 256) return fail(VARQ_ERR_UNSUPPORTED, "varq_attn_fwd: head_dim %d > 256", D);

    AttnArgs a;
    a.q = q->ptr; a.q_dtype = q->dtype; a.qs_b = q->stride_b; a.qs_l = q->stride_l; a.qs_h = q->stride_h;
    a.out = out->ptr; a.o_dtype = out->dtype; a.os_b = out->stride_b; a.os_l = out->stride_l; a.os_h = out->stride_h;
    a.kc = (const int32_t*)k_codes->ptr; a.ks_b = k_codes->stride_b; a.ks_l = k_codes->stride_l; a.ks_h = k_codes->stride_h;
    a.vc = (const int32_t*)v_codes->ptr; a.vs_b = v_codes->stride_b; a.vs_l = v_codes->stride_l; a.vs_h = v_codes->stride_h;
    a.kp = make_param_view(kp);
    a.vp = make_param_view(vp);
    a.B = B; a.H = H; a.Lq = Lq; a.Lk = Lk; a.D = D;
    a.wk = wk; a.wv = wv; a.kpitch = wk;
    a.k16 = words_aligned16(k_codes, wk);
    a.v16 = words_aligned16(v_codes, wv);
    a.scale_log2 = softmax_scale * 1.4426950408889634f;
    a.splits = 1; a.tiles_per_split = 0; a.n_qtiles = 1; a.ws = reinterpret_cast<float*>(workspace);
    // The CUDA-core streaming kernel is memory-bound only while its arithmetic (queries x keys x head_dim on the FMA pipe)
    // stays below the time to stream the packed cache: up to 4 queries at any cache length, and the 1-16-query first scales
    // of a schedule, whose caches are a few hundred tokens at most.  Everything else goes to the tensor cores, where a
    // 128-row tile with few live rows still finishes a long cache sooner.
    const int force = __atomic_load_n(&g_forced_path, __ATOMIC_RELAXED);
    const bool small_q = Lq <= 4 || (Lq <= 16 && Lk <= 256);
    // Between the two: tens of queries over at most a few hundred tokens (the early scales of a schedule), where the tcgen05
    // kernel is bound by its per-CTA set-up; a warp-level tensor-core kernel takes them when the parameters are per key.
    const bool mid_q = Lq > 8 && Lq <= 64 && Lk <= 256;          // measured against both neighbours (B64 H16 and B128 H30, c 64)
    const bool want_mid = force ? (force == VARQ_ATTN_PATH_MID) : mid_q;
    if (want_mid && attn_mid_eligible(a, kb, vb)) return attn_mid_run(a, kb, vb, (cudaStream_t)stream);
    const bool want_tc = force ? (force == VARQ_ATTN_PATH_TC) : !small_q;
    if (want_tc && attn_tc_eligible(a, kb, vb)) return attn_tc_run(a, kb, vb, workspace, workspace_bytes, (cudaStream_t)stream);
    const bool want_stream = force ? (force == VARQ_ATTN_PATH_STREAM) : small_q;
    if (want_stream && attn_stream_eligible(a, kb, vb)) return attn_stream_run(a, kb, vb, workspace, workspace_bytes, (cudaStream_t)stream);
    return attn_small_run(a, kb, vb, workspace, workspace_bytes, (cudaStream_t)stream);
}

extern "C" int varq_attn_force_path(int32_t path) {
    if (path < VARQ_ATTN_PATH_AUTO || path > VARQ_ATTN_PATH_MID) return fail(VARQ_ERR_ARG, "varq_attn_force_path: unknown path %d", path);
    __atomic_store_n(&g_forced_path, (int)path, __ATOMIC_RELAXED);
    return VARQ_OK;
}

extern "C" int varq_device_status(int32_t* status) {
    if (!status) return fail(VARQ_ERR_ARG, "varq_device_status: null pointer");
    int v = 0;
    if (int rc = attn_tc_status(&v)) return rc;
    *status = v;
    return VARQ_OK;
}
