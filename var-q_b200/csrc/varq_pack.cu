// Bit-packing of int8 codes, packed-code dequantisation, and the library's error plumbing.
// One thread owns one int32 word (4 / 8 / 16 codes) so packing needs no cross-lane traffic.
#include <cstdarg>
#include <cstdio>

#include "varq_common.cuh"

namespace varq {

static thread_local char g_err[512] = {0};

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    return fail(VARQ_ERR_CUDA, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

static unsigned long long g_launches = 0;
void count_launches(int n) { __atomic_fetch_add(&g_launches, (unsigned long long)n, __ATOMIC_RELAXED); }

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// A dim the descriptor marks as shared contributes no stride.  For tokens that holds when no row table is given
// (one parameter row describes every token); with a row table the rows are per appended step and keep their stride.
ParamView make_param_view(const varq_qparams_t* p) {
    ParamView v;
    v.scale = p->scale;
    v.zp = p->zp;
    v.row_of_token = p->row_of_token;
    v.row_begin = (p->row_of_token && p->n_rows > 0) ? p->row_begin : nullptr;
    v.n_rows = v.row_begin ? p->n_rows : 0;
    v.sb = p->share_b ? 0 : p->stride_b;
    v.sr = (p->share_l && p->row_of_token == nullptr) ? 0 : p->stride_r;
    v.sh = p->share_h ? 0 : p->stride_h;
    v.sg = p->stride_g;
    v.group = p->group;
    return v;
}

// ------------------------------------------------------------------ int8 <-> words
template <int BITS, bool VEC>
__global__ void pack_int8_kernel(const int8_t* __restrict__ q, long long n_rows, int c, int words_per_row,
                                 int32_t* __restrict__ out) {
    constexpr int VPW = 32 / BITS;
    const long long total = n_rows * words_per_row;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / words_per_row;
        const int w = (int)(i - r * words_per_row);
        const int8_t* src = q + r * c + (long long)w * VPW;
        int8_t v[VPW];
        if constexpr (VEC) {
            if constexpr (VPW == 16) *reinterpret_cast<uint4*>(v) = __ldg(reinterpret_cast<const uint4*>(src));
            else if constexpr (VPW == 8) *reinterpret_cast<uint2*>(v) = __ldg(reinterpret_cast<const uint2*>(src));
            else *reinterpret_cast<uint32_t*>(v) = __ldg(reinterpret_cast<const uint32_t*>(src));
        } else {
            const int n = min(VPW, c - w * VPW);
#pragma unroll
            for (int j = 0; j < VPW; ++j) v[j] = j < n ? src[j] : (int8_t)0;
        }
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < VPW; ++j) word |= ((uint32_t)(int)v[j] & ((1u << BITS) - 1u)) << (j * BITS);
        out[i] = (int32_t)word;
    }
}

template <int BITS, bool VEC>
__global__ void unpack_int8_kernel(const int32_t* __restrict__ words, long long n_rows, int c, int words_per_row,
                                   int8_t* __restrict__ out) {
    constexpr int VPW = 32 / BITS;
    const long long total = n_rows * words_per_row;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / words_per_row;
        const int w = (int)(i - r * words_per_row);
        const uint32_t word = (uint32_t)__ldg(words + i);
        int8_t v[VPW];
#pragma unroll
        for (int j = 0; j < VPW; ++j) v[j] = (int8_t)field<BITS>(word, j);
        int8_t* dst = out + r * c + (long long)w * VPW;
        if constexpr (VEC) {
            if constexpr (VPW == 16) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(v);
            else if constexpr (VPW == 8) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<uint2*>(v);
            else *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<uint32_t*>(v);
        } else {
            const int n = min(VPW, c - w * VPW);
#pragma unroll
            for (int j = 0; j < VPW; ++j)
                if (j < n) dst[j] = v[j];
        }
    }
}

static int grid_for(long long work_items, int threads) {
    long long blocks = (work_items + threads - 1) / threads;
    long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

// ------------------------------------------------------------------ words -> floats
struct DequantArgs {
    const int32_t* codes;
    long long cs_b, cs_l, cs_h;
    void* out;
    long long os_b, os_l, os_h;
    int B, L, H, D, words;
    ParamView p;
};

template <typename T, int BITS, bool VEC>
__global__ void unpack_dequant_kernel(DequantArgs a) {
    constexpr int VPW = 32 / BITS;
    const long long total = (long long)a.B * a.L * a.H * a.words;
    const bool uniform = (a.p.group % VPW) == 0;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int w = (int)(i % a.words);
        long long r = i / a.words;
        // row enumeration follows the code tensor's memory order
        int b, l, h;
        if (a.cs_h <= a.cs_l) { h = (int)(r % a.H); r /= a.H; l = (int)(r % a.L); b = (int)(r / a.L); }
        else                  { l = (int)(r % a.L); r /= a.L; h = (int)(r % a.H); b = (int)(r / a.H); }
        const uint32_t word = (uint32_t)__ldg(a.codes + b * a.cs_b + l * a.cs_l + h * a.cs_h + w);
        const int d0 = w * VPW;
        const int row = a.p.row(l);
        float v[VPW];
        if (uniform) {
            const long long pi = a.p.index(b, row, h, d0);
            const float s = __ldg(a.p.scale + pi);
            const float z = a.p.zp ? __ldg(a.p.zp + pi) : 0.0f;
#pragma unroll
            for (int j = 0; j < VPW; ++j) v[j] = __fmul_rn(__fsub_rn((float)field<BITS>(word, j), z), s);
        } else {
#pragma unroll
            for (int j = 0; j < VPW; ++j) {
                const int d = min(d0 + j, a.D - 1);
                const long long pi = a.p.index(b, row, h, d);
                const float s = __ldg(a.p.scale + pi);
                const float z = a.p.zp ? __ldg(a.p.zp + pi) : 0.0f;
                v[j] = __fmul_rn(__fsub_rn((float)field<BITS>(word, j), z), s);
            }
        }
        T* dst = reinterpret_cast<T*>(a.out) + b * a.os_b + l * a.os_l + h * a.os_h + d0;
        store_vals<T, VPW, VEC>(dst, v, a.D - d0);
    }
}

// Division of n < 2^31 by a fixed divisor d >= 1 as multiply-high + add + shift (Granlund-Montgomery):
// s = ceil(log2 d), m = floor(2^32 (2^s - d) / d) + 1, n / d = (umulhi(n, m) + n) >> s.
struct FastDiv {
    uint32_t m, s, d;
};
static FastDiv make_fastdiv(uint32_t d) {
    FastDiv f;
    f.d = d;
    f.s = 0;
    while ((1ull << f.s) < d) ++f.s;
    f.m = (uint32_t)(((1ull << 32) * ((1ull << f.s) - d)) / d + 1);
    return f;
}
__device__ __forceinline__ void divmod(uint32_t n, const FastDiv& f, uint32_t& q, uint32_t& r) {
    q = (__umulhi(n, f.m) + n) >> f.s;
    r = n - q * f.d;
}

// Fast path of the kernel above for tensors below 2^31 words: the same word-per-thread mapping (stores of
// neighbouring lanes stay contiguous) with 32-bit index arithmetic and divisions by multiply-high.
template <typename T, int BITS>
__global__ void __launch_bounds__(256) unpack_dequant_w32_kernel(DequantArgs a, unsigned total, FastDiv dW, FastDiv dH, FastDiv dL) {
    constexpr int VPW = 32 / BITS;
    const bool h_inner = a.cs_h <= a.cs_l;                       // row enumeration follows the code tensor's memory order
    const bool uniform = (a.p.group % VPW) == 0;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        unsigned r, w, b, l, h, t;
        divmod(i, dW, r, w);
        if (h_inner) { divmod(r, dH, t, h); divmod(t, dL, b, l); }
        else         { divmod(r, dL, t, l); divmod(t, dH, b, h); }
        const uint32_t word = (uint32_t)__ldg(a.codes + b * a.cs_b + l * a.cs_l + h * a.cs_h + w);
        const int row = a.p.row((int)l);
        float v[VPW];
        if (uniform) {
            const long long pi = a.p.index((int)b, row, (int)h, (int)(w * VPW));
            const float s = __ldg(a.p.scale + pi);
            const float z = a.p.zp ? __ldg(a.p.zp + pi) : 0.0f;
#pragma unroll
            for (int j = 0; j < VPW; ++j) v[j] = __fmul_rn(__fsub_rn((float)field<BITS>(word, j), z), s);
        } else {
            // a word spans several groups (per-dim parameters): one parameter pair per value
            const long long p0 = a.p.index((int)b, row, (int)h, 0);
#pragma unroll
            for (int j = 0; j < VPW; ++j) {
                const int d = (int)(w * VPW) + j;
                const long long pi = p0 + (long long)(a.p.group == 1 ? d : d / a.p.group) * a.p.sg;
                const float s = __ldg(a.p.scale + pi);
                const float z = a.p.zp ? __ldg(a.p.zp + pi) : 0.0f;
                v[j] = __fmul_rn(__fsub_rn((float)field<BITS>(word, j), z), s);
            }
        }
        store_vals<T, VPW, true>(reinterpret_cast<T*>(a.out) + b * a.os_b + l * a.os_l + h * a.os_h + w * VPW, v, VPW);
    }
}

template <typename T, int BITS>
static int launch_dequant(const DequantArgs& a, bool vec, cudaStream_t st) {
    const long long total = (long long)a.B * a.L * a.H * a.words;
    if (total == 0) return VARQ_OK;
    const int threads = 256;
    constexpr int VPW = 32 / BITS;
    if (vec && a.D == a.words * VPW && total < (1ll << 31)) {
        unpack_dequant_w32_kernel<T, BITS><<<grid_for(total, threads), threads, 0, st>>>(
            a, (unsigned)total, make_fastdiv((uint32_t)a.words), make_fastdiv((uint32_t)a.H), make_fastdiv((uint32_t)a.L));
        VARQ_CUDA_TRY(cudaGetLastError());
        count_launches(1);
        return VARQ_OK;
    }
    const int blocks = grid_for(total, threads);
    if (vec) unpack_dequant_kernel<T, BITS, true><<<blocks, threads, 0, st>>>(a);
    else     unpack_dequant_kernel<T, BITS, false><<<blocks, threads, 0, st>>>(a);
    VARQ_CUDA_TRY(cudaGetLastError());
    count_launches(1);
    return VARQ_OK;
}

template <int BITS>
static int dispatch_dequant(const DequantArgs& a, int dtype, bool vec, cudaStream_t st) {
    switch (dtype) {
        case VARQ_F32: return launch_dequant<float, BITS>(a, vec, st);
        case VARQ_F16: return launch_dequant<__half, BITS>(a, vec, st);
        default:       return launch_dequant<__nv_bfloat16, BITS>(a, vec, st);
    }
}

}  // namespace varq

using namespace varq;

extern "C" const char* varq_version(void) { return "varq_b200 0.1 (sm_100a)"; }

extern "C" const char* varq_last_error(void) { return g_err; }

extern "C" uint64_t varq_launch_count(void) { return __atomic_load_n(&g_launches, __ATOMIC_RELAXED); }

extern "C" int varq_pack_int8(const int8_t* codes, int64_t n_rows, int32_t c, int32_t bits, int32_t* words,
                              void* stream) {
    if (bits != 2 && bits != 4 && bits != 8) return fail(VARQ_ERR_ARG, "varq_pack_int8: bits must be 2, 4 or 8 (got %d)", bits);
    if (n_rows < 0 || c <= 0) return fail(VARQ_ERR_ARG, "varq_pack_int8: bad shape [%lld, %d]", (long long)n_rows, c);
    if (n_rows == 0) return VARQ_OK;
    if (!codes || !words) return fail(VARQ_ERR_ARG, "varq_pack_int8: null pointer");
    const int vpw = 32 / bits, wpr = (c + vpw - 1) / vpw;
    const bool vec = (c % vpw == 0) && ((reinterpret_cast<uintptr_t>(codes) % vpw) == 0);
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = 256, blocks = grid_for(n_rows * wpr, threads);
#define LAUNCH(B_)                                                                                   \
    if (vec) pack_int8_kernel<B_, true><<<blocks, threads, 0, st>>>(codes, n_rows, c, wpr, words);   \
    else     pack_int8_kernel<B_, false><<<blocks, threads, 0, st>>>(codes, n_rows, c, wpr, words)
    if (bits == 8) { LAUNCH(8); } else if (bits == 4) { LAUNCH(4); } else { LAUNCH(2); }
#undef LAUNCH
    VARQ_CUDA_TRY(cudaGetLastError());
    count_launches(1);
    return VARQ_OK;
}

extern "C" int varq_unpack_int8(const int32_t* words, int64_t n_rows, int32_t c, int32_t bits, int8_t* codes,
                                void* stream) {
    if (bits != 2 && bits != 4 && bits != 8) return fail(VARQ_ERR_ARG, "varq_unpack_int8: bits must be 2, 4 or 8 (got %d)", bits);
    if (n_rows < 0 || c <= 0) return fail(VARQ_ERR_ARG, "varq_unpack_int8: bad shape [%lld, %d]", (long long)n_rows, c);
    if (n_rows == 0) return VARQ_OK;
    if (!codes || !words) return fail(VARQ_ERR_ARG, "varq_unpack_int8: null pointer");
    const int vpw = 32 / bits, wpr = (c + vpw - 1) / vpw;
    const bool vec = (c % vpw == 0) && ((reinterpret_cast<uintptr_t>(codes) % vpw) == 0);
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = 256, blocks = grid_for(n_rows * wpr, threads);
#define LAUNCH(B_)                                                                                     \
    if (vec) unpack_int8_kernel<B_, true><<<blocks, threads, 0, st>>>(words, n_rows, c, wpr, codes);   \
    else     unpack_int8_kernel<B_, false><<<blocks, threads, 0, st>>>(words, n_rows, c, wpr, codes)
    if (bits == 8) { LAUNCH(8); } else if (bits == 4) { LAUNCH(4); } else { LAUNCH(2); }
#undef LAUNCH
    VARQ_CUDA_TRY(cudaGetLastError());
    count_launches(1);
    return VARQ_OK;
}

extern "C" int varq_unpack_dequant(const varq_tensor_t* codes, int32_t B, int32_t L, int32_t H, int32_t D,
                                   int32_t store_bits, const varq_qparams_t* p, const varq_tensor_t* out,
                                   void* stream) {
    if (!codes || !p || !out) return fail(VARQ_ERR_ARG, "varq_unpack_dequant: null descriptor");
    if (store_bits != 2 && store_bits != 4 && store_bits != 8)
        return fail(VARQ_ERR_ARG, "varq_unpack_dequant: store_bits must be 2, 4 or 8 (got %d)", store_bits);
    if (B < 0 || L < 0 || H < 0 || D <= 0) return fail(VARQ_ERR_ARG, "varq_unpack_dequant: bad shape");
    if (!dtype_ok(out->dtype)) return fail(VARQ_ERR_ARG, "varq_unpack_dequant: bad output dtype %d", out->dtype);
    if ((long long)B * L * H == 0) return VARQ_OK;
    if (!codes->ptr || !out->ptr || !p->scale) return fail(VARQ_ERR_ARG, "varq_unpack_dequant: null pointer");
    if (p->group < 1 || p->group > D) return fail(VARQ_ERR_ARG, "varq_unpack_dequant: group must be in [1, D]");
    const int vpw = 32 / store_bits;
    DequantArgs a;
    a.codes = (const int32_t*)codes->ptr;
    a.cs_b = codes->stride_b; a.cs_l = codes->stride_l; a.cs_h = codes->stride_h;
    a.out = out->ptr;
    a.os_b = out->stride_b; a.os_l = out->stride_l; a.os_h = out->stride_h;
    a.B = B; a.L = L; a.H = H; a.D = D; a.words = (D + vpw - 1) / vpw;
    a.p = make_param_view(p);
    const int es = dtype_size(out->dtype);
    const int chunk = (vpw * es) < 16 ? (vpw * es) : 16;
    const bool vec = (D % vpw == 0) && ((reinterpret_cast<uintptr_t>(out->ptr) % chunk) == 0) &&
                     ((out->stride_b * es) % chunk == 0) && ((out->stride_l * es) % chunk == 0) &&
                     ((out->stride_h * es) % chunk == 0);
    cudaStream_t st = (cudaStream_t)stream;
    if (store_bits == 8) return dispatch_dequant<8>(a, out->dtype, vec, st);
    if (store_bits == 4) return dispatch_dequant<4>(a, out->dtype, vec, st);
    return dispatch_dequant<2>(a, out->dtype, vec, st);
}
