// Shared device/host helpers of the varq_b200 library (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "varq_b200.h"

namespace varq {

// ---- host-side error reporting (thread-local message, C ABI returns a code)
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
#define VARQ_CUDA_TRY(expr)                                        \
    do {                                                           \
        cudaError_t _e = (expr);                                   \
        if (_e != cudaSuccess) return ::varq::cuda_fail(_e, #expr); \
    } while (0)

inline int dtype_size(int dt) { return dt == VARQ_F32 ? 4 : 2; }
inline bool dtype_ok(int dt) { return dt == VARQ_F32 || dt == VARQ_F16 || dt == VARQ_BF16; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
int sm_count();
void count_launches(int n);   // bookkeeping behind varq_launch_count()

// ---- order-preserving float <-> uint32 map, so min/max can use integer atomics
__device__ __forceinline__ uint32_t f2ord(float f) {
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ord2f(uint32_t u) {
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

// ---- element conversion
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Load N consecutive elements as fp32.  VEC: p is aligned to min(16, N*sizeof(T)) bytes
// and all N elements exist; otherwise scalar loads of the first n_valid, rest = 0.
template <typename T, int N, bool VEC>
__device__ __forceinline__ void load_vals(const T* __restrict__ p, float (&v)[N], int n_valid) {
    if constexpr (VEC) {
        constexpr int BYTES = N * (int)sizeof(T);
        if constexpr (BYTES >= 16) {
            constexpr int CH = BYTES / 16, PER = 16 / (int)sizeof(T);
            uint4 raw[CH];
#pragma unroll
            for (int i = 0; i < CH; ++i) raw[i] = __ldg(reinterpret_cast<const uint4*>(p) + i);
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                const T* e = reinterpret_cast<const T*>(&raw[i]);
#pragma unroll
                for (int j = 0; j < PER; ++j) v[i * PER + j] = to_f32<T>(e[j]);
            }
        } else {  // 8 bytes: four 16-bit elements
            uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int j = 0; j < N; ++j) v[j] = to_f32<T>(e[j]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < N; ++j) v[j] = (j < n_valid) ? to_f32<T>(p[j]) : 0.0f;
    }
}

// Store N consecutive elements converted from fp32 (same alignment contract).
template <typename T, int N, bool VEC>
__device__ __forceinline__ void store_vals(T* __restrict__ p, const float (&v)[N], int n_valid) {
    if constexpr (VEC) {
        constexpr int BYTES = N * (int)sizeof(T);
        if constexpr (BYTES >= 16) {
            constexpr int CH = BYTES / 16, PER = 16 / (int)sizeof(T);
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                uint4 raw;
                T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
                for (int j = 0; j < PER; ++j) e[j] = from_f32<T>(v[i * PER + j]);
                reinterpret_cast<uint4*>(p)[i] = raw;
            }
        } else {
            uint2 raw;
            T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
            for (int j = 0; j < N; ++j) e[j] = from_f32<T>(v[j]);
            *reinterpret_cast<uint2*>(p) = raw;
        }
    } else {
#pragma unroll
        for (int j = 0; j < N; ++j)
            if (j < n_valid) p[j] = from_f32<T>(v[j]);
    }
}

// Signed field j of a packed word (fields are `BITS` wide, little-endian).
template <int BITS> __device__ __forceinline__ int field(uint32_t w, int j) {
    return ((int)(w << (32 - BITS * (j + 1)))) >> (32 - BITS);
}

// Device-side copy of varq_qparams_t with shared strides zeroed.
struct ParamView {
    const float* scale;
    const float* zp;
    const int32_t* row_of_token;
    const int32_t* row_begin;      // first token of every row (n_rows + 1 entries), or null
    int n_rows;
    long long sb, sr, sh, sg;
    int group;
    __device__ __forceinline__ long long index(int b, int row, int h, int d) const {
        return b * sb + row * sr + h * sh + (long long)(d / group) * sg;
    }
    __device__ __forceinline__ int row(int token) const {
        return row_of_token ? __ldg(row_of_token + token) : token;
    }
};
ParamView make_param_view(const varq_qparams_t* p);

}  // namespace varq
