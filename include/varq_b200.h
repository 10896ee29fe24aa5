/*
 * varq_b200 -- C ABI of the B200 (sm_100a) KV-cache quantization library.
 *
 * The reference project is pure Python and has no FFI of its own; every entry point
 * below names the reference code it replaces (paths inside the reference project).
 * All pointers are DEVICE pointers unless stated otherwise, all work is enqueued on
 * the given CUDA stream (passed as void* = cudaStream_t), and nothing here
 * synchronises the device.  Functions return VARQ_OK or a negative error code and
 * never throw or trap; varq_last_error() gives the message of the calling thread's
 * last failure.
 *
 * Logical tensor shape is always (B, L, H, D): batch, tokens, heads, head_dim.
 * A tensor descriptor carries element strides for B, L and H; D is unit-stride.
 * This covers the reference's 'BLHc' and 'BHLc' layouts (VAR_Q/quant.py:75-95) and
 * the strided q/k/v views cut out of a fused QKV buffer
 * (VAR/models/basic_var.py:123-135) without a staging copy.
 */
#ifndef VARQ_B200_H
#define VARQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VARQ_OK                0
#define VARQ_ERR_ARG          -1   /* null pointer, bad size, bad enum            */
#define VARQ_ERR_UNSUPPORTED  -2   /* combination this build has no kernel for    */
#define VARQ_ERR_CUDA         -3   /* launch or runtime failure                   */
#define VARQ_ERR_WORKSPACE    -4   /* workspace missing or too small              */

#define VARQ_F32  0
#define VARQ_F16  1
#define VARQ_BF16 2

/* A (B, L, H, D) tensor whose last dim is contiguous.  Strides count elements of
 * the tensor's own type (floats, halves, or int32 words for packed codes). */
typedef struct {
    void*   ptr;
    int32_t dtype;          /* VARQ_F32 / F16 / BF16; ignored for packed codes */
    int32_t _pad;
    int64_t stride_b, stride_l, stride_h;
} varq_tensor_t;

/* Quantization parameters of a tensor or of a whole cache.
 *
 * A group is the set of elements that share one scale (and zero-point):
 *   share_b / share_l / share_h = 1 : the group spans the whole batch / all tokens of
 *   the call / all heads;  group = number of consecutive head_dim elements in it.
 * The six reference modes (VAR_Q/quant.py:78-95) map to
 *   G_TENSOR, G_SCALE            : share_b=share_l=share_h=1, group=D
 *   G_SCALE_HEAD_DIM, G_HEAD_DIM : share_b=share_l=1, share_h=0, group=1
 *   G_TOKEN                      : share_b=share_h=1, share_l=0, group=D
 *   G_TOKEN_HEAD                 : share_b=1, share_l=share_h=0, group=D (or smaller)
 * scale[i], zp[i] live at i = b*stride_b + row*stride_r + h*stride_h + (d/group)*stride_g
 * with the stride of a shared dim ignored.  `row` is the token index, or
 * row_of_token[token] when that table is given (modes whose parameters are constant
 * over the tokens of one appended step keep one row per step).
 * zp == NULL means symmetric quantization.
 * row_begin (optional, only read together with row_of_token): row_begin[r] is the first token of row r and
 * row_begin[n_rows] the number of tokens described, i.e. the inverse of row_of_token for rows that cover
 * consecutive tokens (one row per appended step).  Attention uses it to cut its key tiles at step boundaries,
 * which lets per-dim scales that are constant over a step be folded into the queries; without it such
 * groupings are dequantised element by element. */
typedef struct {
    float*         scale;
    float*         zp;
    const int32_t* row_of_token;
    int64_t stride_b, stride_r, stride_h, stride_g;
    int32_t share_b, share_l, share_h, group;
    const int32_t* row_begin;
    int32_t n_rows, _pad;
} varq_qparams_t;

/* Version string, static storage. */
const char* varq_version(void);

/* Message of the calling thread's last failed call (empty string if none). */
const char* varq_last_error(void);

/* Number of kernels this library has launched in the process so far (all threads).
 * No counterpart in the reference; benchmarks use it to report their launch count. */
uint64_t varq_launch_count(void);

/* Every wait inside the kernels is bounded; a wait that expires makes the kernel record a
 * non-zero code and drain instead of hanging.  This call waits for all prior work of the current
 * device (cudaDeviceSynchronize), returns the first such code since the last call (0 = none) and
 * clears it.  HOST pointer.  No counterpart in the reference. */
int varq_device_status(int32_t* status);

/* Pack int8 codes [n_rows, c] into int32 words [n_rows, ceil(c / (32/bits))]:
 * value j of a word occupies bits [j*bits, (j+1)*bits), tail zero-padded.
 * Replaces pack_last_dim_to_int32_triton / _python (VAR_Q/pack_unpack.py:107-134,
 * 177-196) and the Triton kernel _pack2d_kernel (VAR_Q/pack_unpack.py:18-51). */
int varq_pack_int8(const int8_t* codes, int64_t n_rows, int32_t c, int32_t bits,
                   int32_t* words, void* stream);

/* Inverse with sign extension.  Replaces unpack_last_dim_from_int32_triton / _python
 * (VAR_Q/pack_unpack.py:136-162, 198-211) and _unpack2d_kernel (:54-88). */
int varq_unpack_int8(const int32_t* words, int64_t n_rows, int32_t c, int32_t bits,
                     int8_t* codes, void* stream);

/* Bytes of scratch varq_quant_pack needs for this shape and grouping (0 if none). */
size_t varq_quant_workspace_bytes(int32_t B, int32_t L, int32_t H, int32_t D,
                                  int32_t x_dtype, int32_t store_bits,
                                  const varq_qparams_t* grouping);

/* Fused statistics -> scale (/zero-point) -> round -> clamp -> bit-pack of fresh K or V.
 *   symmetric : scale = max(amax|x| / (2^(bits-1)-1), eps); q = clamp(rint(x/scale))
 *   asymmetric: scale = max((max-min) / (2^bits-1), eps); zp = rint(-2^(bits-1) - min/scale);
 *               q = clamp(rint(x/scale) + zp)
 * all in fp32 with true division and round-half-even.  `bits` (2..8) sets the code
 * range, `store_bits` (2, 4 or 8, >= bits) the packed field width.  Codes go to
 * `codes` (int32 words, strides in words), parameters to p->scale / p->zp at row 0
 * (offset the pointers to the row being written).
 * Replaces VAR_Q._compute_scale, _quantize_to_int8 and _pack_last_dim_to_int32 as
 * used by VAR_Q.quant (VAR_Q/quant.py:112-121, 127-131, 140-177). */
int varq_quant_pack(const varq_tensor_t* x, int32_t B, int32_t L, int32_t H, int32_t D,
                    int32_t bits, int32_t store_bits, float eps,
                    const varq_tensor_t* codes, const varq_qparams_t* p,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Producer side of the attention hook in one pass over the fresh q, k, v (views of the fused QKV activation):
 *   q_out = q / max(||q||_2, eps) * scale_mul[h],   k_out = k / max(||k||_2, eps)          (fp32, norms over head_dim)
 * and, in the same read, the min / max statistics of k_out and of v for groupings that are shared over batch and
 * tokens (per-dim, per-step, per-tensor), folded into `k_stats` / `v_stats` (varq_quant_workspace_bytes() bytes each,
 * cleared by this call).  varq_quant_pack_prestats then quantizes from those tables without a statistics pass of its
 * own, so K and V are read once less.  scale_mul may be NULL (= 1); v_in / the statistics pointers may be NULL.
 * Replaces the L2-normalisation of VAR/models/basic_var.py:137-141 and Infinity/infinity/models/basic.py:316-320
 * and the first pass of VAR_Q._compute_scale (VAR_Q/quant.py:112-116). */
int varq_qk_norm_stats(const varq_tensor_t* q_in, const varq_tensor_t* k_in, const varq_tensor_t* v_in,
                       int32_t B, int32_t L, int32_t H, int32_t D, const float* scale_mul, float eps,
                       const varq_tensor_t* q_out, const varq_tensor_t* k_out,
                       const varq_qparams_t* k_grouping, void* k_stats,
                       const varq_qparams_t* v_grouping, void* v_stats, void* stream);

/* varq_quant_pack with the statistics table already filled by varq_qk_norm_stats (same grouping, same tensor):
 * scale / zero-point computation, rounding and packing only.  Same results as varq_quant_pack. */
int varq_quant_pack_prestats(const varq_tensor_t* x, int32_t B, int32_t L, int32_t H, int32_t D,
                             int32_t bits, int32_t store_bits, float eps,
                             const varq_tensor_t* codes, const varq_qparams_t* p,
                             void* stats, size_t stats_bytes, void* stream);

/* varq_quant_pack for callers that may not allocate device memory and have no scratch
 * buffer to lend.  No counterpart in the reference.
 *
 * Who this is for: hosts where every byte of HBM already belongs to someone else's pool --
 * an inference server that handed the whole device to its KV-cache allocator, a plugin
 * loaded into an application that forbids cudaMalloc from plugin code -- and loops that
 * cannot tolerate the device-wide synchronisation an allocation may cost.  Inputs and
 * outputs are still the caller's; only the statistics table that the per-dim, per-token
 * and per-tensor groupings need comes from a fixed array inside the library image.  This
 * function and everything below it call no cudaMalloc / cudaFree and no allocating
 * library routine.
 *
 * Limits and rules:
 *  - the array holds 65536 groups (512 KiB, see varq_quant_static_scratch_bytes()); every
 *    GPU that loads the library keeps it until the process exits.  A grouping with more
 *    groups is refused with VARQ_ERR_WORKSPACE and a message naming both numbers;
 *  - the first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current).  Make that first call during
 *    set-up, before any stream capture begins on that device;
 *  - all calls on a device share the one array and it keeps the previous call's contents;
 *    each call re-zeroes the part it uses on `stream` before accumulating.  Two calls
 *    whose kernels can overlap on the GPU (different streams, or threads racing on one
 *    device) corrupt each other's statistics: serialise them, or use varq_quant_pack
 *    with separate workspaces.
 *  - groupings that keep (token, head) -- per-token-per-head, with or without groups along head_dim -- run in
 *    the single-pass kernels and never touch the array: for them this entry point is varq_quant_pack, but the
 *    size check above still applies to their group count.
 * Results are bit-identical to varq_quant_pack. */
int varq_quant_pack_static(const varq_tensor_t* x, int32_t B, int32_t L, int32_t H, int32_t D,
                           int32_t bits, int32_t store_bits, float eps,
                           const varq_tensor_t* codes, const varq_qparams_t* p, void* stream);

/* Size in bytes of the built-in scratch array used by varq_quant_pack_static. */
size_t varq_quant_static_scratch_bytes(void);

/* Packed codes -> out = (code - zp) * scale, written as fp32, fp16 or bf16.
 * Replaces VAR_Q._unpack_last_dim_from_int32 + _dequantize_from_int8 as used by
 * dequant_current / dequant_all (VAR_Q/quant.py:123-124, 133-137, 208-224). */
int varq_unpack_dequant(const varq_tensor_t* codes, int32_t B, int32_t L, int32_t H, int32_t D,
                        int32_t store_bits, const varq_qparams_t* p,
                        const varq_tensor_t* out, void* stream);

/* Pin the kernel varq_attn_fwd uses for every later call of the process: automatic choice, the general
 * CUDA-core kernel, the streaming CUDA-core kernel, the tcgen05 tensor-core kernel or the warp-level tensor-core
 * kernel of the early scales (MID).  A pinned kernel that cannot take a call (shape, layout, grouping) yields to the
 * next one in the automatic order and finally to the general kernel.  For tests and measurements that compare the kernels on
 * one input; no counterpart in the reference. */
#define VARQ_ATTN_PATH_AUTO   0
#define VARQ_ATTN_PATH_SMALL  1
#define VARQ_ATTN_PATH_STREAM 2
#define VARQ_ATTN_PATH_TC     3
#define VARQ_ATTN_PATH_MID    4
int varq_attn_force_path(int32_t path);

/* Bytes of scratch varq_attn_fwd needs for this shape, whichever kernel it picks: partial results of the
 * key-split CUDA-core kernels, or the per-tile parameter streams that the tensor-core kernel's preparation launch
 * writes (about 8 KB per 64 or 128 cached tokens of every (sample, head); sized for the widest grouping).
 * varq_attn_fwd fails with VARQ_ERR_WORKSPACE when given less. */
size_t varq_attn_workspace_bytes(int32_t B, int32_t H, int32_t Lq, int32_t Lk, int32_t D,
                                 int32_t k_store_bits, int32_t v_store_bits);

/* out = softmax(q k^T * softmax_scale) v over the packed cache, no mask, with
 * k = (k_code - zp_k) * scale_k and v likewise, dequantised on the fly.
 * q, out: (B, Lq, H, D) descriptors; k_codes, v_codes: (B, Lk, H, words) descriptors.
 * The tensor-core kernel holds queries as fp16 (an fp32 query as an fp16 hi + lo pair): elements saturate
 * at +-65504, and 16-bit queries below 2^-14 in magnitude lose low bits.
 * Replaces dequant_all() followed by the attention consumer
 * (VAR_Q/quant.py:216-224 + VAR/models/basic_var.py:156-162;
 *  Infinity/infinity/models/basic.py:327-351). */
int varq_attn_fwd(const varq_tensor_t* q, const varq_tensor_t* k_codes, const varq_tensor_t* v_codes,
                  const varq_qparams_t* kp, const varq_qparams_t* vp,
                  int32_t B, int32_t H, int32_t Lq, int32_t Lk, int32_t D,
                  int32_t k_store_bits, int32_t v_store_bits, float softmax_scale,
                  const varq_tensor_t* out, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VARQ_B200_H */
