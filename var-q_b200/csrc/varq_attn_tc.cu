// Attention over the packed cache on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// Two launches per call.  A small preparation kernel turns the per-key quantisation parameters of one (sample, head) into
// ready-made streams, one block per key tile: the softmax tables, the normaliser record of every key and, where the
// packed-half converters apply, the (key, group) records of K and V.  The main kernel then never loads a parameter from
// global memory with an ordinary load: everything a tile needs arrives by 1-D bulk copies (TMA engine) on mbarriers.
//
// Main kernel: one CTA = one (sample, head) x 128 queries, looping over key tiles.  Warps:
//   0-7        softmax: two threads share query row r (TMEM lane r), each owning half of every tile's keys AND its own
//              output accumulator, so the pair never has to agree on a running maximum: a thread reads its S columns from
//              TMEM 32 at a time, applies the per-key scale / zero-point of K, exponentiates against its own lazily
//              updated reference maximum and writes P (fp16) to shared memory.  The two partial results of a row are
//              merged once, in the epilogue;
//   K and V converters (TcRoles: 4 + 6, or 6 + 4 when K is dequantised): wait for a tile's packed rows, turn them into
//              UMMA operand tiles in shared memory and arrive.  K: exact fp16 integer codes (128B-swizzled, K-major), or an
//              fp16 hi + lo pair of (code - zp) * scale when the scale varies along head_dim per key.  V: unswizzled
//              MN-major tile of D + 16 columns, codes or (code - zp) * scale, whose last 16 columns carry 1 / V-scale and
//              the V zero-point of each key (fp16 hi + lo pairs);
//   MMA warp   waits converged; one elected lane issues tcgen05.mma: S = Q K^T (fp16 x fp16 -> fp32 in TMEM) and
//              (O_half | normaliser sums) += P (V | normaliser columns), so the tensor core adds up exactly the rounded P that
//              it multiplies with V, and commits completion to mbarriers;
//   copy warp  one thread requests tile t + 2 of each stream as soon as the converters have arrived for tile t.
// Per-dim scales that the tokens of an appended step share (the reference's shipped mode) take the dequantising converters
// with a per-(sample, head) table of the steps' parameters and a step index per key.  Only histories of more steps than
// those tables hold fall back to the folded-query mode (Q * s(step) rewritten per step, key tiles cut at step boundaries),
// which keeps the older arrangement: 4 + 3 producer warps that also fetch parameters, write the tables and request their
// own copies, and no copy warp.
// Numerics: integer codes are exact in fp16 and the K scale is applied to S in fp32, so QK^T has
// no rounding beyond Q's; an fp32 Q is split into hi + lo fp16 halves (two MMAs).  P and V are
// rounded to fp16 (bf16 would miss the 1e-3 relative-L2 target by 10x).  A V scale below 2^-20
// is folded as 2^-20 (the error is below 127 * 2^-20 per unit of attention weight).
// Every wait is bounded: on expiry the kernel records a status code and all roles drain out.
#include <cfloat>

#include "varq_attn.cuh"

namespace varq {

// Warp roles of a CTA: 8 softmax warps, KW K-converter warps, VW V-converter warps, the MMA warp, the copy-issue warp.
// The converters are latency-bound (a warp retires an instruction every 6 to 10 cycles), so a tile is spread over as many
// of them as fit: 20 warps keep 96 registers per thread, the next allocation step (24 warps, 80 registers) measured slower.
// The folded-query mode keeps 4 + 3 because its K producers own one query row each.
template <int KM> struct TcRoles {
    static constexpr int KW = KM == 1 ? 6 : 4;            // measured: a dequantised K (two operand tiles) wants more K converters
    static constexpr int VW = KM == 2 ? 3 : KM == 1 ? 4 : 6;            // 20 warps keep 96 registers per thread
    static constexpr int KTHR = KW * 32, VTHR = VW * 32;
    static constexpr int K_WARP0 = 8, V_WARP0 = 8 + KW, MMA_WARP = 8 + KW + VW;
    static constexpr int LOAD_WARP = MMA_WARP + 1;        // issues the bulk copies (not in the folded-query mode)
    static constexpr int THREADS = (MMA_WARP + (KM == 2 ? 1 : 2)) * 32;
};
constexpr int TC_M = 128;
constexpr uint32_t TC_SPIN_LIMIT = 1u << 20;


__device__ int g_tc_status = 0;   // first failure code of any launch since the last read (0 = none)

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the limit expires or another thread has already given up.
// Everything is inline and small: a call here costs a few hundred cycles of register shuffling
// around it, at every one of the ~20 wait sites, and bloats the loops that hold them.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
    uint32_t tries = 0;
#pragma unroll 1
    while (!mbar_try(bar, parity)) {     // a failed try_wait has already been suspended by the hardware for a while
        if (*abort_flag) return false;
        if (++tries >= TC_SPIN_LIMIT) {
            *abort_flag = 1;
            atomicCAS(&g_tc_status, 0, code);
            return false;
        }
    }
    return true;
}
// Three barriers polled together: their probes are independent, so the latencies overlap instead of adding up
// (the third one is optional).  Same bound and abort rules as mbar_wait.
__device__ __forceinline__ bool mbar_wait3(uint64_t* b0, uint32_t p0, uint64_t* b1, uint32_t p1, uint64_t* b2, uint32_t p2, bool use2,
                                           volatile int* abort_flag, int code) {
    uint32_t tries = 0;
#pragma unroll 1
    while (true) {
        const bool d0 = mbar_try(b0, p0), d1 = mbar_try(b1, p1), d2 = use2 ? mbar_try(b2, p2) : true;
        if (d0 && d1 && d2) return true;
        if (*abort_flag) return false;
        if (++tries >= TC_SPIN_LIMIT) {
            *abort_flag = 1;
            atomicCAS(&g_tc_status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Both are called by every lane of the MMA warp with the same operands and executed by one elected lane: the warp stays
// converged, so the descriptors are computed once in uniform registers, which is where the instruction takes them from.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void sts128(void* p, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    *reinterpret_cast<uint4*>(p) = make_uint4(x, y, z, w);
}
__device__ __forceinline__ uint4 lds128(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ float pick(const float4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }


// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 format:
// [0,14) start >> 4 | [16,30) leading byte offset >> 4 | [32,46) stride byte offset >> 4 |
// [46,48) version = 1 | [61,64) layout type (2 = SWIZZLE_128B)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout = 2u) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
}
// The V operand (B of O += P V, MN-major: row = key, column = head_dim) is kept UNSWIZZLED (layout type 0): 8 x 8 core
// matrices of 128 contiguous bytes (8 keys x 16 bytes), key blocks 128 bytes apart, 8-column blocks N * 16 bytes apart.
// Without the 64-column atoms of the swizzled layouts the tile can be D + 16 columns wide: the last 16 columns carry
// the per-key normaliser terms, so one MMA per 16 keys produces the output and the normaliser sums together.
__device__ __forceinline__ uint32_t vtile_off(int key, int d0, int N) {      // byte offset of the 16-byte chunk (key, d0 .. d0 + 7)
    return (uint32_t)((d0 >> 3) * (N * 16) + (key >> 3) * 128 + (key & 7) * 16);
}
// Instruction descriptor, kind::f16: fp16 A and B, fp32 accumulator.
// [4,6) c format (1 = f32) | [7,10) a format (0 = f16) | [10,13) b format | 15 a major | 16 b major
// (0 = K-major, 1 = MN-major) | [17,23) N >> 3 | [24,29) M >> 4
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, int b_mn_major) {
    return (1u << 4) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Byte offset of element (row, col) of a 128B-swizzled operand tile whose 64-column blocks hold
// `rows` rows each (K-major A/B: row = M/N index, col = K index; MN-major B: row = K, col = N).
__device__ __forceinline__ uint32_t tile_off(int row, int col, int rows) {
    return (uint32_t)((col >> 6) * rows * 128 + (row >> 3) * 1024 + (row & 7) * 128 +
                      ((((col & 63) >> 3) ^ (row & 7)) << 4) + ((col & 7) << 1));
}

// ---------------------------------------------------------------- shared-memory plan
// How K reaches the tensor core:
//   KM_EXACT  integer codes; one scale / zero-point per key, applied to S in fp32
//   KM_SPLIT  (code - zp) * scale as an fp16 hi + lo pair of operand tiles, for scales that vary along head_dim: per key
//             (group-wise records) or per appended step (step tables)
//   KM_FOLD   integer codes; scales that vary along head_dim but are constant over the tokens of an appended step are
//             folded into the queries (Q * s as fp16 hi + lo, rewritten when a key tile starts a new step), the
//             zero-point term sum_d q_d s_d z_d is a per-row constant taken off S; key tiles end at step boundaries
constexpr int KM_EXACT = 0, KM_SPLIT = 1, KM_FOLD = 2;
constexpr int TC_MAX_TILES = 384;     // entries of the tile schedule (KM_FOLD)
constexpr int TC_PAR_ENTRIES = 288;   // (key, group) parameter records a producer stages per tile

template <int D, int NQ, int KM> struct TcPlan {
    static constexpr bool KS = KM == KM_SPLIT;
    static constexpr int N = (D == 64) ? 128 : 64;           // keys per tile
    static constexpr int Q_BYTES = TC_M * D * 2;              // one fp16 Q tile
    static constexpr int KV_BYTES = N * D * 2;                // one fp16 K tile
    static constexpr int V_BYTES = N * (D + 16) * 2;          // one fp16 V tile with its 16 normaliser columns
    static constexpr int P_BYTES = TC_M * N * 2;
    static constexpr int PK_BYTES = N * D;                    // packed staging at 8 bits (largest)
    static constexpr int KT = KS ? 2 : 1;                     // K operand tiles per stage (hi, lo when K is dequantised)
    static constexpr int PST = KS ? 1 : 2;                    // P buffers
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = OFF_Q + NQ * Q_BYTES;        // [2][KT]
    static constexpr int OFF_V = OFF_K + 2 * KT * KV_BYTES;   // [2]
    static constexpr int OFF_P = (OFF_V + 2 * V_BYTES + 1023) / 1024 * 1024;   // [PST]
    static constexpr int OFF_PK = OFF_P + PST * P_BYTES;      // [2][K, V]
    // per-key softmax tables, a ring of TAB_SLOTS tiles: K scale, mask bias + log2(V scale), K zp * scale; with a dequantised K
    // the first is a constant and the last is zero, so only the middle row is kept
    static constexpr int TAB_ROWS = KS ? 1 : 3;
    static constexpr int TAB_SLOTS = KM == KM_FOLD ? 4 : 8;
    static constexpr int OFF_KS = OFF_PK + 4 * PK_BYTES;      // float [TAB_SLOTS][TAB_ROWS][N]
    static constexpr int OFF_BAR = OFF_KS + TAB_SLOTS * TAB_ROWS * N * 4;    // mbarriers
    static constexpr int N_BARS = 27;
    static constexpr int OFF_MISC = OFF_BAR + (N_BARS + 1) / 2 * 16;     // tmem base, abort flag (everything below stays 16-byte aligned)
    static constexpr int OFF_PREF = OFF_MISC + 16;            // ParamRef [2]: K and V parameter records of the fp32 converters
    static constexpr int OFF_XCH = OFF_PREF + 2 * 48;         // float [2][128]: the two halves of a row exchange their reference maxima
    static constexpr int OFF_QSUM = OFF_XCH + 2 * 128 * 4;    // float [128]: row sums of Q (zero-point term of K)
    static constexpr int OFF_KPAR = OFF_QSUM + 128 * 4;       // uint2 [TC_PAR_ENTRIES]: staged K parameters of the tile being converted
    static constexpr int OFF_VPAR = OFF_KPAR + TC_PAR_ENTRIES * 8;   // same for V (or fp16 [3][D] when V is per-dim)
    static constexpr int OFF_KRAW = OFF_VPAR + TC_PAR_ENTRIES * 8;   // float [2][TC_PAR_ENTRIES]: raw scales / zero-points of the next K tile
    static constexpr int OFF_VRAW = OFF_KRAW + TC_PAR_ENTRIES * 8;   // same for V
    static constexpr int OFF_ROWC = OFF_VRAW + TC_PAR_ENTRIES * 8;   // KM_FOLD: float [4][128] zero-point constants of the rows, per table slot; float [128] accumulation
    static constexpr int OFF_TILES = OFF_ROWC + (KM == KM_FOLD ? 5 * 128 * 4 : 0);   // KM_FOLD: int2 [TC_MAX_TILES] (first key, keys << 16 | row)
    static constexpr int OFF_VNST = OFF_TILES + (KM == KM_FOLD ? TC_MAX_TILES * 8 : 0);   // uint2 [2][N]: staged normaliser records of a V tile
    static constexpr int TOTAL = OFF_VNST + (KM == KM_FOLD ? 0 : 2 * N * 8);
    // destinations of bulk copies
    static_assert(OFF_PK % 16 == 0 && OFF_KS % 16 == 0 && OFF_KPAR % 16 == 0 && OFF_VPAR % 16 == 0 && OFF_KRAW % 16 == 0 &&
                  OFF_VRAW % 16 == 0 && OFF_VNST % 16 == 0 && PK_BYTES % 16 == 0, "bulk copies need 16-byte aligned destinations");
    // TMEM columns: S double-buffered, then one accumulator per half of the keys:
    // D output columns followed by 16 columns of sum_k P * (small tile)
    static constexpr int ACC_COLS = D + 32;
    static constexpr int TMEM_COLS = 512;
    static constexpr int COL_S = 0, COL_O = 2 * N;
    static_assert(COL_O + 2 * ACC_COLS <= 512, "TMEM plan exceeds 512 columns");
};


// ---- packed integer codes -> fp16 without conversion instructions.
// 0x6400 | u is the fp16 number 1024 + u (0 <= u < 1024); codes are biased to unsigned, placed in
// the low byte of each half with byte permutes, and the bias is removed with one packed subtract.
__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    __half2 r = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
// four unsigned bytes (each = code + bias) -> 4 halves holding 1024 + code + bias
__device__ __forceinline__ void bytes_to_raw4(uint32_t u, uint32_t& h01, uint32_t& h23) {
    h01 = __byte_perm(u, 0x64646464u, 0x4140);
    h23 = __byte_perm(u, 0x64646464u, 0x4342);
}
// Codes<BITS>::raw: one packed word -> 32 / BITS halves holding 1024 + BIAS + code (exact fp16 integers), in field order;
// cvt: the codes themselves.  A caller that wants code - zp subtracts 1024 + BIAS + zp instead of 1024 + BIAS.
template <int BITS> struct Codes;
template <> struct Codes<8> {   // one word -> 4 halves
    static constexpr float BIAS = 128.f;
    static constexpr uint32_t BIAS_H2 = 0x64806480u;                     // 1024 + 128, twice
    static __device__ __forceinline__ void raw(uint32_t w, uint32_t* h) { bytes_to_raw4(w ^ 0x80808080u, h[0], h[1]); }
};
template <> struct Codes<4> {   // one word -> 8 halves
    static constexpr float BIAS = 8.f;
    static constexpr uint32_t BIAS_H2 = 0x64086408u;
    static __device__ __forceinline__ void raw(uint32_t w, uint32_t* h) {
        const uint32_t x = w ^ 0x88888888u;                               // c + 8 per nibble
        const uint32_t lo = x & 0x0F0F0F0Fu, hi = (x >> 4) & 0x0F0F0F0Fu; // fields 0,2,4,6 / 1,3,5,7
        bytes_to_raw4(__byte_perm(lo, hi, 0x5140), h[0], h[1]);
        bytes_to_raw4(__byte_perm(lo, hi, 0x7362), h[2], h[3]);
    }
};
template <> struct Codes<2> {   // one word -> 16 halves
    static constexpr float BIAS = 2.f;
    static constexpr uint32_t BIAS_H2 = 0x64026402u;
    static __device__ __forceinline__ void raw(uint32_t w, uint32_t* h) {
        const uint32_t x = w ^ 0xAAAAAAAAu;                               // c + 2 per field
        const uint32_t t0 = x & 0x03030303u, t1 = (x >> 2) & 0x03030303u; // fields 0,4,8,12 / 1,5,9,13
        const uint32_t t2 = (x >> 4) & 0x03030303u, t3 = (x >> 6) & 0x03030303u;
        const uint32_t a = __byte_perm(t0, t1, 0x5140), b = __byte_perm(t2, t3, 0x5140);   // f0 f1 f4 f5 / f2 f3 f6 f7
        const uint32_t c = __byte_perm(t0, t1, 0x7362), d = __byte_perm(t2, t3, 0x7362);   // f8 f9 f12 f13 / f10 f11 f14 f15
        bytes_to_raw4(__byte_perm(a, b, 0x5410), h[0], h[1]);
        bytes_to_raw4(__byte_perm(a, b, 0x7632), h[2], h[3]);
        bytes_to_raw4(__byte_perm(c, d, 0x5410), h[4], h[5]);
        bytes_to_raw4(__byte_perm(c, d, 0x7632), h[6], h[7]);
    }
};
template <int BITS> __device__ __forceinline__ void codes_cvt(uint32_t w, uint32_t* h) {
    Codes<BITS>::raw(w, h);
#pragma unroll
    for (int i = 0; i < 16 / BITS; ++i) h[i] = h2_sub(h[i], Codes<BITS>::BIAS_H2);
}
__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b), *reinterpret_cast<__half2*>(&c));
    return *reinterpret_cast<uint32_t*>(&r);
}

// Walk over the (key, 16-byte item) pairs of a tile, `nthr` threads abreast.  KEYMAJ: neighbouring lanes take neighbouring
// keys of one item column, which makes the 16-byte operand-tile stores of a quarter-warp land in one 128-byte line
// (several stores per item, so they outweigh the strided read of the packed row); otherwise neighbouring lanes take the
// items of one key (contiguous packed reads).
template <bool KEYMAJ> struct ItemWalk {
    int key, item, rows, nthr, ipr, ishift, it;
    __device__ __forceinline__ void init(int ptid, int rows_, int ipr_, int nthr_) {
        rows = rows_; nthr = nthr_; ipr = ipr_; ishift = __ffs(ipr_) - 1; it = ptid;
        if (KEYMAJ) { item = ptid / rows_; key = ptid - item * rows_; }
        else { key = ptid >> ishift; item = ptid & (ipr_ - 1); }
    }
    __device__ __forceinline__ bool more() const { return KEYMAJ ? item < ipr : key < rows; }
    __device__ __forceinline__ void next() {
        if (KEYMAJ) { key += nthr; while (key >= rows) { key -= rows; ++item; } }
        else { it += nthr; key = it >> ishift; item = it & (ipr - 1); }
    }
};

// An item = IW consecutive packed words of one key (IW = 4 or 2), converted by one thread per trip.  The dequantising
// converters take half-size items when those spread a tile over the threads more evenly (see finer_items); for the exact-code
// converter the extra trips cost more than the balance gains (measured).
template <int IW> __device__ __forceinline__ void lds_words(const uint32_t* p, uint32_t (&w)[IW]) {
    if constexpr (IW == 4) { const uint4 v = lds128(p); w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
    else { const uint2 v = *reinterpret_cast<const uint2*>(p); w[0] = v.x; w[1] = v.y; }
}
// true if items of two words need fewer half-item trips per thread than items of four
__device__ __forceinline__ bool finer_items(int items4, int nthr) {
    return (2 * items4 + nthr - 1) / nthr < 2 * ((items4 + nthr - 1) / nthr);
}
// Exact-code operand tile.
template <int BITS, bool VL = false, int IW = 4>      // VL: the unswizzled V layout
__device__ __noinline__ void codes_tile(unsigned char* tile, const uint32_t* packed, int n_valid, int N, int W, int ptid, int nthr = 128,
                                           int rows = -1) {
    // rows [n_valid, rows) are zero-filled; consumers never read past `rows`
    if (rows < 0) rows = N;
    constexpr int VPW = 32 / BITS;            // codes per word
    constexpr int HW = VPW / 2;               // 32-bit half2 registers per word
    ItemWalk<(BITS < 8) && VL> wk;      // measured: key by key only pays for the unswizzled V tile below 8 bits
#pragma unroll 1
    for (wk.init(ptid, rows, W / IW, nthr); wk.more(); wk.next()) {
        const int key = wk.key, wi = wk.item * IW;
        uint32_t h[IW * HW];
        if (key < n_valid) {
            uint32_t wd[IW];
            lds_words<IW>(packed + key * W + wi, wd);
#pragma unroll
            for (int q = 0; q < IW; ++q) codes_cvt<BITS>(wd[q], h + q * HW);
        } else {
#pragma unroll
            for (int i = 0; i < IW * HW; ++i) h[i] = 0u;
        }
        const int d0 = wi * VPW;              // first head_dim index of the item
        if constexpr (VL) {
            unsigned char* base = tile + vtile_off(key, d0, N);
#pragma unroll
            for (int c = 0; c < IW * HW / 4; ++c) sts128(base + c * (N * 16), h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]);
        } else {
            unsigned char* row = tile + (d0 >> 6) * N * 128 + (key >> 3) * 1024 + (key & 7) * 128;
            const int ch0 = (d0 & 63) >> 3;
#pragma unroll
            for (int c = 0; c < IW * HW / 4; ++c)         // chunks of 8 halves
                sts128(row + (((ch0 + c) ^ (key & 7)) << 4), h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]);
        }
    }
}

// Scale and zero-point of the VPW values of one packed word, kept in registers while consecutive keys of
// a thread share their parameter row (groupings with one row per appended step): a thread always converts
// the same word column of every key it visits, so the parameters change only when the row does.
// What the fp32 converters need of a ParamView, with the (sample, head) part of the index folded into the pointers: small
// enough to travel in registers to an out-of-line routine.
struct ParamRef {     // 40 bytes
    const float* scale;
    const float* zp;
    const int32_t* row_of_token;
    long long sr, sg;
    int group;
    __device__ __forceinline__ int row(int token) const { return row_of_token ? __ldg(row_of_token + token) : token; }
    __device__ __forceinline__ long long index(int r, int d) const { return r * sr + (long long)(d / group) * sg; }
};
__device__ __forceinline__ ParamRef param_ref(const ParamView& pv, int b, int h) {
    const long long base = pv.index(b, 0, h, 0);
    ParamRef r;
    r.scale = pv.scale + base;
    r.zp = pv.zp ? pv.zp + base : nullptr;
    r.row_of_token = pv.row_of_token;
    r.sr = pv.sr; r.sg = pv.sg; r.group = pv.group;
    return r;
}
template <int VPW> struct WordParams {
    float s[VPW], z[VPW];
    int row;
    __device__ __forceinline__ void fetch(const ParamRef& pv, int r, int d0, bool uniform) {
        row = r;
        if (uniform) {
            const long long pi = pv.index(r, d0);
            const float sv = __ldg(pv.scale + pi), zv = pv.zp ? __ldg(pv.zp + pi) : 0.f;
#pragma unroll
            for (int j = 0; j < VPW; ++j) { s[j] = sv; z[j] = zv; }
        } else {
#pragma unroll
            for (int j = 0; j < VPW; ++j) {
                const long long pi = pv.index(r, d0 + j);
                s[j] = __ldg(pv.scale + pi);
                z[j] = pv.zp ? __ldg(pv.zp + pi) : 0.f;
            }
        }
    }
};

// Convert `BITS`-wide codes of one packed word to fp16 and write them to the operand tile.
// EXACT: raw integer codes; otherwise (code - z) * s.
// General V path: (code - zp) * scale in fp32, rounded to fp16, for groupings whose scale varies along
// head_dim (per-dim, group-wise); parameters are fetched per word, or per element when a word spans groups.
template <int BITS>
__device__ __noinline__ void dequant_tile(unsigned char* tile, const uint32_t* packed, int n_valid, int N, int W,
                                             int ptid, const ParamRef* pv_smem, int k0, int nthr = 128) {
    const ParamRef pv = *pv_smem;     // the record lives in shared memory so that the call carries one pointer, not ten registers
    constexpr int VPW = 32 / BITS;
    const int total = min(N, (n_valid + 31) & ~31) * W;
    const int wshift = __ffs(W) - 1;          // W is a power of two
    const bool uniform = (pv.group % VPW) == 0;
    const bool fixed_w = (nthr & (W - 1)) == 0;      // this thread's word column never changes
    WordParams<VPW> wp;
    wp.row = -1;
    for (int idx = ptid; idx < total; idx += nthr) {
        const int key = idx >> wshift, w = idx & (W - 1);
        __half hv[VPW];
        if (key < n_valid) {
            const uint32_t word = packed[idx];
            const int row = pv.row(k0 + key);
            if (row != wp.row || !fixed_w) wp.fetch(pv, row, w * VPW, uniform);
#pragma unroll
            for (int j = 0; j < VPW; ++j) hv[j] = __float2half_rn(((float)field<BITS>(word, j) - wp.z[j]) * wp.s[j]);
        } else {
#pragma unroll
            for (int j = 0; j < VPW; ++j) hv[j] = __float2half_rn(0.f);
        }
        const int d0 = w * VPW;
        if constexpr (VPW == 4) {
            *reinterpret_cast<uint2*>(tile + vtile_off(key, d0, N) + (d0 & 7) * 2) = *reinterpret_cast<uint2*>(hv);
        } else {
#pragma unroll
            for (int c8 = 0; c8 < VPW / 8; ++c8)
                *reinterpret_cast<uint4*>(tile + vtile_off(key, d0 + 8 * c8, N)) = *reinterpret_cast<uint4*>(hv + 8 * c8);
        }
    }
}

// K dequantised to fp32 and split into two fp16 operand tiles, hi = fp16(k) and lo = fp16(k - hi):
// Q (hi + lo) reproduces k to 2^-22, so groupings whose K scale varies along head_dim (per-dim,
// group-wise) keep an essentially exact QK^T at the price of a second MMA.
template <int BITS>
__device__ __noinline__ void dequant_split_tile(unsigned char* tile_hi, unsigned char* tile_lo, const uint32_t* packed,
                                                   int n_valid, int N, int W, int ptid, const ParamRef* pv_smem, int k0, int nthr) {
    const ParamRef pv = *pv_smem;
    constexpr int VPW = 32 / BITS;
    const int total = N * W;
    const int wshift = __ffs(W) - 1;
    const bool uniform = (pv.group % VPW) == 0;
    const bool fixed_w = (nthr & (W - 1)) == 0;       // this thread's word column never changes
    WordParams<VPW> wp;
    wp.row = -1;
    for (int idx = ptid; idx < total; idx += nthr) {
        const int key = idx >> wshift, w = idx & (W - 1);
        __half hh[VPW], hl[VPW];
        if (key < n_valid) {
            const uint32_t word = packed[idx];
            const int row = pv.row(k0 + key);
            if (row != wp.row || !fixed_w) wp.fetch(pv, row, w * VPW, uniform);
#pragma unroll
            for (int j = 0; j < VPW; ++j) {
                const float k = ((float)field<BITS>(word, j) - wp.z[j]) * wp.s[j];
                hh[j] = __float2half_rn(k);
                hl[j] = __float2half_rn(k - __half2float(hh[j]));
            }
        } else {
#pragma unroll
            for (int j = 0; j < VPW; ++j) { hh[j] = __float2half_rn(0.f); hl[j] = hh[j]; }
        }
        const int d0 = w * VPW;
        if constexpr (VPW == 4) {
            *reinterpret_cast<uint2*>(tile_hi + tile_off(key, d0, N)) = *reinterpret_cast<uint2*>(hh);
            *reinterpret_cast<uint2*>(tile_lo + tile_off(key, d0, N)) = *reinterpret_cast<uint2*>(hl);
        } else {
#pragma unroll
            for (int c8 = 0; c8 < VPW / 8; ++c8) {
                *reinterpret_cast<uint4*>(tile_hi + tile_off(key, d0 + 8 * c8, N)) = *reinterpret_cast<uint4*>(hh + 8 * c8);
                *reinterpret_cast<uint4*>(tile_lo + tile_off(key, d0 + 8 * c8, N)) = *reinterpret_cast<uint4*>(hl + 8 * c8);
            }
        }
    }
}

// ---- dequantising producers in packed-half arithmetic.
// The scale and zero-point of every (key, group) of a tile are staged in shared memory as a record
//   x = fp16 pair (s_hi, s_lo), s_hi + s_lo = scale to 2^-22;   y = fp16 pair (zb, zb), zb = 1024 + BIAS + zero-point,
// so that a word's biased codes (1024 + BIAS + code, exact) minus zb are code - zp (exact while |zp| <= 512), and
//   k_hi = RN(d * s_hi),  k_lo = RN(d * s_lo + (d * s_hi - k_hi))      [the inner residual is exact in fp16]
// reproduce (code - zp) * scale to 2^-22 with three packed instructions per two elements.  V is one operand tile:
// RN(d * s_hi + RN(d * s_lo)), i.e. the product rounded once to fp16.
// A tile that holds a record outside those bounds is converted by the fp32 routines above instead.
// The raw parameters of the next tile travel global -> shared memory by 4-byte asynchronous copies, so that no register
// holds them across the out-of-line converter call (a register live across that call is saved to local memory first,
// which would expose the load's latency).  Entry e = key << g_shift | group; a thread only ever touches its own entries.
template <int MAXE> struct ParStage {
    static __device__ __forceinline__ void request(const ParamView& pv, long long base, int k0, int n_valid, int g_shift, int ptid, int nthr,
                                                   float* raw) {
#pragma unroll
        for (int i = 0; i < MAXE; ++i) {
            const int e = ptid + i * nthr, key = e >> g_shift, g = e & ((1 << g_shift) - 1);
            if (key < n_valid) {
                const long long pi = base + pv.row(k0 + key) * pv.sr + (long long)g * pv.sg;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(raw + e)), "l"(pv.scale + pi) : "memory");
                if (pv.zp) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(raw + TC_PAR_ENTRIES + e)), "l"(pv.zp + pi) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // waits for this thread's copies, writes its records; returns true if one of them needs the fp32 routine
    static __device__ __forceinline__ bool build(uint2* par, const float* raw, int n_entries, float bias, bool has_zp, int ptid, int nthr) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        bool slow = false;
#pragma unroll
        for (int i = 0; i < MAXE; ++i) {
            const int e = ptid + i * nthr;
            if (e >= n_entries) continue;
            const float sv = raw[e], zv = has_zp ? raw[TC_PAR_ENTRIES + e] : 0.f;
            const __half s_hi = __float2half_rn(sv);
            const __half s_lo = __float2half_rn(sv - __half2float(s_hi));
            const __half zb = __float2half_rn(1024.f + bias + zv);
            slow = slow || !(fabsf(zv) <= 512.f) || !(sv < 60.f);     // code - zp stays below 2^10, the product inside fp16
            par[e] = make_uint2((uint32_t)__half_as_ushort(s_hi) | ((uint32_t)__half_as_ushort(s_lo) << 16),
                                (uint32_t)__half_as_ushort(zb) * 0x10001u);
        }
        return slow;
    }
};

// K: hi + lo operand tiles from the staged records.
template <int BITS, int IW = 4>
__device__ __noinline__ void group_split_tile(unsigned char* tile_hi, unsigned char* tile_lo, const uint32_t* packed, const uint2* par,
                                              int n_valid, int N, int W, int ptid, int nthr, int g_shift, int grp_shift) {
    constexpr int VPW = 32 / BITS, HW = VPW / 2;
    ItemWalk<false> wk;      // the items of a key share a parameter record: neighbouring lanes read it together
#pragma unroll 1
    for (wk.init(ptid, N, W / IW, nthr); wk.more(); wk.next()) {
        const int key = wk.key, wi = wk.item * IW;
        uint32_t hi[IW * HW], lo[IW * HW];
        if (key < n_valid) {
            uint32_t wd[IW];
            lds_words<IW>(packed + key * W + wi, wd);
#pragma unroll
            for (int q = 0; q < IW; ++q) {
                const uint2 pr = par[(key << g_shift) + (((wi + q) * VPW) >> grp_shift)];
                const uint32_t sh = __byte_perm(pr.x, pr.x, 0x1010), sl = __byte_perm(pr.x, pr.x, 0x3232);
                uint32_t d[HW];
                Codes<BITS>::raw(wd[q], d);
#pragma unroll
                for (int c = 0; c < HW; ++c) {
                    const uint32_t dz = h2_sub(d[c], pr.y);
                    const uint32_t h = h2_mul(dz, sh);
                    const uint32_t e = h2_fma(dz, sh, h ^ 0x80008000u);
                    hi[q * HW + c] = h;
                    lo[q * HW + c] = h2_fma(dz, sl, e);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < IW * HW; ++i) { hi[i] = 0u; lo[i] = 0u; }
        }
        const int d0 = wi * VPW;
        const uint32_t row = (uint32_t)((d0 >> 6) * N * 128 + (key >> 3) * 1024 + (key & 7) * 128);
        const int ch0 = (d0 & 63) >> 3;
#pragma unroll
        for (int c = 0; c < IW * HW / 4; ++c) {
            const uint32_t off = row + (((ch0 + c) ^ (key & 7)) << 4);
            sts128(tile_hi + off, hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
            sts128(tile_lo + off, lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
        }
    }
}

// V: one operand tile RN((code - zp) * scale) from the staged records (rows [n_valid, rows) zero-filled).
template <int BITS, int IW = 4>
__device__ __noinline__ void group_tile(unsigned char* tile, const uint32_t* packed, const uint2* par, int n_valid, int N, int W,
                                        int ptid, int nthr, int rows, int g_shift, int grp_shift) {
    constexpr int VPW = 32 / BITS, HW = VPW / 2;
    ItemWalk<false> wk;
#pragma unroll 1
    for (wk.init(ptid, rows, W / IW, nthr); wk.more(); wk.next()) {
        const int key = wk.key, wi = wk.item * IW;
        uint32_t h[IW * HW];
        if (key < n_valid) {
            uint32_t wd[IW];
            lds_words<IW>(packed + key * W + wi, wd);
#pragma unroll
            for (int q = 0; q < IW; ++q) {
                const uint2 pr = par[(key << g_shift) + (((wi + q) * VPW) >> grp_shift)];
                const uint32_t sh = __byte_perm(pr.x, pr.x, 0x1010), sl = __byte_perm(pr.x, pr.x, 0x3232);
                uint32_t d[HW];
                Codes<BITS>::raw(wd[q], d);
#pragma unroll
                for (int c = 0; c < HW; ++c) {
                    const uint32_t dz = h2_sub(d[c], pr.y);
                    h[q * HW + c] = h2_fma(dz, sh, h2_mul(dz, sl));      // one rounding of (code - zp) * (s_hi + s_lo), to first order
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < IW * HW; ++i) h[i] = 0u;
        }
        const int d0 = wi * VPW;
        unsigned char* base = tile + vtile_off(key, d0, N);
#pragma unroll
        for (int c = 0; c < IW * HW / 4; ++c) sts128(base + c * (N * 16), h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]);
    }
}

// V with one scale / zero-point per head_dim element that all keys of the tile share (per-dim parameters of one appended
// step): s_h[d] + sl_h[d] = scale as an fp16 hi + lo pair, zb_h[d] = fp16 (1024 + BIAS + zero-point), in shared memory.
template <int BITS>
__device__ __noinline__ void perdim_tile(unsigned char* tile, const uint32_t* packed, const __half* s_h, const __half* sl_h, const __half* zb_h,
                                         int n_valid, int N, int W, int ptid, int nthr, int rows) {
    constexpr int VPW = 32 / BITS, HW = VPW / 2;
    ItemWalk<true> wk;
#pragma unroll 1
    for (wk.init(ptid, rows, W >> 2, nthr); wk.more(); wk.next()) {
        const int key = wk.key, wi = wk.item << 2;
        const int d0 = wi * VPW;
        uint32_t h[4 * HW];
        if (key < n_valid) {
            const uint4 pk = lds128(packed + key * W + wi);
            const uint32_t wd[4] = {pk.x, pk.y, pk.z, pk.w};
            const uint32_t* sp = reinterpret_cast<const uint32_t*>(s_h + d0);
            const uint32_t* slp = reinterpret_cast<const uint32_t*>(sl_h + d0);
            const uint32_t* zp = reinterpret_cast<const uint32_t*>(zb_h + d0);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t d[HW];
                Codes<BITS>::raw(wd[q], d);
#pragma unroll
                for (int c = 0; c < HW; ++c) {
                    const uint32_t dz = h2_sub(d[c], zp[q * HW + c]);
                    h[q * HW + c] = h2_fma(dz, sp[q * HW + c], h2_mul(dz, slp[q * HW + c]));
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4 * HW; ++i) h[i] = 0u;
        }
        unsigned char* base = tile + vtile_off(key, d0, N);
#pragma unroll
        for (int c = 0; c < HW; ++c) sts128(base + c * (N * 16), h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]);
    }
}

// ---- per-dim parameters that the tokens of an appended step share, on regular key tiles: every key carries its step index
// (uint16, staged with the tile) and the (sample, head) table [steps][3][D] of fp16 (scale hi, scale lo, 1024 + bias +
// zero-point) is read through the read-only cache: neighbouring lanes convert neighbouring keys, which almost always belong
// to the same step, so a load is one broadcast line.
template <int HW> __device__ __forceinline__ void ldg_pairs(const __half* p, uint32_t (&r)[HW]) {
    if constexpr (HW == 2) { const uint2 v = __ldg(reinterpret_cast<const uint2*>(p)); r[0] = v.x; r[1] = v.y; }
    else {
#pragma unroll
        for (int i = 0; i < HW / 4; ++i) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + i);
            r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
        }
    }
}
// K: hi + lo operand tiles (128B-swizzled, K-major)
template <int BITS>
__device__ __noinline__ void perdim_split_tile(unsigned char* tile_hi, unsigned char* tile_lo, const uint32_t* packed, const uint16_t* step_of_key,
                                               const __half* tab, int D, int n_valid, int N, int W, int ptid, int nthr) {
    constexpr int VPW = 32 / BITS, HW = VPW / 2;
    ItemWalk<true> wk;
#pragma unroll 1
    for (wk.init(ptid, N, W >> 2, nthr); wk.more(); wk.next()) {
        const int key = wk.key, wi = wk.item << 2;
        const int d0 = wi * VPW;
        uint32_t hi[4 * HW], lo[4 * HW];
        if (key < n_valid) {
            const uint4 pk = lds128(packed + key * W + wi);
            const uint32_t wd[4] = {pk.x, pk.y, pk.z, pk.w};
            const __half* row = tab + (int)step_of_key[key] * 3 * D + d0;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t d[HW], sh[HW], sl[HW], zb[HW];
                Codes<BITS>::raw(wd[q], d);
                ldg_pairs<HW>(row + q * VPW, sh);
                ldg_pairs<HW>(row + D + q * VPW, sl);
                ldg_pairs<HW>(row + 2 * D + q * VPW, zb);
#pragma unroll
                for (int c = 0; c < HW; ++c) {
                    const uint32_t dz = h2_sub(d[c], zb[c]);
                    const uint32_t h = h2_mul(dz, sh[c]);
                    const uint32_t e = h2_fma(dz, sh[c], h ^ 0x80008000u);
                    hi[q * HW + c] = h;
                    lo[q * HW + c] = h2_fma(dz, sl[c], e);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4 * HW; ++i) { hi[i] = 0u; lo[i] = 0u; }
        }
        const uint32_t rowo = (uint32_t)((d0 >> 6) * N * 128 + (key >> 3) * 1024 + (key & 7) * 128);
        const int ch0 = (d0 & 63) >> 3;
#pragma unroll
        for (int c = 0; c < HW; ++c) {
            const uint32_t off = rowo + (((ch0 + c) ^ (key & 7)) << 4);
            sts128(tile_hi + off, hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
            sts128(tile_lo + off, lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
        }
    }
}
// V: one operand tile RN((code - zp) * scale) (unswizzled, MN-major; rows [n_valid, rows) zero-filled)
template <int BITS>
__device__ __noinline__ void perdim_steps_tile(unsigned char* tile, const uint32_t* packed, const uint16_t* step_of_key, const __half* tab, int D,
                                               int n_valid, int N, int W, int ptid, int nthr, int rows) {
    constexpr int VPW = 32 / BITS, HW = VPW / 2;
    ItemWalk<true> wk;
#pragma unroll 1
    for (wk.init(ptid, rows, W >> 2, nthr); wk.more(); wk.next()) {
        const int key = wk.key, wi = wk.item << 2;
        const int d0 = wi * VPW;
        uint32_t h[4 * HW];
        if (key < n_valid) {
            const uint4 pk = lds128(packed + key * W + wi);
            const uint32_t wd[4] = {pk.x, pk.y, pk.z, pk.w};
            const __half* row = tab + (int)step_of_key[key] * 3 * D + d0;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t d[HW], sh[HW], sl[HW], zb[HW];
                Codes<BITS>::raw(wd[q], d);
                ldg_pairs<HW>(row + q * VPW, sh);
                ldg_pairs<HW>(row + D + q * VPW, sl);
                ldg_pairs<HW>(row + 2 * D + q * VPW, zb);
#pragma unroll
                for (int c = 0; c < HW; ++c) {
                    const uint32_t dz = h2_sub(d[c], zb[c]);
                    h[q * HW + c] = h2_fma(dz, sh[c], h2_mul(dz, sl[c]));
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4 * HW; ++i) h[i] = 0u;
        }
        unsigned char* base = tile + vtile_off(key, d0, N);
#pragma unroll
        for (int c = 0; c < HW; ++c) sts128(base + c * (N * 16), h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]);
    }
}

// ---- softmax over 32 columns of S held in registers.  Per-key tables (shared memory):
// ks = K scale * softmax_scale * log2(e) (0 past the end), b2 = log2(folded V scale) (-1e30 past the
// end), kzs = K zero-point * ks.
// four consecutive table entries with one 16-byte shared-memory load (tables are 16-byte aligned)
__device__ __forceinline__ float4 tab4(const float* p, int c) { return *reinterpret_cast<const float4*>(p + c); }

// A row keeps its reference maximum until a score exceeds it by more than this (log2 units): P stays below
// 2^12 in fp16 and the accumulators are rescaled rarely.
constexpr float TC_LAZY = 12.f;
constexpr float TC_VS_MIN = 9.5367431640625e-07f;     // 2^-20: smallest V scale folded into P as is
constexpr float TC_AUX_DOWN = 0.015625f;              // 2^-6 on 1 / V-scale so that it stays inside fp16's range
constexpr float TC_AUX_UP = 64.f;
constexpr float TC_ZP_DOWN = 0.00390625f;             // 2^-8 on the V zero-point
constexpr float TC_ZP_UP = 256.f;

// packed fp32 pairs (one instruction for two lanes of work on sm_100)
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// raw scores -> x = s * ks + b2 [- kzs * qsum] in place (log2 domain, V scale folded in); returns their maximum
// KC: the K scale is the same constant `kconst` for every key (a dequantised K carries its own scales)
template <bool KZ, bool KC = false>
__device__ __forceinline__ float chunk_scores(uint32_t (&rw)[32], const float* ks, const float* b2, const float* kzs, float qsum,
                                              float kconst = 0.f) {
    float m0 = -FLT_MAX, m1 = -FLT_MAX;
#pragma unroll
    for (int c = 0; c < 32; c += 4) {
        const float4 s4 = KC ? make_float4(kconst, kconst, kconst, kconst) : tab4(ks, c), b4 = tab4(b2, c);
        float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (KZ) z4 = tab4(kzs, c);
        float x[4];
        fma2(x[0], x[1], __uint_as_float(rw[c]), __uint_as_float(rw[c + 1]), s4.x, s4.y, b4.x, b4.y);
        fma2(x[2], x[3], __uint_as_float(rw[c + 2]), __uint_as_float(rw[c + 3]), s4.z, s4.w, b4.z, b4.w);
        if (KZ) {
            fma2(x[0], x[1], -z4.x, -z4.y, qsum, qsum, x[0], x[1]);
            fma2(x[2], x[3], -z4.z, -z4.w, qsum, qsum, x[2], x[3]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) rw[c + i] = __float_as_uint(x[i]);
        m0 = max3(m0, x[0], x[1]);
        m1 = max3(m1, x[2], x[3]);
    }
    return fmaxf(m0, m1);
}
// x -> P = exp2(x - m) rounded to fp16, packed in pairs
__device__ __forceinline__ void chunk_exp(const uint32_t (&x)[32], float m, uint32_t (&ph)[16]) {
#pragma unroll
    for (int c = 0; c < 32; c += 2) {
        float y0, y1;
        add2(y0, y1, __uint_as_float(x[c]), __uint_as_float(x[c + 1]), -m, -m);
        const __half2 h2 = __floats2half2_rn(ex2(y0), ex2(y1));
        ph[c >> 1] = *reinterpret_cast<const uint32_t*>(&h2);
    }
}

// Out-of-line slow path of the softmax warps: the maximum of this thread's scores over the whole tile
// becomes the reference of the rows that need one, and the accumulator (D output columns + 16 columns of
// normaliser sums) is multiplied by 2^(old - new).  `pv_done` = barrier of the previous tile's O += P V
// (nullptr at the first tile, whose MMA overwrites the accumulator).  Returns the row's reference, NaN if a wait expired.
template <int D, int N, bool KC>
__device__ __noinline__ float new_reference(uint32_t s_addr, int nch, const float* ks, const float* b2, const float* kzs, bool k_zp,
                                            float qsum, float m_used, uint32_t acc, uint64_t* pv_done, uint32_t pv_parity,
                                            volatile int* abort_flag, float kconst) {
    uint32_t rw[32];
    float tm = -FLT_MAX;
#pragma unroll 1
    for (int c = 0; c < nch; ++c) {
        tmem_ld32(s_addr + c * 32, rw);
        tmem_wait_ld();
        tm = fmaxf(tm, KC     ? chunk_scores<false, true>(rw, ks + c * 32, b2 + c * 32, kzs + c * 32, qsum, kconst)
                       : k_zp ? chunk_scores<true>(rw, ks + c * 32, b2 + c * 32, kzs + c * 32, qsum)
                              : chunk_scores<false>(rw, ks + c * 32, b2 + c * 32, kzs + c * 32, qsum));
    }
    float alpha = 1.f;
    if (tm > m_used + TC_LAZY) {
        alpha = ex2(m_used - tm);       // 0 for a row without a reference yet
        m_used = tm;
    }
    if (pv_done == nullptr) return m_used;
    bool ok = mbar_wait(pv_done, pv_parity, abort_flag, 12);   // the accumulator is stable
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) return __int_as_float(0x7fc00000);
    tc_fence_after();
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
        tmem_ld32(acc + c0, rw);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) rw[i] = __float_as_uint(__uint_as_float(rw[i]) * alpha);
        tmem_st32(acc + c0, rw);
    }
    uint32_t ax[16];
    tmem_ld16(acc + D, ax);
    tmem_wait_ld();
#pragma unroll
    for (int i = 0; i < 16; ++i) ax[i] = __float_as_uint(__uint_as_float(ax[i]) * alpha);
    tmem_st16(acc + D, ax);
    tmem_wait_st();
    return m_used;
}

// ---------------------------------------------------------------- preparation kernel
// Everything the main kernel needs per key besides the packed codes, computed once per (sample, head) instead of once per
// query tile: one thread block per key tile, one thread per key.  Block layout (byte offsets in AttnArgs):
//   softmax tables  float [rows][N]   rows = 3 (K scale * softmax_scale * log2 e, mask bias + log2 of the folded V scale,
//                                     K zero-point * that scale) or 1 (the middle row, when K is dequantised)
//   normaliser      uint2 [N]         fp16 (hi, lo) of 2^-6 / V scale and of 2^-8 * V zero-point (1 and 0 when V is dequantised)
//   K records       uint2 [N * groups] + 16-byte trailer     (only for the packed-half converter; see ParStage)
//   V records       the same
// Parameters that the tokens of an appended step share (per-dim scales): the records of a tile are the step index of every
// key (uint16 [N] + trailer), and block 0 of every (sample, head) writes its table [steps][3][D] of fp16 (scale hi, scale lo,
// 1024 + bias + zero-point) behind the tile blocks; every block scans the table's source for out-of-range parameters.
template <int N>
__global__ void __launch_bounds__(N) tc_prepare_kernel(AttnArgs a, int n_tiles, int k_split, int k_ng, int v_ng, int kb, int vb) {
    const int t = threadIdx.x;
    const int j = (int)(blockIdx.x % (unsigned)n_tiles), bh = (int)(blockIdx.x / (unsigned)n_tiles), b = bh / a.H, h = bh - b * a.H;
    const int key = j * N + t;
    const bool valid = key < a.Lk;
    unsigned char* blk = a.prep + (long long)bh * a.prep_bh_stride + (long long)j * a.prep_tile_stride;
    const bool v_exact = a.vp.group == a.D;
    const int krow = valid ? a.kp.row(key) : 0, vrow = valid ? a.vp.row(key) : 0;

    float sc = 0.f, zs = 0.f, vsc = 1.f, vz = 0.f;
    if (valid) {
        if (!k_split) {
            const long long pi = a.kp.index(b, krow, h, 0);
            sc = __ldg(a.kp.scale + pi);
            if (a.kp.zp) zs = __ldg(a.kp.zp + pi);
        }
        if (v_exact) {
            const long long vi = a.vp.index(b, vrow, h, 0);
            vsc = __ldg(a.vp.scale + vi);
            if (a.vp.zp) vz = __ldg(a.vp.zp + vi);
        }
    }
    float* tab = reinterpret_cast<float*>(blk);
    const float b2 = (valid ? 0.f : -1e30f) + __log2f(fmaxf(vsc, TC_VS_MIN));
    if (k_split) {
        tab[t] = b2;
    } else {
        const float scl = sc * a.scale_log2;
        tab[t] = scl;
        tab[N + t] = b2;
        tab[2 * N + t] = zs * scl;
    }
    {
        const float vin = TC_AUX_DOWN * __frcp_rn(fmaxf(vsc, TC_VS_MIN)), vzd = vz * TC_ZP_DOWN;
        const __half vin_hi = __float2half_rn(vin), vz_hi = __float2half_rn(vzd);
        const __half vin_lo = __float2half_rn(vin - __half2float(vin_hi)), vz_lo = __float2half_rn(vzd - __half2float(vz_hi));
        reinterpret_cast<uint2*>(blk + a.prep_off_vn)[t] =
            make_uint2((uint32_t)__half_as_ushort(vin_hi) | ((uint32_t)__half_as_ushort(vin_lo) << 16),
                       (uint32_t)__half_as_ushort(vz_hi) | ((uint32_t)__half_as_ushort(vz_lo) << 16));
    }
    // (key, group) records of the packed-half converters; a record outside their bounds flags the whole tile
    auto records = [&](const ParamView& pv, int row, int ng, int bits, int off, int bytes) {
        if (bytes == 0) return;         // block-uniform
        uint2* rec = reinterpret_cast<uint2*>(blk + off) + t * ng;
        const float bias = bits == 8 ? 128.f : bits == 4 ? 8.f : 2.f;
        bool slow = false;
        for (int g = 0; g < ng; ++g) {
            uint2 r = make_uint2(0u, 0u);
            if (valid) {
                const long long pi = pv.index(b, row, h, g * pv.group);
                const float sv = __ldg(pv.scale + pi), zv = pv.zp ? __ldg(pv.zp + pi) : 0.f;
                const __half s_hi = __float2half_rn(sv);
                const __half s_lo = __float2half_rn(sv - __half2float(s_hi));
                const __half zb = __float2half_rn(1024.f + bias + zv);
                slow = slow || !(fabsf(zv) <= 512.f) || !(sv < 60.f);     // code - zp stays below 2^10, the product inside fp16
                r = make_uint2((uint32_t)__half_as_ushort(s_hi) | ((uint32_t)__half_as_ushort(s_lo) << 16),
                               (uint32_t)__half_as_ushort(zb) * 0x10001u);
            }
            rec[g] = r;
        }
        const int any_slow = __syncthreads_or(slow ? 1 : 0);
        if (t == 0) *reinterpret_cast<uint4*>(blk + off + N * ng * 8) = make_uint4((uint32_t)any_slow, 0u, 0u, 0u);
    };
    auto perdim = [&](const ParamView& pv, int row, int bits, int off, int bytes, const unsigned char* tab_base) {
        reinterpret_cast<uint16_t*>(blk + off)[t] = (uint16_t)row;
        const float bias = bits == 8 ? 128.f : bits == 4 ? 8.f : 2.f;
        __half* tb = reinterpret_cast<__half*>(const_cast<unsigned char*>(tab_base) + (long long)bh * a.prep_tab_bh_stride);
        bool slow = false;
        for (int i = t; i < pv.n_rows * a.D; i += N) {
            const int r = i / a.D, d = i - r * a.D;
            const long long pi = pv.index(b, r, h, d);
            const float sv = __ldg(pv.scale + pi), zv = pv.zp ? __ldg(pv.zp + pi) : 0.f;
            slow = slow || !(fabsf(zv) <= 512.f) || !(sv < 60.f);
            if (j == 0) {
                const __half s_hi = __float2half_rn(sv);
                tb[(r * 3 + 0) * a.D + d] = s_hi;
                tb[(r * 3 + 1) * a.D + d] = __float2half_rn(sv - __half2float(s_hi));
                tb[(r * 3 + 2) * a.D + d] = __float2half_rn(1024.f + bias + zv);
            }
        }
        const int any_slow = __syncthreads_or(slow ? 1 : 0);
        if (t == 0) *reinterpret_cast<uint4*>(blk + off + bytes - 16) = make_uint4((uint32_t)any_slow, 0u, 0u, 0u);
    };
    if (a.tc_k_perdim) perdim(a.kp, krow, kb, a.prep_off_krec, a.prep_krec_bytes, a.prep_ktab);
    else records(a.kp, krow, k_ng, kb, a.prep_off_krec, a.prep_krec_bytes);
    if (a.tc_v_perdim) perdim(a.vp, vrow, vb, a.prep_off_vrec, a.prep_vrec_bytes, a.prep_vtab);
    else records(a.vp, vrow, v_ng, vb, a.prep_off_vrec, a.prep_vrec_bytes);
}

template <int D, int NQ, int KM>
__global__ void __launch_bounds__(TcRoles<KM>::THREADS, 1) attn_tc_kernel(AttnArgs a, int kb, int vb) {
    using P = TcPlan<D, NQ, KM>;
    using R = TcRoles<KM>;
    constexpr int KTHR = R::KTHR, VTHR = R::VTHR, MMA_WARP = R::MMA_WARP;
    constexpr int N = P::N;
    constexpr bool KS = KM == KM_SPLIT, QF = KM == KM_FOLD;
    static_assert(!QF || NQ == 2, "folded queries are fp16 hi + lo pairs");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzle atoms need 1024-byte alignment
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P::OFF_BAR);
    uint64_t* bar_pk = bars;          // [2] packed K rows landed (tx bytes)
    uint64_t* bar_k = bars + 2;       // [2] K operand tile written (128 producers)
    uint64_t* bar_v = bars + 4;       // [2] V operand tile and its normaliser tile written (96 producers)
    uint64_t* bar_s = bars + 6;       // [2] S = Q K^T complete (tcgen05.commit): K stage free again
    uint64_t* bar_p = bars + 8;       // [2] P written (the softmax threads that own real query rows)
    uint64_t* bar_pv = bars + 10;     // [2] O += P V complete (tcgen05.commit): V stage and P buffer free
    uint64_t* bar_o = bars + 12;      // all MMAs complete
    uint64_t* bar_pkv = bars + 17;    // [2] packed V rows landed (tx bytes)
    uint64_t* bar_t = bars + 19;      // [TAB_SLOTS] per-key tables of tile j in place (slot j % TAB_SLOTS): tx bytes, or the K producers (KM_FOLD)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + P::OFF_MISC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + P::OFF_MISC + 4);

    const int tid = threadIdx.x, lane = tid & 31;
    // the warp index through a shuffle: the compiler then knows that it is the same in every lane, keeps the role branches
    // uniform and can hold addresses, descriptors and loop counters of a role in uniform registers
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    // query tile fastest: the tiles of one (sample, head) run together and share its packed rows in L2
    const int qt = (int)(blockIdx.x % (unsigned)a.n_qtiles), bh = (int)(blockIdx.x / (unsigned)a.n_qtiles), b = bh / a.H, h = bh - b * a.H;
    const int q0 = qt * TC_M;
    const int nq = min(TC_M, a.Lq - q0);
    const int wk = a.wk, wv = a.wv;
    // Key tiles: [j * N, j * N + N) cut at Lk, or (KM_FOLD) the schedule in shared memory whose tiles end at step boundaries
    const int2* tiles = reinterpret_cast<const int2*>(smem + P::OFF_TILES);
    int* sched = reinterpret_cast<int*>(smem + P::OFF_MISC + 8);        // KM_FOLD: [0] number of tiles, [1] longest tile
    auto tile_k0 = [&](int j) -> int { if constexpr (QF) return tiles[j].x; else return j * N; };
    auto tile_n = [&](int j) -> int { if constexpr (QF) return tiles[j].y >> 16; else return min(N, a.Lk - j * N); };
    auto tile_row = [&](int j) -> int { return tiles[j].y & 0xffff; };

    const int32_t* kbase = a.kc + b * a.ks_b + h * a.ks_h;
    const int32_t* vbase = a.vc + b * a.vs_b + h * a.vs_h;
    const int aq = (nq + 31) >> 5;                  // TMEM lane quarters that hold real queries
    float* s_qsum = reinterpret_cast<float*>(smem + P::OFF_QSUM);
    // Everything a tile needs arrives by bulk copies on three barriers: the packed K rows (and, for the packed-half converter,
    // the tile's (key, group) records) on bar_pk, the same for V plus the normaliser records on bar_pkv, the softmax tables
    // on bar_t.  In the folded-query mode only the packed rows travel this way.
    const unsigned char* prep_bh = a.prep + (long long)bh * a.prep_bh_stride;
    auto issue_k = [&](int j) {
        const int s = j & 1;
        const uint32_t kbytes = (uint32_t)tile_n(j) * wk * 4;
        if constexpr (QF) {
            mbar_expect_tx(&bar_pk[s], kbytes);
            bulk_copy_g2s(smem + P::OFF_PK + (2 * s) * P::PK_BYTES, kbase + (long long)tile_k0(j) * wk, kbytes, &bar_pk[s]);
        } else {
            const unsigned char* blk = prep_bh + (long long)j * a.prep_tile_stride;
            mbar_expect_tx(&bar_pk[s], kbytes + (uint32_t)a.prep_krec_bytes);
            bulk_copy_g2s(smem + P::OFF_PK + (2 * s) * P::PK_BYTES, kbase + (long long)tile_k0(j) * wk, kbytes, &bar_pk[s]);
            if (a.prep_krec_bytes)
                bulk_copy_g2s(smem + (s ? P::OFF_KRAW : P::OFF_KPAR), blk + a.prep_off_krec, (uint32_t)a.prep_krec_bytes, &bar_pk[s]);
            constexpr uint32_t tab_bytes = P::TAB_ROWS * N * 4;
            uint64_t* bt = &bar_t[j & (P::TAB_SLOTS - 1)];
            mbar_expect_tx(bt, tab_bytes);
            bulk_copy_g2s(smem + P::OFF_KS + (j & (P::TAB_SLOTS - 1)) * tab_bytes, blk, tab_bytes, bt);
        }
    };
    auto issue_v = [&](int j) {
        const int s = j & 1;
        const uint32_t vbytes = (uint32_t)tile_n(j) * wv * 4;
        if constexpr (QF) {
            mbar_expect_tx(&bar_pkv[s], vbytes);
            bulk_copy_g2s(smem + P::OFF_PK + (2 * s + 1) * P::PK_BYTES, vbase + (long long)tile_k0(j) * wv, vbytes, &bar_pkv[s]);
        } else {
            const unsigned char* blk = prep_bh + (long long)j * a.prep_tile_stride;
            mbar_expect_tx(&bar_pkv[s], vbytes + (uint32_t)a.prep_vrec_bytes + N * 8);
            bulk_copy_g2s(smem + P::OFF_PK + (2 * s + 1) * P::PK_BYTES, vbase + (long long)tile_k0(j) * wv, vbytes, &bar_pkv[s]);
            bulk_copy_g2s(smem + P::OFF_VNST + s * N * 8, blk + a.prep_off_vn, N * 8, &bar_pkv[s]);
            if (a.prep_vrec_bytes)
                bulk_copy_g2s(smem + (s ? P::OFF_VRAW : P::OFF_VPAR), blk + a.prep_off_vrec, (uint32_t)a.prep_vrec_bytes, &bar_pkv[s]);
        }
    };

    if (warp == 0) {
        // one lane per mbarrier: [0,2) packed K, [2,4) K tile, [4,6) V tile, [6,8) S, [8,10) P, [10,12) O += P V,
        // 12 all MMAs, [17,19) packed V, [19,27) tables
        if (lane < P::N_BARS) {
            const uint32_t count = (lane >= 2 && lane < 4) || (QF && lane >= 19) ? (uint32_t)KTHR
                                 : (lane >= 4 && lane < 6)   ? (uint32_t)VTHR
                                 : (lane >= 8 && lane < 10)  ? (uint32_t)(64 * aq)     // only the warps that own real query rows take part
                                                             : 1u;
            mbar_init(&bars[lane], count);
        }
        if (lane == 0) *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        int t_first = (a.Lk + N - 1) / N;
        if constexpr (QF) {
            // tile schedule: every row (appended step) is cut into tiles of at most N keys; a lane per row, prefix sums for the slots
            int2* tw = reinterpret_cast<int2*>(smem + P::OFF_TILES);
            int n_tiles = 0, longest = 0;
            for (int r0 = 0; r0 < a.kp.n_rows; r0 += 32) {
                const int r = r0 + lane;
                int beg = 0, end = 0;
                if (r < a.kp.n_rows) { beg = min(__ldg(a.kp.row_begin + r), a.Lk); end = min(__ldg(a.kp.row_begin + r + 1), a.Lk); }
                const int len = max(end - beg, 0), nt = (len + N - 1) / N;
                int incl = nt;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, incl, d);
                    if (lane >= d) incl += up;
                }
                const int base = n_tiles + incl - nt;
                for (int t = 0; t < nt; ++t)
                    if (base + t < TC_MAX_TILES) tw[base + t] = make_int2(beg + t * N, (min(N, len - t * N) << 16) | r);
                n_tiles += __shfl_sync(0xffffffffu, incl, 31);
                longest = max(longest, __reduce_max_sync(0xffffffffu, min(len, N)));
            }
            n_tiles = min(n_tiles, TC_MAX_TILES);      // the host only picks this kernel when the schedule fits
            if (lane == 0) { sched[0] = n_tiles; sched[1] = longest; }
            t_first = n_tiles;
        }
        __syncwarp();
        if (lane == 0) {
            // the first two packed tiles are requested right away; their latency overlaps the rest of the set-up
            for (int j = 0; j < 2 && j < t_first; ++j) { issue_k(j); issue_v(j); }
        }
    }
    if (tid < 128) s_qsum[tid] = 0.f;
    if (warp == MMA_WARP) {   // TMEM allocation by one full warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)P::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int T = QF ? sched[0] : (a.Lk + N - 1) / N;
    const int longest_tile = QF ? sched[1] : min(N, a.Lk);

    if (!QF && (warp < 8 || warp == MMA_WARP)) {
        // ---- Q tile -> shared (fp16 hi [, lo]) by the softmax and MMA warps; the producers are already at work
        constexpr int CH = D / 8;   // 16-byte chunks per row
        const int qtid = warp < 8 ? tid : 256 + lane;
        const bool want_qsum = !KS && a.kp.zp != nullptr;
        // four chunks per thread in flight: the loads of a batch are all issued before the first one is used
        constexpr int QB = 4;
#pragma unroll 1
        for (int i0 = qtid; i0 < TC_M * CH; i0 += QB * 288) {
            float v[QB][8];
#pragma unroll
            for (int u = 0; u < QB; ++u) {
                const int i = i0 + u * 288, r = i / CH, c = i - r * CH;
#pragma unroll
                for (int j = 0; j < 8; ++j) v[u][j] = 0.f;
                if (i < TC_M * CH && r < nq) load_q8(a.q, a.q_dtype, b * a.qs_b + (long long)(q0 + r) * a.qs_l + h * a.qs_h + c * 8, v[u]);
            }
#pragma unroll
            for (int u = 0; u < QB; ++u) {
                const int i = i0 + u * 288, r = i / CH, c = i - r * CH;
                if (i >= TC_M * CH) break;
                // the operand is fp16: a query element beyond its range (an fp32 or bf16 value above 65504) saturates instead
                // of becoming infinite
#pragma unroll
                for (int j = 0; j < 8; ++j) v[u][j] = fminf(fmaxf(v[u][j], -65504.f), 65504.f);
                uint32_t hi[4], lo[4];
                float part = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half2 h = __floats2half2_rn(v[u][2 * j], v[u][2 * j + 1]);
                    const float2 hf = __half22float2(h);
                    const __half2 l = __floats2half2_rn(v[u][2 * j] - hf.x, v[u][2 * j + 1] - hf.y);
                    hi[j] = *reinterpret_cast<const uint32_t*>(&h);
                    lo[j] = *reinterpret_cast<const uint32_t*>(&l);
                    part += v[u][2 * j] + v[u][2 * j + 1];
                }
                const uint32_t off = tile_off(r, c * 8, TC_M);
                sts128(smem + P::OFF_Q + off, hi[0], hi[1], hi[2], hi[3]);
                if constexpr (NQ == 2) sts128(smem + P::OFF_Q + P::Q_BYTES + off, lo[0], lo[1], lo[2], lo[3]);
                if (want_qsum && r < nq) atomicAdd(&s_qsum[r], part);
            }
        }
        fence_async_smem();
        asm volatile("bar.sync 7, 288;" ::: "memory");
    }

    if (warp < 8 && (warp & 3) >= aq) {
        // this warp's TMEM lanes hold no real query: nothing to do until the tear-down
    } else if (warp < 8) {
        // =============================================================== softmax / epilogue
        constexpr int NH = N / 2;                           // keys per thread and tile
        constexpr int DH = D / 2;                           // output columns per thread
        const int quarter = warp & 3, half = warp >> 2;
        const int r = quarter * 32 + lane;                  // query row = TMEM lane
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t acc = lane_base + P::COL_O + half * P::ACC_COLS;     // this thread's accumulator: D + 16 columns
        float* xch = reinterpret_cast<float*>(smem + P::OFF_XCH);
        // the two warps that share a TMEM lane quarter agree on `ok` and meet at a named barrier
        auto pair_sync_and = [&](bool flag) -> bool {
            uint32_t all_ok;
            asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, %2, 64, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(all_ok) : "r"((uint32_t)flag), "r"(3 + quarter) : "memory");
            return all_ok != 0;
        };
        const bool k_zp = !KS && a.kp.zp != nullptr;      // a dequantised K already carries its zero-point
        float qsum = (k_zp && !QF) ? s_qsum[r] : 0.f;       // KM_FOLD: the row's zero-point constant of the tile's step, read per tile
        const float* rowc = reinterpret_cast<const float*>(smem + P::OFF_ROWC);
        float m_used = -FLT_MAX;                            // reference maximum of this thread's keys (log2 domain)
        bool ok = true;
        for (int j = 0; j < T; ++j) {
            const int buf = j & 1;
            // per-key tables visible, S complete, and the P buffer free (the MMA that read it two tiles ago is done)
            ok = ok && mbar_wait3(&bar_t[j & (P::TAB_SLOTS - 1)], (j / P::TAB_SLOTS) & 1, &bar_s[buf], (j >> 1) & 1,
                                  &bar_pv[(j - P::PST) & 1], ((j - P::PST) >> 1) & 1, j >= P::PST, abort_flag, 11);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const float* ks = reinterpret_cast<const float*>(smem + P::OFF_KS) + (j & (P::TAB_SLOTS - 1)) * P::TAB_ROWS * N + half * NH;
            const float* b2 = KS ? ks : ks + N;                 // a dequantised K keeps the middle row only
            const float* kzs = KS ? ks : ks + 2 * N;
            const uint32_t s_addr = lane_base + P::COL_S + buf * N + half * NH;
            // 32-key chunks of this half that hold at least one key
            const int nch = min(NH / 32, max(0, (tile_n(j) - half * NH + 31) >> 5));
            if constexpr (QF) { if (k_zp) qsum = rowc[(j & 3) * 128 + r]; }
            if (nch > 0) {
                tc_fence_after();
                unsigned char* prow = smem + P::OFF_P + (buf & (P::PST - 1)) * P::P_BYTES + (r >> 3) * 1024 + (r & 7) * 128;
                int c = 0;
#pragma unroll 1
                while (c < nch) {
                    uint32_t rw[32];
                    tmem_ld32(s_addr + c * 32, rw);
                    tmem_wait_ld();
                    const float cm = KS     ? chunk_scores<false, true>(rw, ks + c * 32, b2 + c * 32, kzs + c * 32, qsum, a.scale_log2)
                                     : k_zp ? chunk_scores<true>(rw, ks + c * 32, b2 + c * 32, kzs + c * 32, qsum)
                                            : chunk_scores<false>(rw, ks + c * 32, b2 + c * 32, kzs + c * 32, qsum);
                    if (m_used == -FLT_MAX) m_used = cm;    // first chunk this thread ever sees: its maximum is the reference
                    if (__any_sync(0xffffffffu, cm > m_used + TC_LAZY)) {
                        // Rare: some row of this warp meets a score more than 2^12 above its reference.  A new
                        // reference is taken, the accumulator rescaled, and the tile's chunks are redone
                        // (P of earlier chunks was written against the old reference).
                        m_used = new_reference<D, N, KS>(s_addr, nch, ks, b2, kzs, k_zp, qsum, m_used, acc,
                                                         j > 0 ? &bar_pv[(j - 1) & 1] : nullptr, ((j - 1) >> 1) & 1, abort_flag, a.scale_log2);
                        ok = __all_sync(0xffffffffu, m_used == m_used);
                        if (!ok) break;
                        c = 0;
                        continue;
                    }
                    uint32_t ph[16];
                    chunk_exp(rw, m_used, ph);
                    const int col = half * NH + c * 32;     // key index of the chunk inside the tile
                    unsigned char* blk = prow + (col >> 6) * (TC_M * 128);
                    const int ch0 = (col & 63) >> 3;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        sts128(blk + (((ch0 + q4) ^ (r & 7)) << 4), ph[4 * q4], ph[4 * q4 + 1], ph[4 * q4 + 2], ph[4 * q4 + 3]);
                    ++c;
                }
                if (!ok) break;
            }
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(&bar_p[buf]);
        }
        // ---- merge the two halves of a row: o = sum_h w_h (O_h - corr_h) / sum_h w_h L_h, w_h = 2^(m_h - m)
        xch[half * 128 + r] = m_used;
        ok = ok && mbar_wait(bar_o, 0, abort_flag, 14);
        ok = __all_sync(0xffffffffu, ok);
        ok = pair_sync_and(ok);
        if (ok) {
            tc_fence_after();
            const bool two = longest_tile > NH;             // the second half of the keys ever held a key
            const float m_a = half == 0 ? m_used : xch[r], m_b = two ? (half == 1 ? m_used : xch[128 + r]) : -FLT_MAX;
            const float m = fmaxf(m_a, m_b);
            const float w_a = ex2(m_a - m), w_b = two ? ex2(m_b - m) : 0.f;
            const uint32_t acc_a = lane_base + P::COL_O, acc_b = acc_a + P::ACC_COLS;
            uint32_t ax[16];
            tmem_ld16(acc_a + D, ax);
            tmem_wait_ld();
            float den = w_a * (__uint_as_float(ax[0]) + __uint_as_float(ax[1]));
            float cz = w_a * (__uint_as_float(ax[2]) + __uint_as_float(ax[3]));
            if (two) {
                tmem_ld16(acc_b + D, ax);
                tmem_wait_ld();
                den = fmaf(w_b, __uint_as_float(ax[0]) + __uint_as_float(ax[1]), den);
                cz = fmaf(w_b, __uint_as_float(ax[2]) + __uint_as_float(ax[3]), cz);
            }
            const float inv = 1.f / (den * TC_AUX_UP);
            cz *= TC_ZP_UP;
#pragma unroll 1
            for (int c0 = 0; c0 < DH; c0 += 32) {
                uint32_t ra[32], rb[32];
                tmem_ld32(acc_a + half * DH + c0, ra);
                if (two) tmem_ld32(acc_b + half * DH + c0, rb);
                tmem_wait_ld();
                if (r < nq) {
                    const long long off = b * a.os_b + (long long)(q0 + r) * a.os_l + h * a.os_h + half * DH + c0;
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float s = w_a * __uint_as_float(ra[i]);
                        if (two) s = fmaf(w_b, __uint_as_float(rb[i]), s);
                        v[i] = (s - cz) * inv;
                    }
                    store_o_row32(a.out, a.o_dtype, off, v);
                }
            }
        }
        tc_fence_before();
    } else if (warp < R::V_WARP0) {
        if constexpr (QF) {
            // =============================================================== K producers (and per-key tables)
            const int ptid = tid - 256;
            auto issue = [&](int j) {
                const int s = j & 1;
                const uint32_t kbytes = (uint32_t)tile_n(j) * wk * 4;
                mbar_expect_tx(&bar_pk[s], kbytes);
                bulk_copy_g2s(smem + P::OFF_PK + (2 * s) * P::PK_BYTES, kbase + (long long)tile_k0(j) * wk, kbytes, &bar_pk[s]);
            };
            bool ok = true;
            int issued = min(T, 2);                    // tiles 0 and 1 were requested during set-up
            const bool v_exact = a.vp.group == D;
            // per-key parameters of a tile are fetched one tile ahead so the global-load latency is hidden
            float nsc = 0.f, nzs = 0.f, nvsc = 1.f;
            const long long k_par = a.kp.index(b, 0, h, 0), v_par = a.vp.index(b, 0, h, 0);   // (sample, head) part of the parameter index
            auto fetch_params = [&](int j) {
                nsc = 0.f; nzs = 0.f; nvsc = 1.f;
                if (j < T && ptid < tile_n(j)) {
                    const int key = tile_k0(j) + ptid;
                    if constexpr (KM != KM_EXACT) {
                        nsc = 1.f;                       // S needs only softmax_scale * log2(e)
                    } else {
                        const long long pi = k_par + a.kp.row(key) * a.kp.sr;
                        nsc = __ldg(a.kp.scale + pi);
                        if (a.kp.zp) nzs = __ldg(a.kp.zp + pi);
                    }
                    if (v_exact) nvsc = __ldg(a.vp.scale + v_par + a.vp.row(key) * a.vp.sr);
                }
            };
            fetch_params(0);
            // KM_SPLIT: (key, group) records of the tile, staged one tile ahead, for the packed-half converter
            const int k_vpw = 32 / kb;
            const int k_ng = D / a.kp.group;                                   // groups per key
            const bool k_fast = KS && (a.kp.group % k_vpw) == 0 && (a.kp.group & (a.kp.group - 1)) == 0 && N * k_ng <= 2 * KTHR && N * k_ng <= TC_PAR_ENTRIES;
            const int k_gshift = __ffs(k_ng) - 1, k_grp_shift = __ffs(a.kp.group) - 1;
            uint2* kpar = reinterpret_cast<uint2*>(smem + P::OFF_KPAR);
            const ParamRef* k_ref = reinterpret_cast<const ParamRef*>(smem + P::OFF_PREF);
            if (ptid == 0) *reinterpret_cast<ParamRef*>(smem + P::OFF_PREF) = param_ref(a.kp, b, h);
            asm volatile("bar.sync 1, %0;" ::"n"(KTHR) : "memory");
            using KStage = ParStage<2>;            // two records per thread: groups of 32 or more at either head_dim
            float* kraw = reinterpret_cast<float*>(smem + P::OFF_KRAW);
            if (k_fast) KStage::request(a.kp, k_par, tile_k0(0), tile_n(0), k_gshift, ptid, KTHR, kraw);
            // KM_FOLD: the row (appended step) whose scales the Q operand currently carries, and this thread's row constant
            int q_row = -1;
            float my_rowc = 0.f;
            for (int j = 0; j < T; ++j) {
                const int s = j & 1;
                const int n_valid = tile_n(j);
                const int k0 = tile_k0(j);
                const float sc = nsc, zs = nzs, vsc = nvsc;
                const float bias = (ptid < n_valid) ? 0.f : -1e30f;
                fetch_params(j + 1);
                bool slow = !k_fast;
                if (KS && k_fast) {
                    slow = KStage::build(kpar, kraw, n_valid << k_gshift, kb == 8 ? 128.f : kb == 4 ? 8.f : 2.f, a.kp.zp != nullptr, ptid, KTHR);
                    if (j + 1 < T) KStage::request(a.kp, k_par, tile_k0(j + 1), tile_n(j + 1), k_gshift, ptid, KTHR, kraw);   // consumed one tile later
                }
                ok = ok && mbar_wait(&bar_pk[s], (j >> 1) & 1, abort_flag, 21);
                if (j >= 2) ok = ok && mbar_wait(&bar_s[s], ((j - 2) >> 1) & 1, abort_flag, 22);    // K stage is free
                if constexpr (KS) {
                    if (k_fast) {   // records visible to all producers; one record out of bounds sends the whole tile to the fp32 routine
                        uint32_t any_slow;
                        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, 1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                     : "=r"(any_slow) : "r"((uint32_t)slow), "n"(KTHR) : "memory");
                        slow = any_slow != 0;
                    }
                }
                if constexpr (QF) {
                    const int row = tile_row(j);
                    if (row != q_row) {
                        // The tile starts a new step: Q * s(step) replaces the Q operand once S of the previous tile, the last
                        // reader of the old one, is complete.  c = sum_d q_d s_d z_d of every query row goes to the row constants.
                        // A thread keeps one 16-byte chunk column; its query chunks are requested eight at a time, ahead of the wait.
                        constexpr int CH = D / 8;                       // 16-byte chunks per row
                        constexpr int RSTEP = 128 / CH;                 // rows between two chunks of a thread
                        constexpr int BATCH = 8;
                        const int c = ptid % CH, r_first = ptid / CH;
                        float sv[8], szv[8];
    #pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const long long pi = a.kp.index(b, row, h, c * 8 + e);
                            sv[e] = __ldg(a.kp.scale + pi);
                            szv[e] = a.kp.zp ? sv[e] * __ldg(a.kp.zp + pi) : 0.f;
                        }
                        float* racc = reinterpret_cast<float*>(smem + P::OFF_ROWC) + 4 * 128;
                        float v[BATCH][8];
                        auto load_batch = [&](int it0) {
    #pragma unroll
                            for (int u = 0; u < BATCH; ++u) {
                                const int r = r_first + (it0 + u) * RSTEP;
    #pragma unroll
                                for (int e = 0; e < 8; ++e) v[u][e] = 0.f;
                                if (r < nq) load_q8(a.q, a.q_dtype, b * a.qs_b + (long long)(q0 + r) * a.qs_l + h * a.qs_h + c * 8, v[u]);
                            }
                        };
                        load_batch(0);
                        if (j >= 1) ok = ok && mbar_wait(&bar_s[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, 25);
    #pragma unroll 1
                        for (int it0 = 0; it0 < TC_M / RSTEP; it0 += BATCH) {
                            if (it0 > 0) load_batch(it0);
    #pragma unroll
                            for (int u = 0; u < BATCH; ++u) {
                                const int r = r_first + (it0 + u) * RSTEP;
                                uint32_t hi[4], lo[4];
                                float p0 = 0.f, p1 = 0.f;
    #pragma unroll
                                for (int e = 0; e < 4; ++e) {      // packed fp32 pairs: two elements per instruction
                                    float x0, x1;
                                    fma2(p0, p1, v[u][2 * e], v[u][2 * e + 1], szv[2 * e], szv[2 * e + 1], p0, p1);
                                    fma2(x0, x1, v[u][2 * e], v[u][2 * e + 1], sv[2 * e], sv[2 * e + 1], 0.f, 0.f);
                                    x0 = fminf(fmaxf(x0, -65504.f), 65504.f);      // saturate instead of overflowing fp16
                                    x1 = fminf(fmaxf(x1, -65504.f), 65504.f);
                                    const __half2 hh = __floats2half2_rn(x0, x1);
                                    const float2 hf = __half22float2(hh);
                                    float y0, y1;
                                    add2(y0, y1, x0, x1, -hf.x, -hf.y);
                                    const __half2 ll = __floats2half2_rn(y0, y1);
                                    hi[e] = *reinterpret_cast<const uint32_t*>(&hh);
                                    lo[e] = *reinterpret_cast<const uint32_t*>(&ll);
                                }
                                float part = p0 + p1;
                                const uint32_t off = tile_off(r, c * 8, TC_M);
                                sts128(smem + P::OFF_Q + off, hi[0], hi[1], hi[2], hi[3]);
                                sts128(smem + P::OFF_Q + P::Q_BYTES + off, lo[0], lo[1], lo[2], lo[3]);
                                // the CH threads of a row are neighbouring lanes: fold their parts, one of them writes the row's constant
    #pragma unroll
                                for (int m = 1; m < CH; m <<= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
                                if (c == 0) racc[r] = part;
                            }
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        my_rowc = racc[ptid] * a.scale_log2;
                        q_row = row;
                    }
                    reinterpret_cast<float*>(smem + P::OFF_ROWC)[(j & 3) * 128 + ptid] = my_rowc;
                }
                const uint32_t* pk = reinterpret_cast<const uint32_t*>(smem + P::OFF_PK + (2 * s) * P::PK_BYTES);
                unsigned char* tk = smem + P::OFF_K + s * P::KT * P::KV_BYTES;
                if (ok) {
                    if constexpr (KS) {
                        if (!slow) {
                            if (kb == 8) group_split_tile<8>(tk, tk + P::KV_BYTES, pk, kpar, n_valid, N, wk, ptid, KTHR, k_gshift, k_grp_shift);
                            else if (kb == 4) group_split_tile<4>(tk, tk + P::KV_BYTES, pk, kpar, n_valid, N, wk, ptid, KTHR, k_gshift, k_grp_shift);
                            else group_split_tile<2>(tk, tk + P::KV_BYTES, pk, kpar, n_valid, N, wk, ptid, KTHR, k_gshift, k_grp_shift);
                        } else {
                            if (kb == 8) dequant_split_tile<8>(tk, tk + P::KV_BYTES, pk, n_valid, N, wk, ptid, k_ref, k0, KTHR);
                            else if (kb == 4) dequant_split_tile<4>(tk, tk + P::KV_BYTES, pk, n_valid, N, wk, ptid, k_ref, k0, KTHR);
                            else dequant_split_tile<2>(tk, tk + P::KV_BYTES, pk, n_valid, N, wk, ptid, k_ref, k0, KTHR);
                        }
                    } else {
                        const int krows = min(N, ((n_valid + N / 2 - 1) / (N / 2)) * (N / 2));   // softmax reads whole halves of a tile
                        if (kb == 8) codes_tile<8>(tk, pk, n_valid, N, wk, ptid, KTHR, krows);
                        else if (kb == 4) codes_tile<4>(tk, pk, n_valid, N, wk, ptid, KTHR, krows);
                        else codes_tile<2>(tk, pk, n_valid, N, wk, ptid, KTHR, krows);
                    }
                    if (ptid < N) {   // table slot j % 4; the K scale carries softmax_scale * log2(e)
                        float* tab = reinterpret_cast<float*>(smem + P::OFF_KS) + (j & 3) * 3 * N;
                        const float scl = sc * a.scale_log2;
                        const float vsf = fmaxf(vsc, TC_VS_MIN);
                        tab[ptid] = scl;
                        tab[N + ptid] = bias + __log2f(vsf);
                        tab[2 * N + ptid] = QF ? 1.f : zs * scl;      // KM_FOLD: the row constant is subtracted as it is
                    }
                    fence_async_smem();
                    mbar_arrive(&bar_k[s]);
                    mbar_arrive(&bar_t[j & 3]);
                }

                {   // every K producer is done with the packed stage; all 128 take the same decision on `ok`
                    uint32_t all_ok;
                    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                 : "=r"(all_ok) : "r"((uint32_t)ok), "n"(KTHR) : "memory");
                    ok = all_ok != 0;
                }
                if (!ok) break;
                if (ptid == 0 && j + 2 < T) { issue(j + 2); ++issued; }
            }
            if (!ok && ptid == 0) {
                // drain: bulk copies already issued must land before the CTA may exit
                for (int j = 0; j < issued; ++j) {
                    bool landed = false;
                    for (uint32_t i = 0; i < TC_SPIN_LIMIT && !landed; ++i) landed = mbar_try(&bar_pk[j & 1], (j >> 1) & 1);
                }
            }
        } else {
            // =============================================================== K converters
            // A tile's packed rows and parameter records arrive by bulk copy; the converters only wait, convert and arrive.
            const int ptid = tid - 256;
            const int k_ng = D / a.kp.group;                                   // groups per key
            const bool k_fast = KS && a.prep_krec_bytes > 0;                 // records for the packed-half converter were prepared
            const int k_gshift = __ffs(k_ng) - 1, k_grp_shift = __ffs(a.kp.group) - 1;
            const ParamRef* k_ref = reinterpret_cast<const ParamRef*>(smem + P::OFF_PREF);
            const bool k_fine = finer_items(N * wk / 4, KTHR);               // items of two words spread the tile more evenly
            if constexpr (KS) {
                if (ptid == 0) *reinterpret_cast<ParamRef*>(smem + P::OFF_PREF) = param_ref(a.kp, b, h);
                asm volatile("bar.sync 1, %0;" ::"n"(KTHR) : "memory");
            }
            for (int j = 0; j < T; ++j) {
                const int s = j & 1;
                const int n_valid = tile_n(j);
                bool ok = mbar_wait(&bar_pk[s], (j >> 1) & 1, abort_flag, 21);
                if (ok && j >= 2) ok = mbar_wait(&bar_s[s], ((j - 2) >> 1) & 1, abort_flag, 22);    // K stage is free
                if (!ok) break;
                const uint32_t* pk = reinterpret_cast<const uint32_t*>(smem + P::OFF_PK + (2 * s) * P::PK_BYTES);
                unsigned char* tk = smem + P::OFF_K + s * P::KT * P::KV_BYTES;
                if constexpr (KS) {
                    const unsigned char* kst = smem + (s ? P::OFF_KRAW : P::OFF_KPAR);
                    const uint2* kpar = reinterpret_cast<const uint2*>(kst);
                    // the trailer of the record block says whether a record of the tile is outside the packed-half converter's bounds
                    const bool slow = !k_fast || *reinterpret_cast<const uint32_t*>(kst + a.prep_krec_bytes - 16) != 0u;
                    if (!slow && a.tc_k_perdim) {
                        const uint16_t* steps = reinterpret_cast<const uint16_t*>(kst);
                        const __half* ktab = reinterpret_cast<const __half*>(a.prep_ktab + (long long)bh * a.prep_tab_bh_stride);
                        if (kb == 8) perdim_split_tile<8>(tk, tk + P::KV_BYTES, pk, steps, ktab, D, n_valid, N, wk, ptid, KTHR);
                        else if (kb == 4) perdim_split_tile<4>(tk, tk + P::KV_BYTES, pk, steps, ktab, D, n_valid, N, wk, ptid, KTHR);
                        else perdim_split_tile<2>(tk, tk + P::KV_BYTES, pk, steps, ktab, D, n_valid, N, wk, ptid, KTHR);
                    } else if (!slow) {
                        if (kb == 8) { if (k_fine) group_split_tile<8, 2>(tk, tk + P::KV_BYTES, pk, kpar, n_valid, N, wk, ptid, KTHR, k_gshift, k_grp_shift); else group_split_tile<8, 4>(tk, tk + P::KV_BYTES, pk, kpar, n_valid, N, wk, ptid, KTHR, k_gshift, k_grp_shift); }
                        else if (kb == 4) { if (k_fine) group_split_tile<4, 2>(tk, tk + P::KV_BYTES, pk, kpar, n_valid, N, wk, ptid, KTHR, k_gshift, k_grp_shift); else group_split_tile<4, 4>(tk, tk + P::KV_BYTES, pk, kpar, n_valid, N, wk, ptid, KTHR, k_gshift, k_grp_shift); }
                        else { if (k_fine) group_split_tile<2, 2>(tk, tk + P::KV_BYTES, pk, kpar, n_valid, N, wk, ptid, KTHR, k_gshift, k_grp_shift); else group_split_tile<2, 4>(tk, tk + P::KV_BYTES, pk, kpar, n_valid, N, wk, ptid, KTHR, k_gshift, k_grp_shift); }
                    } else {
                        const int k0 = tile_k0(j);
                        if (kb == 8) dequant_split_tile<8>(tk, tk + P::KV_BYTES, pk, n_valid, N, wk, ptid, k_ref, k0, KTHR);
                        else if (kb == 4) dequant_split_tile<4>(tk, tk + P::KV_BYTES, pk, n_valid, N, wk, ptid, k_ref, k0, KTHR);
                        else dequant_split_tile<2>(tk, tk + P::KV_BYTES, pk, n_valid, N, wk, ptid, k_ref, k0, KTHR);
                    }
                } else {
                    const int krows = min(N, ((n_valid + N / 2 - 1) / (N / 2)) * (N / 2));   // softmax reads whole halves of a tile
                    if (kb == 8) codes_tile<8, false>(tk, pk, n_valid, N, wk, ptid, KTHR, krows);
                    else if (kb == 4) codes_tile<4, false>(tk, pk, n_valid, N, wk, ptid, KTHR, krows);
                    else codes_tile<2, false>(tk, pk, n_valid, N, wk, ptid, KTHR, krows);
                }
                fence_async_smem();
                mbar_arrive(&bar_k[s]);
            }
        }
    } else if (warp < MMA_WARP) {
        if constexpr (QF) {
            // =============================================================== V producers
            const int ptid = tid - R::V_WARP0 * 32;
            auto issue = [&](int j) {
                const int s = j & 1;
                const uint32_t vbytes = (uint32_t)tile_n(j) * wv * 4;
                mbar_expect_tx(&bar_pkv[s], vbytes);
                bulk_copy_g2s(smem + P::OFF_PK + (2 * s + 1) * P::PK_BYTES, vbase + (long long)tile_k0(j) * wv, vbytes, &bar_pkv[s]);
            };
            bool ok = true;
            int issued = min(T, 2);                    // tiles 0 and 1 were requested during set-up
            const bool v_exact = a.vp.group == D;
            // The small operand tile of a stage (16 x N fp16, K-major): row 0/1 = hi/lo of 2^-6 / V scale, row 2/3 =
            // hi/lo of 2^-8 * V zero-point of each key; rows 4-15 stay zero for the whole kernel.  Each thread looks
            // after keys ptid and ptid + 96 and fetches their parameters one tile ahead.
            constexpr int KPT = (N + VTHR - 1) / VTHR;
            float nvs[KPT], nvz[KPT];
            const long long v_par = a.vp.index(b, 0, h, 0);     // (sample, head) part of the parameter index
            auto fetch_v = [&](int j) {
    #pragma unroll
                for (int i = 0; i < KPT; ++i) {
                    nvs[i] = 1.f; nvz[i] = 0.f;
                    const int kt = ptid + i * VTHR;
                    if (v_exact && j < T && kt < tile_n(j)) {
                        const long long vi = v_par + a.vp.row(tile_k0(j) + kt) * a.vp.sr;
                        nvs[i] = __ldg(a.vp.scale + vi);
                        if (a.vp.zp) nvz[i] = __ldg(a.vp.zp + vi);
                    }
                }
            };
            fetch_v(0);
            // A V scale that varies along head_dim: (key, group) records staged one tile ahead for the packed-half converter,
            // or, with per-element parameters that a step's tokens share (KM_FOLD tiles lie inside one step), a per-dim table
            const int v_vpw = 32 / vb;
            const int v_ng = D / a.vp.group;
            const bool v_grouped = !v_exact && (a.vp.group % v_vpw) == 0 && (a.vp.group & (a.vp.group - 1)) == 0 && N * v_ng <= 3 * VTHR && N * v_ng <= TC_PAR_ENTRIES;
            const bool v_perdim = QF && !v_exact && !v_grouped && a.vp.row_of_token != nullptr && (D % (4 * v_vpw)) == 0;
            const int v_gshift = __ffs(v_ng) - 1, v_grp_shift = __ffs(a.vp.group) - 1;
            uint2* vpar = reinterpret_cast<uint2*>(smem + P::OFF_VPAR);
            __half* vdim_s = reinterpret_cast<__half*>(smem + P::OFF_VPAR);
            __half* vdim_sl = vdim_s + D;
            __half* vdim_zb = vdim_s + 2 * D;
            const float v_bias = vb == 8 ? 128.f : vb == 4 ? 8.f : 2.f;
            int vdim_row = -1;
            const ParamRef* v_ref = reinterpret_cast<const ParamRef*>(smem + P::OFF_PREF + 48);
            if (ptid == 0) *reinterpret_cast<ParamRef*>(smem + P::OFF_PREF + 48) = param_ref(a.vp, b, h);
            using VStage = ParStage<3>;
            float* vraw = reinterpret_cast<float*>(smem + P::OFF_VRAW);
            if (v_grouped) VStage::request(a.vp, v_par, tile_k0(0), tile_n(0), v_gshift, ptid, VTHR, vraw);
            asm volatile("bar.sync 2, %0;" ::"n"(VTHR) : "memory");
            for (int j = 0; j < T; ++j) {
                const int s = j & 1;
                const int k0 = tile_k0(j);
                const int n_valid = tile_n(j);
                float vs[KPT], vz[KPT];
    #pragma unroll
                for (int i = 0; i < KPT; ++i) { vs[i] = nvs[i]; vz[i] = nvz[i]; }
                fetch_v(j + 1);
                bool slow = !v_grouped && !v_perdim;
                if (v_grouped) {
                    slow = VStage::build(vpar, vraw, n_valid << v_gshift, v_bias, a.vp.zp != nullptr, ptid, VTHR);
                    if (j + 1 < T) VStage::request(a.vp, v_par, tile_k0(j + 1), tile_n(j + 1), v_gshift, ptid, VTHR, vraw);   // consumed one tile later
                } else if (v_perdim) {
                    const int row = a.vp.row(k0);
                    slow = a.vp.row(k0 + n_valid - 1) != row;            // the tile must lie inside one row of V's parameters
                    if (!slow && row != vdim_row) {
                        for (int d = ptid; d < D; d += VTHR) {
                            const long long pi = a.vp.index(b, row, h, d);
                            const float sv = __ldg(a.vp.scale + pi), zv = a.vp.zp ? __ldg(a.vp.zp + pi) : 0.f;
                            const __half s_hi = __float2half_rn(sv);
                            vdim_s[d] = s_hi;
                            vdim_sl[d] = __float2half_rn(sv - __half2float(s_hi));
                            vdim_zb[d] = __float2half_rn(1024.f + v_bias + zv);
                            slow = slow || !(fabsf(zv) <= 512.f) || !(sv < 60.f);
                        }
                    }
                    vdim_row = slow ? -1 : row;
                }
                ok = ok && mbar_wait(&bar_pkv[s], (j >> 1) & 1, abort_flag, 24);
                if (j >= 2) ok = ok && mbar_wait(&bar_pv[s], ((j - 2) >> 1) & 1, abort_flag, 23);   // V stage is free
                if (v_grouped || v_perdim) {   // tables visible to all producers; they agree on the converter
                    uint32_t any_slow;
                    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, 2, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                 : "=r"(any_slow) : "r"((uint32_t)slow), "n"(VTHR) : "memory");
                    slow = any_slow != 0;
                    if (slow) vdim_row = -1;
                }
                const uint32_t* pv = reinterpret_cast<const uint32_t*>(smem + P::OFF_PK + (2 * s + 1) * P::PK_BYTES);
                const int vrows = min(N, (n_valid + 15) & ~15);     // the PV product stops at the 16-key step that holds the last key
                unsigned char* tv = smem + P::OFF_V + s * P::V_BYTES;
                if (ok) {
                    if (v_exact) {
                        if (vb == 8) codes_tile<8, true>(tv, pv, n_valid, N, wv, ptid, VTHR, vrows);
                        else if (vb == 4) codes_tile<4, true>(tv, pv, n_valid, N, wv, ptid, VTHR, vrows);
                        else codes_tile<2, true>(tv, pv, n_valid, N, wv, ptid, VTHR, vrows);
                    } else if (!slow && v_grouped) {
                        if (vb == 8) group_tile<8>(tv, pv, vpar, n_valid, N, wv, ptid, VTHR, vrows, v_gshift, v_grp_shift);
                        else if (vb == 4) group_tile<4>(tv, pv, vpar, n_valid, N, wv, ptid, VTHR, vrows, v_gshift, v_grp_shift);
                        else group_tile<2>(tv, pv, vpar, n_valid, N, wv, ptid, VTHR, vrows, v_gshift, v_grp_shift);
                    } else if (!slow && v_perdim) {
                        if (vb == 8) perdim_tile<8>(tv, pv, vdim_s, vdim_sl, vdim_zb, n_valid, N, wv, ptid, VTHR, vrows);
                        else if (vb == 4) perdim_tile<4>(tv, pv, vdim_s, vdim_sl, vdim_zb, n_valid, N, wv, ptid, VTHR, vrows);
                        else perdim_tile<2>(tv, pv, vdim_s, vdim_sl, vdim_zb, n_valid, N, wv, ptid, VTHR, vrows);
                    } else {
                        if (vb == 8) dequant_tile<8>(tv, pv, n_valid, N, wv, ptid, v_ref, k0, VTHR);
                        else if (vb == 4) dequant_tile<4>(tv, pv, n_valid, N, wv, ptid, v_ref, k0, VTHR);
                        else dequant_tile<2>(tv, pv, n_valid, N, wv, ptid, v_ref, k0, VTHR);
                    }
                    // normaliser columns D .. D + 15 of every key of the tile: 2^-6 / V scale and 2^-8 * V zero-point as fp16 hi + lo
                    // pairs, twelve zeros (every row gets finite values: P is zero for the keys past the end, but 0 * NaN is not)
    #pragma unroll
                    for (int i = 0; i < KPT; ++i) {
                        const int kt = ptid + i * VTHR;
                        if (kt < N) {
                            const float vin = TC_AUX_DOWN * __frcp_rn(fmaxf(vs[i], TC_VS_MIN)), vzd = vz[i] * TC_ZP_DOWN;
                            const __half vin_hi = __float2half_rn(vin), vz_hi = __float2half_rn(vzd);
                            const __half vin_lo = __float2half_rn(vin - __half2float(vin_hi)), vz_lo = __float2half_rn(vzd - __half2float(vz_hi));
                            unsigned char* ax = tv + vtile_off(kt, D, N);
                            sts128(ax, (uint32_t)__half_as_ushort(vin_hi) | ((uint32_t)__half_as_ushort(vin_lo) << 16),
                                   (uint32_t)__half_as_ushort(vz_hi) | ((uint32_t)__half_as_ushort(vz_lo) << 16), 0u, 0u);
                            sts128(ax + N * 16, 0u, 0u, 0u, 0u);
                        }
                    }
                    fence_async_smem();
                    mbar_arrive(&bar_v[s]);
                }

                {
                    uint32_t all_ok;
                    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 2, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                 : "=r"(all_ok) : "r"((uint32_t)ok), "n"(VTHR) : "memory");
                    ok = all_ok != 0;
                }
                if (!ok) break;
                if (ptid == 0 && j + 2 < T) { issue(j + 2); ++issued; }
            }
            if (!ok && ptid == 0) {
                for (int j = 0; j < issued; ++j) {
                    bool landed = false;
                    for (uint32_t i = 0; i < TC_SPIN_LIMIT && !landed; ++i) landed = mbar_try(&bar_pkv[j & 1], (j >> 1) & 1);
                }
            }
        } else {
            // =============================================================== V converters
            const int ptid = tid - R::V_WARP0 * 32;
            const bool v_exact = a.vp.group == D;
            const bool v_grouped = a.prep_vrec_bytes > 0;                    // records for the packed-half converter were prepared
            const int v_ng = D / a.vp.group;
            const int v_gshift = __ffs(v_ng) - 1, v_grp_shift = __ffs(a.vp.group) - 1;
            const ParamRef* v_ref = reinterpret_cast<const ParamRef*>(smem + P::OFF_PREF + 48);
            const bool v_fine = finer_items(N * wv / 4, VTHR);
            if (ptid == 0) *reinterpret_cast<ParamRef*>(smem + P::OFF_PREF + 48) = param_ref(a.vp, b, h);
            asm volatile("bar.sync 2, %0;" ::"n"(VTHR) : "memory");
            for (int j = 0; j < T; ++j) {
                const int s = j & 1;
                const int n_valid = tile_n(j);
                bool ok = mbar_wait(&bar_pkv[s], (j >> 1) & 1, abort_flag, 24);
                if (ok && j >= 2) ok = mbar_wait(&bar_pv[s], ((j - 2) >> 1) & 1, abort_flag, 23);   // V stage is free
                if (!ok) break;
                const uint32_t* pv = reinterpret_cast<const uint32_t*>(smem + P::OFF_PK + (2 * s + 1) * P::PK_BYTES);
                const int vrows = min(N, (n_valid + 15) & ~15);     // the PV product stops at the 16-key step that holds the last key
                unsigned char* tv = smem + P::OFF_V + s * P::V_BYTES;
                if (v_exact) {
                    if (vb == 8) codes_tile<8, true>(tv, pv, n_valid, N, wv, ptid, VTHR, vrows);
                    else if (vb == 4) codes_tile<4, true>(tv, pv, n_valid, N, wv, ptid, VTHR, vrows);
                    else codes_tile<2, true>(tv, pv, n_valid, N, wv, ptid, VTHR, vrows);
                } else {
                    const unsigned char* vst = smem + (s ? P::OFF_VRAW : P::OFF_VPAR);
                    const uint2* vpar = reinterpret_cast<const uint2*>(vst);
                    const bool slow = !v_grouped || *reinterpret_cast<const uint32_t*>(vst + a.prep_vrec_bytes - 16) != 0u;
                    if (!slow && a.tc_v_perdim) {
                        const uint16_t* steps = reinterpret_cast<const uint16_t*>(vst);
                        const __half* vtab = reinterpret_cast<const __half*>(a.prep_vtab + (long long)bh * a.prep_tab_bh_stride);
                        if (vb == 8) perdim_steps_tile<8>(tv, pv, steps, vtab, D, n_valid, N, wv, ptid, VTHR, vrows);
                        else if (vb == 4) perdim_steps_tile<4>(tv, pv, steps, vtab, D, n_valid, N, wv, ptid, VTHR, vrows);
                        else perdim_steps_tile<2>(tv, pv, steps, vtab, D, n_valid, N, wv, ptid, VTHR, vrows);
                    } else if (!slow) {
                        if (vb == 8) { if (v_fine) group_tile<8, 2>(tv, pv, vpar, n_valid, N, wv, ptid, VTHR, vrows, v_gshift, v_grp_shift); else group_tile<8, 4>(tv, pv, vpar, n_valid, N, wv, ptid, VTHR, vrows, v_gshift, v_grp_shift); }
                        else if (vb == 4) { if (v_fine) group_tile<4, 2>(tv, pv, vpar, n_valid, N, wv, ptid, VTHR, vrows, v_gshift, v_grp_shift); else group_tile<4, 4>(tv, pv, vpar, n_valid, N, wv, ptid, VTHR, vrows, v_gshift, v_grp_shift); }
                        else { if (v_fine) group_tile<2, 2>(tv, pv, vpar, n_valid, N, wv, ptid, VTHR, vrows, v_gshift, v_grp_shift); else group_tile<2, 4>(tv, pv, vpar, n_valid, N, wv, ptid, VTHR, vrows, v_gshift, v_grp_shift); }
                    } else {
                        const int k0 = tile_k0(j);
                        if (vb == 8) dequant_tile<8>(tv, pv, n_valid, N, wv, ptid, v_ref, k0, VTHR);
                        else if (vb == 4) dequant_tile<4>(tv, pv, n_valid, N, wv, ptid, v_ref, k0, VTHR);
                        else dequant_tile<2>(tv, pv, n_valid, N, wv, ptid, v_ref, k0, VTHR);
                    }
                }
                // normaliser columns D .. D + 15 of every key of the tile: 2^-6 / V scale and 2^-8 * V zero-point as fp16 hi + lo
                // pairs (prepared per key), twelve zeros
                // (by the highest-numbered threads: they have the fewest items to convert)
                const uint2* vn = reinterpret_cast<const uint2*>(smem + P::OFF_VNST) + s * N;
                for (int kt = VTHR - 1 - ptid; kt < N; kt += VTHR) {
                    const uint2 r = vn[kt];
                    unsigned char* ax = tv + vtile_off(kt, D, N);
                    sts128(ax, r.x, r.y, 0u, 0u);
                    sts128(ax + N * 16, 0u, 0u, 0u, 0u);
                }
                fence_async_smem();
                mbar_arrive(&bar_v[s]);
            }
        }
    } else if (warp == MMA_WARP) {
        // =============================================================== MMA issue (the whole warp waits; one elected lane issues)
        // Order: S(0), S(1), then per tile j: wait P(j) -> S(j+2) -> O += P(j) V(j).  S(j+2) reuses the TMEM
        // columns of S(j), free once P(j) is complete, and goes first because the softmax two tiles ahead
        // waits for it while nobody waits for the accumulator.
        constexpr uint32_t IDESC_S = instr_desc(TC_M, N, 0);
        constexpr uint32_t IDESC_O = instr_desc(TC_M, D + 16, 1);     // output columns and normaliser columns in one product
        bool ok = true;
        // every lane waits; the lanes agree on the outcome so that the warp stays converged for the elected instructions
        auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
            return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, code));
        };
        // descriptors differ from their stage base only in the start-address field (bits 0-13, 16-byte units)
        const uint64_t qd0 = smem_desc(smem_u32(smem + P::OFF_Q), 16, 1024);
        const uint64_t kd0 = smem_desc(smem_u32(smem + P::OFF_K), 16, 1024);
        const uint64_t pd0 = smem_desc(smem_u32(smem + P::OFF_P), 16, 1024);
        // unswizzled MN-major: leading offset = between key blocks (8 keys), stride offset = between 8-column blocks
        const uint64_t vd0 = smem_desc(smem_u32(smem + P::OFF_V), 128, N * 16, 0u);
        // S = Q K^T of tile j.  exact-code K: Q_hi K [+ Q_lo K]; dequantised K: Q_hi K_hi + Q_hi K_lo [+ Q_lo K_hi]
        auto issue_qk = [&](int j) -> bool {
            const int s = j & 1;
            if (!wait_all(&bar_k[s], (j >> 1) & 1, 31)) return false;
            tc_fence_after();
            const uint64_t kd = kd0 + (uint64_t)((s * P::KT * P::KV_BYTES) >> 4);
            bool first = true;
#pragma unroll
            for (int qi = 0; qi < NQ; ++qi) {
#pragma unroll
                for (int ki = 0; ki < P::KT; ++ki) {
                    if (qi == 1 && ki == 1) continue;     // lo x lo is below fp32 resolution
                    const uint64_t qd = qd0 + (uint64_t)((qi * P::Q_BYTES) >> 4), kdk = kd + (uint64_t)((ki * P::KV_BYTES) >> 4);
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        tc_mma_f16(tmem_base + P::COL_S + s * N, qd + (uint64_t)(((kk >> 2) * (TC_M * 128) + (kk & 3) * 32) >> 4),
                                   kdk + (uint64_t)(((kk >> 2) * (N * 128) + (kk & 3) * 32) >> 4), IDESC_S, first ? 0u : 1u);
                        first = false;
                    }
                }
            }
            tc_commit(&bar_s[s]);
            return true;
        };
        // (O_half | sum_k P / V-scale, sum_k P * V zero-point) += P (V | normaliser columns), 16 keys per step; the first half
        // of a tile's keys goes to accumulator 0, the second half to accumulator 1
        bool live0 = false, live1 = false;        // scalars, not an array: a runtime-indexed array would live in local memory
        auto issue_pv = [&](int j) {
            const int s = j & 1;
            const int ksteps = (tile_n(j) + 15) >> 4;                // P columns / V rows past the keys are never read
            const uint64_t pd = pd0 + (uint64_t)(((s & (P::PST - 1)) * P::P_BYTES) >> 4), vd = vd0 + (uint64_t)((s * P::V_BYTES) >> 4);
            // rolled on purpose: the loop is short-lived code that every CTA has to fetch again
            uint64_t pk = pd, vk = vd;
#pragma unroll 1
            for (int kk = 0; kk < ksteps; ++kk) {
                const int hf = kk >= N / 32 ? 1 : 0;
                // the first product into an accumulator overwrites it (with tiles cut at step boundaries the second
                // half of the keys may first appear in a later tile than the first half)
                tc_mma_f16(tmem_base + P::COL_O + hf * P::ACC_COLS, pk, vk, IDESC_O, (hf ? live1 : live0) ? 1u : 0u);
                if (hf) live1 = true; else live0 = true;
                // next 16 keys: 32 bytes further in the K-major P tile (a new 64-key block every fourth step), two key blocks in V
                pk += ((kk & 3) == 3) ? (uint64_t)((TC_M * 128 - 96) >> 4) : 2u;
                vk += (uint64_t)(256 >> 4);
            }
            tc_commit(&bar_pv[s]);
        };
        // Iteration jj issues S(jj) for jj < 2 (nothing to wait for) and from then on waits for P(j), j = jj - 2, and issues
        // S(j + 2) and O += P(j) V(j).  With two P buffers S goes first: the softmax two tiles ahead waits for it while nobody
        // waits for the accumulator.  With one P buffer the next softmax waits for this product to free the buffer, so it goes first.
        for (int jj = 0; jj < T + 2 && ok; ++jj) {
            const int j = jj - 2;
            if (j >= 0) {
                ok = wait_all(&bar_p[j & 1], (j >> 1) & 1, 32);
                if (!ok) break;
                tc_fence_after();
            }
            if (P::PST == 1 && j >= 0) {
                ok = wait_all(&bar_v[j & 1], (j >> 1) & 1, 34);
                if (!ok) break;
                tc_fence_after();
                issue_pv(j);
            }
            if (jj < T) {
                ok = issue_qk(jj);
                if (!ok) break;
            }
            if (P::PST == 2 && j >= 0) {
                ok = wait_all(&bar_v[j & 1], (j >> 1) & 1, 34);
                if (!ok) break;
                tc_fence_after();
                issue_pv(j);
            }
        }
        if (ok) tc_commit(bar_o);
        tc_fence_before();
    } else if (!QF && warp == R::LOAD_WARP) {
        // =============================================================== copy issue (one thread)
        // Tile t goes into the stages of tile t - 2 once the converters have arrived on that tile's operand barriers (their
        // last read of the packed stage).  The table slot of tile t was last read by the softmax of tile t - 8: K(t - 2)
        // converted means S(t - 4) is complete, which was issued after P(t - 6).
        if (lane == 0) {
            bool ok = true;
            int tk = min(T, 2), tv = min(T, 2);          // next tile of each stream (the first two were requested during set-up)
            uint32_t tries = 0;
            while (tk < T || tv < T) {
                bool progress = false;
                if (tk < T && mbar_try(&bar_k[tk & 1], ((tk - 2) >> 1) & 1)) { issue_k(tk); ++tk; progress = true; }
                if (tv < T && mbar_try(&bar_v[tv & 1], ((tv - 2) >> 1) & 1)) { issue_v(tv); ++tv; progress = true; }
                if (progress) { tries = 0; continue; }
                if (*abort_flag) { ok = false; break; }
                if (++tries >= TC_SPIN_LIMIT) {
                    *abort_flag = 1;
                    atomicCAS(&g_tc_status, 0, 41);
                    ok = false;
                    break;
                }
            }
            const int issued = max(tk, tv);
            if (!ok || *abort_flag) {
                // drain: bulk copies already issued must land before the CTA may exit
                for (int t = max(0, issued - 2); t < issued; ++t) {
                    bool landed = false;
                    for (uint32_t i = 0; i < TC_SPIN_LIMIT && !landed; ++i)
                        landed = (t >= tk || (mbar_try(&bar_pk[t & 1], (t >> 1) & 1) &&
                                              mbar_try(&bar_t[t & (P::TAB_SLOTS - 1)], (t / P::TAB_SLOTS) & 1))) &&
                                 (t >= tv || mbar_try(&bar_pkv[t & 1], (t >> 1) & 1));
                }
            }
        }
    }
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)P::TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------- host side
bool attn_tc_eligible(const AttnArgs& a, int kb, int vb) {
    if (a.D != 64 && a.D != 128) return false;
    if ((a.wk & 3) || (a.wv & 3)) return false;                // 16-byte rows for the bulk copies
    if (a.ks_l != a.wk || a.vs_l != a.wv) return false;        // tokens of one (sample, head) contiguous
    if (!a.k16 || !a.v16) return false;
    (void)kb; (void)vb;
    return true;
}

// Records for the packed-half converters exist when the groups are a power of two of whole packed words and a tile's records fit
// their staging buffer (with the trailer): at most 256 (key, group) pairs per tile.
static bool records_apply(int group, int D, int bits, int N) {
    const int vpw = 32 / bits, ng = D / group;
    return group != D && (group % vpw) == 0 && (group & (group - 1)) == 0 && N * ng <= 256;
}
static size_t prep_tile_bytes_max(int N) { return (size_t)3 * N * 4 + (size_t)N * 8 + 2 * (256 * 8 + 16); }
// Per-dim parameters shared by the tokens of a step are served from per-(sample, head) tables of at most this many steps
// (the schedules of the models have 10 to 13); longer histories take the folded-query kernel.
constexpr int TC_MAX_STEPS = 64;
static bool steps_apply(const ParamView& pv, int D, int bits) {
    return pv.group != D && pv.row_of_token != nullptr && pv.n_rows > 0 && pv.n_rows <= TC_MAX_STEPS && (D % (4 * (32 / bits))) == 0;
}

size_t attn_tc_workspace_bytes(int B, int H, int Lk, int D) {
    if (D != 64 && D != 128) return 0;
    const int N = D == 64 ? 128 : 64;
    const size_t tiles = (size_t)(Lk + N - 1) / N;
    const size_t tables = (size_t)2 * TC_MAX_STEPS * 3 * D * 2;       // K and V step tables of one (sample, head)
    return (size_t)B * H * (tiles * prep_tile_bytes_max(N) + tables) + 256;       // + room to align the base
}

template <int D, int NQ, int KM>
static int launch_tc(const AttnArgs& a0, int kb, int vb, void* ws, size_t ws_bytes, cudaStream_t st) {
    AttnArgs a = a0;
    using P = TcPlan<D, NQ, KM>;
    if constexpr (KM != KM_FOLD) {
        constexpr int N = P::N;
        const int T = (a.Lk + N - 1) / N;
        a.tc_k_perdim = KM == KM_SPLIT && steps_apply(a.kp, D, kb);
        a.tc_v_perdim = steps_apply(a.vp, D, vb);
        const bool k_rec = KM == KM_SPLIT && !a.tc_k_perdim && records_apply(a.kp.group, D, kb, N);
        const bool v_rec = !a.tc_v_perdim && records_apply(a.vp.group, D, vb, N);
        const int k_ng = D / a.kp.group, v_ng = D / a.vp.group;
        a.prep_off_vn = P::TAB_ROWS * N * 4;
        a.prep_off_krec = a.prep_off_vn + N * 8;
        a.prep_krec_bytes = a.tc_k_perdim ? N * 2 + 16 : k_rec ? N * k_ng * 8 + 16 : 0;
        a.prep_off_vrec = a.prep_off_krec + a.prep_krec_bytes;
        a.prep_vrec_bytes = a.tc_v_perdim ? N * 2 + 16 : v_rec ? N * v_ng * 8 + 16 : 0;
        a.prep_tile_stride = a.prep_off_vrec + a.prep_vrec_bytes;
        a.prep_bh_stride = (long long)T * a.prep_tile_stride;
        const int tab_k = a.tc_k_perdim ? a.kp.n_rows * 3 * D * 2 : 0, tab_v = a.tc_v_perdim ? a.vp.n_rows * 3 * D * 2 : 0;
        a.prep_tab_bh_stride = tab_k + tab_v;
        const uintptr_t base = (reinterpret_cast<uintptr_t>(ws) + 255) & ~(uintptr_t)255;
        const size_t tiles_bytes = (size_t)a.B * a.H * (size_t)a.prep_bh_stride;
        const size_t need = tiles_bytes + (size_t)a.B * a.H * (size_t)a.prep_tab_bh_stride + (base - reinterpret_cast<uintptr_t>(ws));
        if (!ws || ws_bytes < need)
            return fail(VARQ_ERR_WORKSPACE, "varq_attn_fwd: workspace of %zu bytes needed, %zu given", need, ws_bytes);
        a.prep = reinterpret_cast<unsigned char*>(base);
        a.prep_ktab = a.prep + tiles_bytes;          // tile blocks are multiples of 16 bytes, and so are the tables
        a.prep_vtab = a.prep_ktab + tab_k;
        const long long prep_blocks = (long long)a.B * a.H * T;
        if (prep_blocks > 0x7fffffffLL) return fail(VARQ_ERR_UNSUPPORTED, "varq_attn_fwd: more than 2^31 thread blocks");
        tc_prepare_kernel<N><<<(unsigned)prep_blocks, N, 0, st>>>(a, T, KM == KM_SPLIT ? 1 : 0, k_ng, v_ng, kb, vb);
        VARQ_CUDA_TRY(cudaGetLastError());
        count_launches(1);
    }
    static_assert(P::TOTAL + 1024 <= 227 * 1024, "shared-memory plan exceeds the per-CTA limit");
    const size_t smem = P::TOTAL + 1024;   // slack for the 1024-byte alignment of the swizzled tiles
    static bool configured[64] = {false};    // per device; the attribute is sticky, set it outside any stream capture
    int dev = 0;
    VARQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        VARQ_CUDA_TRY(cudaFuncSetAttribute(attn_tc_kernel<D, NQ, KM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int nqt = (a.Lq + TC_M - 1) / TC_M;
    const long long blocks_1d = (long long)a.B * a.H * nqt;
    if (blocks_1d > 0x7fffffffLL) return fail(VARQ_ERR_UNSUPPORTED, "varq_attn_fwd: more than 2^31 thread blocks");
    a.n_qtiles = nqt;
    attn_tc_kernel<D, NQ, KM><<<(unsigned)blocks_1d, TcRoles<KM>::THREADS, smem, st>>>(a, kb, vb);
    VARQ_CUDA_TRY(cudaGetLastError());
    count_launches(1);
    return VARQ_OK;
}

int attn_tc_run(const AttnArgs& a, int kb, int vb, void* ws, size_t ws_bytes, cudaStream_t st) {
    // fp16 queries, and bf16 queries inside fp16's normal range (2^-14 <= |q| <= 65504), are exact in one fp16 term;
    // larger magnitudes saturate, smaller ones lose low bits (both far outside what a softmax can resolve)
    const bool split_q = a.q_dtype == VARQ_F32;
    const bool varies = a.kp.group != a.D;         // K scale varies along head_dim
    // ... but is constant over the tokens of a step, the steps are known, and their tile schedule fits: fold it into Q
    const int n_max = a.D == 64 ? 128 : 64;
    // (only for histories of more steps than the step tables of the dequantising mode hold)
    const bool fold = varies && !steps_apply(a.kp, a.D, kb) && a.kp.row_of_token && a.kp.row_begin && a.kp.n_rows > 0 &&
                      a.kp.n_rows <= 0xffff && (a.Lk + n_max - 1) / n_max + a.kp.n_rows <= TC_MAX_TILES;
    if (a.D == 64) {
        if (fold) return launch_tc<64, 2, KM_FOLD>(a, kb, vb, ws, ws_bytes, st);
        if (varies) return split_q ? launch_tc<64, 2, KM_SPLIT>(a, kb, vb, ws, ws_bytes, st) : launch_tc<64, 1, KM_SPLIT>(a, kb, vb, ws, ws_bytes, st);
        return split_q ? launch_tc<64, 2, KM_EXACT>(a, kb, vb, ws, ws_bytes, st) : launch_tc<64, 1, KM_EXACT>(a, kb, vb, ws, ws_bytes, st);
    }
    if (fold) return launch_tc<128, 2, KM_FOLD>(a, kb, vb, ws, ws_bytes, st);
    if (varies) return split_q ? launch_tc<128, 2, KM_SPLIT>(a, kb, vb, ws, ws_bytes, st) : launch_tc<128, 1, KM_SPLIT>(a, kb, vb, ws, ws_bytes, st);
    return split_q ? launch_tc<128, 2, KM_EXACT>(a, kb, vb, ws, ws_bytes, st) : launch_tc<128, 1, KM_EXACT>(a, kb, vb, ws, ws_bytes, st);
}

int attn_tc_status(int* out) {
    int v = 0;
    // a symbol copy on the legacy default stream does not wait for kernels on non-blocking streams: wait for the device first
    VARQ_CUDA_TRY(cudaDeviceSynchronize());
    VARQ_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)));
    if (v != 0) {
        const int zero = 0;
        VARQ_CUDA_TRY(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)));
    }
    *out = v;
    return VARQ_OK;
}

}  // namespace varq
