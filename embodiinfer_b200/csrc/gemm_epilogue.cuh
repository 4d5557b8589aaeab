// Pieces shared by the two schedules of the quantised Linear (gemm.cu: one CTA per tile;
// gemm_pair.cu: a CTA pair per 256-token tile): tile constants, the kernel argument block and the
// fused epilogues (scales, bias, residual, GELU table, gate * up, e4m3 / NVFP4 re-encoding).
#pragma once

#include "common.cuh"
#include "ptx.cuh"

#include <cuda.h>

namespace b2 {

// Two service warps (TMA, MMA) plus the epilogue warps.  The plain Linear epilogue is a handful of
// instructions per element and runs on 8 warps; the epilogues that go through the GELU table (lookups, two
// roundings, block scale, exact division, packing) are latency-bound, so they get 16 warps: four per TMEM
// lane partition, each owning 16-feature units (or 32-column chunks) of the tile.
#ifndef B2_GEGLU_EPILOGUE_WARPS
#define B2_GEGLU_EPILOGUE_WARPS 16
#endif
__host__ __device__ constexpr int epilogue_warps(int epi) { return epi != 0 ? B2_GEGLU_EPILOGUE_WARPS : 8; }
constexpr int FIRST_EPILOGUE_WARP = 2;
__host__ __device__ constexpr int gemm_threads(int epi) { return 32 * (FIRST_EPILOGUE_WARP + epilogue_warps(epi)); }
constexpr int TILE_TOKENS = 128;                   // MMA M
constexpr int STAGE_K_BYTES = 128;                 // one swizzle row
constexpr int A_TILE_BYTES = TILE_TOKENS * STAGE_K_BYTES;
constexpr int SCALE_ATOM_BYTES = 512;              // 128 rows x 4 blocks of 16
constexpr int SCALE_ATOMS_PER_STAGE = 4;           // 4 x 64 elements = 256 e2m1 = 128 bytes of K

constexpr int MAX_STAGES = 16;
constexpr int TMEM_COLUMNS = 512;
// NVFP4 scale factors live in TMEM columns 384..479: two sets (alternating by K slice, so the copies for
// one slice never overwrite columns an MMA of the previous slice may still be reading), each 16 columns
// of token scales (4 per 64 elements of K) followed by 32 columns of feature scales (8 per 64 elements).
constexpr int MAX_RESIDENT_KB = 8;                 // K stages of a token tile kept in shared memory (8 x 16 KB)
constexpr int PREFETCH_DISTANCE = 12;              // K stages between an L2 prefetch and its load
constexpr int TMEM_SFA_COLUMNS = 16;               // 4 atoms x 4 columns of token scales per K stage
// A set of scale columns = 16 token-scale columns + 16 per 128-row block of feature scales; sets are
// stacked downwards from column 512 and rotate with the K stages.
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int MAX_COMPACT_GELU = 4096;             // magnitude codes of the GELU table kept in shared memory
constexpr int SMEM_MINIMUM = 120 * 1024;           // keeps a second CTA (and its TMEM request) off the SM

enum { EPI_LINEAR = 0, EPI_GEGLU_BF16 = 1, EPI_GEGLU_FP8 = 2, EPI_GEGLU_NVFP4 = 3, EPI_GELU_BF16 = 4, EPI_GELU_FP8 = 5,
       EPI_ROPE = 6 };          // cluster schedule only: the packed QKV projection with the attention preparation as its epilogue
__host__ __device__ constexpr bool is_gated(int epi) { return epi >= EPI_GEGLU_BF16 && epi <= EPI_GEGLU_NVFP4; }

struct KernelArgs {
    int tokens, features, k_bytes, num_kb;
    int tile_n;                  // TMEM columns per tile (GEGLU: gate half + up half)
    int num_m_tiles, num_n_tiles, total_tiles;
    int stages, accumulators, accumulator_stride, scale_sets, scale_blocks;
    int splits;                  // > 1: K is cut into `splits` ranges computed by different CTAs, see the epilogue
    int resident;                // 1: the CTA keeps its token tile (all of K) and its token scales on chip, see TileWalk
    int kps;                     // paired schedule: K atoms (128 bytes of K) per ring slot
    int up_row_offset;           // row of the first "up" feature in the packed weight
    int scale_column_tiles;      // 512-byte scale atoms per 128-row block
    int act_row_blocks, weight_row_blocks;
    int flags;
    int gelu_lo, gelu_hi;        // bf16 magnitude codes [lo, hi) whose GELU is kept in shared memory (0,0 = none)
    const uint8_t* act_scales;
    const uint8_t* weight_scales;
    const float* act_scale;
    const float* weight_scale;
    const float* weight_scale_up;   // GEGLU: scale of the up rows (nullptr = same as the gate rows)
    const __nv_bfloat16* bias;
    const __nv_bfloat16* residual;
    const uint16_t* gelu_table;
    const float* out_scale;
    void* out;
    uint8_t* out_scales;
    uint8_t* out_blocked;
    unsigned int* status;
    int a_box_bytes;             // bytes of the token box of one K stage: 128 rows, or fewer (a multiple of 8) when the launch has
                                 // one token tile with fewer tokens -- the rows beyond the box are whatever shared memory holds,
                                 // they only feed accumulator rows that are never stored
    // EPI_ROPE (b2_rope_desc): rotary factors, destinations and shapes of the attention preparation
    const float* rope_sine;
    const float* rope_cosine;
    __nv_bfloat16* rope_q;
    __nv_bfloat16* rope_k;
    __nv_bfloat16* rope_v;
    long long rope_batch_stride;
    int rope_tokens, rope_heads, rope_kv_heads, rope_capacity, rope_offset;
    unsigned int* tickets;       // split-K: one arrival counter per tile (zero between launches)
    float* partials;             // split-K: [tile][split][128][tile_n] fp32
};

// ---- epilogue helpers ---------------------------------------------------------

__device__ __forceinline__ uint32_t pack_bf16x2(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&pair);
}

// acc -> the bf16 value the reference's GEMM returns, widened to fp32.
//   plain:        bf16(acc * s)
//   round_scale:  bf16(bf16(acc) * s) with s already rounded to bf16 (nvfp4.py:120)
__device__ __forceinline__ float gemm_value(uint32_t acc_bits, float scale, bool round_scale) {
    float acc = __uint_as_float(acc_bits);
    if (round_scale) acc = round_to_bf16(acc);
    return round_to_bf16(__fmul_rn(acc, scale));
}

__device__ __forceinline__ void store_u4(void* pointer, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    *reinterpret_cast<uint4*>(pointer) = make_uint4(a, b, c, d);
}

// bf16 pair from two floats in one conversion: low half = `low`, high half = `high`.
__device__ __forceinline__ uint32_t cvt_bf16x2(float high, float low) {
    uint32_t packed;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(high), "f"(low));
    return packed;
}

// GELU of one bf16 bit pattern (16 bits), as bf16 bits.  Magnitude codes [lo, lo + span) come from the
// shared-memory copy of the table ([positive | negative] halves).  Below lo the table equals bf16(x/2);
// from lo + span up to the largest finite value it equals x (positive) or -0 (negative): the host verified
// both against the table before choosing the range.  Subnormals, infinities, NaNs (and every value when
// no range was supplied, span == 0) read the full table in global memory.
__device__ __forceinline__ uint32_t gelu_lookup_general(uint32_t code, const KernelArgs& args, uint32_t compact_table,
                                                        uint32_t lo, uint32_t span) {
    const uint32_t magnitude = code & 0x7fffu;
    const uint32_t offset = magnitude - lo;
    const uint32_t negative = code >> 15;
    if (offset < span) {
        uint32_t value;
        asm("ld.shared.u16 %0, [%1];" : "=r"(value) : "r"(compact_table + 2u * (offset + negative * span)));
        return value;
    }
    if (span != 0u && magnitude >= 0x80u && magnitude < 0x7f80u) {
        const float x = __uint_as_float(code << 16);
        return magnitude < lo ? uint32_t(bf16_bits(__fmul_rn(0.5f, x))) : (negative ? 0x8000u : code);
    }
    return uint32_t(__ldg(args.gelu_table + code));
}

// Fills the shared-memory copy of the GELU table ([positive | negative] halves of magnitude codes [lo, hi)) with `threads`
// threads, this one being number `thread`.  Eight loads are issued before the first store: one load per store would
// pay the L2 latency once per entry (the stores are volatile, nothing moves across them).
__device__ __forceinline__ void fill_compact_gelu(const KernelArgs& args, uint32_t compact_table, int thread, int threads) {
    const int span = args.gelu_hi - args.gelu_lo, total = 2 * span;
    for (int first = thread; first < total; first += 8 * threads) {
        uint16_t value[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = first + j * threads;
            value[j] = 0;
            if (i < total) value[j] = __ldg(args.gelu_table + (i < span ? args.gelu_lo + i : 0x8000 + args.gelu_lo + (i - span)));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = first + j * threads;
            if (i < total) asm volatile("st.shared.u16 [%0], %1;" ::"r"(compact_table + 2u * uint32_t(i)), "h"(value[j]) : "memory");
        }
    }
}

// The sixteen gates of one unit as eight bf16x2 words -> their GELUs as eight bf16x2 words.  One test per
// unit (two adds per word: a magnitude m is >= lo iff m + (0x8000 - lo) carries into bit 15, and < hi iff
// m + (0x8000 - hi) does not) picks between straight-line shared-memory lookups and the general path.
__device__ __forceinline__ void gelu_lookup_unit(const uint32_t (&gate)[8], uint32_t (&gelu)[8], const KernelArgs& args,
                                                 uint32_t compact_table, uint32_t lo, uint32_t span) {
    const uint32_t above_lo = (0x8000u - lo) * 0x10001u, above_hi = (0x8000u - (lo + span)) * 0x10001u;
    uint32_t reach_lo = 0xffffffffu, reach_hi = 0u;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        const uint32_t magnitudes = gate[p] & 0x7fff7fffu;
        reach_lo &= magnitudes + above_lo;
        reach_hi |= magnitudes + above_hi;
    }
    if (span != 0u && ((~reach_lo | reach_hi) & 0x80008000u) == 0u) {
        // address of code c: table + 2*(c - lo) for positive c, table + 2*(c - 0x8000 - lo + span) for negative
        const uint32_t origin = compact_table - 2u * lo;
        const uint32_t fold = 0x10000u - 2u * span;
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            const uint32_t first = gate[p] & 0xffffu, second = gate[p] >> 16;
            uint32_t low, high;
            asm("ld.shared.u16 %0, [%1];" : "=r"(low) : "r"(origin + 2u * first - (first >> 15) * fold));
            asm("ld.shared.u16 %0, [%1];" : "=r"(high) : "r"(origin + 2u * second - (second >> 15) * fold));
            gelu[p] = low | (high << 16);
        }
    } else {
#pragma unroll
        for (int p = 0; p < 8; ++p)
            gelu[p] = gelu_lookup_general(gate[p] & 0xffffu, args, compact_table, lo, span) |
                      (gelu_lookup_general(gate[p] >> 16, args, compact_table, lo, span) << 16);
    }
}

// 32 accumulator columns of one token -> 32 bf16 outputs (64 contiguous bytes), in two steps so that a schedule may
// free the accumulator between them: one packed multiply and one two-value conversion per pair, then bias / table /
// residual and 32-byte stores where the row allows them.
// EPI_GELU_*: the bf16 result goes through the GELU table and is stored as bf16 or, divided by *out_scale,
// as e4m3 (32 contiguous bytes) -- SigLIP's fc1 (bias + tanh GELU + the encoder of fc2's input in one launch).
//
// 32 accumulator columns -> the GEMM's bf16 result as 16 bf16x2 words (scales applied, nothing else).
__device__ __forceinline__ void linear_scale_chunk(const uint32_t (&acc)[32], float scale, bool round_scale, uint32_t (&y)[16]) {
    const float2 scale2 = make_float2(scale, scale);
#pragma unroll
    for (int p = 0; p < 16; ++p) {
        float2 value = make_float2(__uint_as_float(acc[2 * p]), __uint_as_float(acc[2 * p + 1]));
        if (round_scale) value = bf16x2_to_float2(float2_to_bf16x2(value));     // nvfp4.py:120: the GEMM's own bf16 output
        y[p] = float2_to_bf16x2(__fmul2_rn(value, scale2));
    }
}

// The rest of the plain / GELU epilogue on those words: bias, table, residual, stores.
template <int EPI>
__device__ __forceinline__ void epilogue_linear_words(uint32_t (&y)[16], const KernelArgs& args, int token, int feature0,
                                                      uint32_t compact_table, const ExactDivider& out_scale, float out_scale_rcp,
                                                      bool true_div) {
    if (args.bias != nullptr) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            if (feature0 + 8 * v < args.features) {
                const uint4 packed = __ldg(reinterpret_cast<const uint4*>(args.bias + feature0 + 8 * v));
                const uint32_t b[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    y[4 * v + i] = float2_to_bf16x2(__fadd2_rn(bf16x2_to_float2(y[4 * v + i]), bf16x2_to_float2(b[i])));
            }
        }
    }
    if (EPI != EPI_LINEAR) {
        const uint32_t lo = uint32_t(args.gelu_lo), span = uint32_t(args.gelu_hi - args.gelu_lo);
        uint32_t in[8], out[8];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int i = 0; i < 8; ++i) in[i] = y[8 * half + i];
            gelu_lookup_unit(in, out, args, compact_table, lo, span);
#pragma unroll
            for (int i = 0; i < 8; ++i) y[8 * half + i] = out[i];
        }
    }
    if (token >= args.tokens) return;
    const int64_t row = int64_t(token) * args.features;
    if (EPI == EPI_GELU_FP8) {
        uint32_t codes[8];
        if (true_div) {
            const float bound = __fmul_rn(1024.0f, out_scale.divisor);
            uint32_t in[8], part[4];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
#pragma unroll
                for (int i = 0; i < 8; ++i) in[i] = y[8 * half + i];
                encode_fp8_words<true, 8>(in, part, out_scale, bound);
#pragma unroll
                for (int i = 0; i < 4; ++i) codes[4 * half + i] = part[i];
            }
        } else {
            const float2 rcp2 = make_float2(out_scale_rcp, out_scale_rcp);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t low = __nv_cvt_float2_to_fp8x2(__fmul2_rn(bf16x2_to_float2(y[2 * i]), rcp2), __NV_SATFINITE, __NV_E4M3);
                const uint32_t high = __nv_cvt_float2_to_fp8x2(__fmul2_rn(bf16x2_to_float2(y[2 * i + 1]), rcp2), __NV_SATFINITE, __NV_E4M3);
                codes[i] = low | (high << 16);
            }
        }
        uint8_t* out8 = static_cast<uint8_t*>(args.out) + row + feature0;
        if (feature0 + 32 <= args.features && aligned32(out8)) {
            st_u8(out8, codes);
        } else {
#pragma unroll
            for (int v = 0; v < 4; ++v)        // 8 features = 8 bytes per step
                if (feature0 + 8 * v < args.features) *reinterpret_cast<uint2*>(out8 + 8 * v) = make_uint2(codes[2 * v], codes[2 * v + 1]);
        }
        return;
    }
    if (args.residual != nullptr) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            if (feature0 + 8 * v < args.features) {
                const uint4 packed = ld_nc_u4(reinterpret_cast<const uint4*>(args.residual + row + feature0 + 8 * v));
                const uint32_t r[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    y[4 * v + i] = float2_to_bf16x2(__fadd2_rn(bf16x2_to_float2(y[4 * v + i]), bf16x2_to_float2(r[i])));
            }
        }
    }
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(args.out) + row + feature0;
    if (feature0 + 32 <= args.features && aligned32(out)) {
        const uint32_t first[8] = {y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7]};
        const uint32_t second[8] = {y[8], y[9], y[10], y[11], y[12], y[13], y[14], y[15]};
        st_u8(out, first);
        st_u8(out + 16, second);
        return;
    }
#pragma unroll
    for (int v = 0; v < 4; ++v)
        if (feature0 + 8 * v < args.features) store_u4(out + 8 * v, y[4 * v], y[4 * v + 1], y[4 * v + 2], y[4 * v + 3]);
}

template <int EPI>
__device__ __forceinline__ void epilogue_linear_chunk(const uint32_t (&acc)[32], const KernelArgs& args, float scale,
                                                      bool round_scale, int token, int feature0, uint32_t compact_table,
                                                      const ExactDivider& out_scale, float out_scale_rcp, bool true_div) {
    uint32_t y[16];
    linear_scale_chunk(acc, scale, round_scale, y);
    epilogue_linear_words<EPI>(y, args, token, feature0, compact_table, out_scale, out_scale_rcp, true_div);
}

// One 16-feature unit of a token's row: 16 gate + 16 up accumulator columns -> 16 hidden values
// h = bf16(bf16(gelu(gate)) * up), stored as bf16, e4m3 or NVFP4 (fusion.cu:5-10, 31-107).  For NVFP4
// the unit is exactly one quantisation block of the next layer's input.  Values travel as bf16 pairs:
// the product of two bf16 numbers is exact in fp32, so the packed bf16 multiply rounds once, like the
// reference's float multiply followed by the bf16 store.
// 16 gate + 16 up accumulator columns -> the two GEMMs' bf16 results as 8 + 8 bf16x2 words.
__device__ __forceinline__ void geglu_scale_unit(const uint32_t (&gate_acc)[16], const uint32_t (&up_acc)[16], float scale,
                                                 float scale_up, bool round_scale, uint32_t (&gate)[8], uint32_t (&up)[8]) {
    const float2 scale2 = make_float2(scale, scale), scale_up2 = make_float2(scale_up, scale_up);
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        float2 g = make_float2(__uint_as_float(gate_acc[2 * p]), __uint_as_float(gate_acc[2 * p + 1]));
        float2 u = make_float2(__uint_as_float(up_acc[2 * p]), __uint_as_float(up_acc[2 * p + 1]));
        if (round_scale) {
            g = bf16x2_to_float2(float2_to_bf16x2(g));
            u = bf16x2_to_float2(float2_to_bf16x2(u));
        }
        gate[p] = float2_to_bf16x2(__fmul2_rn(g, scale2));
        up[p] = float2_to_bf16x2(__fmul2_rn(u, scale_up2));
    }
}

// h = bf16(bf16(gelu(gate)) * up) for the 16 features of a unit, as eight bf16x2 words.
__device__ __forceinline__ void geglu_hidden_words(const uint32_t (&gate)[8], const uint32_t (&up)[8], const KernelArgs& args,
                                                   uint32_t compact_table, uint32_t (&h)[8]) {
    uint32_t gelu[8];
    gelu_lookup_unit(gate, gelu, args, compact_table, uint32_t(args.gelu_lo), uint32_t(args.gelu_hi - args.gelu_lo));
#pragma unroll
    for (int p = 0; p < 8; ++p) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(h[p]) : "r"(gelu[p]), "r"(up[p]));
}

// One 16-value block of the hidden activation -> its 16 e2m1 codes (two words) and its e4m3 block scale, with the
// arithmetic of quantize.cu:85-104 (`out_scale` divides by the global scale g, `by_global` by 6 g).
__device__ __forceinline__ uint2 hidden_block_nvfp4(const uint32_t (&h)[8], const ExactDivider& out_scale, const ExactDivider& by_global,
                                                    uint8_t& code) {
    const float block_max = abs_max_bf16_words(h);
    code = nvfp4_block_scale<true>(block_max, by_global, 0);
    const ExactDivider denominator(__fmul_rn(out_scale.divisor, e4m3_to_float(code)));
    uint2 words;
    if (denominator.fast && __fmul_rn(block_max, denominator.reciprocal) < 1.0e30f) {
        words.x = nvfp4_encode_words_short<true>(h[0], h[1], h[2], h[3], denominator);
        words.y = nvfp4_encode_words_short<true>(h[4], h[5], h[6], h[7], denominator);
    } else {
        float low[8], high[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            low[2 * i] = bf16_lo(h[i]); low[2 * i + 1] = bf16_hi(h[i]);
            high[2 * i] = bf16_lo(h[4 + i]); high[2 * i + 1] = bf16_hi(h[4 + i]);
        }
        words.x = nvfp4_encode_x8<true>(low, denominator, block_max);
        words.y = nvfp4_encode_x8<true>(high, denominator, block_max);
    }
    return words;
}

// The rest of the gated epilogue on those words: table, product, encoding, stores.
template <int EPI>
__device__ __forceinline__ void epilogue_geglu_words(const uint32_t (&gate)[8], const uint32_t (&up)[8], const KernelArgs& args,
                                                     uint32_t compact_table, const ExactDivider& out_scale,
                                                     const ExactDivider& by_global, float out_scale_rcp, bool true_div,
                                                     int token, int feature0) {
    uint32_t h[8];
    geglu_hidden_words(gate, up, args, compact_table, h);
    if (token >= args.tokens || feature0 >= args.features) return;
    const int64_t element = int64_t(token) * args.features + feature0;
    if (EPI == EPI_GEGLU_BF16) {
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(args.out) + element;
        if (aligned32(out)) {
            st_u8(out, h);
        } else {
            store_u4(out, h[0], h[1], h[2], h[3]);
            store_u4(out + 8, h[4], h[5], h[6], h[7]);
        }
    } else if (EPI == EPI_GEGLU_FP8) {
        uint32_t codes[4];
        if (true_div) {
            encode_fp8_words<true, 8>(h, codes, out_scale, __fmul_rn(1024.0f, out_scale.divisor));
        } else {
            const float2 rcp2 = make_float2(out_scale_rcp, out_scale_rcp);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t low = __nv_cvt_float2_to_fp8x2(__fmul2_rn(bf16x2_to_float2(h[2 * i]), rcp2), __NV_SATFINITE, __NV_E4M3);
                const uint32_t high = __nv_cvt_float2_to_fp8x2(__fmul2_rn(bf16x2_to_float2(h[2 * i + 1]), rcp2), __NV_SATFINITE, __NV_E4M3);
                codes[i] = low | (high << 16);
            }
        }
        store_u4(static_cast<uint8_t*>(args.out) + element, codes[0], codes[1], codes[2], codes[3]);
    } else {
        uint8_t code;
        const uint2 words = hidden_block_nvfp4(h, out_scale, by_global, code);
        *reinterpret_cast<uint2*>(static_cast<uint8_t*>(args.out) + (element >> 1)) = words;
        const int block = feature0 >> 4;
        const int blocks_per_row = args.features >> 4;
        if (args.out_scales != nullptr) args.out_scales[int64_t(token) * blocks_per_row + block] = code;
        if (args.out_blocked != nullptr)
            args.out_blocked[scale_tile_offset(token, block, (blocks_per_row + 3) >> 2)] = code;
    }
}

template <int EPI>
__device__ __forceinline__ void epilogue_geglu_unit(const uint32_t (&gate_acc)[16], const uint32_t (&up_acc)[16],
                                                    const KernelArgs& args, uint32_t compact_table, float scale,
                                                    float scale_up, bool round_scale, const ExactDivider& out_scale,
                                                    const ExactDivider& by_global, float out_scale_rcp, bool true_div,
                                                    int token, int feature0) {
    uint32_t gate[8], up[8];
    geglu_scale_unit(gate_acc, up_acc, scale, scale_up, round_scale, gate, up);
    epilogue_geglu_words<EPI>(gate, up, args, compact_table, out_scale, by_global, out_scale_rcp, true_div, token, feature0);
}

// ---- host helpers shared by the two schedules ---------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_entry();
bool make_operand_map(CUtensorMap* map, const void* pointer, int64_t rows, int64_t row_bytes, int box_rows);
bool make_gated_map(CUtensorMap* map, const void* pointer, int64_t features, int64_t row_bytes, int box_rows);

// Paired schedule (gemm_pair.cu): what it would do with a launch (0 columns = it does not apply), and the launch.
struct PairPlan {
    int columns = 0;             // accumulator columns of a tile; 0 = the paired schedule does not apply
    int splits = 1;              // K ranges computed by different SM pairs
    int resident = 0;            // 1: every pair keeps its 256 token rows on chip and streams weights only
    int64_t workspace_need = 0;  // bytes the splits need
};
PairPlan pair_plan(const b2_linear_desc* d, bool geglu, bool split_allowed);
int run_linear_pair(const b2_linear_desc* d, int epilogue, const PairPlan& plan, cudaStream_t stream);

// Cluster schedule for at most 128 tokens (gemm_skinny.cu): what it would do with a launch (0 splits = it does not apply).
struct SkinnyPlan {
    int splits = 0;              // CTAs of a cluster = K ranges of a feature tile; 0 = the schedule does not apply
    int columns = 0;             // accumulator columns: tokens rounded up to 16
    int atoms = 0;               // K atoms (128 bytes of K) of the longest K range
    int tokens_per_rank = 0;     // tokens whose epilogue a CTA of the cluster runs
    int shared_bytes = 0;
    int gelu_span = 0;           // magnitude codes of the GELU table kept in shared memory
};
SkinnyPlan skinny_plan(const b2_linear_desc* d, bool geglu);
bool skinny_rope_supported(const b2_linear_desc* d);
int run_linear_skinny(const b2_linear_desc* d, int epilogue, const SkinnyPlan& plan, cudaStream_t stream);

}  // namespace b2
