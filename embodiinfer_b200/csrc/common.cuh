// Shared device helpers: vector loads, bf16 unpacking, the two reference quantiser
// arithmetics (spec T = torch route, spec C = CUDA route) and the scale-tile offset.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>

#include "../../include/embodiinfer_b200.h"

namespace b2 {

int sm_count();

// ---- programmatic dependent launch -----------------------------------------------------------------
// Consecutive launches of this library on one stream may overlap head and tail: a kernel calls
// `pdl_launch_dependents()` on entry (the next launch of the stream may then be scheduled as soon as every CTA of
// this one has started) and `pdl_wait()` before it first touches memory that an earlier launch may have written
// (it returns once all earlier launches have completed and their writes are visible).  What runs ahead of the wait
// is each kernel's own set-up: barrier initialisation, tensor-memory allocation, descriptor prefetch, index
// arithmetic.  Both calls are no-ops in a launch made without the attribute, and a launch that follows a kernel
// which never triggers (any other library's) simply starts when that kernel has finished.  The reference uses the
// same mechanism in its norm kernels (embodiinfer/backend/cuda/csrc/pdl.cuh).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Host: the launch attribute is set unless B2_PDL=0 is in the environment.
constexpr bool PDL_DEFAULT = true;
bool pdl_enabled();

template <class... Parameters, class... Arguments>
int launch_kernel(void (*kernel)(Parameters...), dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream,
                  Arguments&&... arguments) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = pdl_enabled() ? 1 : 0;
    const cudaError_t error = cudaLaunchKernelEx(&config, kernel, Parameters(arguments)...);
    return error == cudaSuccess ? int(cudaGetLastError()) : int(error);
}

// ---- loads -----------------------------------------------------------------

__device__ __forceinline__ uint4 ld_nc_u4(const uint4* pointer) {
    uint4 value;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w)
                 : "l"(pointer));
    return value;
}

// 32-byte vector access (sm_100): one full DRAM/L2 sector per lane and instruction.  The address must be
// 32-byte aligned.
__device__ __forceinline__ void ld_nc_u8(const void* pointer, uint32_t (&v)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "l"(pointer));
}

__device__ __forceinline__ void st_u8(void* pointer, const uint32_t (&v)[8]) {
    asm volatile("st.global.v8.u32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(pointer), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}

__device__ __forceinline__ bool aligned32(const void* pointer) { return (reinterpret_cast<uintptr_t>(pointer) & 31u) == 0; }

__device__ __forceinline__ float bf16_lo(uint32_t word) { return __uint_as_float(word << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t word) { return __uint_as_float(word & 0xffff0000u); }

__device__ __forceinline__ void unpack_bf16x8(const uint4& packed, float (&v)[8]) {
    v[0] = bf16_lo(packed.x); v[1] = bf16_hi(packed.x);
    v[2] = bf16_lo(packed.y); v[3] = bf16_hi(packed.y);
    v[4] = bf16_lo(packed.z); v[5] = bf16_hi(packed.z);
    v[6] = bf16_lo(packed.w); v[7] = bf16_hi(packed.w);
}

__device__ __forceinline__ float abs_max_bf16x8(const uint4& packed) {
    float v[8];
    unpack_bf16x8(packed, v);
    float maximum = fabsf(v[0]);
#pragma unroll
    for (int i = 1; i < 8; ++i) maximum = fmaxf(maximum, fabsf(v[i]));
    return maximum;
}

// Two bf16 values in one word <-> two floats (low half first).
__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t word) { return make_float2(bf16_lo(word), bf16_hi(word)); }

__device__ __forceinline__ uint32_t float2_to_bf16x2(float2 value) {
    uint32_t packed;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(value.y), "f"(value.x));
    return packed;
}

// max(|a|, |b|) per 16-bit half, NaN-ignoring like fmaxf.
__device__ __forceinline__ uint32_t abs_max_bf16x2(uint32_t a, uint32_t b) {
    const uint32_t x = a & 0x7fff7fffu, y = b & 0x7fff7fffu;
    uint32_t result;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(result) : "r"(x), "r"(y));
    return result;
}

// Largest magnitude among the 2*WORDS bf16 values of `words`.
template <int WORDS>
__device__ __forceinline__ float abs_max_bf16_words(const uint32_t (&words)[WORDS]) {
    uint32_t m = abs_max_bf16x2(words[0], WORDS > 1 ? words[1] : words[0]);
#pragma unroll
    for (int i = 2; i < WORDS; ++i) m = abs_max_bf16x2(m, words[i]);
    return fmaxf(bf16_lo(m), bf16_hi(m));
}

__device__ __forceinline__ float round_to_bf16(float value) {
    return __bfloat162float(__float2bfloat16_rn(value));
}

__device__ __forceinline__ uint16_t bf16_bits(float value) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(value));
}

// ---- scales ----------------------------------------------------------------

// amax -> per-tensor scale.  `bound` is 448 (FP8) or 448*6 (NVFP4).
//   B2_SCALAR_RCP  multiply by the rounded fp32 reciprocal (ATen on CUDA, quantize.cu:54)
//                  instead of dividing (ATen on CPU).
//   B2_CLAMP_TINY  amax.clamp_min(tiny)/bound (nvfp4.py:38) instead of "1.0 for an all-zero tensor".
__device__ __forceinline__ float scale_from_amax(float amax, float bound, int flags) {
    if (flags & B2_CLAMP_TINY) amax = fmaxf(amax, FLT_MIN);
    else if (!(amax > 0.0f)) return 1.0f;
    return (flags & B2_SCALAR_RCP) ? __fmul_rn(amax, __fdiv_rn(1.0f, bound)) : __fdiv_rn(amax, bound);
}

__device__ __forceinline__ float e4m3_to_float(uint8_t code) {
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(code, __NV_E4M3)));
}

__device__ __forceinline__ float clamp_keep_nan(float value, float bound) {
    return value > bound ? bound : (value < -bound ? -bound : value);
}

// ---- exact division by a repeated divisor --------------------------------------
// The reference divides in fp32 (x / scale, x / (g * s_block)); bit-exact codes need the correctly
// rounded quotient.  For a divisor used many times the quotient is rebuilt from the correctly rounded
// reciprocal y = RN(1/b) with one residual step (Markstein): q = RN(a*y), r = a - b*q (exact in an FMA),
// RN(q + r*y) = RN(a/b).  The step is not guaranteed when b's significand is all ones or when the
// residual can underflow/overflow, so those divisors (and non-finite or huge dividends) take the IEEE
// division instead; a zero product keeps its sign, as a true division would.
struct ExactDivider {
    float divisor, reciprocal;
    bool fast;
    __device__ __forceinline__ explicit ExactDivider(float b) : divisor(b) {
        const uint32_t bits = __float_as_uint(b);
        const uint32_t exponent = (bits >> 23) & 0xffu;
        fast = (bits >> 31) == 0 && exponent >= 67u && exponent <= 187u && (bits & 0x7fffffu) != 0x7fffffu;
        reciprocal = fast ? __frcp_rn(b) : 0.0f;
    }
    // From a precomputed (divisor, reciprocal) pair as the constructor above would leave them: the reciprocal is
    // 0.0 exactly when the divisor is outside the range of the short path.
    __device__ __forceinline__ explicit ExactDivider(float2 entry) : divisor(entry.x), reciprocal(entry.y), fast(entry.y != 0.0f) {}
    __device__ __forceinline__ float2 entry() const { return make_float2(divisor, reciprocal); }
    // The residual step alone, for callers that have already established: `fast`, |a * reciprocal| finite.
    // copysign restores the sign of a zero quotient (and changes nothing else: the divisor is positive).
    __device__ __forceinline__ float unchecked(float a) const {
        const float q = __fmul_rn(a, reciprocal);
        return copysignf(__fmaf_rn(__fmaf_rn(-q, divisor, a), reciprocal, q), a);
    }
    // Two quotients at once on the packed fp32 pipe (same arithmetic per lane as `unchecked`).
    __device__ __forceinline__ float2 unchecked2(float2 a) const {
        const float2 r = make_float2(reciprocal, reciprocal), negative = make_float2(-divisor, -divisor);
        const float2 q = __fmul2_rn(a, r);
        const float2 o = __ffma2_rn(__ffma2_rn(q, negative, a), r, q);
        return make_float2(copysignf(o.x, a.x), copysignf(o.y, a.y));
    }
    __device__ __forceinline__ float operator()(float a) const {
        if (fast && fabsf(a) < 1.0e30f) {
            const float q = __fmul_rn(a, reciprocal);
            if (q == 0.0f) return q;
            return __fmaf_rn(__fmaf_rn(-q, divisor, a), reciprocal, q);
        }
        return __fdiv_rn(a, divisor);
    }
};

// ---- FP8 -------------------------------------------------------------------

// Four values -> four e4m3 bytes (first value in the low byte).
//   spec C: fp32 quotient (quantize.cu:62-64).
//   spec T: quotient rounded to bf16, clamped to +-448 (fp8.py:72).
template <bool SPEC_C>
__device__ __forceinline__ uint32_t encode_fp8x4(float a, float b, float c, float d, const ExactDivider& scale) {
    float q[4];
    if (scale.fast) {
        // |x| >= 1024*scale saturates to +-448 whatever x is: clamping there keeps the product finite
        // without changing a code (NaN fails the comparison and stays NaN).
        const float bound = __fmul_rn(1024.0f, scale.divisor);
        const float in[4] = {a, b, c, d};
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = scale.unchecked(fabsf(in[i]) > bound ? copysignf(bound, in[i]) : in[i]);
    } else {
        q[0] = scale(a); q[1] = scale(b); q[2] = scale(c); q[3] = scale(d);
    }
    if (!SPEC_C) {
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = clamp_keep_nan(round_to_bf16(q[i]), 448.0f);
    }
    const uint32_t low = __nv_cvt_float2_to_fp8x2(make_float2(q[0], q[1]), __NV_SATFINITE, __NV_E4M3);
    const uint32_t high = __nv_cvt_float2_to_fp8x2(make_float2(q[2], q[3]), __NV_SATFINITE, __NV_E4M3);
    return low | (high << 16);
}

// Two bf16 values (one word) -> two e4m3 bytes on the divider's short path (caller checked: `scale.fast`
// and |x| <= 1024*scale for both, or x is NaN).  Dropping the reference's clamp to +-448 of spec T changes
// nothing: the saturating conversion maps every finite value beyond 448 and both infinities to +-448 too.
template <bool SPEC_C>
__device__ __forceinline__ uint32_t encode_fp8x2_short(uint32_t word, const ExactDivider& scale) {
    float2 q = scale.unchecked2(bf16x2_to_float2(word));
    if (!SPEC_C) q = bf16x2_to_float2(float2_to_bf16x2(q));
    return uint32_t(__nv_cvt_float2_to_fp8x2(q, __NV_SATFINITE, __NV_E4M3));
}

// 2*WORDS bf16 values -> e4m3 bytes, WORDS/2 output words.  One magnitude test per vector picks the short
// path; vectors holding a value beyond 1024*scale (which saturates whatever it is) take the general one.
template <bool SPEC_C, int WORDS>
__device__ __forceinline__ void encode_fp8_words(const uint32_t (&in)[WORDS], uint32_t (&out)[WORDS / 2],
                                                 const ExactDivider& scale, float short_path_bound) {
    if (scale.fast && abs_max_bf16_words(in) <= short_path_bound) {
#pragma unroll
        for (int i = 0; i < WORDS / 2; ++i)
            out[i] = encode_fp8x2_short<SPEC_C>(in[2 * i], scale) | (encode_fp8x2_short<SPEC_C>(in[2 * i + 1], scale) << 16);
    } else {
#pragma unroll
        for (int i = 0; i < WORDS / 2; ++i)
            out[i] = encode_fp8x4<SPEC_C>(bf16_lo(in[2 * i]), bf16_hi(in[2 * i]), bf16_lo(in[2 * i + 1]), bf16_hi(in[2 * i + 1]), scale);
    }
}

// Same, but the caller supplies already-divided values (used by fused epilogues).
__device__ __forceinline__ uint32_t pack_fp8x4(float a, float b, float c, float d) {
    const uint32_t low = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t high = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return low | (high << 16);
}

// ---- NVFP4 -----------------------------------------------------------------

// e4m3 scale of one 16-element block.
//   spec C: e4m3(min(448, max/(6*g)))                      quantize.cu:85-86
//   spec T: e4m3(clamp(max/6/g, tiny, 448))                nvfp4.py:40
//   `by_global` divides by 6*g (spec C) or by g (spec T).
template <bool SPEC_C>
__device__ __forceinline__ uint8_t nvfp4_block_scale(float block_max, const ExactDivider& by_global, int flags) {
    float raw;
    if (SPEC_C) {
        raw = fminf(448.0f, by_global(block_max));
    } else {
        const float sixth = (flags & B2_SCALAR_RCP) ? __fmul_rn(block_max, __fdiv_rn(1.0f, 6.0f))
                                                    : __fdiv_rn(block_max, 6.0f);
        raw = by_global(sixth);
        raw = raw < FLT_MIN ? FLT_MIN : (raw > 448.0f ? 448.0f : raw);
    }
    return uint8_t(__nv_cvt_float_to_fp8(raw, __NV_SATFINITE, __NV_E4M3));
}

// Torch-route e2m1 code: bucketize(|v|) with ties toward zero, NaN -> 7, sign = v < 0 (nvfp4.py:42-44).
__device__ __forceinline__ uint32_t e2m1_bucketize(float value) {
    const float a = fabsf(value);
    uint32_t magnitude = uint32_t(a > 0.25f) + uint32_t(a > 0.75f) + uint32_t(a > 1.25f) + uint32_t(a > 1.75f) +
                         uint32_t(a > 2.5f) + uint32_t(a > 3.5f) + uint32_t(a > 5.0f);
    if (a != a) magnitude = 7u;
    return magnitude | (value < 0.0f ? 8u : 0u);
}

// Same code as e2m1_bucketize without the seven comparisons.  Below 2 the e2m1 grid is uniform (step 0.5)
// and "ties toward zero" is ceil(2a - 0.5), exact in fp32 for a >= 0.25 and of the right sign below; from
// 2 up the code is the float's exponent and top mantissa bit after a round-half-down of the bits beneath
// (adding 0x1fffff, one less than half a step, so exact ties do not carry).  Values beyond 6, infinities
// and NaN (whose bit pattern exceeds every number's) end at 7.
__device__ __forceinline__ uint32_t e2m1_bucketize_fast(float value) {
    const float a = fabsf(value);
    const uint32_t low = uint32_t(__float2int_ru(__fmaf_rn(a, 2.0f, -0.5f)));
    const uint32_t high = ((__float_as_uint(a) + 0x1fffffu) >> 22) - 252u;
    const uint32_t magnitude = min(a < 2.0f ? low : high, 7u);
    return magnitude | (value < 0.0f ? 8u : 0u);
}

// Eight bf16 values in four words -> eight nibbles, on the divider's short path (caller checked
// `denominator.fast` and that block_max / denominator is finite).
template <bool SPEC_C>
__device__ __forceinline__ uint32_t nvfp4_encode_words_short(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3,
                                                            const ExactDivider& denominator) {
    const uint32_t words[4] = {w0, w1, w2, w3};
    uint32_t codes = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 q = denominator.unchecked2(bf16x2_to_float2(words[i]));
        uint32_t byte;
        if (SPEC_C) byte = uint32_t(__nv_cvt_float2_to_fp4x2(q, __NV_E2M1, cudaRoundNearest)) & 0xffu;
        else byte = e2m1_bucketize_fast(q.x) | (e2m1_bucketize_fast(q.y) << 4);
        codes |= byte << (8 * i);
    }
    return codes;
}

// Eight values of one half-block -> eight nibbles, first value in the lowest nibble.
//   spec C: x/den (0 when den == 0), hardware round-to-nearest-even e2m1   quantize.cu:91-95
//   spec T: clamp(x/den, +-6) then bucketize                               nvfp4.py:41-44
//   `block_max` is the largest magnitude of the block the eight values belong to; when the divisor is
//   in the divider's safe range and block_max/den is finite, all eight quotients take the short path.
template <bool SPEC_C>
__device__ __forceinline__ uint32_t nvfp4_encode_x8(const float (&v)[8], const ExactDivider& denominator, float block_max) {
    uint32_t word = 0;
    const bool short_path = denominator.fast && __fmul_rn(block_max, denominator.reciprocal) < 1.0e30f;
    if (SPEC_C && short_path) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t byte = __nv_cvt_float2_to_fp4x2(
                make_float2(denominator.unchecked(v[2 * i]), denominator.unchecked(v[2 * i + 1])), __NV_E2M1, cudaRoundNearest);
            word |= (byte & 0xffu) << (8 * i);
        }
    } else if (SPEC_C) {
        const bool positive = denominator.divisor > 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float first = positive ? denominator(v[2 * i]) : 0.0f;
            const float second = positive ? denominator(v[2 * i + 1]) : 0.0f;
            const uint32_t byte = __nv_cvt_float2_to_fp4x2(make_float2(first, second), __NV_E2M1, cudaRoundNearest);
            word |= (byte & 0xffu) << (8 * i);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float normalized = clamp_keep_nan(short_path ? denominator.unchecked(v[i]) : denominator(v[i]), 6.0f);
            word |= e2m1_bucketize(normalized) << (4 * i);
        }
    }
    return word;
}

// The dividers by global * e4m3(code) for the 127 non-negative finite e4m3 codes (code 127 is NaN: its entry takes
// the general path like the constructor would).  Called by the first 128 threads of a block; the caller
// synchronises the block afterwards.
__device__ __forceinline__ void fill_denominator_table(float2* table, float global) {
    if (threadIdx.x < 128) table[threadIdx.x] = ExactDivider(__fmul_rn(global, e4m3_to_float(uint8_t(threadIdx.x)))).entry();
}

// One 16-element block held as eight bf16x2 words -> 16 nibbles (two words) and the block's e4m3 scale.
// `denominators`: nullptr, or this launch's table (shared memory, 128 entries, see `fill_denominator_table`) of the
// dividers by global * e4m3(code): the block's divider is then two loads instead of a conversion, a product and a
// reciprocal.
template <bool SPEC_C>
__device__ __forceinline__ uint2 nvfp4_encode_block(const uint32_t (&w)[8], float global, const ExactDivider& by_global,
                                                    int flags, uint8_t& scale_code, const float2* denominators = nullptr) {
    const float maximum = abs_max_bf16_words(w);
    scale_code = nvfp4_block_scale<SPEC_C>(maximum, by_global, flags);
    const ExactDivider denominator = denominators != nullptr ? ExactDivider(denominators[scale_code & 127u])
                                                            : ExactDivider(__fmul_rn(global, e4m3_to_float(scale_code)));
    uint2 codes;
    if (denominator.fast && __fmul_rn(maximum, denominator.reciprocal) < 1.0e30f) {
        codes.x = nvfp4_encode_words_short<SPEC_C>(w[0], w[1], w[2], w[3], denominator);
        codes.y = nvfp4_encode_words_short<SPEC_C>(w[4], w[5], w[6], w[7], denominator);
    } else {
        float low[8], high[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            low[2 * i] = bf16_lo(w[i]); low[2 * i + 1] = bf16_hi(w[i]);
            high[2 * i] = bf16_lo(w[4 + i]); high[2 * i + 1] = bf16_hi(w[4 + i]);
        }
        codes.x = nvfp4_encode_x8<SPEC_C>(low, denominator, maximum);
        codes.y = nvfp4_encode_x8<SPEC_C>(high, denominator, maximum);
    }
    return codes;
}

// Byte offset of the scale of (row, 16-element block) in the 128x4-tile layout
// (nvfp4.py:14-25, quantize.cu:97-101).  One tile is 512 bytes: 32 rows x 16 bytes,
// each 16-byte row holding [row, row+32, row+64, row+96] x 4 blocks.
__host__ __device__ __forceinline__ int64_t scale_tile_offset(int row, int block, int column_tiles) {
    return (int64_t(row >> 7) * column_tiles + (block >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 +
           (block & 3);
}

// ---- launchers shared between translation units ---------------------------------

int launch_tensor_scale(const void* input, int64_t count, float bound, int flags, void* scratch, void* scale,
                        cudaStream_t stream);
int launch_fp8_encode(const void* input, void* output, const void* scale, int64_t count, int flags,
                      cudaStream_t stream);
int launch_nvfp4_encode(const void* input, void* output, void* scales, void* blocked, const void* global, int rows,
                        int columns, int flags, cudaStream_t stream);

}  // namespace b2
