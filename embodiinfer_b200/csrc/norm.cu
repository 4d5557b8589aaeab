// RMSNorm producer in front of the quantised projections: residual update (two bf16 rounding points),
// mean of squares, affine or adaptive modulation, one rounding to bf16, then the activation encoder
// (e4m3 at a static scale, NVFP4 spec C, or plain bf16) -- one launch, one read of the row.
//
// Arithmetic follows the reference kernels step by step (embodiinfer/backend/cuda/csrc/norm_quant.cu:
// norm_fp8_reduce 114-171, norm_fp4_reduce 173-251, the 8-columns-per-lane variants 254-369 and 381-514,
// and the given-mean kernels 5-89): every product and sum is a separate fp32 operation (no fused
// multiply-add), and the sum of squares is taken in the order of the kernel the reference would launch for
// the width, because fp32 addition is not associative:
//   * columns 1024 and 2048 (dispatch at norm_quant.cu:523-546): lane t adds its columns 8t..8t+7 in
//     order, a 32-lane butterfly (xor 16, 8, 4, 2, 1) follows, then a butterfly over the warp totals;
//   * other widths: lane t of 256 adds columns t, t+256, ... in order, then a halving tree over 256 partials.
// Here each thread always owns 8 consecutive columns per vector (16-byte loads and stores).  Widths 1024 and
// 2048 run one warp per row with the row in registers; for the strided order a block of 256 threads stages
// the rounded row in shared memory and re-reads it in the reference's order.
//
// HBM-bound: per row 2*columns bytes in (4*columns with an update), 2*columns out for the residual, and
// columns (e4m3), 9/16*columns (NVFP4) or 2*columns (bf16) out for the result.
#include "common.cuh"

namespace b2 {

constexpr int NORM_THREADS = 256;       // strided order: the reference's reduction width
constexpr int NORM_MAX_VECTORS = 4;     // 8-column vectors per thread in the strided order (8192 columns)

struct NormArgs {
    const __nv_bfloat16* input;
    const __nv_bfloat16* update;
    const __nv_bfloat16* update_gate;
    const float* scale;
    const float* modulation;
    const float* mean;
    const float* global;
    __nv_bfloat16* residual;
    uint8_t* output;
    uint8_t* scales;
    uint8_t* blocked;
    __nv_bfloat16* gate;
    float* inverse;
    int rows, columns, tokens;
    bool evict_last;
};

__device__ __forceinline__ void store_residual_vector(__nv_bfloat16* destination, const uint4& value, bool evict_last) {
    if (!evict_last) {
        *reinterpret_cast<uint4*>(destination) = value;
        return;
    }
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(destination), "r"(value.x),
                 "r"(value.y), "r"(value.z), "r"(value.w), "l"(policy)
                 : "memory");
}


__device__ __forceinline__ uint4 pack_bf16x8(const float (&v)[8]) {
    uint4 packed;
    packed.x = float2_to_bf16x2(make_float2(v[0], v[1]));
    packed.y = float2_to_bf16x2(make_float2(v[2], v[3]));
    packed.z = float2_to_bf16x2(make_float2(v[4], v[5]));
    packed.w = float2_to_bf16x2(make_float2(v[6], v[7]));
    return packed;
}

// r = bf16(input + (gate ? bf16(update * gate) : update)) for 8 columns, both operands already loaded.
__device__ __forceinline__ uint4 apply_update(const NormArgs& a, const uint4& input, const uint4& update, int64_t gate_base,
                                              int column) {
    float v[8], delta[8];
    unpack_bf16x8(input, v);
    unpack_bf16x8(update, delta);
    if (a.update_gate != nullptr) {
        float factor[8];
        unpack_bf16x8(ld_nc_u4(reinterpret_cast<const uint4*>(a.update_gate + gate_base + column)), factor);
#pragma unroll
        for (int i = 0; i < 8; ++i) delta[i] = round_to_bf16(__fmul_rn(delta[i], factor[i]));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fadd_rn(v[i], delta[i]);
    return pack_bf16x8(v);
}

// Packed fp32 product and sum (`mul.rn.f32x2`, `add.rn.f32x2`).  Used where no product feeds a sum directly.
__device__ __forceinline__ float2 mul2_rn(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float2 add2_rn(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

// y = bf16((r * inverse) * (1 + scale))  or  bf16((r * inverse) * (1 + m_scale) + m_shift) for the 8 packed
// values of `r`, returned packed.  Two columns per instruction on the packed fp32 pipe (`mul.rn.f32x2`,
// `add.rn.f32x2`: each lane rounds like the scalar operation).
__device__ __forceinline__ uint4 affine_vector(const NormArgs& a, int64_t modulation_base, int column, float inverse,
                                               const uint4& r) {
    const float* multiplier = a.modulation != nullptr ? a.modulation + modulation_base + column : a.scale + column;
    const float4 m0 = *reinterpret_cast<const float4*>(multiplier), m1 = *reinterpret_cast<const float4*>(multiplier + 4);
    const float2 m[4] = {make_float2(m0.x, m0.y), make_float2(m0.z, m0.w), make_float2(m1.x, m1.y), make_float2(m1.z, m1.w)};
    const float2 inverse2 = make_float2(inverse, inverse), one = make_float2(1.0f, 1.0f);
    const uint32_t words[4] = {r.x, r.y, r.z, r.w};
    uint32_t y[4];
    if (a.modulation != nullptr) {
        const float* shift = a.modulation + modulation_base + a.columns + column;
        const float4 s0 = *reinterpret_cast<const float4*>(shift), s1 = *reinterpret_cast<const float4*>(shift + 4);
        const float2 s[4] = {make_float2(s0.x, s0.y), make_float2(s0.z, s0.w), make_float2(s1.x, s1.y), make_float2(s1.z, s1.w)};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // the shift is added with the scalar intrinsic: a packed product followed by a packed sum came back
            // fused (one rounding instead of two: 1 bf16 result in 30,000 differs), explicit `.rn` or not
            const float2 scaled = mul2_rn(mul2_rn(bf16x2_to_float2(words[i]), inverse2), add2_rn(one, m[i]));
            y[i] = float2_to_bf16x2(make_float2(__fadd_rn(scaled.x, s[i].x), __fadd_rn(scaled.y, s[i].y)));
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            y[i] = float2_to_bf16x2(mul2_rn(mul2_rn(bf16x2_to_float2(words[i]), inverse2), add2_rn(one, m[i])));
    }
    return make_uint4(y[0], y[1], y[2], y[3]);
}

__device__ __forceinline__ void write_gate_vector(const NormArgs& a, int64_t modulation_base, int64_t gate_base, int column) {
    const float* source = a.modulation + modulation_base + 2 * a.columns + column;
    const float4 g0 = *reinterpret_cast<const float4*>(source), g1 = *reinterpret_cast<const float4*>(source + 4);
    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    *reinterpret_cast<uint4*>(a.gate + gate_base + column) = pack_bf16x8(g);
}

__device__ __forceinline__ float rounded_reciprocal(float value) { return __fdiv_rn(1.0f, value); }
__device__ __forceinline__ float rounded_product(float a, float b) { return __fmul_rn(a, b); }

// The encoder behind the norm; the scale arithmetic that does not depend on the data is done once per thread.
template <int BITS>
struct Encoder {
    float global, reciprocal;
    bool divide;
    ExactDivider by_global;
    const float2* denominators = nullptr;    // NVFP4: the block's table of dividers by global * e4m3(code), in shared memory
    __device__ __forceinline__ Encoder(const NormArgs& a, const float2* table)
        : global(BITS == 16 ? 1.0f : *a.global), reciprocal(rounded_reciprocal(global)), divide(a.mean != nullptr),
          by_global(rounded_product(6.0f, global)), denominators(BITS == 4 ? table : nullptr) {}
    // Scale (and, for e4m3, the multiplier) given by value, as the layer-norm entry points of the reference take them.
    __device__ __forceinline__ Encoder(float global_scale, float multiplier, const float2* table)
        : global(global_scale), reciprocal(multiplier), divide(false), by_global(rounded_product(6.0f, global_scale)),
          denominators(BITS == 4 ? table : nullptr) {}

    // `y`: eight bf16 values, packed.  Every lane of the warp calls this (the NVFP4 block maximum is exchanged
    // with the neighbouring lane); lanes without a vector pass valid = false.
    template <class Args>
    __device__ __forceinline__ void store(const Args& a, int row, int64_t base, int column, bool valid, const uint4& y) const {
        if (BITS == 16) {
            if (valid) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.output) + base + column) = y;
        } else if (BITS == 8) {
            if (!valid) return;
            const uint32_t words[4] = {y.x, y.y, y.z, y.w};
            uint32_t codes[4];
            if (divide) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 v = bf16x2_to_float2(words[i]);
                    codes[i] = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(v.x, global), __fdiv_rn(v.y, global)), __NV_SATFINITE, __NV_E4M3);
                }
            } else {
                const float2 factor = make_float2(reciprocal, reciprocal);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    codes[i] = __nv_cvt_float2_to_fp8x2(__fmul2_rn(bf16x2_to_float2(words[i]), factor), __NV_SATFINITE, __NV_E4M3);
            }
            uint2 packed;
            packed.x = codes[0] | (codes[1] << 16);
            packed.y = codes[2] | (codes[3] << 16);
            *reinterpret_cast<uint2*>(a.output + base + column) = packed;
        } else {
            // A 16-element block is shared by an even lane and its odd neighbour.
            const uint32_t words[4] = {valid ? y.x : 0u, valid ? y.y : 0u, valid ? y.z : 0u, valid ? y.w : 0u};
            float maximum = abs_max_bf16_words(words);
            maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, 1));
            if (!valid) return;
            const uint8_t code = nvfp4_block_scale<true>(maximum, by_global, 0);
            const ExactDivider denominator = denominators != nullptr ? ExactDivider(denominators[code & 127u])
                                                                    : ExactDivider(__fmul_rn(global, e4m3_to_float(code)));
            uint32_t codes;
            if (denominator.fast && __fmul_rn(maximum, denominator.reciprocal) < 1.0e30f) {
                codes = nvfp4_encode_words_short<true>(words[0], words[1], words[2], words[3], denominator);
            } else {
                float values[8];
                unpack_bf16x8(y, values);
                codes = nvfp4_encode_x8<true>(values, denominator, maximum);
            }
            *reinterpret_cast<uint32_t*>(a.output + (base + column) / 2) = codes;
            if (((column >> 3) & 1) == 0) {
                const int block = column >> 4, blocks_per_row = a.columns >> 4;
                a.blocked[scale_tile_offset(row, block, (blocks_per_row + 3) >> 2)] = code;
                if (a.scales != nullptr) a.scales[int64_t(row) * blocks_per_row + block] = code;
            }
        }
    }
};

__device__ __forceinline__ float sum_squares_of_vector(const uint4& packed) {
    float v[8];
    unpack_bf16x8(packed, v);
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) sum = __fadd_rn(sum, __fmul_rn(v[j], v[j]));
    return sum;
}

__device__ __forceinline__ float warp_butterfly_sum(float sum) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, offset));
    return sum;
}

// The reference's butterfly over its 8 warp totals (xor 4, 2, 1), absent warps counting 0.0.
__device__ __forceinline__ float combine_warp_totals(const float (&t)[8]) {
    return __fadd_rn(__fadd_rn(__fadd_rn(t[0], t[4]), __fadd_rn(t[2], t[6])),
                     __fadd_rn(__fadd_rn(t[1], t[5]), __fadd_rn(t[3], t[7])));
}

// Sum of squares in the order of the 256-lane strided reference kernels: `row` is the bf16-rounded row in
// shared memory, `partials` 256 floats.
__device__ __forceinline__ float sum_squares_strided(const __nv_bfloat16* row, int columns, float* partials) {
    float sum = 0.0f;
    for (int column = threadIdx.x; column < columns; column += NORM_THREADS) {
        const float value = __bfloat162float(row[column]);
        sum = __fadd_rn(sum, __fmul_rn(value, value));
    }
    partials[threadIdx.x] = sum;
    __syncthreads();
#pragma unroll
    for (int stride = NORM_THREADS / 2; stride >= 32; stride >>= 1) {
        if (threadIdx.x < stride) partials[threadIdx.x] = __fadd_rn(partials[threadIdx.x], partials[threadIdx.x + stride]);
        __syncthreads();
    }
    // Strides 16..1 pair lane t with lane t+stride of the first warp: the same additions as the tree in
    // shared memory, taken with shuffles (lanes at or beyond `stride` compute values nobody reads).
    float value = partials[threadIdx.x & 31];
#pragma unroll
    for (int stride = 16; stride > 0; stride >>= 1) value = __fadd_rn(value, __shfl_down_sync(0xffffffffu, value, stride));
    return __shfl_sync(0xffffffffu, value, 0);
}

enum NormOrder { ORDER_LANES8 = 0, ORDER_STRIDED = 1 };

// One block per row.  ORDER_LANES8 (widths 1024 / 2048, few rows): columns/8 threads, one vector each, the
// reference's block shape.  ORDER_STRIDED (other widths): 256 threads, up to NORM_MAX_VECTORS vectors each.
template <int BITS, int ORDER>
__global__ void __launch_bounds__(NORM_THREADS)
norm_encode_block_kernel(const NormArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float2 denominator_table[BITS == 4 ? 128 : 1];
    if (BITS == 4) {
        fill_denominator_table(denominator_table, *a.global);
        __syncthreads();
    }
    constexpr int VECTORS = ORDER == ORDER_LANES8 ? 1 : NORM_MAX_VECTORS;
    extern __shared__ __align__(16) uint8_t norm_shared[];
    __shared__ float partials[ORDER == ORDER_LANES8 ? 8 : NORM_THREADS];
    const int row = blockIdx.x;
    const int batch = row / a.tokens;
    const int64_t base = int64_t(row) * a.columns, gate_base = int64_t(batch) * a.columns;
    const int64_t modulation_base = int64_t(batch) * 3 * a.columns;
    uint4 packed[VECTORS], update[VECTORS];
    bool valid[VECTORS];
#pragma unroll
    for (int i = 0; i < VECTORS; ++i) {
        const int column = (threadIdx.x + i * NORM_THREADS) * 8;
        valid[i] = column < a.columns;
        if (valid[i]) packed[i] = ld_nc_u4(reinterpret_cast<const uint4*>(a.input + base + column));
        if (valid[i] && a.update != nullptr) update[i] = ld_nc_u4(reinterpret_cast<const uint4*>(a.update + base + column));
    }
#pragma unroll
    for (int i = 0; i < VECTORS; ++i) {
        if (!valid[i]) continue;
        const int column = (threadIdx.x + i * NORM_THREADS) * 8;
        if (a.update != nullptr) packed[i] = apply_update(a, packed[i], update[i], gate_base, column);
        if (a.residual != nullptr) store_residual_vector(a.residual + base + column, packed[i], a.evict_last);
    }
    float inverse;
    if (a.mean != nullptr) {
        inverse = rsqrtf(__fadd_rn(a.mean[row], 1.0e-6f));
    } else {
        float total;
        if (ORDER == ORDER_LANES8) {
            const float sum = warp_butterfly_sum(sum_squares_of_vector(packed[0]));
            if ((threadIdx.x & 31) == 0) partials[threadIdx.x >> 5] = sum;
            __syncthreads();
            float totals[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) totals[i] = i < int(blockDim.x >> 5) ? partials[i] : 0.0f;
            total = combine_warp_totals(totals);
        } else {
            __nv_bfloat16* staged = reinterpret_cast<__nv_bfloat16*>(norm_shared);
#pragma unroll
            for (int i = 0; i < VECTORS; ++i)
                if (valid[i]) *reinterpret_cast<uint4*>(staged + (threadIdx.x + i * NORM_THREADS) * 8) = packed[i];
            __syncthreads();
            total = sum_squares_strided(staged, a.columns, partials);
        }
        inverse = rsqrtf(__fadd_rn(__fmul_rn(total, __fdiv_rn(1.0f, float(a.columns))), 1.0e-6f));
    }
    if (a.inverse != nullptr && threadIdx.x == 0) a.inverse[row] = inverse;
    const Encoder<BITS> encoder(a, denominator_table);
    const bool write_gate = a.gate != nullptr && row == batch * a.tokens;
#pragma unroll
    for (int i = 0; i < VECTORS; ++i) {
        const int column = (threadIdx.x + i * NORM_THREADS) * 8;
        uint4 y = make_uint4(0u, 0u, 0u, 0u);
        if (valid[i]) {
            y = affine_vector(a, modulation_base, column, inverse, packed[i]);
            if (write_gate) write_gate_vector(a, modulation_base, gate_base, column);
        }
        encoder.store(a, row, base, column, valid[i], y);
    }
}

// Widths 1024 and 2048 with many rows: one warp per row, the whole row in registers (VECTORS = columns / 256
// packed vectors per lane, every load of the row in flight before any arithmetic), no shared memory and no
// block barrier.  The reference's thread t = lane + 32*i is this lane's vector i, so the 32-lane butterfly of
// the reference's warp i is a butterfly over vector i of all lanes.
constexpr int NORM_ROWS_PER_BLOCK = 4;
constexpr int NORM_WARP_ROWS_THRESHOLD = 4096;     // below this a warp per row leaves most SMs idle

template <int BITS, int VECTORS>
__global__ void __launch_bounds__(NORM_ROWS_PER_BLOCK * 32)
norm_encode_warp_kernel(const NormArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float2 denominator_table[BITS == 4 ? 128 : 1];
    if (BITS == 4) {
        fill_denominator_table(denominator_table, *a.global);
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * NORM_ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (row >= a.rows) return;                                   // the whole warp leaves together
    const int batch = row / a.tokens;
    const int64_t base = int64_t(row) * a.columns, gate_base = int64_t(batch) * a.columns;
    const int64_t modulation_base = int64_t(batch) * 3 * a.columns;
    uint4 packed[VECTORS];
#pragma unroll
    for (int i = 0; i < VECTORS; ++i) packed[i] = ld_nc_u4(reinterpret_cast<const uint4*>(a.input + base + (lane + 32 * i) * 8));
    if (a.update != nullptr) {
        uint4 update[VECTORS];
#pragma unroll
        for (int i = 0; i < VECTORS; ++i) update[i] = ld_nc_u4(reinterpret_cast<const uint4*>(a.update + base + (lane + 32 * i) * 8));
#pragma unroll
        for (int i = 0; i < VECTORS; ++i) packed[i] = apply_update(a, packed[i], update[i], gate_base, (lane + 32 * i) * 8);
    }
    if (a.residual != nullptr) {
#pragma unroll
        for (int i = 0; i < VECTORS; ++i) store_residual_vector(a.residual + base + (lane + 32 * i) * 8, packed[i], a.evict_last);
    }
    float inverse;
    if (a.mean != nullptr) {
        inverse = rsqrtf(__fadd_rn(a.mean[row], 1.0e-6f));
    } else {
        float totals[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) totals[i] = i < VECTORS ? warp_butterfly_sum(sum_squares_of_vector(packed[i < VECTORS ? i : 0])) : 0.0f;
        inverse = rsqrtf(__fadd_rn(__fmul_rn(combine_warp_totals(totals), __fdiv_rn(1.0f, float(a.columns))), 1.0e-6f));
    }
    if (a.inverse != nullptr && lane == 0) a.inverse[row] = inverse;
    const Encoder<BITS> encoder(a, denominator_table);
    const bool write_gate = a.gate != nullptr && row == batch * a.tokens;
#pragma unroll
    for (int i = 0; i < VECTORS; ++i) {
        const int column = (lane + 32 * i) * 8;
        const uint4 y = affine_vector(a, modulation_base, column, inverse, packed[i]);
        if (write_gate) write_gate_vector(a, modulation_base, gate_base, column);
        encoder.store(a, row, base, column, true, y);
    }
}

template <int BITS>
static int launch_norm_bits(const NormArgs& a, cudaStream_t stream) {
    int status;
    const bool lanes8 = a.columns == 1024 || a.columns == 2048;
    const int blocks = (a.rows + NORM_ROWS_PER_BLOCK - 1) / NORM_ROWS_PER_BLOCK;
    if (BITS == 4 && lanes8) {
        // NVFP4: the row-per-block shape at every row count.  The encoder's arithmetic, not memory, bounds this kernel, and a
        // thread that holds one 8-column vector leaves the scheduler more warps to hide it with than a lane that holds 64
        // columns of a whole row (17920 x 2048 with update and residual: 69 us against 76 us; the reference's kernel: 64 us).
        status = launch_kernel(norm_encode_block_kernel<BITS, ORDER_LANES8>, dim3(unsigned(a.rows)), dim3(unsigned(a.columns / 8)), size_t(0), stream, a);
    } else if (lanes8 && a.rows >= NORM_WARP_ROWS_THRESHOLD && a.columns == 2048) {
        status = launch_kernel(norm_encode_warp_kernel<BITS, 8>, dim3(unsigned(blocks)), dim3(unsigned(NORM_ROWS_PER_BLOCK * 32)), size_t(0), stream, a);
    } else if (lanes8 && a.rows >= NORM_WARP_ROWS_THRESHOLD) {
        status = launch_kernel(norm_encode_warp_kernel<BITS, 4>, dim3(unsigned(blocks)), dim3(unsigned(NORM_ROWS_PER_BLOCK * 32)), size_t(0), stream, a);
    } else if (lanes8) {
        status = launch_kernel(norm_encode_block_kernel<BITS, ORDER_LANES8>, dim3(unsigned(a.rows)), dim3(unsigned(a.columns / 8)), size_t(0), stream, a);
    } else {
        status = launch_kernel(norm_encode_block_kernel<BITS, ORDER_STRIDED>, dim3(unsigned(a.rows)), dim3(unsigned(NORM_THREADS)), size_t(size_t(a.columns) * 2), stream, a);
    }
    return status == 0 ? B2_OK : B2_E_DRIVER;
}

int launch_norm_quant(const b2_norm_desc* d, cudaStream_t stream) {
    NormArgs a;
    a.input = static_cast<const __nv_bfloat16*>(d->input);
    a.update = static_cast<const __nv_bfloat16*>(d->update);
    a.update_gate = static_cast<const __nv_bfloat16*>(d->update_gate);
    a.scale = static_cast<const float*>(d->scale);
    a.modulation = static_cast<const float*>(d->modulation);
    a.mean = static_cast<const float*>(d->mean);
    a.global = static_cast<const float*>(d->global);
    a.residual = static_cast<__nv_bfloat16*>(d->residual);
    a.output = static_cast<uint8_t*>(d->output);
    a.scales = static_cast<uint8_t*>(d->scales);
    a.blocked = static_cast<uint8_t*>(d->blocked);
    a.gate = static_cast<__nv_bfloat16*>(d->gate);
    a.inverse = static_cast<float*>(d->inverse);
    a.rows = d->rows;
    a.columns = d->columns;
    a.tokens = d->tokens;
    a.evict_last = (d->flags & B2_NORM_RESIDUAL_EVICT_LAST) != 0;
    if (d->bits == 16) return launch_norm_bits<16>(a, stream);
    if (d->bits == 8) return launch_norm_bits<8>(a, stream);
    return launch_norm_bits<4>(a, stream);
}

// ---- LayerNorm producer (the SigLIP tower) ------------------------------------------------------------
// embodiinfer/backend/cuda/csrc/norm_quant.cu:564-687 (e4m3 / bf16) and 797-931 (NVFP4), compiled by the
// reference without fused multiply-add, so every operation below is a separate fp32 rounding:
//   r = update ? bf16(input + update) : input
//   per thread (8 columns, pairs (x, y)):  sum = sum + (x + y);  sq = sq + (x*x + y*y)
//   32-lane butterflies, then butterflies over the warp totals of a 160-thread (columns <= 1152) or
//   256-thread block; mean = sum / columns;  var = max(0, sq / columns - mean*mean);  inv = rsqrtf(var + 1e-6)
//   y = bf16((((r - mean) * inv) * weight) + bias), then e4m3(y * multiplier), NVFP4 spec C at the global
//   scale, or y itself.
// WARP_ROW = true: one warp per row holding WARPS vectors per lane (the reference's thread t = lane + 32*i);
// false: one block of 32*WARPS threads per row, one vector per thread (few rows).
struct LayerNormArgs {
    const __nv_bfloat16* input;
    const __nv_bfloat16* update;
    const __nv_bfloat16* weight;
    const __nv_bfloat16* bias;
    __nv_bfloat16* residual;
    uint8_t* output;
    uint8_t* scales;
    uint8_t* blocked;
    float* statistics;      // optional [rows, 2]: mean, inverse deviation
    float scale_value;      // bits 8: multiplier; bits 4: global scale
    int rows, columns;
};

__device__ __forceinline__ void layer_sums_of_vector(const uint4& packed, float& sum, float& squares) {
    float v[8];
    unpack_bf16x8(packed, v);
    sum = 0.0f;
    squares = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        sum = __fadd_rn(sum, __fadd_rn(v[2 * j], v[2 * j + 1]));
        squares = __fadd_rn(squares, __fadd_rn(__fmul_rn(v[2 * j], v[2 * j]), __fmul_rn(v[2 * j + 1], v[2 * j + 1])));
    }
}

template <int BITS, int WARPS, bool WARP_ROW>
__global__ void __launch_bounds__(WARP_ROW ? NORM_ROWS_PER_BLOCK * 32 : WARPS * 32)
layer_norm_encode_kernel(const LayerNormArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float2 denominator_table[BITS == 4 ? 128 : 1];
    if (BITS == 4) {
        fill_denominator_table(denominator_table, a.scale_value);
        __syncthreads();
    }
    constexpr int VECTORS = WARP_ROW ? WARPS : 1;
    __shared__ float block_totals[2][8];
    const int lane = threadIdx.x & 31;
    const int row = WARP_ROW ? blockIdx.x * NORM_ROWS_PER_BLOCK + (threadIdx.x >> 5) : blockIdx.x;
    if (row >= a.rows) return;                                   // WARP_ROW only: the whole warp leaves together
    const int64_t base = int64_t(row) * a.columns;
    uint4 packed[VECTORS], update[VECTORS];
    bool valid[VECTORS];
#pragma unroll
    for (int i = 0; i < VECTORS; ++i) {
        const int column = (WARP_ROW ? lane + 32 * i : int(threadIdx.x)) * 8;
        valid[i] = column < a.columns;
        packed[i] = make_uint4(0u, 0u, 0u, 0u);
        if (valid[i]) packed[i] = ld_nc_u4(reinterpret_cast<const uint4*>(a.input + base + column));
        if (valid[i] && a.update != nullptr) update[i] = ld_nc_u4(reinterpret_cast<const uint4*>(a.update + base + column));
    }
    float sums[8], squares[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) sums[i] = squares[i] = 0.0f;
#pragma unroll
    for (int i = 0; i < VECTORS; ++i) {
        const int column = (WARP_ROW ? lane + 32 * i : int(threadIdx.x)) * 8;
        if (valid[i] && a.update != nullptr) {
            float v[8], delta[8];
            unpack_bf16x8(packed[i], v);
            unpack_bf16x8(update[i], delta);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __fadd_rn(v[j], delta[j]);
            packed[i] = pack_bf16x8(v);
        }
        if (valid[i] && a.residual != nullptr) *reinterpret_cast<uint4*>(a.residual + base + column) = packed[i];
        float sum, square;
        layer_sums_of_vector(packed[i], sum, square);            // an absent vector is all zeros: both sums 0.0
        sums[i] = warp_butterfly_sum(sum);
        squares[i] = warp_butterfly_sum(square);
    }
    if (!WARP_ROW) {
        if (lane == 0) {
            block_totals[0][threadIdx.x >> 5] = sums[0];
            block_totals[1][threadIdx.x >> 5] = squares[0];
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            sums[i] = i < WARPS ? block_totals[0][i] : 0.0f;
            squares[i] = i < WARPS ? block_totals[1][i] : 0.0f;
        }
    }
    const float width = float(a.columns);
    const float mean = __fdiv_rn(combine_warp_totals(sums), width);
    const float variance = fmaxf(0.0f, __fsub_rn(__fdiv_rn(combine_warp_totals(squares), width), __fmul_rn(mean, mean)));
    const float deviation = rsqrtf(__fadd_rn(variance, 1.0e-6f));
    if (a.statistics != nullptr && (WARP_ROW ? lane == 0 : threadIdx.x == 0)) {
        a.statistics[2 * row] = mean;
        a.statistics[2 * row + 1] = deviation;
    }
    const Encoder<BITS> encoder(BITS == 4 ? a.scale_value : 1.0f, a.scale_value, denominator_table);
#pragma unroll
    for (int i = 0; i < VECTORS; ++i) {
        const int column = (WARP_ROW ? lane + 32 * i : int(threadIdx.x)) * 8;
        float y[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        if (valid[i]) {
            float weight[8], bias[8];
            unpack_bf16x8(packed[i], y);
            unpack_bf16x8(*reinterpret_cast<const uint4*>(a.weight + column), weight);
            unpack_bf16x8(*reinterpret_cast<const uint4*>(a.bias + column), bias);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                y[j] = round_to_bf16(__fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(y[j], mean), deviation), weight[j]), bias[j]));
        }
        encoder.store(a, row, base, column, valid[i], pack_bf16x8(y));
    }
}

template <int BITS>
static int launch_layer_norm_bits(const LayerNormArgs& a, cudaStream_t stream) {
    int status;
    const int blocks = (a.rows + NORM_ROWS_PER_BLOCK - 1) / NORM_ROWS_PER_BLOCK;
    const bool narrow = a.columns <= 1152;                       // the reference's 160-thread block (norm_quant.cu:681)
    if (a.rows >= NORM_WARP_ROWS_THRESHOLD) {
        if (narrow) status = launch_kernel(layer_norm_encode_kernel<BITS, 5, true>, dim3(unsigned(blocks)), dim3(unsigned(NORM_ROWS_PER_BLOCK * 32)), size_t(0), stream, a);
        else status = launch_kernel(layer_norm_encode_kernel<BITS, 8, true>, dim3(unsigned(blocks)), dim3(unsigned(NORM_ROWS_PER_BLOCK * 32)), size_t(0), stream, a);
    } else {
        if (narrow) status = launch_kernel(layer_norm_encode_kernel<BITS, 5, false>, dim3(unsigned(a.rows)), dim3(unsigned(160)), size_t(0), stream, a);
        else status = launch_kernel(layer_norm_encode_kernel<BITS, 8, false>, dim3(unsigned(a.rows)), dim3(unsigned(256)), size_t(0), stream, a);
    }
    return status == 0 ? B2_OK : B2_E_DRIVER;
}

int launch_layer_norm_quant(const void* input, const void* update, const void* weight, const void* bias, void* residual,
                            void* output, void* scales, void* blocked, void* statistics, float scale_value, int rows,
                            int columns, int bits, cudaStream_t stream) {
    LayerNormArgs a;
    a.input = static_cast<const __nv_bfloat16*>(input);
    a.update = static_cast<const __nv_bfloat16*>(update);
    a.weight = static_cast<const __nv_bfloat16*>(weight);
    a.bias = static_cast<const __nv_bfloat16*>(bias);
    a.residual = static_cast<__nv_bfloat16*>(residual);
    a.output = static_cast<uint8_t*>(output);
    a.scales = static_cast<uint8_t*>(scales);
    a.blocked = static_cast<uint8_t*>(blocked);
    a.statistics = static_cast<float*>(statistics);
    a.scale_value = scale_value;
    a.rows = rows;
    a.columns = columns;
    if (bits == 16) return launch_layer_norm_bits<16>(a, stream);
    if (bits == 8) return launch_layer_norm_bits<8>(a, stream);
    return launch_layer_norm_bits<4>(a, stream);
}

// ---- attention output [B, H, S, D] -> encoded rows [B*S, H*D] ---------------------------------------------
// embodiinfer/backend/cuda/csrc/norm_quant.cu:689-795 (cc_bhsd_fp8 / cc_bhsd_fp4): the transpose in front of the
// output projection fused with its activation encoder.  e4m3: x * multiplier (the reference passes the
// reciprocal of the activation scale by value); NVFP4: spec C at the global scale; bits 16: the plain
// transposing copy.  One 8-element vector per thread, grid-stride; a head's D elements are contiguous in the
// source, a row's H*D elements in the destination, so both sides move whole 16-byte vectors.
struct BhsdArgs {
    const __nv_bfloat16* input;
    uint8_t* output;
    uint8_t* scales;
    uint8_t* blocked;
    float scale_value;
    int64_t stride_b, stride_h, stride_s;
    int batch, heads, tokens, head_dim, columns;
};

constexpr int BHSD_THREADS = 256;

template <int BITS>
__global__ void __launch_bounds__(BHSD_THREADS)
bhsd_encode_kernel(const BhsdArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float2 denominator_table[BITS == 4 ? 128 : 1];
    if (BITS == 4) {
        fill_denominator_table(denominator_table, a.scale_value);
        __syncthreads();
    }
    const int vectors_per_row = a.columns >> 3;
    const int64_t total = int64_t(a.batch) * a.tokens * vectors_per_row;
    const int64_t rounded = (total + 31) & ~int64_t(31);        // whole warps enter the loop: NVFP4 pairs exchange maxima
    const Encoder<BITS> encoder(BITS == 4 ? a.scale_value : 1.0f, a.scale_value, denominator_table);
    for (int64_t index = int64_t(blockIdx.x) * BHSD_THREADS + threadIdx.x; index < rounded; index += int64_t(gridDim.x) * BHSD_THREADS) {
        const bool valid = index < total;
        const int row = int(index / vectors_per_row);           // b * tokens + s
        const int column = int(index - int64_t(row) * vectors_per_row) * 8;
        uint4 y = make_uint4(0u, 0u, 0u, 0u);
        if (valid) {
            const int b = row / a.tokens, s = row - b * a.tokens;
            const int h = column / a.head_dim, d = column - h * a.head_dim;
            y = ld_nc_u4(reinterpret_cast<const uint4*>(a.input + b * a.stride_b + h * a.stride_h + s * a.stride_s + d));
        }
        encoder.store(a, row, int64_t(row) * a.columns, column, valid, y);
    }
}

int launch_bhsd_quant(const void* input, void* output, void* scales, void* blocked, float scale_value, int64_t stride_b,
                      int64_t stride_h, int64_t stride_s, int batch, int heads, int tokens, int head_dim, int bits,
                      cudaStream_t stream) {
    BhsdArgs a;
    a.input = static_cast<const __nv_bfloat16*>(input);
    a.output = static_cast<uint8_t*>(output);
    a.scales = static_cast<uint8_t*>(scales);
    a.blocked = static_cast<uint8_t*>(blocked);
    a.scale_value = scale_value;
    a.stride_b = stride_b;
    a.stride_h = stride_h;
    a.stride_s = stride_s;
    a.batch = batch;
    a.heads = heads;
    a.tokens = tokens;
    a.head_dim = head_dim;
    a.columns = heads * head_dim;
    const int64_t total = int64_t(batch) * tokens * (a.columns >> 3);
    const int64_t wanted = (total + BHSD_THREADS - 1) / BHSD_THREADS;
    const int blocks = int(wanted < int64_t(sm_count()) * 16 ? wanted : int64_t(sm_count()) * 16);
    int status;
    if (bits == 16) status = launch_kernel(bhsd_encode_kernel<16>, dim3(unsigned(blocks)), dim3(unsigned(BHSD_THREADS)), size_t(0), stream, a);
    else if (bits == 8) status = launch_kernel(bhsd_encode_kernel<8>, dim3(unsigned(blocks)), dim3(unsigned(BHSD_THREADS)), size_t(0), stream, a);
    else status = launch_kernel(bhsd_encode_kernel<4>, dim3(unsigned(blocks)), dim3(unsigned(BHSD_THREADS)), size_t(0), stream, a);
    return status == 0 ? B2_OK : B2_E_DRIVER;
}

}  // namespace b2
