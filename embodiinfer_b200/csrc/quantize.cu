// Activation quantisers for sm_100a: bf16 -> FP8 e4m3 (per-tensor scale) and
// bf16 -> NVFP4 (e2m1 codes, e4m3 scale per 16 elements, fp32 global scale).
//
// HBM-bound kernels: every thread moves 16 bytes per load, the tensor amax is
// reduced with warp shuffles and one atomic per CTA, and the NVFP4 encoder
// writes the block scales directly in the 128x4 tile order the block-scaled
// tensor-core instruction consumes.
//
// Two arithmetics of the reference are reproduced bit for bit and selected by
// `flags` (see embodiinfer_b200.h):
//   spec T  embodiinfer/backend/torch/fp8.py:66-73, backend/torch/nvfp4.py:28-46
//   spec C  embodiinfer/backend/cuda/csrc/quantize.cu:38-104
#include "common.cuh"

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

namespace b2 {

constexpr int QUANT_THREADS = 256;

// ---------------------------------------------------------------------------
// tensor amax -> scale.  scratch[0] accumulates the amax bit pattern (non-negative
// floats order like unsigned integers), scratch[1] counts finished CTAs.  The last
// CTA publishes the scale and puts both words back to zero, so the same scratch
// serves the next call on the stream without a memset.

__global__ void __launch_bounds__(QUANT_THREADS)
tensor_scale_kernel(const uint4* __restrict__ input, int64_t vectors, const __nv_bfloat16* __restrict__ tail,
                    int tail_count, float bound, int flags, unsigned int* scratch, float* scale) {
    pdl_launch_dependents();
    pdl_wait();
    float maximum = 0.0f;
    const int64_t stride = int64_t(gridDim.x) * QUANT_THREADS;
    for (int64_t index = int64_t(blockIdx.x) * QUANT_THREADS + threadIdx.x; index < vectors; index += stride) {
        const uint4 packed = ld_nc_u4(input + index);
        maximum = fmaxf(maximum, abs_max_bf16x8(packed));
    }
    if (blockIdx.x == 0 && int(threadIdx.x) < tail_count)
        maximum = fmaxf(maximum, fabsf(__bfloat162float(tail[threadIdx.x])));
#pragma unroll
    for (int delta = 16; delta; delta >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, delta));
    __shared__ float warp_max[QUANT_THREADS / 32];
    __shared__ bool last_block;
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = maximum;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int warp = 1; warp < QUANT_THREADS / 32; ++warp) maximum = fmaxf(maximum, warp_max[warp]);
        atomicMax(scratch, __float_as_uint(maximum));
        __threadfence();
        const unsigned int ticket = atomicAdd(scratch + 1, 1u);
        last_block = ticket == gridDim.x - 1;
    }
    __syncthreads();
    if (last_block && threadIdx.x == 0) {
        __threadfence();
        const float total = __uint_as_float(atomicExch(scratch, 0u));
        scratch[1] = 0u;
        *scale = scale_from_amax(total, bound, flags);
    }
}

// ---------------------------------------------------------------------------
// FP8 encode: 8 bf16 in (16 bytes), 8 e4m3 out (8 bytes) per thread per step.

template <bool SPEC_C>
__global__ void __launch_bounds__(QUANT_THREADS)
fp8_encode_kernel(const uint4* __restrict__ input, uint2* __restrict__ output, int64_t vectors,
                  const __nv_bfloat16* __restrict__ tail_in, uint8_t* __restrict__ tail_out, int tail_count,
                  const float* __restrict__ scale_pointer, int flags) {
    pdl_launch_dependents();
    pdl_wait();
    float scale_value = __ldg(scale_pointer);
    if (!SPEC_C && (flags & B2_DIVISOR_BF16)) scale_value = __bfloat162float(__float2bfloat16(scale_value));
    const ExactDivider scale(scale_value);
    const int64_t stride = int64_t(gridDim.x) * QUANT_THREADS;
    for (int64_t index = int64_t(blockIdx.x) * QUANT_THREADS + threadIdx.x; index < vectors; index += stride) {
        const uint4 packed = ld_nc_u4(input + index);
        float v[8];
        unpack_bf16x8(packed, v);
        uint2 out;
        out.x = encode_fp8x4<SPEC_C>(v[0], v[1], v[2], v[3], scale);
        out.y = encode_fp8x4<SPEC_C>(v[4], v[5], v[6], v[7], scale);
        output[index] = out;
    }
    if (blockIdx.x == 0 && int(threadIdx.x) < tail_count) {
        const float value = __bfloat162float(tail_in[threadIdx.x]);
        tail_out[threadIdx.x] = uint8_t(encode_fp8x4<SPEC_C>(value, 0.0f, 0.0f, 0.0f, scale) & 0xffu);
    }
}

// Wide variant for 32-byte aligned tensors: 16 bf16 in (one 32-byte load), 16 e4m3 out (one 16-byte store)
// per thread and step, two steps in flight per thread, packed fp32 arithmetic.
template <bool SPEC_C>
__global__ void __launch_bounds__(QUANT_THREADS)
fp8_encode_wide_kernel(const uint8_t* __restrict__ input, uint4* __restrict__ output, int64_t vectors,
                       const float* __restrict__ scale_pointer, int flags) {
    pdl_launch_dependents();
    pdl_wait();
    float scale_value = __ldg(scale_pointer);
    if (!SPEC_C && (flags & B2_DIVISOR_BF16)) scale_value = __bfloat162float(__float2bfloat16(scale_value));
    const ExactDivider scale(scale_value);
    const float bound = __fmul_rn(1024.0f, scale_value);
    const int64_t stride = int64_t(gridDim.x) * QUANT_THREADS;
    for (int64_t index = int64_t(blockIdx.x) * QUANT_THREADS + threadIdx.x; index < vectors; index += 2 * stride) {
        const int64_t second = index + stride;
        const bool has_second = second < vectors;
        uint32_t a[8], b[8];
        ld_nc_u8(input + index * 32, a);
        if (has_second) ld_nc_u8(input + second * 32, b);
        uint32_t out[4];
        encode_fp8_words<SPEC_C, 8>(a, out, scale, bound);
        output[index] = make_uint4(out[0], out[1], out[2], out[3]);
        if (has_second) {
            encode_fp8_words<SPEC_C, 8>(b, out, scale, bound);
            output[second] = make_uint4(out[0], out[1], out[2], out[3]);
        }
    }
}

// ---------------------------------------------------------------------------
// NVFP4 encode.  Two adjacent threads own one 16-element block (8 elements, one
// 16-byte load each); the pair's maximum crosses with a single shuffle.  Eight
// adjacent threads therefore cover four blocks = one 4-byte word of the tiled
// scale layout, which the first of them stores whole when the row width allows.

template <bool SPEC_C>
__global__ void __launch_bounds__(QUANT_THREADS)
nvfp4_encode_kernel(const uint4* __restrict__ input, uint32_t* __restrict__ output, uint8_t* __restrict__ scales,
                    uint8_t* __restrict__ blocked, const float* __restrict__ global_pointer, int rows, int columns,
                    int flags) {
    pdl_launch_dependents();
    pdl_wait();
    const int vectors_per_row = columns >> 3;
    const int blocks_per_row = columns >> 4;
    const int column_tiles = (blocks_per_row + 3) >> 2;
    const int64_t total = int64_t(rows) * vectors_per_row;
    const float global = __ldg(global_pointer);
    const ExactDivider by_global(SPEC_C ? __fmul_rn(6.0f, global) : global);
    const bool whole_words = (blocks_per_row & 3) == 0;
    const int64_t stride = int64_t(gridDim.x) * QUANT_THREADS;
    // The loop condition is uniform per warp.  `total` is a multiple of 2 (a row holds whole
    // blocks), so both threads of a pair are active together; the shuffle mask follows the
    // active lanes.
    const int lane = threadIdx.x & 31;
    for (int64_t warp_base = int64_t(blockIdx.x) * QUANT_THREADS + (threadIdx.x - lane); warp_base < total;
         warp_base += stride) {
        const int64_t index = warp_base + lane;
        const bool active = index < total;
        const unsigned int mask = __ballot_sync(0xffffffffu, active);
        if (!active) continue;
        const uint4 packed = ld_nc_u4(input + index);
        float v[8];
        unpack_bf16x8(packed, v);
        float maximum = abs_max_bf16x8(packed);
        maximum = fmaxf(maximum, __shfl_xor_sync(mask, maximum, 1));
        const uint8_t scale_code = nvfp4_block_scale<SPEC_C>(maximum, by_global, flags);
        const ExactDivider denominator(__fmul_rn(global, e4m3_to_float(scale_code)));
        output[index] = nvfp4_encode_x8<SPEC_C>(v, denominator, maximum);
        // 32-bit index arithmetic whenever the matrix allows it (a 64-bit division costs dozens of instructions)
        const int row = total <= 0x7fffffff ? int(uint32_t(index) / uint32_t(vectors_per_row)) : int(index / vectors_per_row);
        const int vector = int(index - int64_t(row) * vectors_per_row);
        const int block = vector >> 1;
        if (whole_words) {
            // lanes 0,2,4,6 of each group of eight hold the four scale bytes of one word
            const int base = (threadIdx.x & 31) & ~7;
            unsigned int word = scale_code;
            word |= (unsigned int)__shfl_sync(mask, (unsigned int)scale_code, base + 2) << 8;
            word |= (unsigned int)__shfl_sync(mask, (unsigned int)scale_code, base + 4) << 16;
            word |= (unsigned int)__shfl_sync(mask, (unsigned int)scale_code, base + 6) << 24;
            if ((threadIdx.x & 7) == 0) {
                if (blocked != nullptr)
                    *reinterpret_cast<uint32_t*>(blocked + scale_tile_offset(row, block, column_tiles)) = word;
                if (scales != nullptr)
                    *reinterpret_cast<uint32_t*>(scales + int64_t(row) * blocks_per_row + block) = word;
            }
        } else if ((vector & 1) == 0) {
            if (blocked != nullptr) blocked[scale_tile_offset(row, block, column_tiles)] = scale_code;
            if (scales != nullptr) scales[int64_t(row) * blocks_per_row + block] = scale_code;
        }
    }
}

// Wide variant for 32-byte aligned matrices: one thread owns whole 16-element blocks (one 32-byte load and
// one 8-byte store of codes each), so the block maximum needs no shuffle and the scale arithmetic runs once
// per block.  BLOCKS = 2 (rows of a multiple of 32 elements): two adjacent blocks per thread, both loads in
// flight before any arithmetic, 16-byte code stores, and two adjacent threads assemble a 4-byte word of
// scale bytes; BLOCKS = 1: four adjacent threads do.
template <bool SPEC_C, int BLOCKS>
__global__ void __launch_bounds__(QUANT_THREADS)
nvfp4_encode_wide_kernel(const uint8_t* __restrict__ input, uint8_t* __restrict__ output, uint8_t* __restrict__ scales,
                         uint8_t* __restrict__ blocked, const float* __restrict__ global_pointer, int rows, int columns,
                         int flags) {
    pdl_launch_dependents();
    pdl_wait();
    const int blocks_per_row = columns >> 4;
    const int column_tiles = (blocks_per_row + 3) >> 2;
    const int items_per_row = blocks_per_row / BLOCKS;                 // one item = BLOCKS adjacent blocks of one row
    const int64_t total = int64_t(rows) * items_per_row;
    const float global = __ldg(global_pointer);
    const ExactDivider by_global(SPEC_C ? __fmul_rn(6.0f, global) : global);
    __shared__ float2 denominators[128];
    fill_denominator_table(denominators, global);
    __syncthreads();
    const bool whole_words = (blocks_per_row & 3) == 0;
    constexpr int LANES_PER_WORD = 4 / BLOCKS;
    const int64_t stride = int64_t(gridDim.x) * QUANT_THREADS;
    const int lane = threadIdx.x & 31;
    // warp-uniform loop: `total` is a multiple of LANES_PER_WORD whenever whole words are stored, so the
    // lanes of a scale word are active together
    // (row, item in row) of this thread's item, advanced by the grid stride without a division per item
    const int64_t first_index = int64_t(blockIdx.x) * QUANT_THREADS + threadIdx.x;
    int row = int(first_index / items_per_row);
    int item_in_row = int(first_index - int64_t(row) * items_per_row);
    const int row_step = int(stride / items_per_row), item_step = int(stride - int64_t(row_step) * items_per_row);
    // the loads of the next item are issued before the arithmetic of the current one (one item of look-ahead)
    uint32_t ahead[BLOCKS][8];
    {
        const int64_t first = first_index;
        if (first < total) {
#pragma unroll
            for (int b = 0; b < BLOCKS; ++b) ld_nc_u8(input + (first * BLOCKS + b) * 32, ahead[b]);
        }
    }
    for (int64_t warp_base = int64_t(blockIdx.x) * QUANT_THREADS + (threadIdx.x - lane); warp_base < total;
         warp_base += stride, row += row_step, item_in_row += item_step) {
        if (item_in_row >= items_per_row) {
            item_in_row -= items_per_row;
            ++row;
        }
        const int64_t index = warp_base + lane;
        const bool active = index < total;
        const unsigned int mask = __ballot_sync(0xffffffffu, active);
        if (!active) continue;
        uint32_t w[BLOCKS][8];
#pragma unroll
        for (int b = 0; b < BLOCKS; ++b)
#pragma unroll
            for (int i = 0; i < 8; ++i) w[b][i] = ahead[b][i];
        if (index + stride < total) {
#pragma unroll
            for (int b = 0; b < BLOCKS; ++b) ld_nc_u8(input + ((index + stride) * BLOCKS + b) * 32, ahead[b]);
        }
        uint8_t code[BLOCKS];
        uint2 codes[BLOCKS];
#pragma unroll
        for (int b = 0; b < BLOCKS; ++b) codes[b] = nvfp4_encode_block<SPEC_C>(w[b], global, by_global, flags, code[b], denominators);
        if (BLOCKS == 2) *reinterpret_cast<uint4*>(output + index * 16) = make_uint4(codes[0].x, codes[0].y, codes[BLOCKS - 1].x, codes[BLOCKS - 1].y);
        else *reinterpret_cast<uint2*>(output + index * 8) = codes[0];
        const int block = item_in_row * BLOCKS;
        if (whole_words) {
            const int base = lane & ~(LANES_PER_WORD - 1);
            unsigned int mine = code[0];
            if (BLOCKS == 2) mine |= (unsigned int)code[BLOCKS - 1] << 8;
            unsigned int word = 0;
#pragma unroll
            for (int i = 0; i < LANES_PER_WORD; ++i) word |= __shfl_sync(mask, mine, base + i) << (8 * BLOCKS * i);
            if ((lane & (LANES_PER_WORD - 1)) == 0) {
                if (blocked != nullptr)
                    *reinterpret_cast<uint32_t*>(blocked + scale_tile_offset(row, block, column_tiles)) = word;
                if (scales != nullptr)
                    *reinterpret_cast<uint32_t*>(scales + int64_t(row) * blocks_per_row + block) = word;
            }
        } else {
#pragma unroll
            for (int b = 0; b < BLOCKS; ++b) {
                if (blocked != nullptr) blocked[scale_tile_offset(row, block + b, column_tiles)] = code[b];
                if (scales != nullptr) scales[int64_t(row) * blocks_per_row + block + b] = code[b];
            }
        }
    }
}

// ---------------------------------------------------------------------------
// host side

static int grid_for(int64_t work_items, int per_block) {
    const int64_t wanted = (work_items + per_block - 1) / per_block;
    const int64_t cap = int64_t(sm_count()) * 8;
    return int(wanted < 1 ? 1 : (wanted < cap ? wanted : cap));
}

int launch_tensor_scale(const void* input, int64_t count, float bound, int flags, void* scratch, void* scale,
                        cudaStream_t stream) {
    const int64_t vectors = count >> 3;
    const int tail = int(count & 7);
    const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(input);
    tensor_scale_kernel<<<grid_for(vectors, QUANT_THREADS * 4), QUANT_THREADS, 0, stream>>>(
        static_cast<const uint4*>(input), vectors, base + vectors * 8, tail, bound, flags,
        static_cast<unsigned int*>(scratch), static_cast<float*>(scale));
    return int(cudaGetLastError());
}

int launch_fp8_encode(const void* input, void* output, const void* scale, int64_t count, int flags,
                      cudaStream_t stream) {
    const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(input);
    uint8_t* out_base = static_cast<uint8_t*>(output);
    if ((reinterpret_cast<uintptr_t>(input) & 31u) == 0 && (reinterpret_cast<uintptr_t>(output) & 15u) == 0 && count >= 16) {
        // whole 16-element vectors on the wide kernel, the rest (< 16 elements) on the narrow one below
        const int64_t wide = count >> 4;
        const int grid = grid_for(wide, QUANT_THREADS * 2);
        if (flags & B2_SPEC_C)
            launch_kernel(fp8_encode_wide_kernel<true>, dim3(unsigned(grid)), dim3(unsigned(QUANT_THREADS)), size_t(0), stream, 
                static_cast<const uint8_t*>(input), static_cast<uint4*>(output), wide, static_cast<const float*>(scale), flags);
        else
            launch_kernel(fp8_encode_wide_kernel<false>, dim3(unsigned(grid)), dim3(unsigned(QUANT_THREADS)), size_t(0), stream, 
                static_cast<const uint8_t*>(input), static_cast<uint4*>(output), wide, static_cast<const float*>(scale), flags);
        const cudaError_t error = cudaGetLastError();
        if (error != cudaSuccess || (count & 15) == 0) return int(error);
        base += wide * 16;
        out_base += wide * 16;
        count &= 15;
        input = base;
        output = out_base;
    }
    const int64_t vectors = count >> 3;
    const int tail = int(count & 7);
    const int grid = grid_for(vectors, QUANT_THREADS * 2);
    if (flags & B2_SPEC_C)
        launch_kernel(fp8_encode_kernel<true>, dim3(unsigned(grid)), dim3(unsigned(QUANT_THREADS)), size_t(0), stream, 
            static_cast<const uint4*>(input), static_cast<uint2*>(output), vectors, base + vectors * 8,
            out_base + vectors * 8, tail, static_cast<const float*>(scale), flags);
    else
        launch_kernel(fp8_encode_kernel<false>, dim3(unsigned(grid)), dim3(unsigned(QUANT_THREADS)), size_t(0), stream, 
            static_cast<const uint4*>(input), static_cast<uint2*>(output), vectors, base + vectors * 8,
            out_base + vectors * 8, tail, static_cast<const float*>(scale), flags);
    return int(cudaGetLastError());
}

int launch_nvfp4_encode(const void* input, void* output, void* scales, void* blocked, const void* global, int rows,
                        int columns, int flags, cudaStream_t stream) {
    if ((reinterpret_cast<uintptr_t>(input) & 31u) == 0 && (reinterpret_cast<uintptr_t>(output) & 15u) == 0) {
        const bool pairs = (columns & 31) == 0;
        const int grid = grid_for(int64_t(rows) * (columns >> (pairs ? 5 : 4)), QUANT_THREADS);
        const uint8_t* in = static_cast<const uint8_t*>(input);
        uint8_t* out = static_cast<uint8_t*>(output);
        uint8_t* row_major = static_cast<uint8_t*>(scales);
        uint8_t* tiled = static_cast<uint8_t*>(blocked);
        const float* g = static_cast<const float*>(global);
        if (flags & B2_SPEC_C) {
            if (pairs) launch_kernel(nvfp4_encode_wide_kernel<true, 2>, dim3(unsigned(grid)), dim3(unsigned(QUANT_THREADS)), size_t(0), stream, in, out, row_major, tiled, g, rows, columns, flags);
            else launch_kernel(nvfp4_encode_wide_kernel<true, 1>, dim3(unsigned(grid)), dim3(unsigned(QUANT_THREADS)), size_t(0), stream, in, out, row_major, tiled, g, rows, columns, flags);
        } else {
            if (pairs) launch_kernel(nvfp4_encode_wide_kernel<false, 2>, dim3(unsigned(grid)), dim3(unsigned(QUANT_THREADS)), size_t(0), stream, in, out, row_major, tiled, g, rows, columns, flags);
            else launch_kernel(nvfp4_encode_wide_kernel<false, 1>, dim3(unsigned(grid)), dim3(unsigned(QUANT_THREADS)), size_t(0), stream, in, out, row_major, tiled, g, rows, columns, flags);
        }
        return int(cudaGetLastError());
    }
    const int64_t total = int64_t(rows) * (columns >> 3);
    const int grid = grid_for(total, QUANT_THREADS * 2);
    if (flags & B2_SPEC_C)
        launch_kernel(nvfp4_encode_kernel<true>, dim3(unsigned(grid)), dim3(unsigned(QUANT_THREADS)), size_t(0), stream, 
            static_cast<const uint4*>(input), static_cast<uint32_t*>(output), static_cast<uint8_t*>(scales),
            static_cast<uint8_t*>(blocked), static_cast<const float*>(global), rows, columns, flags);
    else
        launch_kernel(nvfp4_encode_kernel<false>, dim3(unsigned(grid)), dim3(unsigned(QUANT_THREADS)), size_t(0), stream, 
            static_cast<const uint4*>(input), static_cast<uint32_t*>(output), static_cast<uint8_t*>(scales),
            static_cast<uint8_t*>(blocked), static_cast<const float*>(global), rows, columns, flags);
    return int(cudaGetLastError());
}

}  // namespace b2
