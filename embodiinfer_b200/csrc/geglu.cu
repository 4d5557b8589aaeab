// Stand-alone gated-GELU epilogue: h = bf16(bf16(gelu(gate)) * up), stored as bf16,
// e4m3 or NVFP4.  It serves callers whose gate/up come from somewhere other than the
// fused tensor-core kernel (gemm.cu fuses the same arithmetic into its epilogue).
// HBM-bound: one 16-byte load per operand per thread, GELU from the 128 KiB table
// (L2-resident), 16-byte / 8-byte / 4-byte stores.
//
// Arithmetic follows embodiinfer/backend/cuda/csrc/fusion.cu:5-10 (two bf16 rounding
// points), :64-107 (FP8: multiply by the reciprocal scale) and :31-62 (NVFP4).
#include "common.cuh"

namespace b2 {

constexpr int GEGLU_THREADS = 256;

__device__ __forceinline__ float gelu_times_up(uint32_t gate_bits, float up, bool has_up, const uint16_t* table) {
    const float gelu = bf16_lo(uint32_t(__ldg(table + gate_bits)));
    return has_up ? round_to_bf16(__fmul_rn(gelu, up)) : gelu;
}

__device__ __forceinline__ void hidden_x8(const uint4& gate, const uint4& up, bool has_up, const uint16_t* table,
                                          float (&h)[8]) {
    float u[8];
    unpack_bf16x8(up, u);
    const uint32_t words[4] = {gate.x, gate.y, gate.z, gate.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        h[2 * i] = gelu_times_up(words[i] & 0xffffu, u[2 * i], has_up, table);
        h[2 * i + 1] = gelu_times_up(words[i] >> 16, u[2 * i + 1], has_up, table);
    }
}

// BITS 16 or 8.  `vectors_per_row` 8-element vectors per row; rows are `row_stride` elements apart.
template <int BITS>
__global__ void __launch_bounds__(GEGLU_THREADS)
geglu_vector_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up, void* __restrict__ output,
                    const float* __restrict__ scale_pointer, int rows, int vectors_per_row, int64_t row_stride,
                    const uint16_t* __restrict__ table, int flags) {
    const int64_t total = int64_t(rows) * vectors_per_row;
    float scale = 1.0f, reciprocal = 1.0f;
    if (BITS == 8) {
        scale = __ldg(scale_pointer);
        reciprocal = __fdiv_rn(1.0f, scale);
    }
    const bool true_div = (flags & B2_GEGLU_TRUE_DIV) != 0;
    const ExactDivider divide(scale);
    const bool has_up = up != nullptr;
    const int64_t stride = int64_t(gridDim.x) * GEGLU_THREADS;
    for (int64_t index = int64_t(blockIdx.x) * GEGLU_THREADS + threadIdx.x; index < total; index += stride) {
        const int64_t row = index / vectors_per_row;
        const int64_t vector = index - row * vectors_per_row;
        const int64_t offset = row * row_stride + vector * 8;
        const uint4 g = ld_nc_u4(reinterpret_cast<const uint4*>(gate + offset));
        const uint4 u = has_up ? ld_nc_u4(reinterpret_cast<const uint4*>(up + offset)) : make_uint4(0, 0, 0, 0);
        float h[8];
        hidden_x8(g, u, has_up, table, h);
        if (BITS == 16) {
            uint4 out;
            out.x = uint32_t(bf16_bits(h[0])) | (uint32_t(bf16_bits(h[1])) << 16);
            out.y = uint32_t(bf16_bits(h[2])) | (uint32_t(bf16_bits(h[3])) << 16);
            out.z = uint32_t(bf16_bits(h[4])) | (uint32_t(bf16_bits(h[5])) << 16);
            out.w = uint32_t(bf16_bits(h[6])) | (uint32_t(bf16_bits(h[7])) << 16);
            static_cast<uint4*>(output)[index] = out;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = true_div ? divide(h[i]) : __fmul_rn(h[i], reciprocal);
            uint2 out;
            out.x = pack_fp8x4(h[0], h[1], h[2], h[3]);
            out.y = pack_fp8x4(h[4], h[5], h[6], h[7]);
            static_cast<uint2*>(output)[index] = out;
        }
    }
}

// One element per thread for widths that are not a multiple of eight.
template <int BITS>
__global__ void __launch_bounds__(GEGLU_THREADS)
geglu_scalar_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up, void* __restrict__ output,
                    const float* __restrict__ scale_pointer, int rows, int columns, int64_t row_stride,
                    const uint16_t* __restrict__ table, int flags) {
    const int64_t total = int64_t(rows) * columns;
    const bool true_div = (flags & B2_GEGLU_TRUE_DIV) != 0;
    const bool has_up = up != nullptr;
    const int64_t stride = int64_t(gridDim.x) * GEGLU_THREADS;
    for (int64_t index = int64_t(blockIdx.x) * GEGLU_THREADS + threadIdx.x; index < total; index += stride) {
        const int64_t row = index / columns;
        const int64_t offset = row * row_stride + (index - row * columns);
        const float upv = has_up ? __bfloat162float(up[offset]) : 0.0f;
        const float h = gelu_times_up(__bfloat16_as_ushort(gate[offset]), upv, has_up, table);
        if (BITS == 16) {
            static_cast<__nv_bfloat16*>(output)[index] = __float2bfloat16_rn(h);
        } else {
            const float scale = __ldg(scale_pointer);
            const float q = true_div ? __fdiv_rn(h, scale) : __fmul_rn(h, __fdiv_rn(1.0f, scale));
            static_cast<uint8_t*>(output)[index] = uint8_t(pack_fp8x4(q, 0.0f, 0.0f, 0.0f) & 0xffu);
        }
    }
}

// NVFP4 output: two threads per 16-element block, as in the activation quantiser.
__global__ void __launch_bounds__(GEGLU_THREADS)
geglu_nvfp4_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up, uint32_t* __restrict__ output,
                   uint8_t* __restrict__ scales, uint8_t* __restrict__ blocked, const float* __restrict__ global_pointer,
                   int rows, int columns, int64_t row_stride, const uint16_t* __restrict__ table) {
    const int vectors_per_row = columns >> 3;
    const int blocks_per_row = columns >> 4;
    const int column_tiles = (blocks_per_row + 3) >> 2;
    const int64_t total = int64_t(rows) * vectors_per_row;
    const float global = __ldg(global_pointer);
    const ExactDivider by_global(__fmul_rn(6.0f, global));
    const bool has_up = up != nullptr;
    const int lane = threadIdx.x & 31;
    const int64_t stride = int64_t(gridDim.x) * GEGLU_THREADS;
    for (int64_t warp_base = int64_t(blockIdx.x) * GEGLU_THREADS + (threadIdx.x - lane); warp_base < total;
         warp_base += stride) {
        const int64_t index = warp_base + lane;
        const bool active = index < total;
        const unsigned int mask = __ballot_sync(0xffffffffu, active);
        if (!active) continue;
        const int row = total <= 0x7fffffff ? int(uint32_t(index) / uint32_t(vectors_per_row)) : int(index / vectors_per_row);
        const int vector = int(index - int64_t(row) * vectors_per_row);
        const int64_t offset = int64_t(row) * row_stride + int64_t(vector) * 8;
        const uint4 g = ld_nc_u4(reinterpret_cast<const uint4*>(gate + offset));
        const uint4 u = has_up ? ld_nc_u4(reinterpret_cast<const uint4*>(up + offset)) : make_uint4(0, 0, 0, 0);
        float h[8];
        hidden_x8(g, u, has_up, table, h);
        float maximum = fabsf(h[0]);
#pragma unroll
        for (int i = 1; i < 8; ++i) maximum = fmaxf(maximum, fabsf(h[i]));
        maximum = fmaxf(maximum, __shfl_xor_sync(mask, maximum, 1));
        const uint8_t scale_code = nvfp4_block_scale<true>(maximum, by_global, 0);
        const ExactDivider denominator(__fmul_rn(global, e4m3_to_float(scale_code)));
        output[index] = nvfp4_encode_x8<true>(h, denominator, maximum);
        if ((vector & 1) == 0) {
            const int block = vector >> 1;
            if (blocked != nullptr) blocked[scale_tile_offset(row, block, column_tiles)] = scale_code;
            if (scales != nullptr) scales[int64_t(row) * blocks_per_row + block] = scale_code;
        }
    }
}

static int geglu_grid(int64_t work_items) {
    const int64_t wanted = (work_items + GEGLU_THREADS - 1) / GEGLU_THREADS;
    const int64_t cap = int64_t(sm_count()) * 16;
    return int(wanted < 1 ? 1 : (wanted < cap ? wanted : cap));
}

int launch_geglu(const void* gate, const void* up, void* output, void* scales, void* blocked, const void* scale,
                 int rows, int columns, int64_t row_stride, int bits, const void* table, int flags,
                 cudaStream_t stream) {
    const __nv_bfloat16* g = static_cast<const __nv_bfloat16*>(gate);
    const __nv_bfloat16* u = static_cast<const __nv_bfloat16*>(up);
    const uint16_t* t = static_cast<const uint16_t*>(table);
    const float* s = static_cast<const float*>(scale);
    const bool vectorised = columns % 8 == 0 && row_stride % 8 == 0 &&
                            (reinterpret_cast<uintptr_t>(gate) & 15u) == 0 &&
                            (up == nullptr || (reinterpret_cast<uintptr_t>(up) & 15u) == 0);
    if (bits == 4) {
        if (columns % 16 != 0 || !vectorised) return B2_E_UNSUPPORTED;
        const int64_t total = int64_t(rows) * (columns >> 3);
        geglu_nvfp4_kernel<<<geglu_grid(total), GEGLU_THREADS, 0, stream>>>(
            g, u, static_cast<uint32_t*>(output), static_cast<uint8_t*>(scales), static_cast<uint8_t*>(blocked), s, rows,
            columns, row_stride, t);
    } else if (vectorised) {
        const int64_t total = int64_t(rows) * (columns >> 3);
        if (bits == 8)
            geglu_vector_kernel<8><<<geglu_grid(total), GEGLU_THREADS, 0, stream>>>(g, u, output, s, rows, columns >> 3,
                                                                                   row_stride, t, flags);
        else
            geglu_vector_kernel<16><<<geglu_grid(total), GEGLU_THREADS, 0, stream>>>(g, u, output, s, rows, columns >> 3,
                                                                                    row_stride, t, flags);
    } else {
        const int64_t total = int64_t(rows) * columns;
        if (bits == 8)
            geglu_scalar_kernel<8><<<geglu_grid(total), GEGLU_THREADS, 0, stream>>>(g, u, output, s, rows, columns, row_stride,
                                                                                   t, flags);
        else
            geglu_scalar_kernel<16><<<geglu_grid(total), GEGLU_THREADS, 0, stream>>>(g, u, output, s, rows, columns, row_stride,
                                                                                    t, flags);
    }
    return int(cudaGetLastError());
}

}  // namespace b2
