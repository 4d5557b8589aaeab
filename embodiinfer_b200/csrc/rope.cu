// Attention preparation after the packed QKV projection: split the [rows, q_dim + 2*kv_dim] bf16 result,
// rotate queries and keys, and write queries as [B, heads, T, D] and keys / values straight into the
// attention's key/value buffers [B, kv_heads, S, D] at a token offset (the action expert appends its ten
// tokens behind the prefix's keys/values; the prefix tower writes at offset 0).  One launch replaces the
// split, two rotations (five elementwise kernels each), the transposes and the two buffer copies.
//
// Rotation arithmetic is the reference's (embodiinfer/backend/torch/rotary.py:24-27, contract
// "fp32_rope_bf16_output"): fp32 factors, separate multiplies and add/subtract (no fused multiply-add), one
// rounding to bf16:  out[:h] = bf16(x[:h]*cos - x[h:]*sin),  out[h:] = bf16(x[h:]*cos + x[:h]*sin).
// HBM-bound and tiny: 16-byte loads and stores, one thread per 8 elements of a half head.
#include "common.cuh"

namespace b2 {

constexpr int ROPE_THREADS = 256;

__global__ void __launch_bounds__(ROPE_THREADS)
rope_split_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ sine, const float* __restrict__ cosine,
                  __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out, __nv_bfloat16* __restrict__ v_out,
                  int batch, int tokens, int heads, int kv_heads, int head_dim, int64_t factor_batch_stride,
                  int kv_capacity, int kv_offset) {
    pdl_launch_dependents();
    pdl_wait();
    const int half = head_dim >> 1;
    const int vectors_per_half = half >> 3;                       // 8 elements per thread
    const int total_heads = heads + 2 * kv_heads;                 // q heads, k heads, v heads of one token
    const int64_t total = int64_t(batch) * tokens * total_heads * vectors_per_half;
    const int row_width = total_heads * head_dim;
    for (int64_t index = int64_t(blockIdx.x) * ROPE_THREADS + threadIdx.x; index < total;
         index += int64_t(gridDim.x) * ROPE_THREADS) {
        const int vector = int(index % vectors_per_half);
        const int head = int((index / vectors_per_half) % total_heads);
        const int64_t row = index / (int64_t(vectors_per_half) * total_heads);     // b * tokens + t
        const int token = int(row % tokens);
        const int b = int(row / tokens);
        const __nv_bfloat16* source = qkv + row * row_width + head * head_dim + vector * 8;
        const uint4 first = ld_nc_u4(reinterpret_cast<const uint4*>(source));
        const uint4 second = ld_nc_u4(reinterpret_cast<const uint4*>(source + half));
        __nv_bfloat16* destination;
        bool rotate = true;
        if (head < heads) {
            destination = q_out + ((int64_t(b) * heads + head) * tokens + token) * head_dim;
        } else if (head < heads + kv_heads) {
            destination = k_out + ((int64_t(b) * kv_heads + (head - heads)) * kv_capacity + kv_offset + token) * head_dim;
        } else {
            destination = v_out + ((int64_t(b) * kv_heads + (head - heads - kv_heads)) * kv_capacity + kv_offset + token) * head_dim;
            rotate = false;
        }
        destination += vector * 8;
        if (!rotate) {
            *reinterpret_cast<uint4*>(destination) = first;
            *reinterpret_cast<uint4*>(destination + half) = second;
            continue;
        }
        const float* s = sine + b * factor_batch_stride + int64_t(token) * half + vector * 8;
        const float* c = cosine + b * factor_batch_stride + int64_t(token) * half + vector * 8;
        float x[8], y[8];
        unpack_bf16x8(first, x);
        unpack_bf16x8(second, y);
        uint32_t low[4], high[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float c0 = __ldg(c + 2 * i), c1 = __ldg(c + 2 * i + 1), s0 = __ldg(s + 2 * i), s1 = __ldg(s + 2 * i + 1);
            const float2 a = make_float2(__fsub_rn(__fmul_rn(x[2 * i], c0), __fmul_rn(y[2 * i], s0)),
                                         __fsub_rn(__fmul_rn(x[2 * i + 1], c1), __fmul_rn(y[2 * i + 1], s1)));
            const float2 d = make_float2(__fadd_rn(__fmul_rn(y[2 * i], c0), __fmul_rn(x[2 * i], s0)),
                                         __fadd_rn(__fmul_rn(y[2 * i + 1], c1), __fmul_rn(x[2 * i + 1], s1)));
            low[i] = float2_to_bf16x2(a);
            high[i] = float2_to_bf16x2(d);
        }
        *reinterpret_cast<uint4*>(destination) = make_uint4(low[0], low[1], low[2], low[3]);
        *reinterpret_cast<uint4*>(destination + half) = make_uint4(high[0], high[1], high[2], high[3]);
    }
}

int launch_rope_split(const void* qkv, const void* sine, const void* cosine, void* q_out, void* k_out, void* v_out, int batch,
                      int tokens, int heads, int kv_heads, int head_dim, int64_t factor_batch_stride, int kv_capacity,
                      int kv_offset, cudaStream_t stream) {
    const int64_t total = int64_t(batch) * tokens * (heads + 2 * kv_heads) * (head_dim >> 4);
    const int64_t wanted = (total + ROPE_THREADS - 1) / ROPE_THREADS;
    const int64_t cap = int64_t(sm_count()) * 8;
    const int grid = int(wanted < 1 ? 1 : (wanted < cap ? wanted : cap));
    const int status = launch_kernel(rope_split_kernel, dim3(unsigned(grid)), dim3(unsigned(ROPE_THREADS)), size_t(0), stream,
                                     static_cast<const __nv_bfloat16*>(qkv), static_cast<const float*>(sine), static_cast<const float*>(cosine),
        static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_out), static_cast<__nv_bfloat16*>(v_out), batch, tokens,
        heads, kv_heads, head_dim, factor_batch_stride, kv_capacity, kv_offset);
    return status;
}

}  // namespace b2
