// Camera frames to model inputs: uint8 [cameras, H, W, 3] -> (x / 255) * 2 - 1, written either as the
// reference's fp32 planes [cameras, 3, H, W] (embodiinfer/backend/cuda/csrc/camera_frames.cu:11-22,
// cc_normalize_frames) or directly as the bf16 patch rows [cameras * (H/p) * (W/p), 3*p*p] that the SigLIP patch
// embedding multiplies (embodiinfer/policies/pi05/inference/vision.py:593-602:
// images.bfloat16().view(b, 3, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5).reshape(b * gh * gw, 3*p*p)), which
// skips the fp32 image and the permuting copy.
//
// The three steps round separately, as on the host (fp32 division, product, difference; the reference builds
// its kernel without fused multiply-add).  A byte has 256 values, so each block evaluates the expression once
// per value into a shared table and the pixels index it: the result is the expression's, bit for bit.
#include "common.cuh"

namespace b2 {

constexpr int FRAME_THREADS = 256;

__device__ __forceinline__ float normalized_byte(int value) {
    return __fsub_rn(__fmul_rn(__fdiv_rn(float(value), 255.0f), 2.0f), 1.0f);
}

__global__ void __launch_bounds__(FRAME_THREADS)
normalize_frames_kernel(const uint8_t* __restrict__ frames, float* __restrict__ images, int pixels, int64_t count) {
    __shared__ float table[256];
    table[threadIdx.x] = normalized_byte(threadIdx.x);
    __syncthreads();
    for (int64_t index = int64_t(blockIdx.x) * FRAME_THREADS + threadIdx.x; index < count; index += int64_t(gridDim.x) * FRAME_THREADS) {
        const int64_t camera = index / pixels;
        const int64_t pixel = index - camera * pixels;
        const uint8_t* source = frames + index * 3;
        float* target = images + camera * 3 * pixels + pixel;
#pragma unroll
        for (int channel = 0; channel < 3; ++channel) target[int64_t(channel) * pixels] = table[source[channel]];
    }
}

// One thread per four consecutive columns of a patch row (8-byte stores; 3*p*p is a multiple of 4).
__global__ void __launch_bounds__(FRAME_THREADS)
frames_to_patches_kernel(const uint8_t* __restrict__ frames, __nv_bfloat16* __restrict__ patches, int height, int width,
                         int patch, int64_t groups) {
    __shared__ float table[256];
    table[threadIdx.x] = normalized_byte(threadIdx.x);
    __syncthreads();
    const int grid_w = width / patch, grid_h = height / patch;
    const int area = patch * patch, columns = 3 * area, groups_per_row = columns >> 2;
    for (int64_t index = int64_t(blockIdx.x) * FRAME_THREADS + threadIdx.x; index < groups; index += int64_t(gridDim.x) * FRAME_THREADS) {
        const int64_t row = index / groups_per_row;               // (camera * grid_h + gy) * grid_w + gx
        const int first = int(index - row * groups_per_row) * 4;
        const int gx = int(row % grid_w), gy = int((row / grid_w) % grid_h);
        const int64_t camera = row / (int64_t(grid_w) * grid_h);
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int column = first + i;
            const int channel = column / area, inside = column - channel * area;
            const int py = inside / patch, px = inside - py * patch;
            const int64_t y = int64_t(gy) * patch + py, x = int64_t(gx) * patch + px;
            v[i] = table[frames[((camera * height + y) * width + x) * 3 + channel]];
        }
        uint2 packed;
        packed.x = float2_to_bf16x2(make_float2(v[0], v[1]));
        packed.y = float2_to_bf16x2(make_float2(v[2], v[3]));
        *reinterpret_cast<uint2*>(patches + row * columns + first) = packed;
    }
}

// Pillow's 8-bit two-pass bilinear resample (22-bit fixed-point taps, half-unit rounding offset, clamp to a byte
// after EACH pass), centred on a black canvas, then the normalisation above
// (embodiinfer/backend/cuda/csrc/camera_frames.cu:24-88, cc_resize_frames; the taps come from the host,
// embodiinfer/backend/cuda/camera_frames.py:64-90).  The reference runs the horizontal pass into a uint8 scratch
// and the vertical pass in a second launch; here one thread per canvas pixel evaluates the horizontal sums of the
// source rows its vertical taps touch and rounds each to a byte exactly as the scratch would hold it, so there is
// no scratch and one launch.  The recomputation (each horizontal sum is needed by up to `column_taps` output rows)
// is integer work on frames that sit in the L2.
constexpr int RESAMPLE_BITS = 22;

__device__ __forceinline__ int clip_to_byte(int sum) {
    const int value = sum >> RESAMPLE_BITS;
    return value < 0 ? 0 : (value > 255 ? 255 : value);
}

__global__ void __launch_bounds__(FRAME_THREADS)
resize_frames_kernel(const uint8_t* __restrict__ frames, float* __restrict__ images, const int* __restrict__ row_bounds,
                     const int* __restrict__ row_weights, int row_taps, const int* __restrict__ column_bounds,
                     const int* __restrict__ column_weights, int column_taps, int height, int width, int out_height,
                     int out_width, int canvas_height, int canvas_width, int top, int left, int64_t count) {
    __shared__ float table[256];
    table[threadIdx.x] = normalized_byte(threadIdx.x);
    __syncthreads();
    const int64_t pixels = int64_t(canvas_height) * canvas_width;
    for (int64_t index = int64_t(blockIdx.x) * FRAME_THREADS + threadIdx.x; index < count; index += int64_t(gridDim.x) * FRAME_THREADS) {
        const int64_t camera = index / pixels;
        const int64_t pixel = index - camera * pixels;
        const int y = int(pixel / canvas_width) - top, x = int(pixel % canvas_width) - left;
        int value[3] = {0, 0, 0};
        if (y >= 0 && y < out_height && x >= 0 && x < out_width) {
            const int first_row = column_bounds[2 * y], used_rows = column_bounds[2 * y + 1];
            const int first_column = row_bounds[2 * x], used_columns = row_bounds[2 * x + 1];
            const int* vertical = column_weights + int64_t(y) * column_taps;
            const int* horizontal = row_weights + int64_t(x) * row_taps;
            int sums[3] = {1 << (RESAMPLE_BITS - 1), 1 << (RESAMPLE_BITS - 1), 1 << (RESAMPLE_BITS - 1)};
            for (int i = 0; i < used_rows; ++i) {
                const uint8_t* source = frames + ((camera * height + first_row + i) * width + first_column) * 3;
                int across[3] = {1 << (RESAMPLE_BITS - 1), 1 << (RESAMPLE_BITS - 1), 1 << (RESAMPLE_BITS - 1)};
                for (int j = 0; j < used_columns; ++j) {
                    const int weight = horizontal[j];
                    across[0] += int(source[3 * j + 0]) * weight;
                    across[1] += int(source[3 * j + 1]) * weight;
                    across[2] += int(source[3 * j + 2]) * weight;
                }
                const int weight = vertical[i];
                sums[0] += clip_to_byte(across[0]) * weight;
                sums[1] += clip_to_byte(across[1]) * weight;
                sums[2] += clip_to_byte(across[2]) * weight;
            }
            value[0] = clip_to_byte(sums[0]);
            value[1] = clip_to_byte(sums[1]);
            value[2] = clip_to_byte(sums[2]);
        }
        float* target = images + camera * 3 * pixels + pixel;
        target[0] = table[value[0]];
        target[pixels] = table[value[1]];
        target[2 * pixels] = table[value[2]];
    }
}

static int blocks_for(int64_t items) {
    const int64_t wanted = (items + FRAME_THREADS - 1) / FRAME_THREADS, limit = int64_t(sm_count()) * 16;
    return int(wanted < limit ? wanted : limit);
}

int launch_normalize_frames(const void* frames, void* images, int cameras, int pixels, cudaStream_t stream) {
    const int64_t count = int64_t(cameras) * pixels;
    normalize_frames_kernel<<<blocks_for(count), FRAME_THREADS, 0, stream>>>(static_cast<const uint8_t*>(frames),
                                                                           static_cast<float*>(images), pixels, count);
    return cudaGetLastError() == cudaSuccess ? B2_OK : B2_E_DRIVER;
}

int launch_frames_to_patches(const void* frames, void* patches, int cameras, int height, int width, int patch,
                             cudaStream_t stream) {
    const int64_t groups = int64_t(cameras) * (height / patch) * (width / patch) * (3 * patch * patch / 4);
    frames_to_patches_kernel<<<blocks_for(groups), FRAME_THREADS, 0, stream>>>(
        static_cast<const uint8_t*>(frames), static_cast<__nv_bfloat16*>(patches), height, width, patch, groups);
    return cudaGetLastError() == cudaSuccess ? B2_OK : B2_E_DRIVER;
}

int launch_resize_frames(const void* frames, void* images, const void* row_bounds, const void* row_weights, int row_taps,
                         const void* column_bounds, const void* column_weights, int column_taps, int cameras, int height,
                         int width, int out_height, int out_width, int canvas_height, int canvas_width, int top, int left,
                         cudaStream_t stream) {
    const int64_t count = int64_t(cameras) * canvas_height * canvas_width;
    resize_frames_kernel<<<blocks_for(count), FRAME_THREADS, 0, stream>>>(
        static_cast<const uint8_t*>(frames), static_cast<float*>(images), static_cast<const int*>(row_bounds),
        static_cast<const int*>(row_weights), row_taps, static_cast<const int*>(column_bounds),
        static_cast<const int*>(column_weights), column_taps, height, width, out_height, out_width, canvas_height,
        canvas_width, top, left, count);
    return cudaGetLastError() == cudaSuccess ? B2_OK : B2_E_DRIVER;
}

}  // namespace b2
