// Tensor amax -> scale without any caller-provided or allocated scratch.
//
// Some hosts of this library cannot allocate device memory at the point where they need the
// activation scale: a robot-control loop that was handed a fixed arena of raw device pointers by
// another runtime, or a serving process that forbids cudaMalloc after start-up because it
// synchronises the whole device and stalls the other streams.  b2_tensor_scale asks such a caller for
// an 8-byte zeroed scratch buffer; this variant keeps its scratch inside the library instead.
//
// The scratch is a file-scope __device__ array: every GPU that loads the library holds these
// B2_STATIC_SCRATCH_BYTES until the process exits.  One array per device is shared by all calls, so
// two calls that overlap on the same GPU (different streams, or different threads) race on it; calls
// ordered on one stream are safe.  The array keeps whatever the last call left: the partial maxima are
// rewritten by every launch before they are read, and the arrival counter is cleared by a memset that
// the entry point puts on the stream ahead of the kernel.
#include "common.cuh"

#include <mutex>

namespace b2 {

constexpr int STATIC_THREADS = 256;
constexpr int STATIC_ELEMENTS_PER_CTA = 16384;                 // 64 elements per thread
constexpr int STATIC_SLOTS = 4096;                             // one partial maximum per CTA
constexpr int64_t STATIC_MAX_COUNT = int64_t(STATIC_SLOTS) * STATIC_ELEMENTS_PER_CTA;

struct StaticScratch {
    float partial[STATIC_SLOTS];
    unsigned int arrivals;
    unsigned int padding[63];
};
static_assert(sizeof(StaticScratch) == B2_STATIC_SCRATCH_BYTES, "header and kernel disagree on the scratch size");
static_assert(STATIC_MAX_COUNT == B2_STATIC_SCALE_MAX_COUNT, "header and kernel disagree on the maximum count");

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) StaticScratch static_scratch;

__global__ void __launch_bounds__(STATIC_THREADS)
tensor_scale_static_kernel(const __nv_bfloat16* __restrict__ input, int64_t count, float bound, int flags,
                           StaticScratch* scratch, float* scale) {
    const int64_t begin = int64_t(blockIdx.x) * STATIC_ELEMENTS_PER_CTA;
    const int64_t end = begin + STATIC_ELEMENTS_PER_CTA < count ? begin + STATIC_ELEMENTS_PER_CTA : count;
    float maximum = 0.0f;
    // `begin` is a multiple of 8 elements and the base pointer is 16-byte aligned: whole vectors first
    const int64_t vectors = (end - begin) >> 3;
    const uint4* vector_input = reinterpret_cast<const uint4*>(input + begin);
    for (int64_t index = threadIdx.x; index < vectors; index += STATIC_THREADS)
        maximum = fmaxf(maximum, abs_max_bf16x8(ld_nc_u4(vector_input + index)));
    for (int64_t index = begin + (vectors << 3) + threadIdx.x; index < end; index += STATIC_THREADS)
        maximum = fmaxf(maximum, fabsf(__bfloat162float(input[index])));
#pragma unroll
    for (int delta = 16; delta; delta >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, delta));
    __shared__ float warp_max[STATIC_THREADS / 32];
    __shared__ bool last_block;
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = maximum;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int warp = 1; warp < STATIC_THREADS / 32; ++warp) maximum = fmaxf(maximum, warp_max[warp]);
        scratch->partial[blockIdx.x] = maximum;
        __threadfence();
        last_block = atomicAdd(&scratch->arrivals, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!last_block) return;
    __threadfence();
    float total = 0.0f;
    for (int slot = threadIdx.x; slot < int(gridDim.x); slot += STATIC_THREADS)
        total = fmaxf(total, *(volatile float*)&scratch->partial[slot]);
#pragma unroll
    for (int delta = 16; delta; delta >>= 1) total = fmaxf(total, __shfl_xor_sync(0xffffffffu, total, delta));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = total;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int warp = 1; warp < STATIC_THREADS / 32; ++warp) total = fmaxf(total, warp_max[warp]);
        *scale = scale_from_amax(total, bound, flags);
    }
}

// Device address of the array on the current device, looked up once per device.
static int static_scratch_address(StaticScratch** address) {
    static StaticScratch* cached[64] = {nullptr};
    static std::mutex lock;
    int device = 0;
    cudaError_t error = cudaGetDevice(&device);
    if (error != cudaSuccess) return int(error);
    if (device < 0 || device >= 64) return B2_E_UNSUPPORTED;
    std::lock_guard<std::mutex> guard(lock);
    if (cached[device] == nullptr) {
        void* pointer = nullptr;
        error = cudaGetSymbolAddress(&pointer, static_scratch);
        if (error != cudaSuccess) return int(error);
        cached[device] = static_cast<StaticScratch*>(pointer);
    }
    *address = cached[device];
    return B2_OK;
}

int launch_tensor_scale_static(const void* input, int64_t count, float bound, int flags, void* scale,
                               cudaStream_t stream) {
    if (count > STATIC_MAX_COUNT) return B2_E_TOO_LARGE;
    StaticScratch* scratch = nullptr;
    const int status = static_scratch_address(&scratch);
    if (status != B2_OK) return status;
    cudaError_t error = cudaMemsetAsync(&scratch->arrivals, 0, sizeof(unsigned int), stream);
    if (error != cudaSuccess) return int(error);
    const int grid = int((count + STATIC_ELEMENTS_PER_CTA - 1) / STATIC_ELEMENTS_PER_CTA);
    tensor_scale_static_kernel<<<grid, STATIC_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(input), count,
                                                                   bound, flags, scratch, static_cast<float*>(scale));
    return int(cudaGetLastError());
}

}  // namespace b2
