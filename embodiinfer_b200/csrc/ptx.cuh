// Thin inline-PTX wrappers for the sm_100a features the kernels use:
// mbarrier, TMA (cp.async.bulk[.tensor]), tcgen05 (TMEM alloc / mma / cp / ld / commit).
// No cluster multicast is used anywhere: every load targets the issuing CTA only.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

namespace b2 {

// Status words a kernel may leave in the caller-visible status buffer.
enum : unsigned int {
    STATUS_OK = 0,
    STATUS_WAIT_PRODUCER = 0x101,   // TMA producer gave up waiting for a free stage
    STATUS_WAIT_MMA_FULL = 0x102,   // MMA issuer gave up waiting for a filled stage
    STATUS_WAIT_MMA_TMEM = 0x103,   // MMA issuer gave up waiting for a drained accumulator
    STATUS_WAIT_EPILOGUE = 0x104,   // epilogue gave up waiting for a finished accumulator
    STATUS_WAIT_DRAIN = 0x105,      // producer gave up waiting for its copies in flight
    STATUS_WAIT_SPLIT = 0x106,      // split K: a CTA gave up waiting for the other K ranges of its tile
    STATUS_WAIT_EXCHANGE = 0x107,   // cluster split K: a CTA gave up waiting for the partial sums of its cluster
    STATUS_WAIT_ATTENTION_EXCHANGE = 0x108,   // split attention: a CTA gave up waiting for the partial rows of its cluster
};

// Upper bound, in SM clock cycles, for any single wait (about a second).
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* pointer) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait.  After the first expiry the caller's `failed` flag stays set and
// every later wait of that thread returns at once, so a broken pipeline drains in
// bounded time instead of spinning.  The first expiry records `code` in *status.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, bool& failed,
                                          unsigned int* status, unsigned int code) {
    if (mbar_try_wait(bar, parity)) return true;
    if (failed) return false;
    const long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > WAIT_LIMIT_CYCLES) {
            failed = true;
            if (status != nullptr) atomicCAS(status, 0u, code);
            return false;
        }
    }
    return true;
}

// One lane of a fully converged warp.  The roles that feed the asynchronous units (TMA, tensor pipe) run
// their loops on all 32 lanes and predicate only the issuing instructions with this: the address and
// descriptor arithmetic then stays warp-uniform, which the compiler keeps in uniform registers, the
// operand form those instructions take.  The same loop run by a single thread of a diverged warp needs
// a register-to-uniform move per operand and issues each tcgen05 instruction several times more slowly
// (measured: 8 scale copies + 4 MMAs per K stage in 322 cycles instead of 535).
__device__ __forceinline__ bool elect_one() {
    uint32_t elected;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(elected));
    return elected != 0;
}

// ---- TMA -----------------------------------------------------------------

__device__ __forceinline__ void tma_prefetch_descriptor(const void* tensor_map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tensor_map)) : "memory");
}

// 2-D tiled load into this CTA's shared memory; x is the innermost coordinate.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tensor_map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// Three-dimensional box (x innermost): used for the packed [gate; up] weight, whose two row ranges of a tile
// arrive with one instruction as planes z = 0 (gate) and z = 1 (up), one behind the other in shared memory.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tensor_map, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ void tma_prefetch_l2_3d(const void* tensor_map, int x, int y, int z) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
                 ::"l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}

// Hints the L2 to fetch one box of a tensor map / a byte range ahead of the loads that will need it.
__device__ __forceinline__ void tma_prefetch_l2_2d(const void* tensor_map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                 ::"l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(src)), "r"(bytes) : "memory");
}

// Untiled bulk copy global -> this CTA's shared memory (16-byte aligned, size % 16 == 0).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
        : "memory");
}

// ---- tcgen05 ---------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Makes the mbarrier track completion of all tcgen05 operations issued so far by this thread.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], e4m3 operands, fp32 accumulate.
__device__ __forceinline__ void mma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Block-scaled e2m1 x e2m1 with one ue4m3 scale per 16 elements, scales read from TMEM.
__device__ __forceinline__ void mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// Shared memory -> TMEM: 32 rows x 16 bytes, replicated into the four 32-lane partitions.
__device__ __forceinline__ void tc_copy_32x128b_x4(uint32_t dst_tmem, uint64_t src_desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(dst_tmem), "l"(src_desc) : "memory");
}

// Each thread of the warp reads 32 consecutive fp32 columns of its own TMEM lane.
__device__ __forceinline__ void tmem_load_32x32(uint32_t address, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(address)
        : "memory");
}

__device__ __forceinline__ void tmem_load_32x16(uint32_t address, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(address)
        : "memory");
}

__device__ __forceinline__ void tmem_load_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- descriptors -----------------------------------------------------------

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes and
// which was written with the 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_address) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_address & 0x3FFFF) >> 4);   // start address
    desc |= static_cast<uint64_t>(1) << 16;                          // leading byte offset (unused with swizzle)
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;                  // stride byte offset: 8 rows * 128 B
    desc |= static_cast<uint64_t>(1) << 46;                          // descriptor version for sm_100
    desc |= static_cast<uint64_t>(2) << 61;                          // SWIZZLE_128B
    return desc;
}

// Descriptor for an unswizzled 32-row x 16-byte scale-factor atom (rows 16 bytes apart).
__device__ __forceinline__ uint64_t smem_desc_scale_atom(uint32_t smem_address) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_address & 0x3FFFF) >> 4);
    desc |= static_cast<uint64_t>(128 >> 4) << 32;                   // 8 rows * 16 B between row groups
    desc |= static_cast<uint64_t>(1) << 46;
    return desc;
}

// A descriptor whose address field alone varies: the low word is (address >> 4) plus the constant low bits,
// so stepping through a tile is one 32-bit add (the 14-bit address field never carries: shared memory ends
// below 2^18).
__device__ __forceinline__ uint64_t desc_from_words(uint32_t low, uint32_t high) {
    uint64_t desc;
    asm("mov.b64 %0, {%1, %2};" : "=l"(desc) : "r"(low), "r"(high));
    return desc;
}

// Instruction descriptor, kind::f8f6f4, e4m3 x e4m3 -> fp32, both operands K-major.
__device__ __forceinline__ uint32_t idesc_f8(uint32_t m, uint32_t n) {
    return (1u << 4)            // D format fp32
         | (0u << 7)            // A = e4m3
         | (0u << 10)           // B = e4m3
         | ((n >> 3) << 17)
         | ((m >> 4) << 24);
}

// Instruction descriptor, kind::mxf4nvf4, e2m1 x e2m1, ue4m3 scales, both K-major, K = 64.
__device__ __forceinline__ uint32_t idesc_nvf4(uint32_t m, uint32_t n) {
    return (1u << 7)            // A = e2m1
         | (1u << 10)           // B = e2m1
         | ((n >> 3) << 17)
         | (0u << 23)           // scale format ue4m3
         | ((m >> 4) << 24);
}

// ---- thread-block clusters: rank, barrier, distributed shared memory ----------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}

// Hardware barrier over every thread of every CTA of the cluster (release / acquire: shared-memory writes made
// before the arrive, to any CTA of the cluster, are visible after the wait).  Each thread calls both, once per phase.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }

// Address, in the cluster's shared window, of this CTA's shared address `local` in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t cluster_map_shared(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}

__device__ __forceinline__ void cluster_store_u4(uint32_t remote, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

}  // namespace b2
