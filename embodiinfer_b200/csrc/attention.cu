// Multi-query attention for the Gemma-shaped towers: head dimension 256, one key/value head shared by all query
// heads, no mask (the prefix attends to itself; the action expert's ten-token chunk attends to prefix + chunk).
//
//   out[b, h, t, :] = softmax(q[b, h, t, :] . k[b, :, :]^T / sqrt(256)) v[b, :, :]
//
// It replaces the attention the reference computes between its QKV projection and its output projection
// (embodiinfer/backend/torch/attention.py:97-106, `SDPAAttention`: torch's scaled_dot_product_attention on
// [B, H, T, D] queries and [B, 1, S, D] keys / values, bf16) and, for the ten-query case, the job of
// backend/cuda/csrc/mqa_decode_attention.cu:170-393 -- not that kernel's structure (it merges key splits behind a grid
// barrier that spins without a bound).
//
// Because every query head reads the same keys and values, the H x T query rows of one batch element are one matrix:
// a CTA takes 128 of those rows and walks the keys in tiles of 64.
//   warp 0      TMA producer: the query tile once, then key and value tiles through two-stage rings
//   warp 1      tensor-memory owner and MMA issuer: S = Q K^T (128 x 64, K = 256) and O += P V (128 x 256, K = 64),
//               bf16 operands, fp32 accumulators in tensor memory; V is used as it lies in memory ([key][d], the MN-major
//               operand form), no transpose anywhere
//   warps 2-5   one thread per query row: scores from tensor memory, running reference and sum (base-2 exponentials of
//               scores pre-multiplied by log2(e)/16), probabilities as bf16 into shared memory in the operand layout the
//               second MMA reads, rescaling of the output accumulator when the reference moved, final 1/sum and store
// S is double-buffered, so the scores of the next key tile are computed while this one's probabilities are formed.
// Every wait is bounded and reports through the status word, as in the GEMM kernels.
//
// Few rows (one observation's ten-token chunk is 80 rows: a single CTA walking all ten key tiles): the keys are cut
// across the CTAs of a thread-block cluster instead (SPLIT).  Every CTA runs the loop above on its own key tiles and
// ends with an unnormalised output, a reference m and a sum l per row; the rows are dealt to the CTAs in runs of T, each
// CTA sends every other CTA the rows that one owns (one bulk copy per owner through distributed shared memory) and the
// owner combines them in rank order:
//   out = sum_r 2^(m_r - M) O_r / sum_r 2^(m_r - M) l_r,   M = max_r m_r.
// A partial row travels as 256 fp16 values c_r O_r with c_r the power of two that brings the row's largest magnitude
// into [1, 2) (so no range of inputs overflows and the rounding, 2^-11 of the row's maximum, is a quarter of the
// output's own bf16 rounding), followed by m_r, l_r and 1 / c_r in fp32: 528 bytes instead of 1040 -- the exchange moves
// every row to its owner at some 18 bytes per cycle and SM, which is what bounds these launches.
// The exchange buffers lie over the query / key / value stages, which are dead by then in every CTA of the cluster: a
// hardware cluster barrier separates the two uses.
#include "gemm_epilogue.cuh"

#include <cuda.h>
#include <cuda_fp16.h>

#include <type_traits>

namespace b2 {

namespace {

constexpr int ATT_D = 256;                       // head dimension
constexpr int ATT_ROWS = 128;                    // query rows per CTA
constexpr int ATT_KEYS = 64;                     // keys per tile
constexpr int ATT_ATOM_BYTES = 128;              // bytes of one swizzled row: 64 bf16
constexpr int ATT_D_ATOMS = ATT_D * 2 / ATT_ATOM_BYTES;      // 4 column groups of 64 elements
constexpr uint32_t Q_ATOM_BYTES = ATT_ROWS * ATT_ATOM_BYTES;  // 16 KB
constexpr uint32_t KV_ATOM_BYTES = ATT_KEYS * ATT_ATOM_BYTES; // 8 KB
constexpr uint32_t Q_BYTES = ATT_D_ATOMS * Q_ATOM_BYTES;      // 64 KB
constexpr uint32_t KV_STAGE_BYTES = ATT_D_ATOMS * KV_ATOM_BYTES;   // 32 KB
constexpr uint32_t P_BYTES = ATT_ROWS * ATT_ATOM_BYTES;       // 16 KB: 128 rows x 64 keys of bf16
constexpr int ATT_THREADS = 32 * 6;
constexpr int ATT_SHARED_BYTES = 1024 + int(Q_BYTES + 4 * KV_STAGE_BYTES + 2 * P_BYTES) + 256;
constexpr uint32_t TMEM_S = 0, TMEM_O = 128;     // two score buffers of 64 columns, then 256 output columns
constexpr uint32_t SPLIT_ROW_BYTES = 528;        // 256 outputs as fp16, then reference, sum and row scale as fp32, 4 bytes of padding:
                                                 // rows start 4 banks apart

__device__ __forceinline__ bool mbar_try_wait_cluster_scope(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

__device__ __forceinline__ void bulk_copy_rows_to_cluster(uint32_t dst, uint32_t src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "r"(src), "r"(bytes), "r"(bar) : "memory");
}

// Instruction descriptor, kind::f16: bf16 x bf16 -> fp32, A K-major, B K-major or MN-major.
__device__ __forceinline__ uint32_t idesc_bf16(uint32_t m, uint32_t n, bool b_mn_major) {
    return (1u << 4)            // D format fp32
         | (1u << 7)            // A = bf16
         | (1u << 10)           // B = bf16
         | (uint32_t(b_mn_major) << 16)
         | ((n >> 3) << 17)
         | ((m >> 4) << 24);
}

// Shared-memory descriptor of an MN-major operand written by TMA with the 128-byte swizzle as [k][64 elements]:
// a 128-byte row holds 64 consecutive MN elements of one k; 8 consecutive k are 1024 bytes apart per group (stride
// byte offset), the next 64 MN elements start `mn_group_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t smem_address, uint32_t mn_group_bytes) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_address & 0x3FFFF) >> 4);
    desc |= static_cast<uint64_t>(mn_group_bytes >> 4) << 16;
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;
    desc |= static_cast<uint64_t>(1) << 46;
    desc |= static_cast<uint64_t>(2) << 61;
    return desc;
}

__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tmem_store_32x32(uint32_t address, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(address), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Four bf16 pairs -> eight e4m3 codes at a static multiplier: the arithmetic of the stand-alone output encoder
// (bhsd_encode_kernel, bits 8): e4m3(bf16 value * multiplier), saturating.
__device__ __forceinline__ uint2 encode_row_words(const uint32_t (&words)[4], float multiplier) {
    const float2 factor = make_float2(multiplier, multiplier);
    uint32_t codes[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        codes[i] = __nv_cvt_float2_to_fp8x2(__fmul2_rn(bf16x2_to_float2(words[i]), factor), __NV_SATFINITE, __NV_E4M3);
    return make_uint2(codes[0] | (codes[1] << 16), codes[2] | (codes[3] << 16));
}

// Eight values of an NVFP4 block whose other eight the neighbouring lane (lane ^ 1) holds -> eight e2m1 codes and the
// block's e4m3 scale: the arithmetic of the stand-alone output encoder (bhsd_encode_kernel, bits 4; quantize.cu:85-104).
// Every lane of the warp calls this.
__device__ __forceinline__ uint32_t encode_half_block_nvfp4(const uint32_t (&words)[4], float global, const ExactDivider& by_global,
                                                            uint8_t& scale_code) {
    float maximum = abs_max_bf16_words(words);
    maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, 1));
    scale_code = nvfp4_block_scale<true>(maximum, by_global, 0);
    const ExactDivider denominator(__fmul_rn(global, e4m3_to_float(scale_code)));
    if (denominator.fast && __fmul_rn(maximum, denominator.reciprocal) < 1.0e30f)
        return nvfp4_encode_words_short<true>(words[0], words[1], words[2], words[3], denominator);
    float values[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        values[2 * i] = bf16_lo(words[i]);
        values[2 * i + 1] = bf16_hi(words[i]);
    }
    return nvfp4_encode_x8<true>(values, denominator, maximum);
}

struct AttentionArgs {
    __nv_bfloat16* out;          // [batch, heads * queries, 256], or nullptr when `codes` is given
    uint8_t* codes;              // e4m3 [batch * queries, heads * 256]: the encoded rows of the output projection, or nullptr
    float multiplier;            // codes = e4m3(bf16(out) * multiplier)
    uint8_t* blocked;            // given: `codes` are e2m1 pairs [batch * queries, heads * 128] instead, with their e4m3 block
                                 // scales here in 128 x 4 tile order (the stand-alone output encoder's bits = 4 form)
    uint8_t* block_scales;       // the same block scales row-major [batch * queries, heads * 16], or nullptr
    float global_scale;          // NVFP4: the projection's static global scale
    int queries;                 // queries per head (row of a batch element = head * queries + query)
    unsigned int* status;
    int rows_per_batch;          // heads * queries
    int keys;                    // keys (= values) per batch element
    int tiles_per_batch;
    float scale_log2;            // log2(e) / sqrt(256)
    int splits;                  // SPLIT: CTAs of a cluster = key ranges of one 128-row tile
    int rows_per_rank;           // SPLIT: rows whose partial results a CTA combines (T)
};

template <bool SPLIT>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attention_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                 const __grid_constant__ CUtensorMap v_map, const AttentionArgs args) {
    pdl_launch_dependents();
    extern __shared__ uint8_t shared_raw[];
    const uint32_t base = (smem_u32(shared_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = base;
    const uint32_t k_smem = q_smem + Q_BYTES;                 // [2 stages]
    const uint32_t v_smem = k_smem + 2 * KV_STAGE_BYTES;      // [2 stages]
    const uint32_t p_smem = v_smem + 2 * KV_STAGE_BYTES;      // [2 buffers]
    const uint32_t bars = p_smem + 2 * P_BYTES;
    const uint32_t q_full = bars;
    const uint32_t k_full = bars + 8, k_empty = bars + 24, v_full = bars + 40, v_empty = bars + 56;      // [2] each
    const uint32_t s_full = bars + 72, s_free = bars + 88, p_ready = bars + 104, p_free = bars + 120;    // [2] each
    const uint32_t o_done = bars + 136;
    const uint32_t tmem_slot = bars + 144;
    const uint32_t receive_bar = bars + 152;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t splits = SPLIT ? uint32_t(args.splits) : 1u;
    const uint32_t rank = SPLIT ? cluster_cta_rank() : 0u;
    const int work = SPLIT ? int(blockIdx.x) / args.splits : int(blockIdx.x);
    const int batch = work / args.tiles_per_batch;
    const int tile = work - batch * args.tiles_per_batch;
    const int row0 = tile * ATT_ROWS;                                   // within the batch element
    const int all_key_tiles = (args.keys + ATT_KEYS - 1) / ATT_KEYS;
    const int first_key_tile = SPLIT ? int(rank) * all_key_tiles / args.splits : 0;
    const int num_key_tiles = SPLIT ? (int(rank) + 1) * all_key_tiles / args.splits - first_key_tile : all_key_tiles;   // of this CTA (>= 1)
    // SPLIT: rows of the tile that exist, and the exchange buffers over the dead operand stages
    int tile_rows = args.rows_per_batch - row0;
    if (tile_rows > ATT_ROWS) tile_rows = ATT_ROWS;
    const uint32_t staging = base;
    const uint32_t receive_base = staging + uint32_t(tile_rows) * SPLIT_ROW_BYTES;

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&q_map);
        tma_prefetch_descriptor(&k_map);
        tma_prefetch_descriptor(&v_map);
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full + 8 * i, 1);
            mbar_init(k_empty + 8 * i, 1);
            mbar_init(v_full + 8 * i, 1);
            mbar_init(v_empty + 8 * i, 1);
            mbar_init(s_full + 8 * i, 1);
            mbar_init(s_free + 8 * i, 4);        // the four softmax warps
            mbar_init(p_ready + 8 * i, 4);
            mbar_init(p_free + 8 * i, 1);
        }
        mbar_init(o_done, 1);
        if (SPLIT) mbar_init(receive_bar, 1);
        fence_barrier_init();
        if (SPLIT) {      // the bytes this CTA will receive: a partial row from every CTA for each row it owns
            int owned = tile_rows - int(rank) * args.rows_per_rank;
            owned = owned < 0 ? 0 : (owned > args.rows_per_rank ? args.rows_per_rank : owned);
            mbar_expect_tx(receive_bar, splits * uint32_t(owned) * SPLIT_ROW_BYTES);
        }
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLUMNS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");
    pdl_wait();

    bool failed = false;
    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer
        const int q_row = batch * args.rows_per_batch + row0;
        const int kv_row = batch * args.keys;
        if (elect_one()) {
            mbar_expect_tx(q_full, Q_BYTES);
            for (int a = 0; a < ATT_D_ATOMS; ++a) tma_load_2d(q_smem + a * Q_ATOM_BYTES, &q_map, q_full, a * ATT_ATOM_BYTES, q_row);
        }
        __syncwarp();
        for (int j = 0; j < num_key_tiles; ++j) {
            const int b = j & 1;
            const uint32_t parity = uint32_t(j >> 1) & 1u;
            mbar_wait(k_empty + 8 * b, parity ^ 1u, failed, args.status, STATUS_WAIT_PRODUCER);
            __syncwarp();
            if (elect_one()) {
                mbar_expect_tx(k_full + 8 * b, KV_STAGE_BYTES);
                for (int a = 0; a < ATT_D_ATOMS; ++a)
                    tma_load_2d(k_smem + b * KV_STAGE_BYTES + a * KV_ATOM_BYTES, &k_map, k_full + 8 * b, a * ATT_ATOM_BYTES, kv_row + (first_key_tile + j) * ATT_KEYS);
            }
            __syncwarp();
            mbar_wait(v_empty + 8 * b, parity ^ 1u, failed, args.status, STATUS_WAIT_PRODUCER);
            __syncwarp();
            if (elect_one()) {
                mbar_expect_tx(v_full + 8 * b, KV_STAGE_BYTES);
                for (int a = 0; a < ATT_D_ATOMS; ++a)
                    tma_load_2d(v_smem + b * KV_STAGE_BYTES + a * KV_ATOM_BYTES, &v_map, v_full + 8 * b, a * ATT_ATOM_BYTES, kv_row + (first_key_tile + j) * ATT_KEYS);
            }
            __syncwarp();
        }
        // do not leave while a copy is in flight: the last fill of every stage has landed when the MMAs that read it were
        // issued, and those complete before the row threads finish; the waits below only bound the abnormal path
        bool drain_failed = false;
        mbar_wait(q_full, 0u, drain_failed, args.status, STATUS_WAIT_DRAIN);
        for (int b = 0; b < 2 && b < num_key_tiles; ++b) {
            const int last = ((num_key_tiles - 1 - b) / 2) * 2 + b;      // last tile that used stage b
            mbar_wait(k_full + 8 * b, uint32_t(last >> 1) & 1u, drain_failed, args.status, STATUS_WAIT_DRAIN);
            mbar_wait(v_full + 8 * b, uint32_t(last >> 1) & 1u, drain_failed, args.status, STATUS_WAIT_DRAIN);
        }
        if (SPLIT) {
            cluster_arrive();
            cluster_wait();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer
        const uint32_t idesc_scores = idesc_bf16(ATT_ROWS, ATT_KEYS, false);
        const uint32_t idesc_output = idesc_bf16(ATT_ROWS, ATT_D, true);
        const uint64_t k_major = smem_desc_sw128(0);
        const uint32_t k_major_low = uint32_t(k_major), k_major_high = uint32_t(k_major >> 32);
        const uint64_t mn_major = smem_desc_sw128_mn(0, KV_ATOM_BYTES);
        const uint32_t mn_major_low = uint32_t(mn_major), mn_major_high = uint32_t(mn_major >> 32);
        // Descriptor address field: the low 18 bits of the shared address, in units of 16 bytes.  The mask matters: in a
        // cluster launch the shared window of every CTA but rank 0 has bits above those, which would spill into the
        // leading-byte-offset field next to it (the K-major operands ignore that field, the MN-major V operand does not).
        auto field = [](uint32_t address) { return (address & 0x3FFFFu) >> 4; };
        mbar_wait(q_full, 0u, failed, args.status, STATUS_WAIT_MMA_FULL);
        tc_fence_after_sync();
        auto scores = [&](int j) {          // S[j & 1] = Q K_j^T
            const int b = j & 1;
            const uint32_t parity = uint32_t(j >> 1) & 1u;
            mbar_wait(k_full + 8 * b, parity, failed, args.status, STATUS_WAIT_MMA_FULL);
            mbar_wait(s_free + 8 * b, parity ^ 1u, failed, args.status, STATUS_WAIT_MMA_TMEM);
            tc_fence_after_sync();
            __syncwarp();
            if (elect_one()) {
                const uint32_t d_tmem = tmem_base + TMEM_S + uint32_t(b) * ATT_KEYS;
#pragma unroll
                for (int a = 0; a < ATT_D_ATOMS; ++a) {
                    const uint32_t q_low = k_major_low + field(q_smem + a * Q_ATOM_BYTES);
                    const uint32_t k_low = k_major_low + field(k_smem + b * KV_STAGE_BYTES + a * KV_ATOM_BYTES);
#pragma unroll
                    for (int s = 0; s < 4; ++s)          // 16 elements of D = 32 bytes per MMA
                        mma_bf16(d_tmem, desc_from_words(q_low + 2 * s, k_major_high), desc_from_words(k_low + 2 * s, k_major_high),
                                 idesc_scores, (a | s) != 0);
                }
                tc_commit(k_empty + 8 * b);
                tc_commit(s_full + 8 * b);
            }
            __syncwarp();
        };
        auto output = [&](int j) {          // O += P[j & 1] V_j
            const int b = j & 1;
            const uint32_t parity = uint32_t(j >> 1) & 1u;
            mbar_wait(v_full + 8 * b, parity, failed, args.status, STATUS_WAIT_MMA_FULL);
            mbar_wait(p_ready + 8 * b, parity, failed, args.status, STATUS_WAIT_MMA_TMEM);
            tc_fence_after_sync();
            __syncwarp();
            if (elect_one()) {
                const uint32_t p_low = k_major_low + field(p_smem + b * P_BYTES);
                const uint32_t v_low = mn_major_low + field(v_smem + b * KV_STAGE_BYTES);
#pragma unroll
                for (int s = 0; s < ATT_KEYS / 16; ++s)   // 16 keys per MMA: 32 bytes along a row of P, 16 rows (2048 bytes) of V
                    mma_bf16(tmem_base + TMEM_O, desc_from_words(p_low + 2 * s, k_major_high),
                             desc_from_words(v_low + s * (2048 >> 4), mn_major_high), idesc_output, (j | s) != 0);
                tc_commit(v_empty + 8 * b);
                tc_commit(p_free + 8 * b);
                tc_commit(o_done);
            }
            __syncwarp();
        };
        scores(0);
        for (int j = 0; j < num_key_tiles; ++j) {
            if (j + 1 < num_key_tiles) scores(j + 1);
            output(j);
        }
        if (SPLIT) {
            cluster_arrive();
            cluster_wait();
        }
    } else {
        // ------------------------------------------------------------- one thread per query row
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                 // row of the tile = tensor-memory lane
        const uint32_t lane_address = tmem_base + (uint32_t(quarter * 32) << 16);
        float running_max = -INFINITY, running_sum = 0.0f;
        for (int j = 0; j < num_key_tiles; ++j) {
            const int b = j & 1;
            const uint32_t parity = uint32_t(j >> 1) & 1u;
            mbar_wait(s_full + 8 * b, parity, failed, args.status, STATUS_WAIT_EPILOGUE);
            tc_fence_after_sync();
            uint32_t raw[2][32];
            tmem_load_32x32(lane_address + TMEM_S + uint32_t(b) * ATT_KEYS, raw[0]);
            tmem_load_32x32(lane_address + TMEM_S + uint32_t(b) * ATT_KEYS + 32, raw[1]);
            tmem_load_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free + 8 * b);      // the scores of key tile j + 2 may overwrite this buffer
            const int valid = args.keys - (first_key_tile + j) * ATT_KEYS;     // keys of this tile that exist
            if (valid < ATT_KEYS) {                          // last tile: keys beyond the end never win the maximum and add nothing
#pragma unroll
                for (int half = 0; half < 2; ++half)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (half * 32 + i >= valid) raw[half][i] = __float_as_uint(-INFINITY);
            }
            // of the raw scores (the scale is positive); four independent chains, this thread is alone on its scheduler
            float partial_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int half = 0; half < 2; ++half)
#pragma unroll
                for (int i = 0; i < 32; ++i) partial_max[i & 3] = fmaxf(partial_max[i & 3], __uint_as_float(raw[half][i]));
            const float tile_max = fmaxf(fmaxf(partial_max[0], partial_max[1]), fmaxf(partial_max[2], partial_max[3])) * args.scale_log2;
            // The exponentials are taken relative to a reference that follows the row maximum lazily: it moves only when
            // the maximum has grown by more than 2^8 since it was set (probabilities then stay below 256, far inside the
            // range of bf16 and fp32, and the final division by the sum is exact whatever the reference), so the output
            // accumulator in tensor memory is rescaled a few times per row instead of once per key tile.
            const bool move = tile_max > running_max + 8.0f;                  // always on the first tile (running_max = -inf)
            const float new_max = move ? tile_max : running_max;
            const float correction = move ? exp2_approx(running_max - new_max) : 1.0f;      // 0 on the first tile
            running_max = new_max;
            float partial_sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t packed[2][16];
#pragma unroll
            for (int half = 0; half < 2; ++half)
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    // 2^(score * log2(e)/16 - reference) in one multiply-add per value
                    const float p0 = exp2_approx(__fmaf_rn(__uint_as_float(raw[half][2 * i]), args.scale_log2, -new_max));
                    const float p1 = exp2_approx(__fmaf_rn(__uint_as_float(raw[half][2 * i + 1]), args.scale_log2, -new_max));
                    packed[half][i] = float2_to_bf16x2(make_float2(p0, p1));
                    partial_sum[i & 3] += p0 + p1;
                }
            const float tile_sum = (partial_sum[0] + partial_sum[1]) + (partial_sum[2] + partial_sum[3]);
            running_sum = running_sum * correction + tile_sum;
            // P[b]: row `row`, 64 keys = 128 bytes = 8 chunks of 16 bytes, chunk c stored at c ^ (row % 8) (128-byte swizzle)
            mbar_wait(p_free + 8 * b, parity ^ 1u, failed, args.status, STATUS_WAIT_EPILOGUE);
            const uint32_t p_row = p_smem + b * P_BYTES + uint32_t(row >> 3) * 1024u + uint32_t(row & 7) * 128u;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint32_t* w = &packed[c >> 2][(c & 3) * 4];
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + uint32_t((c ^ (row & 7)) * 16)), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
            }
            // the accumulator holds the sum over the tiles before this one in units of the old maximum
            if (j > 0) {
                mbar_wait(o_done, uint32_t(j - 1) & 1u, failed, args.status, STATUS_WAIT_EPILOGUE);
                tc_fence_after_sync();
                if (__any_sync(0xffffffffu, correction != 1.0f)) {
#pragma unroll 1
                    for (int chunk = 0; chunk < ATT_D / 32; ++chunk) {
                        uint32_t o[32];
                        tmem_load_32x32(lane_address + TMEM_O + chunk * 32, o);
                        tmem_load_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * correction);
                        tmem_store_32x32(lane_address + TMEM_O + chunk * 32, o);
                    }
                    tmem_store_wait();
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // P, written by these threads, is read by the tensor core
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready + 8 * b);
        }
        mbar_wait(o_done, uint32_t(num_key_tiles - 1) & 1u, failed, args.status, STATUS_WAIT_EPILOGUE);
        tc_fence_after_sync();
        const bool row_exists = row0 + row < args.rows_per_batch;
        if (SPLIT) {
            // (a) this CTA's partial rows into its own shared memory (the operand stages are dead: every MMA of this CTA has
            //     completed): the row's largest magnitude first, then the scaled values as fp16
            const int reader = (warp - 2) * 32 + lane;
            const uint32_t my_row = staging + uint32_t(row) * SPLIT_ROW_BYTES;
            float largest = 0.0f;
#pragma unroll 1
            for (int chunk = 0; chunk < ATT_D / 32; chunk += 2) {       // two loads in flight per wait
                uint32_t o[2][32];
                tmem_load_32x32(lane_address + TMEM_O + chunk * 32, o[0]);
                tmem_load_32x32(lane_address + TMEM_O + chunk * 32 + 32, o[1]);
                tmem_load_wait();
                float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    part[i & 3] = fmaxf(part[i & 3], fabsf(__uint_as_float(o[0][i])));
                    part[i & 3] = fmaxf(part[i & 3], fabsf(__uint_as_float(o[1][i])));
                }
                largest = fmaxf(fmaxf(largest, fmaxf(part[0], part[1])), fmaxf(part[2], part[3]));
            }
            // 2^-(exponent of the largest magnitude); 1 for an all-zero row and for infinities / NaNs (which then travel as they are)
            uint32_t exponent = __float_as_uint(largest) & 0x7f800000u;
            const bool unscaled = exponent == 0u || exponent == 0x7f800000u;
            if (exponent > 0x7e000000u) exponent = 0x7e000000u;            // keeps the scale itself a normal number
            const float row_scale = unscaled ? 1.0f : __uint_as_float(0x7f000000u - exponent);
            const float row_unscale = unscaled ? 1.0f : __uint_as_float(exponent);          // 1 / row_scale, exactly
#pragma unroll 1
            for (int chunk = 0; chunk < ATT_D / 32; chunk += 2) {
                uint32_t o[2][32];
                tmem_load_32x32(lane_address + TMEM_O + chunk * 32, o[0]);
                tmem_load_32x32(lane_address + TMEM_O + chunk * 32 + 32, o[1]);
                tmem_load_wait();
                if (row_exists) {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t h[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const __half2 pair = __floats2half2_rn(__uint_as_float(o[half][2 * i]) * row_scale, __uint_as_float(o[half][2 * i + 1]) * row_scale);
                            h[i] = *reinterpret_cast<const uint32_t*>(&pair);
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + uint32_t((chunk + half) * 64 + q * 16)),
                                         "r"(h[4 * q]), "r"(h[4 * q + 1]), "r"(h[4 * q + 2]), "r"(h[4 * q + 3]) : "memory");
                    }
                }
            }
            if (row_exists)
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + 512u), "f"(running_max), "f"(running_sum), "f"(row_unscale), "f"(0.0f) : "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the copies below read these rows through the async proxy
            // (b) first cluster barrier: every CTA of the cluster has finished with its operand stages, so partial rows may
            //     land on them
            cluster_arrive();
            cluster_wait();
            if (uint32_t(reader) < splits) {      // one copy per thread, starting with the next rank: no owner is everyone's first
                const uint32_t step = uint32_t(reader) + 1u;
                const uint32_t r = rank + step < splits ? rank + step : rank + step - splits;
                const int first = int(r) * args.rows_per_rank;
                int count = tile_rows - first;
                if (count > args.rows_per_rank) count = args.rows_per_rank;
                if (count > 0)
                    bulk_copy_rows_to_cluster(cluster_map_shared(receive_base + rank * uint32_t(args.rows_per_rank) * SPLIT_ROW_BYTES, r),
                                              staging + uint32_t(first) * SPLIT_ROW_BYTES, uint32_t(count) * SPLIT_ROW_BYTES,
                                              cluster_map_shared(receive_bar, r));
            }
            // (c) the rows this CTA owns: weights 2^(m_r - M) / sum_r 2^(m_r - M) l_r per row, then the weighted sum in rank
            //     order, 16 bytes of a row per thread and step
            if (!failed) {
                const long long start = clock64();
                while (!mbar_try_wait_cluster_scope(receive_bar, 0u)) {
                    if (clock64() - start > WAIT_LIMIT_CYCLES) {
                        failed = true;
                        if (args.status != nullptr) atomicCAS(args.status, 0u, STATUS_WAIT_ATTENTION_EXCHANGE);
                        break;
                    }
                }
            }
            const int first_row = int(rank) * args.rows_per_rank;
            int owned = tile_rows - first_row;
            if (owned > args.rows_per_rank) owned = args.rows_per_rank;
            const uint32_t rank_stride = uint32_t(args.rows_per_rank) * SPLIT_ROW_BYTES;
            __nv_bfloat16* tile_out = args.out + (int64_t(batch) * args.rows_per_batch + row0 + first_row) * ATT_D;
            // The cluster size is a compile-time constant of the loop body (one copy per size, chosen below): with a run-time
            // bound every partial row is its own basic block and the single warp of a scheduler crawls through them.
            const ExactDivider by_global(__fmul_rn(6.0f, args.global_scale));
            auto combine = [&](auto size_tag) {
                constexpr uint32_t SIZE = decltype(size_tag)::value;
                for (int slot = reader; slot < owned * 32; slot += 128) {
                    const uint32_t local = uint32_t(slot) >> 5, column = uint32_t(slot) & 31u;      // 16 bytes = 8 values of a row
                    const uint32_t row_address = receive_base + local * SPLIT_ROW_BYTES;
                    // the row's weights 2^(m_r - M) / (c_r sum_r 2^(m_r - M) l_r): every thread works them out for its own slot
                    // (the loads are the same address across a warp), which is cheaper than a table, a barrier and idle warps
                    float weight[SIZE];
                    {
                        float4 tail[SIZE];
#pragma unroll
                        for (uint32_t r = 0; r < SIZE; ++r)
                            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(tail[r].x), "=f"(tail[r].y), "=f"(tail[r].z), "=f"(tail[r].w)
                                         : "r"(row_address + r * rank_stride + 512u) : "memory");
                        float top = tail[0].x;
#pragma unroll
                        for (uint32_t r = 1; r < SIZE; ++r) top = fmaxf(top, tail[r].x);
                        float total = 0.0f;
#pragma unroll
                        for (uint32_t r = 0; r < SIZE; ++r) {
                            const float w = exp2_approx(tail[r].x - top);
                            total = __fmaf_rn(w, tail[r].y, total);
                            weight[r] = w * tail[r].z;
                        }
                        const float inverse = __fdividef(1.0f, total);
#pragma unroll
                        for (uint32_t r = 0; r < SIZE; ++r) weight[r] *= inverse;
                    }
                    uint4 part[SIZE];
#pragma unroll
                    for (uint32_t r = 0; r < SIZE; ++r)
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(part[r].x), "=r"(part[r].y), "=r"(part[r].z), "=r"(part[r].w)
                                     : "r"(row_address + column * 16u + r * rank_stride) : "memory");
                    float total[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (uint32_t r = 0; r < SIZE; ++r) {
                        const uint32_t words[4] = {part[r].x, part[r].y, part[r].z, part[r].w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 pair = __half22float2(*reinterpret_cast<const __half2*>(&words[i]));
                            total[2 * i] = __fmaf_rn(weight[r], pair.x, total[2 * i]);
                            total[2 * i + 1] = __fmaf_rn(weight[r], pair.y, total[2 * i + 1]);
                        }
                    }
                    const uint32_t words[4] = {float2_to_bf16x2(make_float2(total[0], total[1])), float2_to_bf16x2(make_float2(total[2], total[3])),
                                               float2_to_bf16x2(make_float2(total[4], total[5])), float2_to_bf16x2(make_float2(total[6], total[7]))};
                    if (args.codes != nullptr) {
                        // row (head, query) of the batch element -> row batch * queries + query, columns of that head
                        const int tile_row = row0 + first_row + int(local);
                        const int head = tile_row / args.queries, query = tile_row - head * args.queries;
                        const int64_t width = int64_t(args.rows_per_batch / args.queries) * ATT_D;
                        const int64_t out_row = int64_t(batch) * args.queries + query;
                        const int64_t element = out_row * width + head * ATT_D + column * 8u;
                        if (args.blocked != nullptr) {
                            // a warp's 32 slots are the 32 column groups of one row: lanes 2j and 2j + 1 hold one block
                            uint8_t scale_code;
                            const uint32_t nibbles = encode_half_block_nvfp4(words, args.global_scale, by_global, scale_code);
                            *reinterpret_cast<uint32_t*>(args.codes + (element >> 1)) = nibbles;
                            if ((column & 1u) == 0u) {
                                const int block = (head * ATT_D + int(column) * 8) >> 4, blocks_per_row = int(width >> 4);
                                args.blocked[scale_tile_offset(int(out_row), block, (blocks_per_row + 3) >> 2)] = scale_code;
                                if (args.block_scales != nullptr) args.block_scales[out_row * blocks_per_row + block] = scale_code;
                            }
                        } else {
                            *reinterpret_cast<uint2*>(args.codes + element) = encode_row_words(words, args.multiplier);
                        }
                    } else {
                        *reinterpret_cast<uint4*>(tile_out + local * ATT_D + column * 8u) = make_uint4(words[0], words[1], words[2], words[3]);
                    }
                }
            };
            switch (splits) {
                case 2: combine(std::integral_constant<uint32_t, 2>{}); break;
                case 3: combine(std::integral_constant<uint32_t, 3>{}); break;
                case 4: combine(std::integral_constant<uint32_t, 4>{}); break;
                case 5: combine(std::integral_constant<uint32_t, 5>{}); break;
                case 6: combine(std::integral_constant<uint32_t, 6>{}); break;
                case 7: combine(std::integral_constant<uint32_t, 7>{}); break;
                case 8: combine(std::integral_constant<uint32_t, 8>{}); break;
                case 9: combine(std::integral_constant<uint32_t, 9>{}); break;
                case 10: combine(std::integral_constant<uint32_t, 10>{}); break;
                case 11: combine(std::integral_constant<uint32_t, 11>{}); break;
                case 12: combine(std::integral_constant<uint32_t, 12>{}); break;
                case 13: combine(std::integral_constant<uint32_t, 13>{}); break;
                case 14: combine(std::integral_constant<uint32_t, 14>{}); break;
                case 15: combine(std::integral_constant<uint32_t, 15>{}); break;
                default: combine(std::integral_constant<uint32_t, 16>{}); break;
            }
        } else {
        const float inverse = 1.0f / running_sum;
        __nv_bfloat16* destination = args.out + (int64_t(batch) * args.rows_per_batch + row0 + row) * ATT_D;
#pragma unroll 1
        for (int group = 0; group < ATT_D / 128; ++group) {      // four 32-column loads in flight per wait
            uint32_t o[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_load_32x32(lane_address + TMEM_O + group * 128 + c * 32, o[c]);
            tmem_load_wait();
            if (row_exists) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t words[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        words[i] = float2_to_bf16x2(make_float2(__uint_as_float(o[c][2 * i]) * inverse, __uint_as_float(o[c][2 * i + 1]) * inverse));
                    if (args.codes != nullptr) {
                        const int tile_row = row0 + row;
                        const int head = tile_row / args.queries, query = tile_row - head * args.queries;
                        const int64_t width = int64_t(args.rows_per_batch / args.queries) * ATT_D;
                        const int64_t out_row = int64_t(batch) * args.queries + query;
                        const int64_t element = out_row * width + head * ATT_D + group * 128 + c * 32;
                        if (args.blocked != nullptr) {      // two whole blocks of this row
                            const ExactDivider out_scale(args.global_scale), by_global(__fmul_rn(6.0f, args.global_scale));
                            const uint32_t first[8] = {words[0], words[1], words[2], words[3], words[4], words[5], words[6], words[7]};
                            const uint32_t second[8] = {words[8], words[9], words[10], words[11], words[12], words[13], words[14], words[15]};
                            uint8_t code[2];
                            const uint2 low = hidden_block_nvfp4(first, out_scale, by_global, code[0]);
                            const uint2 high = hidden_block_nvfp4(second, out_scale, by_global, code[1]);
                            *reinterpret_cast<uint4*>(args.codes + (element >> 1)) = make_uint4(low.x, low.y, high.x, high.y);
                            const int block = (head * ATT_D + group * 128 + c * 32) >> 4, blocks_per_row = int(width >> 4);
#pragma unroll
                            for (int half = 0; half < 2; ++half) {
                                args.blocked[scale_tile_offset(int(out_row), block + half, (blocks_per_row + 3) >> 2)] = code[half];
                                if (args.block_scales != nullptr) args.block_scales[out_row * blocks_per_row + block + half] = code[half];
                            }
                        } else {
                        uint8_t* encoded = args.codes + element;
                        uint2 part[4];
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            const uint32_t four[4] = {words[4 * v], words[4 * v + 1], words[4 * v + 2], words[4 * v + 3]};
                            part[v] = encode_row_words(four, args.multiplier);
                        }
                        *reinterpret_cast<uint4*>(encoded) = make_uint4(part[0].x, part[0].y, part[1].x, part[1].y);
                        *reinterpret_cast<uint4*>(encoded + 16) = make_uint4(part[2].x, part[2].y, part[3].x, part[3].y);
                        }
                    } else {
                    const uint32_t first[8] = {words[0], words[1], words[2], words[3], words[4], words[5], words[6], words[7]};
                    const uint32_t second[8] = {words[8], words[9], words[10], words[11], words[12], words[13], words[14], words[15]};
                    st_u8(destination + group * 128 + c * 32, first);
                    st_u8(destination + group * 128 + c * 32 + 16, second);
                    }
                }
            }
        }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLUMNS);
    }
    if (SPLIT) {
        // second cluster barrier: no CTA leaves while a copy still reads its shared memory or writes another CTA's (every
        // owner has seen all its bytes by the time it arrives here)
        asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory");
        cluster_wait();
    }
}

}  // namespace

// `out`: bf16 [batch, heads, queries, 256]; or, with `codes` given and no `out`, e4m3 [batch * queries, heads * 256] at
// `multiplier`; or, with `blocked` given as well, e2m1 pairs [batch * queries, heads * 128] with their block scales at
// `global_scale` (`block_scales`: the row-major copy, optional).
int launch_attention(const void* q, const void* k, const void* v, void* out, void* codes, float multiplier, void* block_scales,
                     void* blocked, float global_scale, int batch, int heads, int queries, int keys, int head_dim, void* status,
                     cudaStream_t stream) {
    if (head_dim != ATT_D) return B2_E_UNSUPPORTED;
    const int64_t rows_per_batch = int64_t(heads) * queries;
    if (rows_per_batch * batch >= (int64_t(1) << 31) || int64_t(keys) * batch >= (int64_t(1) << 31)) return B2_E_TOO_LARGE;
    static bool configured[64] = {false};
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64 && !configured[device]) {
        cudaError_t error = cudaFuncSetAttribute(attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SHARED_BYTES);
        if (error == cudaSuccess)
            error = cudaFuncSetAttribute(attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SHARED_BYTES);
        if (error != cudaSuccess) return int(error);
        configured[device] = true;
    }
    CUtensorMap q_map, k_map, v_map;
    if (!make_operand_map(&q_map, q, rows_per_batch * batch, ATT_D * 2, ATT_ROWS)) return B2_E_DRIVER;
    if (!make_operand_map(&k_map, k, int64_t(keys) * batch, ATT_D * 2, ATT_KEYS)) return B2_E_DRIVER;
    if (!make_operand_map(&v_map, v, int64_t(keys) * batch, ATT_D * 2, ATT_KEYS)) return B2_E_DRIVER;
    AttentionArgs args{};
    args.out = static_cast<__nv_bfloat16*>(out);
    args.codes = static_cast<uint8_t*>(codes);
    args.multiplier = multiplier;
    args.blocked = static_cast<uint8_t*>(blocked);
    args.block_scales = static_cast<uint8_t*>(block_scales);
    args.global_scale = global_scale;
    args.queries = queries;
    args.status = static_cast<unsigned int*>(status);
    args.rows_per_batch = int(rows_per_batch);
    args.keys = keys;
    args.tiles_per_batch = int((rows_per_batch + ATT_ROWS - 1) / ATT_ROWS);
    args.scale_log2 = 1.4426950408889634f / 16.0f;
    args.splits = 1;
    args.rows_per_rank = 0;
    // Few CTAs and several key tiles: the keys of a tile are cut across a cluster, as long as all clusters of the launch run
    // at once and the partial rows of a tile (sent and received) fit over the operand stages.
    const int key_tiles = (keys + ATT_KEYS - 1) / ATT_KEYS;
    const int tiles = batch * args.tiles_per_batch;
    // How many clusters of each size the device runs at once is asked of the driver, once per device (sizes above 8 are the
    // opt-in ones; a size the device does not schedule reports 0): a launch takes the largest cluster, up to one CTA per
    // key tile, whose clusters are all resident together.
    static int resident_clusters[64][17] = {};
    static bool probed[64] = {false};
    if (device >= 0 && device < 64 && !probed[device]) {
        const bool wide = cudaFuncSetAttribute(attention_kernel<true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        for (int size = 2; size <= 16; ++size) {
            resident_clusters[device][size] = 0;
            if (size > 8 && !wide) continue;
            cudaLaunchConfig_t probe = {};
            probe.gridDim = dim3(unsigned(size));
            probe.blockDim = dim3(ATT_THREADS);
            probe.dynamicSmemBytes = size_t(ATT_SHARED_BYTES);
            cudaLaunchAttribute cluster;
            cluster.id = cudaLaunchAttributeClusterDimension;
            cluster.val.clusterDim.x = unsigned(size);
            cluster.val.clusterDim.y = 1;
            cluster.val.clusterDim.z = 1;
            probe.attrs = &cluster;
            probe.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, attention_kernel<true>, &probe) == cudaSuccess) resident_clusters[device][size] = clusters;
        }
        cudaGetLastError();
        probed[device] = true;
    }
    int splits = 1;
    if (device >= 0 && device < 64) {
        for (int size = key_tiles < 16 ? key_tiles : 16; size >= 2; --size) {
            if (size > 8 && size != key_tiles) continue;                 // beyond 8 only for one CTA per key tile
            if (size <= 8 && (size & (size - 1)) != 0 && size != key_tiles) continue;      // else powers of two
            if (tiles <= resident_clusters[device][size]) {
                splits = size;
                break;
            }
        }
    }
    if (splits > 1 && args.tiles_per_batch == 1) {
        const int rows = int(rows_per_batch);
        const int rows_per_rank = (rows + splits - 1) / splits;
        const int64_t exchange = int64_t(rows) * SPLIT_ROW_BYTES + int64_t(splits) * rows_per_rank * SPLIT_ROW_BYTES;
        if (exchange <= int64_t(Q_BYTES + 4 * KV_STAGE_BYTES + 2 * P_BYTES)) {
            args.splits = splits;
            args.rows_per_rank = rows_per_rank;
        }
    }
    if (args.splits > 1) {
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(unsigned(tiles * args.splits));
        config.blockDim = dim3(ATT_THREADS);
        config.dynamicSmemBytes = size_t(ATT_SHARED_BYTES);
        config.stream = stream;
        cudaLaunchAttribute attributes[2];
        attributes[0].id = cudaLaunchAttributeClusterDimension;
        attributes[0].val.clusterDim.x = unsigned(args.splits);
        attributes[0].val.clusterDim.y = 1;
        attributes[0].val.clusterDim.z = 1;
        attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[1].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attributes;
        config.numAttrs = pdl_enabled() ? 2 : 1;
        const cudaError_t error = cudaLaunchKernelEx(&config, attention_kernel<true>, q_map, k_map, v_map, args);
        return error == cudaSuccess ? int(cudaGetLastError()) : int(error);
    }
    return launch_kernel(attention_kernel<false>, dim3(unsigned(tiles)), dim3(ATT_THREADS), size_t(ATT_SHARED_BYTES), stream,
                         q_map, k_map, v_map, args);
}

}  // namespace b2
