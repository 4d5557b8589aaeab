// Quantised Linear for a handful of tokens (the action expert's 10 .. 128 rows): the weight is the MMA's "A"
// operand, the tokens are its "B" operand, and K is cut across the CTAs of a thread-block cluster.
//
// Why a schedule of its own.  A tcgen05.mma with M = 128 takes some 75 cycles however few columns it has (the
// 128 x 32-byte "A" slice has to be read from shared memory), so with the tokens as "A" a launch of 10 tokens
// spends one such MMA per 32 or 64 features and 32 bytes of K: 1024 features x 4096 of K are 4096 MMAs, on the 16
// or 32 CTAs the feature tiles give, each walking all of K.  Here the 128 rows of "A" are 128 features, all of
// them useful: the same launch is 1024 MMAs, and because a tile no longer has to keep its K together they spread
// over eight times as many CTAs:
//
//   grid     = feature tiles (128 rows: plain; 64 gate rows + 64 up rows: gated) x S, clusters of S = 1, 2, 4 or 8
//   CTA r    = K atoms [r * num_kb / S, (r + 1) * num_kb / S) of its tile, every atom in its own shared-memory stage
//              (filled once: no ring, no "empty" barriers), accumulator [128 features x tokens] in tensor memory
//   exchange = the tokens are dealt to the S CTAs in runs of T = ceil(tokens / S).  Every CTA lays its partial sums out
//              as [token][128 features] fp32 rows in its own shared memory (over the operand stages, which are dead
//              by then) and sends each CTA the rows of the tokens that CTA owns with one bulk copy through distributed
//              shared memory, counted in bytes on the owner's barrier (scalar remote stores plus remote arrivals took
//              ~90 cycles per token and ~400 per arrival).  The owner adds the S partial rows in rank order (so the
//              result does not depend on timing) and runs the ordinary fused epilogue on them -- by then a token's
//              features are contiguous again, and the epilogue code is the one the other schedules use.
//
// Warps: 0 = TMA producer, 1 = tensor memory + MMA issuer, 2..5 = accumulator readers / epilogue (one per 32-lane
// partition).  The weight boxes are prefetched into the L2 before the dependency wait of the launch, so they travel
// from HBM while the previous kernel of the stream is still finishing.  Every mbarrier wait is bounded (ptx.cuh); the
// two hardware cluster barriers are reached by every thread on every path.
#include "common.cuh"
#include "gemm_epilogue.cuh"

#include <cuda.h>

#include <mutex>

namespace b2 {

constexpr int SKINNY_THREADS = 32 * 6;
constexpr int SKINNY_ROW_FLOATS = 132;           // 128 partial sums + 4 of padding: rows start 4 banks apart
constexpr int SKINNY_MAX_TOKENS = 128;

__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
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

// Bounded wait whose acquire covers writes made by other CTAs of the cluster before their (release.cluster) arrivals.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, bool& failed, unsigned int* status,
                                                  unsigned int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (failed) return false;
    const long long start = clock64();
    while (!mbar_try_wait_cluster(bar, parity)) {
        if (clock64() - start > WAIT_LIMIT_CYCLES) {
            failed = true;
            if (status != nullptr) atomicCAS(status, 0u, code);
            return false;
        }
    }
    return true;
}

// Bulk copy from this CTA's shared memory into a CTA of the cluster (`dst` and `bar` are shared::cluster addresses of
// that CTA); the bytes are counted on `bar` as they land.  16-byte aligned, size % 16 == 0.
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t dst, uint32_t src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "r"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory"); }

__device__ __forceinline__ float4 ld_shared_f4(uint32_t address) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(address) : "memory");
    return v;
}

// KernelArgs as this schedule reads it: tile_n = token columns of the accumulator (tokens rounded up to 16),
// num_n_tiles = feature tiles, splits = cluster size S, stages = K atoms of the longest K range, a_box_bytes = bytes of
// the token box of one K atom, kps = tokens per CTA of the exchange (T).
template <int KIND, int EPI>
__global__ void __launch_bounds__(SKINNY_THREADS, 1)
skinny_linear_kernel(const __grid_constant__ CUtensorMap act_map, const __grid_constant__ CUtensorMap weight_map,
                     const KernelArgs args) {
    constexpr bool GEGLU = is_gated(EPI);
    constexpr bool ROPE = EPI == EPI_ROPE;      // tile = 64 features of a head and their 64 rotation partners (two planes, like gate / up)
    constexpr bool USES_TABLE = EPI != EPI_LINEAR && !ROPE;
    constexpr bool NVFP4 = KIND == B2_KIND_NVFP4;
    constexpr uint32_t WEIGHT_BYTES = 128 * STAGE_K_BYTES;
    constexpr uint32_t SCALE_PART_BYTES = SCALE_ATOMS_PER_STAGE * SCALE_ATOM_BYTES;
    pdl_launch_dependents();
    extern __shared__ uint8_t shared_raw[];
    const uint32_t base = (smem_u32(shared_raw) + 1023u) & ~1023u;
    const int columns = args.tile_n;
    const uint32_t splits = uint32_t(args.splits);
    const uint32_t rank = cluster_cta_rank();
    const int tile = int(blockIdx.x) / args.splits;
    const int kb_begin = int(rank) * args.num_kb / args.splits;
    const int kb_end = (int(rank) + 1) * args.num_kb / args.splits;
    const int atoms = kb_end - kb_begin;
    const int tokens_per_rank = args.kps;

    // shared memory: [stages x (weight rows 16 KB | token rows)][NVFP4: stages x (weight scale atoms | token scale atoms)]
    //                  (later, from the start: this CTA's partial sums, `tokens` rows of 132 floats)
    //                [receive buffer: S x T rows of 132 floats][barriers][GELU table]
    constexpr uint32_t ROW_BYTES = SKINNY_ROW_FLOATS * 4u;
    const uint32_t stage_bytes = WEIGHT_BYTES + uint32_t(args.a_box_bytes);
    const uint32_t scale_base = base + uint32_t(args.stages) * stage_bytes;
    const uint32_t operand_bytes = uint32_t(args.stages) * (stage_bytes + (NVFP4 ? 2u * SCALE_PART_BYTES : 0u));
    const uint32_t staging_bytes = uint32_t(args.tokens) * ROW_BYTES;
    const uint32_t receive_base = base + (operand_bytes > staging_bytes ? operand_bytes : staging_bytes);
    const uint32_t barrier_base = receive_base + splits * uint32_t(tokens_per_rank) * (SKINNY_ROW_FLOATS * 4u);
    const uint32_t full_bar = barrier_base;                        // [stages]
    const uint32_t acc_full_bar = barrier_base + 8 * MAX_STAGES;
    const uint32_t receive_bar = acc_full_bar + 8;
    const uint32_t tmem_slot = receive_bar + 8;
    const uint32_t table_bar = tmem_slot + 8;
    const uint32_t compact_table = barrier_base + 8 * MAX_STAGES + 48;     // 16-byte aligned
    // The GELU table's range comes in with two bulk copies when both halves are 16-byte aligned multiples of 16 bytes
    // (b2_gelu_table_range chooses such ranges), else entry by entry.
    const int table_span = args.gelu_hi - args.gelu_lo;
    const bool bulk_table = USES_TABLE && table_span > 0 && (args.gelu_lo & 7) == 0 && (table_span & 7) == 0 &&
                            (reinterpret_cast<uintptr_t>(args.gelu_table) & 15u) == 0;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int f0 = tile * (GEGLU ? 64 : 128);

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&act_map);
        tma_prefetch_descriptor(&weight_map);
        for (int s = 0; s < args.stages; ++s) mbar_init(full_bar + 8 * s, 1);
        mbar_init(acc_full_bar, 1);
        mbar_init(receive_bar, 1);
        mbar_init(table_bar, 1);
        fence_barrier_init();
        // the table is a constant of the model: its copies do not wait for the launches before this one
        if (bulk_table) {
            mbar_expect_tx(table_bar, 4u * uint32_t(table_span));
            bulk_load(compact_table, args.gelu_table + args.gelu_lo, 2u * uint32_t(table_span), table_bar);
            bulk_load(compact_table + 2u * uint32_t(table_span), args.gelu_table + 0x8000 + args.gelu_lo, 2u * uint32_t(table_span), table_bar);
        } else {
            mbar_arrive(table_bar);
        }
        // the bytes this CTA will receive: S partial rows for each token it owns (none: the phase completes at once)
        int owned = args.tokens - int(rank) * tokens_per_rank;
        owned = owned < 0 ? 0 : (owned > tokens_per_rank ? tokens_per_rank : owned);
        mbar_expect_tx(receive_bar, splits * uint32_t(owned) * ROW_BYTES);
    }
    if (warp == 0) {
        // the weights are not written by the launches this one may overlap with in any way that matters to a
        // prefetch: it only moves lines into the L2, the loads below still read them after the dependency wait
        if (elect_one()) {
            for (int i = 0; i < atoms; ++i) {
                if (ROPE) tma_prefetch_l2_3d(&weight_map, (kb_begin + i) * STAGE_K_BYTES, (tile & 1) * 64, 2 * (tile >> 1));
                else if (GEGLU) tma_prefetch_l2_3d(&weight_map, (kb_begin + i) * STAGE_K_BYTES, f0, 0);
                else tma_prefetch_l2_2d(&weight_map, (kb_begin + i) * STAGE_K_BYTES, f0);
            }
        }
        __syncwarp();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLUMNS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    // first cluster barrier: every CTA's receive barrier is initialised (fence.mbarrier_init above) before another CTA's
    // copies count bytes on it (the wait is further down, right before the copies are issued)
    cluster_arrive_relaxed();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");
    pdl_wait();

    bool failed = false;
    const int num_kb = args.num_kb;
    const int last_kb_mmas = ((args.k_bytes - (num_kb - 1) * STAGE_K_BYTES) + 31) / 32;
    const int tail_atoms = args.scale_column_tiles - (num_kb - 1) * SCALE_ATOMS_PER_STAGE;

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer: every K atom at once
        if (elect_one()) {
            const uint8_t* weight_scales = NVFP4 ? args.weight_scales + int64_t(tile) * args.scale_column_tiles * SCALE_ATOM_BYTES : nullptr;
            for (int i = 0; i < atoms; ++i) {
                const int kb = kb_begin + i;
                const uint32_t bar = full_bar + 8 * i;
                const uint32_t a_smem = base + uint32_t(i) * stage_bytes;
                const uint32_t copy_bytes = uint32_t(kb == num_kb - 1 ? tail_atoms : SCALE_ATOMS_PER_STAGE) * SCALE_ATOM_BYTES;
                mbar_expect_tx(bar, stage_bytes + (NVFP4 ? 2u * copy_bytes : 0u));
                if (ROPE) tma_load_3d(a_smem, &weight_map, bar, kb * STAGE_K_BYTES, (tile & 1) * 64, 2 * (tile >> 1));
                else if (GEGLU) tma_load_3d(a_smem, &weight_map, bar, kb * STAGE_K_BYTES, f0, 0);
                else tma_load_2d(a_smem, &weight_map, bar, kb * STAGE_K_BYTES, f0);
                tma_load_2d(a_smem + WEIGHT_BYTES, &act_map, bar, kb * STAGE_K_BYTES, 0);
                if (NVFP4) {
                    const uint32_t s_smem = scale_base + uint32_t(i) * 2u * SCALE_PART_BYTES;
                    const int64_t offset = int64_t(kb) * SCALE_PART_BYTES;
                    bulk_load(s_smem, weight_scales + offset, copy_bytes, bar);
                    bulk_load(s_smem + SCALE_PART_BYTES, args.act_scales + offset, copy_bytes, bar);
                }
            }
        }
        __syncwarp();
        // do not leave while a copy is in flight (on the normal path the MMA warp has seen them all long before)
        bool drain_failed = false;
        for (int i = 0; i < atoms; ++i) mbar_wait(full_bar + 8 * i, 0u, drain_failed, args.status, STATUS_WAIT_DRAIN);
        mbar_wait(table_bar, 0u, drain_failed, args.status, STATUS_WAIT_DRAIN);
        cluster_wait();
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer
        const uint32_t idesc = NVFP4 ? idesc_nvf4(128, uint32_t(columns)) : idesc_f8(128, uint32_t(columns));
        const uint64_t operand_desc = smem_desc_sw128(0);
        const uint32_t operand_low = uint32_t(operand_desc), operand_high = uint32_t(operand_desc >> 32);
        const uint32_t scale_desc_high = uint32_t(smem_desc_scale_atom(0) >> 32);
        for (int i = 0; i < atoms; ++i) {
            mbar_wait(full_bar + 8 * i, 0u, failed, args.status, STATUS_WAIT_MMA_FULL);
            tc_fence_after_sync();
            __syncwarp();
            if (elect_one()) {
                constexpr uint32_t ATOM = SCALE_ATOM_BYTES >> 4;
                const uint32_t a_smem = base + uint32_t(i) * stage_bytes;
                // (address field = low 18 bits: in a cluster every CTA but rank 0 has shared-window bits above them)
                const uint32_t a_low = operand_low + ((a_smem & 0x3FFFFu) >> 4);
                const uint32_t b_low = operand_low + (((a_smem + WEIGHT_BYTES) & 0x3FFFFu) >> 4);
                // NVFP4: every atom has its own 32 columns of tensor memory (16 of weight scales, 16 of token scales)
                const uint32_t sfa_tmem = tmem_base + uint32_t(TMEM_COLUMNS) - 32u * uint32_t(i + 1);
                const uint32_t sfb_tmem = sfa_tmem + 16u;
                const uint32_t scale_low = ((scale_base + uint32_t(i) * 2u * SCALE_PART_BYTES) & 0x3FFFFu) >> 4;
                const int count = kb_begin + i == num_kb - 1 ? last_kb_mmas : SCALE_ATOMS_PER_STAGE;
#pragma unroll
                for (int j = 0; j < SCALE_ATOMS_PER_STAGE; ++j) {
                    if (j < count) {
                        if (NVFP4) {
                            tc_copy_32x128b_x4(sfa_tmem + j * 4, desc_from_words(scale_low + j * ATOM, scale_desc_high));
                            tc_copy_32x128b_x4(sfb_tmem + j * 4, desc_from_words(scale_low + (SCALE_PART_BYTES >> 4) + j * ATOM, scale_desc_high));
                        }
                        const uint32_t accumulate = (i != 0 || j != 0) ? 1u : 0u;
                        const uint64_t a_desc = desc_from_words(a_low + 2 * j, operand_high);
                        const uint64_t b_desc = desc_from_words(b_low + 2 * j, operand_high);
                        if (NVFP4) mma_nvf4(tmem_base, a_desc, b_desc, idesc, sfa_tmem + j * 4, sfb_tmem + j * 4, accumulate);
                        else mma_f8f6f4(tmem_base, a_desc, b_desc, idesc, accumulate);
                    }
                }
            }
            __syncwarp();
        }
        if (elect_one()) tc_commit(acc_full_bar);
        __syncwarp();
        cluster_wait();
    } else {
        // ------------------------------------------------------------- accumulator readers, exchange, epilogue
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;              // feature row of the tile (gated: 64 gate rows, then 64 up rows)
        const int reader = (warp - FIRST_EPILOGUE_WARP) * 32 + lane;
        const bool round_scale = (args.flags & B2_LINEAR_ROUND_SCALE_BF16) != 0;
        float scale = __fmul_rn(__ldg(args.act_scale), __ldg(args.weight_scale));
        if (round_scale) scale = round_to_bf16(scale);
        float scale_up = scale;
        if (GEGLU && args.weight_scale_up != nullptr) {
            scale_up = __fmul_rn(__ldg(args.act_scale), __ldg(args.weight_scale_up));
            if (round_scale) scale_up = round_to_bf16(scale_up);
        }
        float out_scale_value = 1.0f, out_scale_rcp = 1.0f;
        if (EPI == EPI_GEGLU_FP8 || EPI == EPI_GEGLU_NVFP4 || EPI == EPI_GELU_FP8) {
            out_scale_value = __ldg(args.out_scale);
            out_scale_rcp = __fdiv_rn(1.0f, out_scale_value);
        }
        const ExactDivider out_scale(out_scale_value);
        const ExactDivider by_global(__fmul_rn(6.0f, out_scale_value));
        const bool true_div = (args.flags & B2_GEGLU_TRUE_DIV) != 0;
        // The shared-memory copy of the GELU table is filled here, by the warps that will read it, while the operands are
        // on their way (the table is a constant of the model; the barrier after the staging orders it before its use).
        if (USES_TABLE && !bulk_table) fill_compact_gelu(args, compact_table, reader, 128);

        // (a) this CTA's partial sums as [token][feature row] in its own shared memory, then one copy per owner:
        //     rows [r T, r T + T) -> owner r's receive buffer at [this rank * T ...]
        mbar_wait(acc_full_bar, 0u, failed, args.status, STATUS_WAIT_EPILOGUE);
        tc_fence_after_sync();
        const uint32_t lane_address = tmem_base + (uint32_t(quarter * 32) << 16);
        const uint32_t staging = base + uint32_t(row) * 4u;
        for (int group = 0; group * 16 < args.tokens; ++group) {
            uint32_t v[16];
            tmem_load_32x16(lane_address + uint32_t(group * 16), v);
            tmem_load_wait();
#pragma unroll
            for (int c = 0; c < 16; ++c)
                if (group * 16 + c < args.tokens)
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(staging + uint32_t(group * 16 + c) * ROW_BYTES), "r"(v[c]) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the copies below read these rows through the async proxy
        asm volatile("bar.sync 1, 128;" ::: "memory");
        cluster_wait();
        if (uint32_t(reader) < splits) {      // one copy per thread, starting with the next rank: no owner is everyone's first
            const uint32_t step = uint32_t(reader) + 1u;
            const uint32_t r = rank + step < splits ? rank + step : rank + step - splits;
            const int first = int(r) * tokens_per_rank;
            int count = args.tokens - first;
            if (count > tokens_per_rank) count = tokens_per_rank;
            if (count > 0)
                bulk_copy_to_cluster(cluster_map_shared(receive_base + rank * uint32_t(tokens_per_rank) * ROW_BYTES, r),
                                     base + uint32_t(first) * ROW_BYTES, uint32_t(count) * ROW_BYTES,
                                     cluster_map_shared(receive_bar, r));
        }

        // (b) the tokens this CTA owns: all 128 threads add the S partial rows in rank order, one 16-byte column each
        //     (the eight loads of a column are independent, so they are in flight together), into the rank-0 row ...
        mbar_wait_cluster(receive_bar, 0u, failed, args.status, STATUS_WAIT_EXCHANGE);
        const int first_token = int(rank) * tokens_per_rank;
        int owned = args.tokens - first_token;
        if (owned > tokens_per_rank) owned = tokens_per_rank;
        const uint32_t rank_stride = uint32_t(tokens_per_rank) * ROW_BYTES;
        for (int slot = reader; slot < owned * 32; slot += 128) {
            const uint32_t address = receive_base + uint32_t(slot >> 5) * ROW_BYTES + uint32_t(slot & 31) * 16u;
            float4 p[8];
#pragma unroll
            for (uint32_t r = 0; r < 8; ++r)
                if (r < splits) p[r] = ld_shared_f4(address + r * rank_stride);
            float4 total = p[0];
#pragma unroll
            for (uint32_t r = 1; r < 8; ++r) {
                if (r < splits) {
                    total.x = __fadd_rn(total.x, p[r].x); total.y = __fadd_rn(total.y, p[r].y);
                    total.z = __fadd_rn(total.z, p[r].z); total.w = __fadd_rn(total.w, p[r].w);
                }
            }
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(address), "f"(total.x), "f"(total.y), "f"(total.z), "f"(total.w) : "memory");
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (USES_TABLE) mbar_wait(table_bar, 0u, failed, args.status, STATUS_WAIT_EPILOGUE);
        //     ... then the fused epilogue on 32-feature chunks (16-feature units of gate and up) of those rows
        for (int item = reader; item < owned * 4; item += 128) {
            const int local = item >> 2, part = item & 3;
            const int token = first_token + local;
            const uint32_t sums = receive_base + uint32_t(local) * ROW_BYTES;
            if (ROPE) {
                // 16 features of a half head (sums in floats [16 part, 16 part + 16)) and their partners 128 features on (64
                // floats further): the projection's bf16 result, then b2_rope_split's rotation, queries / keys / values to
                // their places
                uint32_t acc[32];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 x = ld_shared_f4(sums + uint32_t(part) * 64u + 16u * q), y = ld_shared_f4(sums + 256u + uint32_t(part) * 64u + 16u * q);
                    acc[4 * q] = __float_as_uint(x.x); acc[4 * q + 1] = __float_as_uint(x.y);
                    acc[4 * q + 2] = __float_as_uint(x.z); acc[4 * q + 3] = __float_as_uint(x.w);
                    acc[16 + 4 * q] = __float_as_uint(y.x); acc[16 + 4 * q + 1] = __float_as_uint(y.y);
                    acc[16 + 4 * q + 2] = __float_as_uint(y.z); acc[16 + 4 * q + 3] = __float_as_uint(y.w);
                }
                uint32_t words[16];
                linear_scale_chunk(acc, scale, round_scale, words);
                const int head = tile >> 1, first_dim = (tile & 1) * 64 + part * 16;
                const int b = token / args.rope_tokens, t = token - b * args.rope_tokens;
                __nv_bfloat16* destination;
                bool rotate = true;
                if (head < args.rope_heads) {
                    destination = args.rope_q + ((int64_t(b) * args.rope_heads + head) * args.rope_tokens + t) * 256;
                } else if (head < args.rope_heads + args.rope_kv_heads) {
                    destination = args.rope_k + ((int64_t(b) * args.rope_kv_heads + (head - args.rope_heads)) * args.rope_capacity + args.rope_offset + t) * 256;
                } else {
                    destination = args.rope_v + ((int64_t(b) * args.rope_kv_heads + (head - args.rope_heads - args.rope_kv_heads)) * args.rope_capacity + args.rope_offset + t) * 256;
                    rotate = false;
                }
                destination += first_dim;
                uint32_t low[8], high[8];
                if (rotate) {
                    const float* s = args.rope_sine + b * args.rope_batch_stride + int64_t(t) * 128 + first_dim;
                    const float* c = args.rope_cosine + b * args.rope_batch_stride + int64_t(t) * 128 + first_dim;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float2 x = bf16x2_to_float2(words[i]), y = bf16x2_to_float2(words[8 + i]);
                        const float c0 = __ldg(c + 2 * i), c1 = __ldg(c + 2 * i + 1), s0 = __ldg(s + 2 * i), s1 = __ldg(s + 2 * i + 1);
                        low[i] = float2_to_bf16x2(make_float2(__fsub_rn(__fmul_rn(x.x, c0), __fmul_rn(y.x, s0)), __fsub_rn(__fmul_rn(x.y, c1), __fmul_rn(y.y, s1))));
                        high[i] = float2_to_bf16x2(make_float2(__fadd_rn(__fmul_rn(y.x, c0), __fmul_rn(x.x, s0)), __fadd_rn(__fmul_rn(y.y, c1), __fmul_rn(x.y, s1))));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) { low[i] = words[i]; high[i] = words[8 + i]; }
                }
                store_u4(destination, low[0], low[1], low[2], low[3]);
                store_u4(destination + 8, low[4], low[5], low[6], low[7]);
                store_u4(destination + 128, high[0], high[1], high[2], high[3]);
                store_u4(destination + 136, high[4], high[5], high[6], high[7]);
            } else if (GEGLU) {
                // 16 features: gate sums in floats [16 part, 16 part + 16), up sums 64 floats further
                uint32_t gate_acc[16], up_acc[16];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 g = ld_shared_f4(sums + uint32_t(part) * 64u + 16u * q), u = ld_shared_f4(sums + 256u + uint32_t(part) * 64u + 16u * q);
                    gate_acc[4 * q] = __float_as_uint(g.x); gate_acc[4 * q + 1] = __float_as_uint(g.y);
                    gate_acc[4 * q + 2] = __float_as_uint(g.z); gate_acc[4 * q + 3] = __float_as_uint(g.w);
                    up_acc[4 * q] = __float_as_uint(u.x); up_acc[4 * q + 1] = __float_as_uint(u.y);
                    up_acc[4 * q + 2] = __float_as_uint(u.z); up_acc[4 * q + 3] = __float_as_uint(u.w);
                }
                epilogue_geglu_unit<GEGLU ? EPI : EPI_GEGLU_BF16>(gate_acc, up_acc, args, compact_table, scale, scale_up, round_scale,
                                                                 out_scale, by_global, out_scale_rcp, true_div, token, f0 + part * 16);
            } else {
                uint32_t acc[32];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const float4 v = ld_shared_f4(sums + uint32_t(part) * 128u + 16u * q);
                    acc[4 * q] = __float_as_uint(v.x); acc[4 * q + 1] = __float_as_uint(v.y);
                    acc[4 * q + 2] = __float_as_uint(v.z); acc[4 * q + 3] = __float_as_uint(v.w);
                }
                epilogue_linear_chunk<(GEGLU || ROPE) ? EPI_LINEAR : EPI>(acc, args, scale, round_scale, token, f0 + part * 32, compact_table,
                                                                out_scale, out_scale_rcp, true_div);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLUMNS);
    }
    // second cluster barrier: no CTA leaves while a copy still reads its shared memory or writes another CTA's (every
    // owner has seen all its bytes by the time it arrives here)
    cluster_arrive_relaxed();
    cluster_wait();
}

// ---------------------------------------------------------------------------
// host side

// Clusters of 2, 4 and 8 CTAs of this kernel that the device runs at once (one CTA per SM: 120 KB of shared memory at
// least), asked of the driver once per device; a cluster sits inside one GPC, so the answer is not SMs / size.
static int resident_clusters(int size) {
    static int answers[64][9] = {};
    static bool probed[64] = {false};
    static std::mutex lock;
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64) return sm_count() / size - 2;
    std::lock_guard<std::mutex> guard(lock);
    if (!probed[device]) {
        cudaFuncSetAttribute(skinny_linear_kernel<B2_KIND_FP8, EPI_LINEAR>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
        for (int candidate = 2; candidate <= 8; candidate *= 2) {
            cudaLaunchConfig_t probe = {};
            probe.gridDim = dim3(unsigned(candidate));
            probe.blockDim = dim3(unsigned(SKINNY_THREADS));
            probe.dynamicSmemBytes = size_t(SMEM_MINIMUM);
            cudaLaunchAttribute cluster;
            cluster.id = cudaLaunchAttributeClusterDimension;
            cluster.val.clusterDim.x = unsigned(candidate);
            cluster.val.clusterDim.y = 1;
            cluster.val.clusterDim.z = 1;
            probe.attrs = &cluster;
            probe.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, skinny_linear_kernel<B2_KIND_FP8, EPI_LINEAR>, &probe) != cudaSuccess || clusters <= 0)
                clusters = sm_count() / candidate - (candidate == 8 ? 4 : candidate == 4 ? 4 : 2);      // the guess used before the query
            answers[device][candidate] = clusters;
        }
        cudaGetLastError();
        probed[device] = true;
    }
    return answers[device][size];
}

// Cluster size for `tiles` feature tiles and `num_kb` K atoms: the largest of 8, 4, 2 whose clusters are all resident at
// once and that leaves every CTA at least one K atom.
static int skinny_cluster(int tiles, int num_kb) {
    if (num_kb >= 8 && tiles <= resident_clusters(8)) return 8;
    if (num_kb >= 4 && tiles <= resident_clusters(4)) return 4;
    if (num_kb >= 2 && tiles <= resident_clusters(2)) return 2;
    return 1;
}

// Whether this schedule applies to a launch, and whether it is the faster one.  Both times were measured on the action
// expert's projections (FP8 and NVFP4; 10 .. 120 tokens; 1024 .. 4096 features; K = 1024 .. 4096) and follow
//   tile schedule    ~ fixed + a per 128 elements of K  (one CTA walks all of K of its tile: a ~ 150 ns, gated ~ 270 ns)
//   cluster schedule ~ fixed + 200 ns per K atom of a CTA + 26 ns per token (staging, exchange and epilogue grow with
//                      the tokens; the K of a CTA shrinks with the cluster size)
// with the cluster schedule's fixed part 140 ns (FP8) / 460 ns (NVFP4) below the tile schedule's.  B2_LINEAR_CLUSTER skips
// the comparison.
SkinnyPlan skinny_plan(const b2_linear_desc* d, bool geglu) {
    SkinnyPlan plan;
    if (d->tokens > SKINNY_MAX_TOKENS || d->feature_tile != 0) return plan;
    if (d->flags & (B2_LINEAR_SINGLE_CTA | B2_LINEAR_PAIRS | B2_LINEAR_STREAM_TOKENS)) return plan;
    const bool nvfp4 = d->kind == B2_KIND_NVFP4;
    if (geglu && nvfp4 && (!(d->flags & B2_LINEAR_PAIRED_GATE_UP_SCALES) || d->features % 64 != 0)) return plan;
    const bool rope = d->rope != nullptr;                 // only this schedule has the attention preparation as an epilogue
    const int k_bytes = nvfp4 ? d->width / 2 : d->width;
    const int num_kb = (k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES;
    const int columns = (d->tokens + 15) / 16 * 16;
    const int tiles = geglu ? (d->features + 63) / 64 : (d->features + 127) / 128;
    int span = 0;
    if (d->epilogue != B2_EPI_LINEAR && d->gelu_lo >= 0x80 && d->gelu_hi > d->gelu_lo && d->gelu_hi <= 0x7f80 &&
        d->gelu_hi - d->gelu_lo <= MAX_COMPACT_GELU)
        span = d->gelu_hi - d->gelu_lo;
    for (int splits = skinny_cluster(tiles, num_kb); splits >= 1; splits /= 2) {
        const int atoms = (num_kb + splits - 1) / splits;
        const int tokens_per_rank = (d->tokens + splits - 1) / splits;
        const int stage_bytes = 128 * STAGE_K_BYTES + columns * STAGE_K_BYTES + (nvfp4 ? 2 * SCALE_ATOMS_PER_STAGE * SCALE_ATOM_BYTES : 0);
        const int64_t operand_bytes = int64_t(atoms) * stage_bytes, staging_bytes = int64_t(d->tokens) * SKINNY_ROW_FLOATS * 4;
        const int64_t bytes = 1024 + (operand_bytes > staging_bytes ? operand_bytes : staging_bytes) +
                              int64_t(splits) * tokens_per_rank * SKINNY_ROW_FLOATS * 4 + 8 * MAX_STAGES + 64 + 4 * span;
        if (atoms <= MAX_STAGES && bytes <= SMEM_LIMIT && (!nvfp4 || columns + 32 * atoms <= TMEM_COLUMNS)) {
            if (!(d->flags & B2_LINEAR_CLUSTER) && !rope) {
                const int64_t waves = (int64_t(tiles) * splits + sm_count() - 1) / sm_count();
                const int64_t tile_ns = (nvfp4 ? 460 : 140) + int64_t(geglu ? 270 : 150) * (d->width / 128);
                const int64_t cluster_ns = waves * (200 * int64_t(atoms) + 26 * int64_t(d->tokens));
                if (cluster_ns >= tile_ns) return plan;
            }
            plan.splits = splits;
            plan.columns = columns;
            plan.atoms = atoms;
            plan.tokens_per_rank = tokens_per_rank;
            plan.shared_bytes = int(bytes < SMEM_MINIMUM ? SMEM_MINIMUM : bytes);
            plan.gelu_span = span;
            return plan;
        }
    }
    return plan;
}

// A launch with `d->rope` set that the EPI_ROPE epilogue handles (run_linear returns B2_E_UNSUPPORTED otherwise).
bool skinny_rope_supported(const b2_linear_desc* d) {
    const b2_rope_desc* r = d->rope;
    if (r == nullptr) return false;
    if (d->kind != B2_KIND_FP8 || d->epilogue != B2_EPI_LINEAR || d->out_format != B2_OUT_BF16 || d->bias != nullptr || d->residual != nullptr)
        return false;
    if (r->head_dim != 256 || r->batch <= 0 || r->tokens <= 0 || r->heads <= 0 || r->kv_heads <= 0) return false;
    if (d->tokens != r->batch * r->tokens || d->tokens > SKINNY_MAX_TOKENS || d->features != (r->heads + 2 * r->kv_heads) * 256) return false;
    if (r->kv_offset < 0 || r->kv_offset + r->tokens > r->kv_capacity || r->factor_batch_stride < 0) return false;
    if (r->sine == nullptr || r->cosine == nullptr || r->q_out == nullptr || r->k_out == nullptr || r->v_out == nullptr) return false;
    const uintptr_t alignment = reinterpret_cast<uintptr_t>(r->sine) | reinterpret_cast<uintptr_t>(r->cosine) |
                                reinterpret_cast<uintptr_t>(r->q_out) | reinterpret_cast<uintptr_t>(r->k_out) | reinterpret_cast<uintptr_t>(r->v_out);
    return (alignment & 15u) == 0;
}

// The packed QKV weight [(heads + 2 kv heads) * 256, row_bytes] as [row_bytes][128 rows][2 halves per head ...]: one box of
// 64 rows x 128 bytes x 2 halves lands as [64 features of a half head | their 64 rotation partners].
static bool make_rope_map(CUtensorMap* map, const void* pointer, int64_t total_heads, int64_t row_bytes) {
    EncodeTiledFn encode = encode_tiled_entry();
    if (encode == nullptr) return false;
    const cuuint64_t dims[3] = {cuuint64_t(row_bytes), 128, cuuint64_t(2 * total_heads)};
    const cuuint64_t strides[2] = {cuuint64_t(row_bytes), cuuint64_t(row_bytes) * 128};
    const cuuint32_t box[3] = {cuuint32_t(STAGE_K_BYTES), 64, 2};
    const cuuint32_t element_strides[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(pointer), dims, strides, box, element_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int KIND, int EPI>
static int launch_skinny(const CUtensorMap& act_map, const CUtensorMap& weight_map, const KernelArgs& args, int shared_bytes,
                         cudaStream_t stream) {
    static bool configured[64] = {false};
    static std::mutex lock;
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64) {
        std::lock_guard<std::mutex> guard(lock);
        if (!configured[device]) {
            const cudaError_t error = cudaFuncSetAttribute(skinny_linear_kernel<KIND, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
            if (error != cudaSuccess) return int(error);
            configured[device] = true;
        }
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(unsigned(args.num_n_tiles * args.splits));
    config.blockDim = dim3(unsigned(SKINNY_THREADS));
    config.dynamicSmemBytes = size_t(shared_bytes);
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
    const cudaError_t error = cudaLaunchKernelEx(&config, skinny_linear_kernel<KIND, EPI>, act_map, weight_map, args);
    return error == cudaSuccess ? int(cudaGetLastError()) : int(error);
}

// `d` has passed run_linear's checks; `epilogue` is the EPI_* it resolved.
int run_linear_skinny(const b2_linear_desc* d, int epilogue, const SkinnyPlan& plan, cudaStream_t stream) {
    const bool nvfp4 = d->kind == B2_KIND_NVFP4;
    const bool geglu = is_gated(epilogue);
    KernelArgs args{};
    args.tokens = d->tokens;
    args.features = d->features;
    args.k_bytes = nvfp4 ? d->width / 2 : d->width;
    args.num_kb = (args.k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES;
    args.tile_n = plan.columns;
    args.num_m_tiles = 1;
    args.num_n_tiles = geglu ? (d->features + 63) / 64 : (d->features + 127) / 128;
    args.total_tiles = args.num_n_tiles;
    args.stages = plan.atoms;
    args.splits = plan.splits;
    args.kps = plan.tokens_per_rank;
    args.a_box_bytes = plan.columns * STAGE_K_BYTES;
    args.up_row_offset = d->features;
    args.scale_column_tiles = nvfp4 ? (d->width / 16 + 3) / 4 : 0;
    args.act_row_blocks = 1;
    args.weight_row_blocks = ((geglu ? 2 : 1) * d->features + 127) / 128;
    args.flags = d->flags;
    args.gelu_lo = args.gelu_hi = 0;
    if (plan.gelu_span > 0) {
        args.gelu_lo = d->gelu_lo;
        args.gelu_hi = d->gelu_hi;
    }
    args.act_scales = static_cast<const uint8_t*>(d->act_scales);
    args.weight_scales = static_cast<const uint8_t*>(d->weight_scales);
    args.act_scale = static_cast<const float*>(d->act_scale);
    args.weight_scale = static_cast<const float*>(d->weight_scale);
    args.weight_scale_up = geglu ? static_cast<const float*>(d->weight_scale_up) : nullptr;
    args.bias = static_cast<const __nv_bfloat16*>(d->bias);
    args.residual = static_cast<const __nv_bfloat16*>(d->residual);
    args.gelu_table = static_cast<const uint16_t*>(d->gelu_table);
    args.out_scale = static_cast<const float*>(d->out_scale);
    args.out = d->out;
    args.out_scales = static_cast<uint8_t*>(d->out_scales);
    args.out_blocked = static_cast<uint8_t*>(d->out_blocked);
    args.status = static_cast<unsigned int*>(d->status);

    CUtensorMap act_map, weight_map;
    if (!make_operand_map(&act_map, d->act, d->tokens, args.k_bytes, plan.columns)) return B2_E_DRIVER;
    if (epilogue == EPI_ROPE) {
        const b2_rope_desc* r = d->rope;
        args.rope_sine = static_cast<const float*>(r->sine);
        args.rope_cosine = static_cast<const float*>(r->cosine);
        args.rope_q = static_cast<__nv_bfloat16*>(r->q_out);
        args.rope_k = static_cast<__nv_bfloat16*>(r->k_out);
        args.rope_v = static_cast<__nv_bfloat16*>(r->v_out);
        args.rope_batch_stride = r->factor_batch_stride;
        args.rope_tokens = r->tokens;
        args.rope_heads = r->heads;
        args.rope_kv_heads = r->kv_heads;
        args.rope_capacity = r->kv_capacity;
        args.rope_offset = r->kv_offset;
        if (!make_rope_map(&weight_map, d->weight, r->heads + 2 * r->kv_heads, args.k_bytes)) return B2_E_DRIVER;
        return launch_skinny<B2_KIND_FP8, EPI_ROPE>(act_map, weight_map, args, plan.shared_bytes, stream);
    }
    if (geglu ? !make_gated_map(&weight_map, d->weight, d->features, args.k_bytes, 64)
              : !make_operand_map(&weight_map, d->weight, d->features, args.k_bytes, 128))
        return B2_E_DRIVER;

#define B2_SKINNY_CASE(KIND_VALUE, EPI_VALUE) \
    case EPI_VALUE: return launch_skinny<KIND_VALUE, EPI_VALUE>(act_map, weight_map, args, plan.shared_bytes, stream)
    if (nvfp4) {
        switch (epilogue) {
            B2_SKINNY_CASE(B2_KIND_NVFP4, EPI_LINEAR);
            B2_SKINNY_CASE(B2_KIND_NVFP4, EPI_GEGLU_BF16);
            B2_SKINNY_CASE(B2_KIND_NVFP4, EPI_GEGLU_FP8);
            B2_SKINNY_CASE(B2_KIND_NVFP4, EPI_GEGLU_NVFP4);
            B2_SKINNY_CASE(B2_KIND_NVFP4, EPI_GELU_BF16);
            B2_SKINNY_CASE(B2_KIND_NVFP4, EPI_GELU_FP8);
            default: return B2_E_UNSUPPORTED;
        }
    }
    switch (epilogue) {
        B2_SKINNY_CASE(B2_KIND_FP8, EPI_LINEAR);
        B2_SKINNY_CASE(B2_KIND_FP8, EPI_GEGLU_BF16);
        B2_SKINNY_CASE(B2_KIND_FP8, EPI_GEGLU_FP8);
        B2_SKINNY_CASE(B2_KIND_FP8, EPI_GEGLU_NVFP4);
        B2_SKINNY_CASE(B2_KIND_FP8, EPI_GELU_BF16);
        B2_SKINNY_CASE(B2_KIND_FP8, EPI_GELU_FP8);
        default: return B2_E_UNSUPPORTED;
    }
#undef B2_SKINNY_CASE
}

}  // namespace b2
