// Quantised Linear, paired schedule: two CTAs of a thread-block cluster (two SMs) compute one tile of
// 256 tokens x BN features with `tcgen05.mma.cta_group::2`.
//
// Why pairs.  With one CTA per 128-token tile (gemm.cu) every K stage moves 128 token rows and BN weight
// rows into shared memory for 128 x BN x 128 bytes of tensor work; the kernel is then bound by operand bytes
// per MMA (L2 -> SM traffic several times the algorithmic bytes, tensor pipe under 20 % busy).  A pair shares
// the weight tile: each CTA loads its own 128 token rows and only HALF of the weight rows (BN/2), the
// hardware reads the other half from the peer's shared memory, and each SM accumulates its own 128 tokens x
// BN features in its own tensor memory.  Operand bytes per MMA drop by a third at BN = 256, and a weight byte
// crosses L2 -> SM once per 256 tokens instead of once per 128.
//
// Roles per CTA (same warp layout as the single-CTA kernel, so the epilogues are shared code):
//   warp 0      TMA producer: this CTA's token rows, its half of the weight rows, (NVFP4) its scale atoms.
//               Every copy completes on the LEADER's `full` barrier (`cp.async.bulk.tensor...cta_group::2`,
//               no multicast anywhere: each CTA issues plain loads of its own operands).
//   warp 1      allocates tensor memory (both CTAs, `cta_group::2`); in the leader (cluster rank 0) it issues
//               the scale copies and the MMAs for both SMs and commits to barriers in both CTAs.
//   warps 2..   epilogue of this CTA's 128 tokens; the accumulator is handed back to the leader's MMA warp
//               through a barrier in the leader's shared memory (the peer arrives remotely).
//
// Every wait is bounded (ptx.cuh); an expired wait leaves a code in the status word and the kernel drains.
// The cluster barriers at entry and exit are hardware barriers that every thread reaches after at most its
// bounded waits.
#include "gemm_epilogue.cuh"

#include <cuda.h>

#include <mutex>
#include <type_traits>

namespace b2 {


constexpr int PAIR_TOKENS = 2 * TILE_TOKENS;
constexpr int PAIR_MAX_SPLITS = 4;

// ---- cta_group::2 forms of the tcgen05 / TMA instructions -------------------------------------------------

__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

// The barrier at the same shared-memory offset in every CTA of `mask` receives one arrival when all tcgen05
// operations issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}

__device__ __forceinline__ void mma_f8f6f4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_nvf4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// Shared memory -> tensor memory in both CTAs of the pair: each reads its own shared memory at the descriptor's
// offset and writes its own tensor memory.
__device__ __forceinline__ void tc_copy_32x128b_x4_pair(uint32_t dst_tmem, uint64_t src_desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(dst_tmem), "l"(src_desc) : "memory");
}

// Tiled load into THIS CTA's shared memory whose completion bytes are counted on a barrier that may live in the
// peer CTA (`bar` is a shared::cluster address).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tensor_map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// Instruction descriptors for the pair: M = 256 (128 rows per CTA).
__device__ __forceinline__ uint32_t idesc_f8_pair(uint32_t n) { return idesc_f8(PAIR_TOKENS, n); }
__device__ __forceinline__ uint32_t idesc_nvf4_pair(uint32_t n) { return idesc_nvf4(PAIR_TOKENS, n); }

// Work items of a cluster.
//   streaming: item = cluster + i * clusters over the n-major list (token pair inner), so the clusters that run side
//       by side share a weight slab (it comes from HBM once and from the L2 afterwards); every K stage loads token
//       rows and weight rows.
//   resident:  the cluster stays on one token pair (cluster % pairs) and walks the feature tiles r, r + G, r + 2G ...
//       (r = cluster / pairs, G = clusters on that pair).  Each CTA loads its 128 token rows for all of K once
//       (shared memory; NVFP4: their scales into tensor memory) and a K stage loads weights only.  Clusters c, c+1 ..
//       of different token pairs start on the same feature tile, so the slab sharing through the L2 stays.
struct PairWalk {
    int item, step, m_pair, n_tile;
    int tile, split, kb_begin, kb_end;      // split K: the work item is (tile, split) and covers K stages [kb_begin, kb_end)
    bool resident;
    __device__ __forceinline__ explicit PairWalk(const KernelArgs& args)
        : item(int(blockIdx.x) >> 1), step(int(gridDim.x) >> 1), resident(args.resident != 0) {
        if (resident) {
            const int cluster = item, clusters = step;
            m_pair = cluster % args.num_m_tiles;
            n_tile = cluster / args.num_m_tiles;
            step = (clusters - m_pair + args.num_m_tiles - 1) / args.num_m_tiles;
            tile = split = kb_begin = 0;
            kb_end = args.num_kb;
        } else {
            decompose(args);
        }
    }
    __device__ __forceinline__ void decompose(const KernelArgs& args) {
        tile = item;
        split = 0;
        kb_begin = 0;
        kb_end = args.num_kb;
        if (args.splits > 1) {
            tile = item / args.splits;
            split = item - tile * args.splits;
            kb_begin = split * args.num_kb / args.splits;
            kb_end = (split + 1) * args.num_kb / args.splits;
        }
        n_tile = tile / args.num_m_tiles;
        m_pair = tile - n_tile * args.num_m_tiles;
    }
    __device__ __forceinline__ bool valid(const KernelArgs& args) const {
        return resident ? n_tile < args.num_n_tiles : item < args.total_tiles * args.splits;
    }
    __device__ __forceinline__ void next(const KernelArgs& args) {
        if (resident) {
            n_tile += step;
        } else {
            item += step;
            decompose(args);
        }
    }
};

// KernelArgs as the pair kernel reads them: num_m_tiles = token PAIRS, tile_n = BN (columns of one CTA's
// accumulator), scale_blocks = 128-row blocks of feature scales per tile (1 or 2), a_box_bytes unused.
//
// SPLIT (plain epilogue only): K is cut into `splits` ranges computed by different clusters, one work item each (the
// host launches exactly tiles x splits clusters, all resident at once).  Every CTA leaves its fp32 partial sums (its
// 128 token rows x BN) in the workspace, the CTAs of a tile meet at a counter, and then EACH of them adds the
// partial sums of its own share of the tile's columns in split order and runs the epilogue on that share: the
// fix-up is as parallel as the main loop, and the result does not depend on timing.  The meeting is a bounded wait.
template <int KIND, int EPI, bool SPLIT>
__global__ void __launch_bounds__(gemm_threads(EPI), 1)
pair_linear_kernel(const __grid_constant__ CUtensorMap act_map, const __grid_constant__ CUtensorMap weight_map,
                   const __grid_constant__ CUtensorMap act_scale_map, const __grid_constant__ CUtensorMap weight_scale_map,
                   const KernelArgs args) {
    constexpr bool GEGLU = is_gated(EPI);
    constexpr bool USES_TABLE = EPI != EPI_LINEAR;
    constexpr bool NVFP4 = KIND == B2_KIND_NVFP4;
    pdl_launch_dependents();
    extern __shared__ uint8_t shared_raw[];
    const uint32_t base = (smem_u32(shared_raw) + 1023u) & ~1023u;
    const int BN = args.tile_n;
    const int features_per_tile = GEGLU ? BN / 2 : BN;
    const uint32_t rank = cluster_cta_rank();
    const bool leader = rank == 0;
    // shared memory: [resident token rows: num_kb x 16 KB][stages x (token tile 16 KB unless resident | half weight tile)]
    //                [stages x (token atoms unless resident | feature atoms)][barriers][GELU table]
    const bool resident = args.resident != 0;
    const uint32_t kps = uint32_t(args.kps);                      // K atoms (128 bytes of K) per ring slot: 1, or 2 in the resident order
    const uint32_t a_stage_bytes = resident ? 0u : uint32_t(A_TILE_BYTES);
    const uint32_t b_tile_bytes = uint32_t(BN / 2) * STAGE_K_BYTES;
    const uint32_t stage_bytes = a_stage_bytes + kps * b_tile_bytes;
    constexpr uint32_t SCALE_PART_BYTES = SCALE_ATOMS_PER_STAGE * SCALE_ATOM_BYTES;
    const uint32_t token_part_bytes = resident ? 0u : SCALE_PART_BYTES;
    const uint32_t feature_part_bytes = uint32_t(args.scale_blocks) * SCALE_PART_BYTES;      // feature atoms of one K atom
    const uint32_t scale_stage_bytes = NVFP4 ? token_part_bytes + kps * feature_part_bytes : 0u;
    const uint32_t panel_base = base;
    const uint32_t stage_base = panel_base + (resident ? uint32_t(args.num_kb) * A_TILE_BYTES : 0u);
    const uint32_t scale_base = stage_base + uint32_t(args.stages) * stage_bytes;
    const uint32_t barrier_base = scale_base + uint32_t(args.stages) * scale_stage_bytes;
    const uint32_t full_bar = barrier_base;                       // [stages]  used in the leader only
    const uint32_t empty_bar = barrier_base + 8 * MAX_STAGES;     // [stages]  one per CTA
    const uint32_t acc_full_bar = barrier_base + 16 * MAX_STAGES; // [2]       one per CTA
    const uint32_t acc_empty_bar = acc_full_bar + 16;             // [2]       used in the leader only
    const uint32_t panel_bar = acc_empty_bar + 16;                // [MAX_RESIDENT_KB] leader only: both CTAs' token rows of K stage kb landed
    const uint32_t tmem_slot = panel_bar + 8 * MAX_RESIDENT_KB;
    const uint32_t compact_table = tmem_slot + 16;                // 2 * (gelu_hi - gelu_lo) bf16 entries
    // the leader's barriers as the peer addresses them
    const uint32_t full_bar_leader = cluster_map_shared(full_bar, 0u);
    const uint32_t acc_empty_bar_leader = cluster_map_shared(acc_empty_bar, 0u);
    const uint32_t panel_bar_leader = cluster_map_shared(panel_bar, 0u);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&act_map);
        tma_prefetch_descriptor(&weight_map);
        if (NVFP4) {
            tma_prefetch_descriptor(&act_scale_map);
            tma_prefetch_descriptor(&weight_scale_map);
        }
        for (int s = 0; s < args.stages; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar + 8 * b, 1);
            mbar_init(acc_empty_bar + 8 * b, 2 * epilogue_warps(EPI));     // the epilogue warps of both CTAs
        }
        for (int kb = 0; kb < MAX_RESIDENT_KB; ++kb) mbar_init(panel_bar + 8 * kb, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, TMEM_COLUMNS);
        tmem_relinquish_pair();
    }
    // Both CTAs' barriers and tensor memory exist before either touches the other's.
    tc_fence_before_sync();
    cluster_arrive();
    cluster_wait();
    tc_fence_after_sync();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");
    // The shared-memory copy of the GELU table is the epilogue warps' business only: they fill it (the table is a
    // constant of the model, so this may run ahead of the launches before this one) and meet at their own barrier,
    // while the producer and the MMA warp are already at work.
    if (USES_TABLE && warp >= FIRST_EPILOGUE_WARP) {
        fill_compact_gelu(args, compact_table, int(threadIdx.x) - 32 * FIRST_EPILOGUE_WARP, 32 * epilogue_warps(EPI));
        asm volatile("bar.sync 1, %0;" ::"r"(32 * epilogue_warps(EPI)) : "memory");
    }

    pdl_wait();

    bool failed = false;
    const int num_kb = args.num_kb;
    const int last_kb_mmas = ((args.k_bytes - (num_kb - 1) * STAGE_K_BYTES) + 31) / 32;
    // bytes one CTA brings per stage; boxes that reach beyond a matrix are filled with zeros and still count in full
    const uint32_t atom_tx_bytes = a_stage_bytes + b_tile_bytes + (NVFP4 ? token_part_bytes + feature_part_bytes : 0u);   // per K atom

    using Yes = std::true_type;
    using No = std::false_type;
    const bool paired_scales = GEGLU && (args.flags & B2_LINEAR_PAIRED_GATE_UP_SCALES) != 0;
    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer (both CTAs)
        auto producer_role = [&](auto order_tag) {
            constexpr int ORDER = decltype(order_tag)::value;      // 0 streaming, 1 resident, 2 resident with two K atoms per slot
            constexpr bool RESIDENT = ORDER != 0;
            constexpr int KPS = ORDER == 2 ? 2 : 1;
            int stage = 0;
            uint32_t phase = 0;
            uint32_t filled = 0, fill_parity = 0;
            PairWalk walk(args);
            const bool panel_loaded = RESIDENT && walk.valid(args);
            if (panel_loaded) {
                // this CTA's 128 token rows for all of K, once; (NVFP4) their scale atoms travel through the first slots of
                // the stage ring, from where the MMA warp moves them into tensor memory for good
                const int m0 = walk.m_pair * PAIR_TOKENS + int(rank) * TILE_TOKENS;
                if (elect_one()) {
                    for (int kb = 0; kb < num_kb; ++kb) {
                        if (leader) mbar_expect_tx(panel_bar + 8 * kb, 2u * A_TILE_BYTES);
                        tma_load_2d_pair(panel_base + uint32_t(kb) * A_TILE_BYTES, &act_map, panel_bar_leader + 8 * kb, kb * STAGE_K_BYTES, m0);
                    }
                }
                __syncwarp();
                if (NVFP4) {
                    const int token_atom_row = (2 * walk.m_pair + int(rank)) * args.scale_column_tiles;
                    for (int kb = 0; kb < num_kb; kb += KPS) {
                        mbar_wait(empty_bar + 8 * stage, phase ^ 1u, failed, args.status, STATUS_WAIT_PRODUCER);
                        __syncwarp();
                        filled |= 1u << stage;
                        fill_parity = (fill_parity & ~(1u << stage)) | (phase << stage);
                        if (elect_one()) {
                            const int atoms = min(KPS, num_kb - kb);
                            if (leader) mbar_expect_tx(full_bar + 8 * stage, 2u * uint32_t(atoms) * SCALE_PART_BYTES);
#pragma unroll
                            for (int k = 0; k < KPS; ++k)
                                if (k < atoms)
                                    tma_load_2d_pair(scale_base + uint32_t(stage) * scale_stage_bytes + uint32_t(k) * SCALE_PART_BYTES, &act_scale_map,
                                                     full_bar_leader + 8 * stage, 0, token_atom_row + (kb + k) * SCALE_ATOMS_PER_STAGE);
                        }
                        __syncwarp();
                        if (++stage == args.stages) { stage = 0; phase ^= 1u; }
                    }
                }
            }
            for (; walk.valid(args); walk.next(args)) {
                const int m0 = walk.m_pair * PAIR_TOKENS + int(rank) * TILE_TOKENS;
                const int f0 = walk.n_tile * features_per_tile;
                // this CTA's half of the weight tile: plain -> rows [f0 + rank*BN/2, +BN/2); gated -> the gate rows (leader)
                // or the up rows (peer) of features [f0, f0 + BN/2)
                const int weight_row = GEGLU ? int(rank) * args.up_row_offset + f0 : f0 + int(rank) * (BN / 2);
                // scale atoms: token rows of this CTA; feature rows of the WHOLE tile (every SM scales all BN columns).
                // With the paired gate/up layout the 64 gate + 64 up rows of feature tile n form the n-th 128-row block.
                const int token_atom_row = (2 * walk.m_pair + int(rank)) * args.scale_column_tiles;
                int feature_atom_row[2];
                feature_atom_row[0] = (paired_scales ? walk.n_tile : (f0 >> 7)) * args.scale_column_tiles;
                feature_atom_row[1] = (GEGLU ? ((args.up_row_offset + f0) >> 7) : (f0 >> 7) + 1) * args.scale_column_tiles;
                for (int kb = walk.kb_begin; kb < walk.kb_end; kb += KPS) {
                    mbar_wait(empty_bar + 8 * stage, phase ^ 1u, failed, args.status, STATUS_WAIT_PRODUCER);
                    __syncwarp();
                    filled |= 1u << stage;
                    fill_parity = (fill_parity & ~(1u << stage)) | (phase << stage);
                    if (elect_one()) {
                        const uint32_t bar = full_bar_leader + 8 * stage;
                        const uint32_t slot_smem = stage_base + uint32_t(stage) * stage_bytes;
                        const uint32_t s_smem = scale_base + uint32_t(stage) * scale_stage_bytes;
                        const int atoms = min(KPS, walk.kb_end - kb);
                        if (leader) mbar_expect_tx(full_bar + 8 * stage, 2u * uint32_t(atoms) * atom_tx_bytes);
#pragma unroll
                        for (int k = 0; k < KPS; ++k) {
                            if (k < atoms) {
                                const int k0 = (kb + k) * STAGE_K_BYTES;
                                const int atom = (kb + k) * SCALE_ATOMS_PER_STAGE;
                                if (!RESIDENT) tma_load_2d_pair(slot_smem, &act_map, bar, k0, m0);
                                tma_load_2d_pair(slot_smem + a_stage_bytes + uint32_t(k) * b_tile_bytes, &weight_map, bar, k0, weight_row);
                                if (NVFP4) {
                                    const uint32_t f_smem = s_smem + token_part_bytes + uint32_t(k) * feature_part_bytes;
                                    if (!RESIDENT) tma_load_2d_pair(s_smem, &act_scale_map, bar, 0, token_atom_row + atom);
                                    tma_load_2d_pair(f_smem, &weight_scale_map, bar, 0, feature_atom_row[0] + atom);
                                    if (args.scale_blocks == 2)
                                        tma_load_2d_pair(f_smem + SCALE_PART_BYTES, &weight_scale_map, bar, 0, feature_atom_row[1] + atom);
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (++stage == args.stages) { stage = 0; phase ^= 1u; }
                }
            }
            // The leader does not leave while a copy of the pair is still in flight: wait (bounded) for the last fill of
            // every stage.  On the normal path these have all completed already.
            if (leader) {
                bool drain_failed = false;
                for (int s = 0; s < args.stages; ++s)
                    if (filled & (1u << s))
                        mbar_wait(full_bar + 8 * s, (fill_parity >> s) & 1u, drain_failed, args.status, STATUS_WAIT_DRAIN);
                if (panel_loaded)
                    for (int kb = 0; kb < num_kb; ++kb) mbar_wait(panel_bar + 8 * kb, 0u, drain_failed, args.status, STATUS_WAIT_DRAIN);
            }
        };
        if (!resident) producer_role(std::integral_constant<int, 0>{});
        else if (args.kps == 2) producer_role(std::integral_constant<int, 2>{});
        else producer_role(std::integral_constant<int, 1>{});
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer (leader only)
        // The tcgen05 instructions of a ring slot are few, but the barrier waits, the election and the operand
        // arithmetic around them are a dependent chain of a hundred-odd instructions that this one warp works through
        // slot after slot while sharing its scheduler with four epilogue warps: everything a slot needs is computed
        // before the election, and the elected lane then issues the copies and MMAs back to back.
        if (leader) {
            auto mma_role = [&](auto order_tag, auto two_blocks_tag, auto lag_tag) {
                constexpr int ORDER = decltype(order_tag)::value;      // 0 streaming, 1 resident, 2 resident with two K atoms per slot
                constexpr bool RESIDENT = ORDER != 0;
                constexpr int KPS = ORDER == 2 ? 2 : 1;
                constexpr bool TWO = decltype(two_blocks_tag)::value;
                // LAG: fewer sets of feature-scale columns than K atoms in the ring, so a set's reuse needs its own wait.
                // With one set per atom of every slot (the usual case) the set is free whenever the slot's `full` barrier
                // has completed again: the producer refilled the slot only after the MMAs that read it, and its scales,
                // had completed.
                constexpr bool LAG = decltype(lag_tag)::value;
                static_assert(!(LAG && KPS == 2), "two atoms per slot need a scale set per atom");
                const uint32_t idesc = NVFP4 ? idesc_nvf4_pair(uint32_t(BN)) : idesc_f8_pair(uint32_t(BN));
                const uint64_t operand_desc = smem_desc_sw128(0);
                const uint32_t operand_low = uint32_t(operand_desc), operand_high = uint32_t(operand_desc >> 32);
                const uint64_t scale_desc = smem_desc_scale_atom(0);
                const uint32_t scale_desc_high = uint32_t(scale_desc >> 32);
                const uint32_t set_columns = uint32_t((RESIDENT ? 0 : TMEM_SFA_COLUMNS) + 16 * args.scale_blocks);
                // resident order: the token scales of all K stages sit in tensor memory right after the accumulators
                const uint32_t resident_sfa = tmem_base + uint32_t(args.accumulators * args.accumulator_stride);
                constexpr uint32_t ATOM = SCALE_ATOM_BYTES >> 4, PART = SCALE_ATOMS_PER_STAGE * ATOM;
                const bool two_accumulators = args.accumulators == 2;
                int stage = 0;
                uint32_t phase = 0;
                int local_tile = 0;
                PairWalk walk(args);
                if (RESIDENT && NVFP4 && walk.valid(args)) {
                    // the first ring slots carry the token scale atoms of both CTAs: into tensor memory, slot freed
                    for (int kb = 0; kb < num_kb; kb += KPS) {
                        mbar_wait(full_bar + 8 * stage, phase, failed, args.status, STATUS_WAIT_MMA_FULL);
                        tc_fence_after_sync();
                        __syncwarp();
                        if (elect_one()) {
                            const uint32_t atom_low = (scale_base + uint32_t(stage) * scale_stage_bytes) >> 4;
#pragma unroll
                            for (int k = 0; k < KPS; ++k)
                                if (kb + k < num_kb) {
#pragma unroll
                                    for (int j = 0; j < SCALE_ATOMS_PER_STAGE; ++j)
                                        tc_copy_32x128b_x4_pair(resident_sfa + uint32_t((kb + k) * TMEM_SFA_COLUMNS + j * 4),
                                                                desc_from_words(atom_low + k * PART + j * ATOM, scale_desc_high));
                                }
                            tc_commit_pair(empty_bar + 8 * stage, 3);
                        }
                        __syncwarp();
                        if (++stage == args.stages) { stage = 0; phase ^= 1u; }
                    }
                }
                int set = 0, lag_stage = stage, issued = 0;
                uint32_t lag_phase = phase;
                for (; walk.valid(args); walk.next(args), ++local_tile) {
                    const int f0 = walk.n_tile * features_per_tile;
                    // a 64- or 128-column tile that starts inside a 128-row scale block starts at that block's column
                    const uint32_t scale_column = (GEGLU || BN == 256) ? 0u : uint32_t((f0 & 127) >> 5);
                    const int buffer = two_accumulators ? local_tile & 1 : 0;
                    const uint32_t use = uint32_t(two_accumulators ? local_tile >> 1 : local_tile);
                    const uint32_t d_tmem = tmem_base + uint32_t(buffer * args.accumulator_stride);
                    // the epilogue has drained this accumulator's last use
                    mbar_wait(acc_empty_bar + 8 * buffer, (use & 1u) ^ 1u, failed, args.status, STATUS_WAIT_MMA_TMEM);
                    tc_fence_after_sync();
                    for (int kb = walk.kb_begin; kb < walk.kb_end; kb += KPS) {
                        mbar_wait(full_bar + 8 * stage, phase, failed, args.status, STATUS_WAIT_MMA_FULL);
                        if (RESIDENT && local_tile == 0) {       // first pass over K: the token rows may still be landing
                            mbar_wait(panel_bar + 8 * kb, 0u, failed, args.status, STATUS_WAIT_MMA_FULL);
                            if (KPS == 2 && kb + 1 < num_kb) mbar_wait(panel_bar + 8 * (kb + 1), 0u, failed, args.status, STATUS_WAIT_MMA_FULL);
                        }
                        if (NVFP4 && LAG) {
                            // a set of scale columns is overwritten only after the MMAs that last read it have completed
                            if (issued >= args.scale_sets) {
                                mbar_wait(empty_bar + 8 * lag_stage, lag_phase, failed, args.status, STATUS_WAIT_MMA_TMEM);
                                if (++lag_stage == args.stages) { lag_stage = 0; lag_phase ^= 1u; }
                            }
                            ++issued;
                        }
                        tc_fence_after_sync();
                        // every operand of the slot's instructions, before the election
                        const uint32_t slot_smem = stage_base + uint32_t(stage) * stage_bytes;
                        const uint32_t atom_low = (scale_base + uint32_t(stage) * scale_stage_bytes) >> 4;
                        uint32_t a_low[KPS], b_low[KPS], sfa_tmem[KPS], sfb_tmem[KPS], feature_low[KPS];
                        int count[KPS];
#pragma unroll
                        for (int k = 0; k < KPS; ++k) {
                            const int atom_kb = kb + k;
                            a_low[k] = operand_low + ((RESIDENT ? panel_base + uint32_t(atom_kb) * A_TILE_BYTES : slot_smem) >> 4);
                            b_low[k] = operand_low + ((slot_smem + a_stage_bytes + uint32_t(k) * b_tile_bytes) >> 4);
                            const uint32_t set_tmem = tmem_base + uint32_t(TMEM_COLUMNS) - set_columns * uint32_t((LAG ? set : stage * KPS + k) + 1);
                            sfa_tmem[k] = RESIDENT ? resident_sfa + uint32_t(atom_kb * TMEM_SFA_COLUMNS) : set_tmem;
                            sfb_tmem[k] = RESIDENT ? set_tmem : set_tmem + TMEM_SFA_COLUMNS;
                            feature_low[k] = atom_low + (RESIDENT ? uint32_t(k * args.scale_blocks) * PART : PART);
                            count[k] = atom_kb >= walk.kb_end ? 0 : (atom_kb == num_kb - 1 ? last_kb_mmas : SCALE_ATOMS_PER_STAGE);
                        }
                        const bool full_slot = count[KPS - 1] == SCALE_ATOMS_PER_STAGE && (KPS == 1 || count[0] == SCALE_ATOMS_PER_STAGE);
                        const bool last_slot = kb + KPS >= walk.kb_end;
                        __syncwarp();
                        if (elect_one()) {
                            // `limit` is a literal except in a slot with a ragged or missing K atom
                            auto issue = [&](auto full_tag) {
                                constexpr bool FULL = decltype(full_tag)::value;
#pragma unroll
                                for (int k = 0; k < KPS; ++k) {
                                    const int limit = FULL ? SCALE_ATOMS_PER_STAGE : count[k];
                                    if (NVFP4) {
#pragma unroll
                                        for (int j = 0; j < SCALE_ATOMS_PER_STAGE; ++j) {
                                            if (j < limit) {
                                                if (!RESIDENT) tc_copy_32x128b_x4_pair(sfa_tmem[k] + j * 4, desc_from_words(atom_low + j * ATOM, scale_desc_high));
                                                tc_copy_32x128b_x4_pair(sfb_tmem[k] + j * (TWO ? 8 : 4), desc_from_words(feature_low[k] + j * ATOM, scale_desc_high));
                                                if (TWO)
                                                    tc_copy_32x128b_x4_pair(sfb_tmem[k] + j * 8 + 4, desc_from_words(feature_low[k] + PART + j * ATOM, scale_desc_high));
                                            }
                                        }
                                    }
#pragma unroll
                                    for (int j = 0; j < SCALE_ATOMS_PER_STAGE; ++j) {
                                        if (j < limit) {
                                            const uint32_t accumulate = (j == 0 && k == 0) ? uint32_t(kb != walk.kb_begin) : 1u;
                                            const uint64_t a_desc = desc_from_words(a_low[k] + 2 * j, operand_high);
                                            const uint64_t b_desc = desc_from_words(b_low[k] + 2 * j, operand_high);
                                            if (NVFP4)
                                                mma_nvf4_pair(d_tmem, a_desc, b_desc, idesc, sfa_tmem[k] + j * 4,
                                                              sfb_tmem[k] + j * (TWO ? 8 : 4) + scale_column, accumulate);
                                            else
                                                mma_f8f6f4_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
                                        }
                                    }
                                }
                            };
                            if (full_slot) issue(Yes{});
                            else issue(No{});
                            tc_commit_pair(empty_bar + 8 * stage, 3);     // the slot is free again in both CTAs
                            if (last_slot) tc_commit_pair(acc_full_bar + 8 * buffer, 3);
                        }
                        __syncwarp();
                        if (NVFP4 && LAG && ++set == args.scale_sets) set = 0;
                        if (++stage == args.stages) { stage = 0; phase ^= 1u; }
                    }
                }
            };
            using Order0 = std::integral_constant<int, 0>;
            using Order1 = std::integral_constant<int, 1>;
            using Order2 = std::integral_constant<int, 2>;
            const bool two_blocks = NVFP4 && args.scale_blocks == 2;
            const bool lag = NVFP4 && args.scale_sets < args.stages * args.kps;
            if (resident && args.kps == 2) {
                if (two_blocks) mma_role(Order2{}, Yes{}, No{}); else mma_role(Order2{}, No{}, No{});
            } else if (lag) {
                if (resident) { if (two_blocks) mma_role(Order1{}, Yes{}, Yes{}); else mma_role(Order1{}, No{}, Yes{}); }
                else { if (two_blocks) mma_role(Order0{}, Yes{}, Yes{}); else mma_role(Order0{}, No{}, Yes{}); }
            } else {
                if (resident) { if (two_blocks) mma_role(Order1{}, Yes{}, No{}); else mma_role(Order1{}, No{}, No{}); }
                else { if (two_blocks) mma_role(Order0{}, Yes{}, No{}); else mma_role(Order0{}, No{}, No{}); }
            }
        }
    } else {
        // ------------------------------------------------------------- epilogue (both CTAs, own 128 tokens)
        const int quarter = warp & 3;
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
        constexpr int WARPS_PER_QUARTER = epilogue_warps(EPI) / 4;
        const int part = (warp - FIRST_EPILOGUE_WARP) >> 2;
        const bool two_accumulators = args.accumulators == 2;
        int local_tile = 0;
        for (PairWalk walk(args); walk.valid(args); walk.next(args), ++local_tile) {
            const int token0 = walk.m_pair * PAIR_TOKENS + int(rank) * TILE_TOKENS + quarter * 32;
            const int token = token0 + lane;
            const int f0 = walk.n_tile * features_per_tile;
            const int buffer = two_accumulators ? local_tile & 1 : 0;
            const uint32_t use = uint32_t(two_accumulators ? local_tile >> 1 : local_tile);
            mbar_wait(acc_full_bar + 8 * buffer, use & 1u, failed, args.status, STATUS_WAIT_EPILOGUE);
            tc_fence_after_sync();
            const uint32_t lane_address = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(buffer * args.accumulator_stride);
            const bool warp_has_tokens = token0 < args.tokens;      // else: padding rows only
            // The accumulator goes back to the MMA warp as soon as this warp's columns sit in registers as bf16
            // words (scales applied): the table look-ups, the encoding and the stores then overlap the next tile's
            // main loop even when only one accumulator fits in tensor memory.
            auto release = [&]() {
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (leader) mbar_arrive(acc_empty_bar + 8 * buffer);
                    else mbar_arrive_cluster(acc_empty_bar_leader + 8 * buffer);
                }
            };
            if constexpr (SPLIT) {
                // (a) this CTA's partial sums (valid token rows) -> its slot of the workspace, the accumulator goes back
                const int64_t slot_floats = int64_t(TILE_TOKENS) * BN;
                float* slots = args.partials + (int64_t(walk.tile) * args.splits * 2 + rank) * slot_floats;   // [split][rank][128][BN], this rank
                // A slot is laid out [BN / 4 column groups][128 rows][4 floats]: the 32 lanes of a warp (32 token rows)
                // write, and later read, 512 contiguous bytes per instruction.
                // This CTA's own share of the columns (chunks [c0, c1) of 32) never leaves tensor memory: only the other
                // chunks are written, and the accumulator is kept until the sums are done (a cluster has one work item).
                const int row = quarter * 32 + lane;
                const int chunks = BN / 32;
                const int c0 = walk.split * chunks / args.splits, c1 = (walk.split + 1) * chunks / args.splits;
                uint4* mine = reinterpret_cast<uint4*>(slots + int64_t(walk.split) * 2 * slot_floats) + row;
                for (int chunk = part; chunk < chunks && warp_has_tokens; chunk += WARPS_PER_QUARTER) {
                    if (chunk >= c0 && chunk < c1) continue;
                    uint32_t v[32];
                    tmem_load_32x32(lane_address + chunk * 32, v);
                    tmem_load_wait();
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        __stcg(mine + (chunk * 8 + i) * TILE_TOKENS, make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
                }
                // (b) meet the other splits of this tile (same rank): one thread counts in and waits, bounded
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"r"(32 * epilogue_warps(EPI)) : "memory");
                unsigned int* arrived = args.tickets + 4 * walk.tile + rank;          // per tile: arrived[2], departed[2]
                unsigned int* departed = arrived + 2;
                if (threadIdx.x == 32 * FIRST_EPILOGUE_WARP) {
                    atomicAdd(arrived, 1u);
                    const long long start = clock64();
                    unsigned int seen = 0, ok = 1;
                    while (true) {
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(arrived) : "memory");
                        if (seen >= unsigned(args.splits)) break;
                        if (clock64() - start > WAIT_LIMIT_CYCLES) {
                            ok = 0;
                            if (args.status != nullptr) atomicCAS(args.status, 0u, unsigned(STATUS_WAIT_SPLIT));
                            break;
                        }
                    }
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(tmem_slot + 8), "r"(ok) : "memory");
                }
                asm volatile("bar.sync 1, %0;" ::"r"(32 * epilogue_warps(EPI)) : "memory");
                unsigned int met;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(met) : "r"(tmem_slot + 8) : "memory");
                // (c) this split's share of the columns: the other splits' partial sums (up to three: every load of a
                // 16-column group is issued before the first addition) and its own from tensor memory, added in split
                // order whichever CTA does it; then the plain epilogue
                const float4* row_sums = reinterpret_cast<const float4*>(slots) + row;
                for (int chunk = c0 + part; chunk < c1 && warp_has_tokens && met; chunk += WARPS_PER_QUARTER) {
                    uint32_t first[32];
                    tmem_load_32x32(lane_address + chunk * 32, first);
                    tmem_load_wait();
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        float4 piece[PAIR_MAX_SPLITS][4];
#pragma unroll
                        for (int q = 0; q < PAIR_MAX_SPLITS; ++q)
                            if (q < args.splits && q != walk.split) {
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    piece[q][j] = __ldcg(row_sums + int64_t(q) * 2 * (slot_floats / 4) + (chunk * 8 + half * 4 + j) * TILE_TOKENS);
                            }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                            for (int q = 0; q < PAIR_MAX_SPLITS; ++q)
                                if (q < args.splits) {
                                    float4 term = piece[q][j];
                                    if (q == walk.split)
                                        term = make_float4(__uint_as_float(first[half * 16 + 4 * j]), __uint_as_float(first[half * 16 + 4 * j + 1]),
                                                           __uint_as_float(first[half * 16 + 4 * j + 2]), __uint_as_float(first[half * 16 + 4 * j + 3]));
                                    if (q == 0) {
                                        total = term;
                                    } else {
                                        total.x = __fadd_rn(total.x, term.x); total.y = __fadd_rn(total.y, term.y);
                                        total.z = __fadd_rn(total.z, term.z); total.w = __fadd_rn(total.w, term.w);
                                    }
                                }
                            first[half * 16 + 4 * j] = __float_as_uint(total.x); first[half * 16 + 4 * j + 1] = __float_as_uint(total.y);
                            first[half * 16 + 4 * j + 2] = __float_as_uint(total.z); first[half * 16 + 4 * j + 3] = __float_as_uint(total.w);
                        }
                    }
                    epilogue_linear_chunk<EPI_LINEAR>(first, args, scale, round_scale, token, f0 + chunk * 32, compact_table, out_scale,
                                                      out_scale_rcp, true_div);
                }
                release();
                // (d) the last CTA to leave puts both counters back to zero for the next launch
                asm volatile("bar.sync 1, %0;" ::"r"(32 * epilogue_warps(EPI)) : "memory");
                if (threadIdx.x == 32 * FIRST_EPILOGUE_WARP && met) {
                    if (atomicAdd(departed, 1u) == unsigned(args.splits - 1)) {
                        *arrived = 0u;
                        *departed = 0u;
                    }
                }
            } else if (GEGLU) {
                constexpr int UNITS_PER_WARP = (128 / 16 + WARPS_PER_QUARTER - 1) / WARPS_PER_QUARTER;   // at most 128 features per tile
                const int units = features_per_tile / 16;
                uint32_t gate[UNITS_PER_WARP][8], up[UNITS_PER_WARP][8];
#pragma unroll
                for (int u = 0; u < UNITS_PER_WARP; ++u) {       // one unit's 32 accumulator registers at a time (96-register budget)
                    const int unit = part + u * WARPS_PER_QUARTER;
                    if (unit < units && warp_has_tokens) {
                        uint32_t first[16], second[16];
                        tmem_load_32x16(lane_address + unit * 16, first);
                        tmem_load_32x16(lane_address + BN / 2 + unit * 16, second);
                        tmem_load_wait();
                        geglu_scale_unit(first, second, scale, scale_up, round_scale, gate[u], up[u]);
                    }
                }
                release();
#pragma unroll
                for (int u = 0; u < UNITS_PER_WARP; ++u) {
                    const int unit = part + u * WARPS_PER_QUARTER;
                    if (unit < units && warp_has_tokens)
                        epilogue_geglu_words<GEGLU ? EPI : EPI_GEGLU_BF16>(gate[u], up[u], args, compact_table, out_scale, by_global,
                                                                          out_scale_rcp, true_div, token, f0 + unit * 16);
                }
            } else {
                constexpr int CHUNKS_PER_WARP = (256 / 32 + WARPS_PER_QUARTER - 1) / WARPS_PER_QUARTER;  // at most 256 features per tile
                const int chunks = features_per_tile / 32;
                uint32_t y[CHUNKS_PER_WARP][16];
                // accumulator chunks in flight per thread: two (64 registers) with the eight-warp plain epilogue, one
                // with the sixteen-warp table epilogues, whose threads have 96 registers
                constexpr int IN_FLIGHT = WARPS_PER_QUARTER == 2 ? 2 : 1;
#pragma unroll
                for (int c = 0; c < CHUNKS_PER_WARP; c += IN_FLIGHT) {
                    uint32_t first[IN_FLIGHT][32];
#pragma unroll
                    for (int i = 0; i < IN_FLIGHT; ++i) {
                        const int chunk = part + (c + i) * WARPS_PER_QUARTER;
                        if (c + i < CHUNKS_PER_WARP && chunk < chunks && warp_has_tokens) tmem_load_32x32(lane_address + chunk * 32, first[i]);
                    }
                    tmem_load_wait();
#pragma unroll
                    for (int i = 0; i < IN_FLIGHT; ++i) {
                        const int chunk = part + (c + i) * WARPS_PER_QUARTER;
                        if (c + i < CHUNKS_PER_WARP && chunk < chunks && warp_has_tokens) linear_scale_chunk(first[i], scale, round_scale, y[c + i]);
                    }
                }
                release();
#pragma unroll
                for (int c = 0; c < CHUNKS_PER_WARP; ++c) {
                    const int chunk = part + c * WARPS_PER_QUARTER;
                    if (chunk < chunks && warp_has_tokens)
                        epilogue_linear_words<GEGLU ? EPI_LINEAR : EPI>(y[c], args, token, f0 + chunk * 32, compact_table, out_scale,
                                                                        out_scale_rcp, true_div);
                }
            }
        }
    }

    // Neither CTA leaves (or frees tensor memory) while the other may still read its shared memory, write its
    // barriers or run MMAs into its tensor memory.
    tc_fence_before_sync();
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, TMEM_COLUMNS);
    }
}

// ---------------------------------------------------------------------------
// host side

// Scale atoms ([row blocks][column tiles] x 512 bytes, the 128x4-tile layout) as a matrix of 512-byte rows: one box =
// the four atoms of a K stage.  Rows beyond the array read as zero.
static bool make_atom_map(CUtensorMap* map, const void* pointer, int64_t atoms) {
    EncodeTiledFn encode = encode_tiled_entry();
    if (encode == nullptr) return false;
    const cuuint64_t dims[2] = {cuuint64_t(SCALE_ATOM_BYTES / 4), cuuint64_t(atoms)};
    const cuuint64_t strides[1] = {cuuint64_t(SCALE_ATOM_BYTES)};
    const cuuint32_t box[2] = {cuuint32_t(SCALE_ATOM_BYTES / 4), cuuint32_t(SCALE_ATOMS_PER_STAGE)};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(pointer), dims, strides, box, element_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int KIND, int EPI, bool SPLIT>
static int launch_pair_variant(const CUtensorMap& act_map, const CUtensorMap& weight_map, const CUtensorMap& act_scale_map,
                       const CUtensorMap& weight_scale_map, const KernelArgs& args, int shared_bytes, cudaStream_t stream) {
    static bool configured[64] = {false};
    static std::mutex lock;
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64) {
        std::lock_guard<std::mutex> guard(lock);
        if (!configured[device]) {
            const cudaError_t error = cudaFuncSetAttribute(pair_linear_kernel<KIND, EPI, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
            if (error != cudaSuccess) return int(error);
            configured[device] = true;
        }
    }
    const int items = args.total_tiles * args.splits;
    const int clusters = items < sm_count() / 2 ? items : sm_count() / 2;      // resident: at least one cluster per token pair (pair_plan)
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(unsigned(2 * clusters));
    config.blockDim = dim3(unsigned(gemm_threads(EPI)));
    config.dynamicSmemBytes = size_t(shared_bytes);
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 2;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = pdl_enabled() ? 2 : 1;
    const cudaError_t error = cudaLaunchKernelEx(&config, pair_linear_kernel<KIND, EPI, SPLIT>, act_map, weight_map, act_scale_map,
                                                 weight_scale_map, args);
    return error == cudaSuccess ? int(cudaGetLastError()) : int(error);
}

template <int KIND, int EPI>
static int launch_pair(const CUtensorMap& act_map, const CUtensorMap& weight_map, const CUtensorMap& act_scale_map,
                       const CUtensorMap& weight_scale_map, const KernelArgs& args, int shared_bytes, cudaStream_t stream) {
    if constexpr (EPI == EPI_LINEAR) {
        if (args.splits > 1)
            return launch_pair_variant<KIND, EPI, true>(act_map, weight_map, act_scale_map, weight_scale_map, args, shared_bytes, stream);
    }
    return launch_pair_variant<KIND, EPI, false>(act_map, weight_map, act_scale_map, weight_scale_map, args, shared_bytes, stream);
}

constexpr int64_t PAIR_TICKET_BYTES = 1024;      // per tile: arrived[2], departed[2] (uint32); zero between launches

// Shared memory outside the stage ring and the resident token rows.
static int pair_fixed_bytes(int gelu_span) {
    return 1024 /* alignment slack */ + 16 * MAX_STAGES + 8 * MAX_RESIDENT_KB + 128 + 4 * gelu_span;
}

static int compact_gelu_span(const b2_linear_desc* d) {
    if (d->epilogue != B2_EPI_LINEAR && d->gelu_lo >= 0x80 && d->gelu_hi > d->gelu_lo && d->gelu_hi <= 0x7f80 &&
        d->gelu_hi - d->gelu_lo <= MAX_COMPACT_GELU)
        return d->gelu_hi - d->gelu_lo;
    return 0;
}

// The resident order for a tile of `columns` accumulator columns: does everything fit, and is it worth it?
//   shared memory: the token rows of all of K (num_kb x 16 KB per CTA) beside at least four weight stages;
//   tensor memory: the accumulators (two when they fit), the token scales of all of K, two or more feature-scale sets;
//   work: at least two tiles per SM pair on average, so that loading the token rows once is amortised.
static bool pair_resident_fits(const b2_linear_desc* d, int columns, int scale_blocks, int num_kb, int pairs, int64_t tiles) {
    if (d->flags & B2_LINEAR_STREAM_TOKENS) return false;
    const bool nvfp4 = d->kind == B2_KIND_NVFP4;
    const int clusters = sm_count() / 2;
    if (num_kb > MAX_RESIDENT_KB || pairs > clusters || tiles < 2 * int64_t(clusters)) return false;
    constexpr int SCALE_PART_BYTES = SCALE_ATOMS_PER_STAGE * SCALE_ATOM_BYTES;
    const int stage_bytes = (columns / 2) * STAGE_K_BYTES + (nvfp4 ? scale_blocks * SCALE_PART_BYTES : 0);
    const int stages = (SMEM_LIMIT - pair_fixed_bytes(compact_gelu_span(d)) - num_kb * A_TILE_BYTES) / stage_bytes;
    if (stages < 4) return false;
    if (nvfp4) {
        const int free_columns = TMEM_COLUMNS - columns - num_kb * TMEM_SFA_COLUMNS;
        if (free_columns < 2 * 16 * scale_blocks) return false;
    }
    return true;
}

// What the paired schedule would do with this launch: accumulator columns (0 = it does not apply), K splits, the
// workspace bytes the splits need, and whether the token rows stay on chip.
//   Pairs apply to more than one 128-token tile.  Feature scales are read as whole 128-row blocks: plain tiles of 128
//   or 256 features, gated tiles of 128 + 128 in the bundle's order, or gated tiles of 64 + 64 in the paired gate/up
//   layout (B2_LINEAR_PAIRED_GATE_UP_SCALES), which only the resident order reads.
//   A pair computes 256 token rows whether they exist or not.  In the streaming order, when the last pair would be
//   mostly padding (560 tokens: 768 rows of work on pairs against 640 on single CTAs) the single-CTA schedule is as
//   fast or faster (measured: 560 x 16384 x 2048 FP8 28.0 vs 27.1 us); with equal padding, or enough tokens for it not
//   to matter, pairs win by 6-20 % (8192 x 1152 x 4304 FP8 51.6 vs 64.4 us; 8960 x 32768 x 2048 gated FP8 480 vs 543
//   us).  B2_LINEAR_PAIRS asks for pairs regardless.
//   Resident order (K of at most eight stages, at least two tiles per SM pair): a K stage carries weights only, half
//   the bytes of the streaming order and a third of the single-CTA schedule's, which is what bounds those; it is
//   taken whatever the padding.
//   Split K (plain epilogue, caller-provided workspace): when 256-column tiles leave more than half of the SM pairs
//   idle and K is long (560 x 2048 x 16384: 24 tiles for 74 pairs), K is cut so that tiles x splits fills one wave;
//   that launch runs on pairs whatever the padding.
PairPlan pair_plan(const b2_linear_desc* d, bool geglu, bool split_allowed) {
    PairPlan plan;
    if (d->tokens <= TILE_TOKENS) return plan;
    if (d->flags & B2_LINEAR_SINGLE_CTA) return plan;
    const bool nvfp4 = d->kind == B2_KIND_NVFP4;
    const bool paired_scales = (d->flags & B2_LINEAR_PAIRED_GATE_UP_SCALES) != 0;
    const int pairs = (d->tokens + PAIR_TOKENS - 1) / PAIR_TOKENS;
    const int clusters = sm_count() / 2;
    const int k_bytes = nvfp4 ? d->width / 2 : d->width;
    const int num_kb = (k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES;
    if (paired_scales) {
        // 64 gate + 64 up rows per scale block: tiles of 128 columns, resident order only
        if (!(geglu && nvfp4) || (d->feature_tile != 0 && d->feature_tile != 64) || d->features % 64 != 0) return plan;
        if (!pair_resident_fits(d, 128, 1, num_kb, pairs, int64_t(pairs) * (d->features / 64))) return plan;
        plan.columns = 128;
        plan.resident = 1;
        return plan;
    }
    if (!geglu && d->epilogue == B2_EPI_LINEAR && split_allowed && (d->feature_tile == 0 || d->feature_tile == 256)) {
        const int64_t tiles = int64_t(pairs) * ((d->features + 255) / 256);
        int count = int(clusters / (tiles > 0 ? tiles : 1));
        if (count > PAIR_MAX_SPLITS) count = PAIR_MAX_SPLITS;
        while (count > 1 && num_kb / count < 20) --count;        // the fix-up costs about as much as a dozen K atoms
        if (count > 1 && tiles * 16 <= PAIR_TICKET_BYTES) {
            plan.columns = 256;
            plan.splits = count;
            plan.workspace_need = PAIR_TICKET_BYTES + tiles * count * 2 * TILE_TOKENS * 256 * 4;
            return plan;
        }
    }
    int columns = 0;
    if (geglu) {
        if (d->feature_tile != 0 && d->feature_tile != 128) return plan;
        if (nvfp4 && d->features % 128 != 0) return plan;
        columns = 256;
    } else if (d->feature_tile == 128 || d->feature_tile == 256) {
        columns = d->feature_tile;
    } else if (d->feature_tile != 0) {
        return plan;
    } else {
        // fill the machine: the wider tile moves fewer operand bytes per MMA, the narrower one gives more work items
        const int64_t wide_items = int64_t(pairs) * ((d->features + 255) / 256);
        columns = wide_items >= clusters ? 256 : 128;
    }
    const int features_per_tile = geglu ? columns / 2 : columns;
    const int64_t tiles = int64_t(pairs) * ((d->features + features_per_tile - 1) / features_per_tile);
    const int64_t pair_rows = int64_t(pairs) * PAIR_TOKENS;
    const int64_t single_rows = int64_t((d->tokens + TILE_TOKENS - 1) / TILE_TOKENS) * TILE_TOKENS;
    const bool little_padding = pair_rows == single_rows || d->tokens >= 2048;
    // Gated 256-column tiles have one accumulator, so the main loop pauses while it is drained; with a token pair that
    // is mostly padding the clusters of the resident order that sit on it finish early and the rest decide the time
    // (560 x 2 x 16384 x 2048 NVFP4: resident 40.6 us, streaming 36.0 us; 8960 tokens: 322 against 335 us).
    const bool resident = pair_resident_fits(d, columns, columns > 128 ? 2 : 1, num_kb, pairs, tiles) && (!geglu || little_padding);
    const bool gated_nvfp4_prefill = geglu && nvfp4 && d->tokens >= 512;      // measured faster on pairs whatever the padding
    if (!resident && !(d->flags & B2_LINEAR_PAIRS) && !little_padding && !gated_nvfp4_prefill) return plan;
    plan.columns = columns;
    plan.resident = resident ? 1 : 0;
    return plan;
}

int run_linear_pair(const b2_linear_desc* d, int epilogue, const PairPlan& plan, cudaStream_t stream) {
    const bool nvfp4 = d->kind == B2_KIND_NVFP4;
    const bool geglu = is_gated(epilogue);
    const int tile_columns = plan.columns;
    const int splits = plan.splits;
    const bool paired_scales = (d->flags & B2_LINEAR_PAIRED_GATE_UP_SCALES) != 0;
    KernelArgs args{};
    args.tokens = d->tokens;
    args.features = d->features;
    args.k_bytes = nvfp4 ? d->width / 2 : d->width;
    args.num_kb = (args.k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES;
    args.num_m_tiles = (d->tokens + PAIR_TOKENS - 1) / PAIR_TOKENS;
    args.tile_n = tile_columns;
    const int features_per_tile = geglu ? tile_columns / 2 : tile_columns;
    args.num_n_tiles = (d->features + features_per_tile - 1) / features_per_tile;
    args.total_tiles = args.num_m_tiles * args.num_n_tiles;
    args.splits = splits;
    args.resident = plan.resident;
    args.tickets = nullptr;
    args.partials = nullptr;
    if (splits > 1) {
        args.tickets = static_cast<unsigned int*>(d->workspace);
        args.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(d->workspace) + PAIR_TICKET_BYTES);
    }
    args.scale_blocks = tile_columns > 128 ? 2 : 1;
    args.up_row_offset = d->features;
    args.scale_column_tiles = nvfp4 ? (d->width / 16 + 3) / 4 : 0;
    args.act_row_blocks = (d->tokens + 127) / 128;
    const int weight_rows = (geglu ? 2 : 1) * d->features;
    args.weight_row_blocks = paired_scales ? args.num_n_tiles : (weight_rows + 127) / 128;
    args.flags = d->flags;
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
    args.gelu_lo = args.gelu_hi = 0;
    if (compact_gelu_span(d) != 0) {
        args.gelu_lo = d->gelu_lo;
        args.gelu_hi = d->gelu_hi;
    }

    // tensor memory: accumulators from column 0, (resident NVFP4) the token scales of all of K behind them, (NVFP4) sets
    // of scale columns stacked down from column 512
    const int resident_columns = plan.resident && nvfp4 ? args.num_kb * TMEM_SFA_COLUMNS : 0;
    const int set_columns = (plan.resident ? 0 : TMEM_SFA_COLUMNS) + 16 * args.scale_blocks;
    if (nvfp4) {
        args.accumulators = 2 * tile_columns + resident_columns + 2 * set_columns <= TMEM_COLUMNS ? 2 : 1;
        args.accumulator_stride = tile_columns;
    } else {
        args.accumulators = 2;
        args.accumulator_stride = 256;
    }
    constexpr int SCALE_PART_BYTES = SCALE_ATOMS_PER_STAGE * SCALE_ATOM_BYTES;
    int stage_bytes = (plan.resident ? 0 : A_TILE_BYTES) + (tile_columns / 2) * STAGE_K_BYTES +
                      (nvfp4 ? ((plan.resident ? 0 : 1) + args.scale_blocks) * SCALE_PART_BYTES : 0);
    const int panel_bytes = plan.resident ? args.num_kb * A_TILE_BYTES : 0;
    const int fixed_bytes = pair_fixed_bytes(args.gelu_hi - args.gelu_lo);
    const int ring_bytes = SMEM_LIMIT - fixed_bytes - panel_bytes;
    const int sets_available = nvfp4 ? (TMEM_COLUMNS - args.accumulators * args.accumulator_stride - resident_columns) / set_columns : 0;
    // Resident order: two K atoms per ring slot when four such slots fit (and a scale set per atom): the MMA warp then
    // passes its barrier waits, its election and its commit once per 256 bytes of K instead of once per 128, and that
    // fixed part is most of what a K atom costs it at 128-column tiles.
    args.kps = 1;
    if (plan.resident && args.num_kb >= 2 && ring_bytes / (2 * stage_bytes) >= 4 && (!nvfp4 || sets_available >= 8)) {
        args.kps = 2;
        stage_bytes *= 2;
    }
    int stages = ring_bytes / stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) return B2_E_UNSUPPORTED;
    args.scale_sets = 1;
    if (nvfp4) {
        args.scale_sets = sets_available;
        if (args.kps == 2 && stages > sets_available / 2) stages = sets_available / 2;
        if (args.scale_sets > stages * args.kps) args.scale_sets = stages * args.kps;
        if (args.scale_sets < 2) return B2_E_UNSUPPORTED;
    }
    args.stages = stages;
    int shared_bytes = fixed_bytes + panel_bytes + stages * stage_bytes;
    if (shared_bytes < SMEM_MINIMUM) shared_bytes = SMEM_MINIMUM;

    CUtensorMap act_map, weight_map, act_scale_map, weight_scale_map;
    if (!make_operand_map(&act_map, d->act, d->tokens, args.k_bytes, TILE_TOKENS)) return B2_E_DRIVER;
    if (!make_operand_map(&weight_map, d->weight, weight_rows, args.k_bytes, tile_columns / 2)) return B2_E_DRIVER;
    if (nvfp4) {
        if (!make_atom_map(&act_scale_map, d->act_scales, int64_t(args.act_row_blocks) * args.scale_column_tiles)) return B2_E_DRIVER;
        if (!make_atom_map(&weight_scale_map, d->weight_scales, int64_t(args.weight_row_blocks) * args.scale_column_tiles))
            return B2_E_DRIVER;
    } else {
        act_scale_map = act_map;          // never dereferenced by the FP8 kernels
        weight_scale_map = weight_map;
    }

#define B2_PAIR_CASE(kind, epi) \
    case epi: return launch_pair<kind, epi>(act_map, weight_map, act_scale_map, weight_scale_map, args, shared_bytes, stream)
    if (nvfp4) {
        switch (epilogue) {
            B2_PAIR_CASE(B2_KIND_NVFP4, EPI_LINEAR);
            B2_PAIR_CASE(B2_KIND_NVFP4, EPI_GEGLU_BF16);
            B2_PAIR_CASE(B2_KIND_NVFP4, EPI_GEGLU_FP8);
            B2_PAIR_CASE(B2_KIND_NVFP4, EPI_GEGLU_NVFP4);
            B2_PAIR_CASE(B2_KIND_NVFP4, EPI_GELU_BF16);
            B2_PAIR_CASE(B2_KIND_NVFP4, EPI_GELU_FP8);
            default: return B2_E_UNSUPPORTED;
        }
    }
    switch (epilogue) {
        B2_PAIR_CASE(B2_KIND_FP8, EPI_LINEAR);
        B2_PAIR_CASE(B2_KIND_FP8, EPI_GEGLU_BF16);
        B2_PAIR_CASE(B2_KIND_FP8, EPI_GEGLU_FP8);
        B2_PAIR_CASE(B2_KIND_FP8, EPI_GEGLU_NVFP4);
        B2_PAIR_CASE(B2_KIND_FP8, EPI_GELU_BF16);
        B2_PAIR_CASE(B2_KIND_FP8, EPI_GELU_FP8);
        default: return B2_E_UNSUPPORTED;
    }
#undef B2_PAIR_CASE
}

}  // namespace b2
