// Quantised Linear on the 5th-generation tensor cores (sm_100a).
//
//   out[token, feature] = epilogue( sum_k act[token, k] * weight[feature, k] )
//
// Both operands are K-major in global memory.  A tile is 128 tokens (the MMA "A"
// operand, one token per TMEM lane) by BN features (the "B" operand, one feature per
// TMEM column).  TMA brings 128-byte-wide K slices of both into 128-byte-swizzled
// shared-memory stages; one thread issues `tcgen05.mma` (kind::f8f6f4 for e4m3,
// kind::mxf4nvf4 with a ue4m3 scale per 16 elements for e2m1) into fp32 accumulators
// in tensor memory.  Because a token's features lie along the columns of its own lane,
// an epilogue thread owns whole 16-element quantisation blocks of the output row and
// writes 16-byte vectors: no shuffles, no transposition.
//
// One persistent CTA per SM, ten or eighteen warps:
//   warp 0      TMA producer (all lanes run the loop, an elected lane issues)
//   warp 1      TMEM owner and tcgen05 issuer (scale-factor copies and MMAs; same scheme)
//   warps 2..   epilogue; warps w, w+4, ... share a 32-lane TMEM partition and split the columns
// Accumulators are double-buffered in TMEM whenever two fit, so the epilogue of one
// tile overlaps the main loop of the next.  Tiles that share a weight slab are
// consecutive in the schedule, so the slab comes from HBM once and from L2 afterwards.
//
// Gated MLP: the gate rows and the up rows of the packed [2F, K] weight land in one
// shared-memory B tile ([gate BN/2 rows | up BN/2 rows]); one MMA fills columns
// [0, BN/2) with gate and [BN/2, BN) with up, so an epilogue thread finds gate and up
// of the same feature in its own lane.
//
// Every wait is bounded (ptx.cuh); an expired wait leaves a code in the status word.
#include "common.cuh"
#include "gemm_epilogue.cuh"

#include <cstdlib>

#include <cuda.h>

#include <mutex>
#include <type_traits>

namespace b2 {

// Which tiles a CTA computes, in which order.
//   streaming (default): tile = blockIdx.x + i * gridDim.x over the n-major tile list (token tile inner), so
//       the CTAs running side by side share a weight slab and every K stage loads a token tile and a
//       weight tile.
//   resident: the CTA stays on one token tile (blockIdx.x % num_m_tiles) and walks the feature tiles
//       r, r + G, r + 2G ... (r = blockIdx.x / num_m_tiles, G = CTAs on that token tile).  The token tile
//       and its scales are loaded once for all of K (shared memory / TMEM), and a K stage loads weights
//       only: less than half the bytes per MMA, which is what bounds the streaming order at 128 tokens.
struct TileWalk {
    int m_tile, n_tile, step, linear;
    int tile, split, kb_begin, kb_end;       // streaming order only: tile index, K range [kb_begin, kb_end) of this work item
    bool resident;
    __device__ __forceinline__ void decompose(const KernelArgs& args) {
        tile = linear;
        split = 0;
        kb_begin = 0;
        kb_end = args.num_kb;
        if (args.splits > 1) {
            tile = linear / args.splits;
            split = linear - tile * args.splits;
            kb_begin = split * args.num_kb / args.splits;
            kb_end = (split + 1) * args.num_kb / args.splits;
        }
        n_tile = tile / args.num_m_tiles;
        m_tile = tile - n_tile * args.num_m_tiles;
    }
    __device__ __forceinline__ explicit TileWalk(const KernelArgs& args) : resident(args.resident != 0) {
        tile = split = kb_begin = 0;
        kb_end = args.num_kb;
        if (resident) {
            m_tile = int(blockIdx.x) % args.num_m_tiles;
            n_tile = int(blockIdx.x) / args.num_m_tiles;
            step = (int(gridDim.x) - m_tile + args.num_m_tiles - 1) / args.num_m_tiles;
            linear = 0;
        } else {
            linear = blockIdx.x;
            step = gridDim.x;
            decompose(args);
        }
    }
    __device__ __forceinline__ bool valid(const KernelArgs& args) const {
        return resident ? n_tile < args.num_n_tiles : linear < args.total_tiles * args.splits;
    }
    __device__ __forceinline__ void next(const KernelArgs& args) {
        if (resident) {
            n_tile += step;
        } else {
            linear += step;
            decompose(args);
        }
    }
};

// ---- the kernel ---------------------------------------------------------------

// SPLIT selects how K is cut across CTAs (each variant is its own kernel, so the fix-up's registers stay out of
// the unsplit kernels):
//   SPLIT_NONE     one CTA computes all of K of its tiles;
//   SPLIT_GLOBAL   partial sums go through a caller-provided workspace in global memory, the CTA that draws a
//                  tile's last ticket adds them (any number of token tiles; opt-in);
enum SplitMode { SPLIT_NONE = 0, SPLIT_GLOBAL = 1 };

template <int KIND, int EPI, int SPLIT_MODE>
__global__ void __launch_bounds__(gemm_threads(EPI), 1)
linear_kernel(const __grid_constant__ CUtensorMap act_map, const __grid_constant__ CUtensorMap weight_map,
              const KernelArgs args) {
    constexpr bool SPLIT_K = SPLIT_MODE == SPLIT_GLOBAL;
    constexpr bool GEGLU = is_gated(EPI);
    constexpr bool USES_TABLE = EPI != EPI_LINEAR;
    pdl_launch_dependents();
    extern __shared__ uint8_t shared_raw[];
    const uint32_t base = (smem_u32(shared_raw) + 1023u) & ~1023u;
    const int BN = args.tile_n;
    const int features_per_tile = GEGLU ? BN / 2 : BN;
    // shared memory: [resident token tile: num_kb x 16 KB][resident token scales: num_kb x 2 KB]
    //                [stages x (token tile unless resident | weight tile)][stages x scale atoms][barriers][GELU table]
    const bool resident = args.resident != 0;
    // A ring slot holds `kps` K atoms (128 bytes of K each): 1, or 2 / 4 for launches whose CTAs have a single tile and a
    // long K, where the waits, the election and the commit of a slot (some 400 cycles of the MMA warp) dwarf the MMAs of one atom
    const uint32_t kps = uint32_t(args.kps);
    const uint32_t a_stage_bytes = resident ? 0u : uint32_t(args.a_box_bytes);
    const uint32_t atom_bytes = a_stage_bytes + uint32_t(BN) * STAGE_K_BYTES;            // operands of one K atom
    const uint32_t stage_bytes = kps * atom_bytes;
    constexpr uint32_t SCALE_PART_BYTES = SCALE_ATOMS_PER_STAGE * SCALE_ATOM_BYTES;     // one operand's atoms of a K atom
    const uint32_t token_part_bytes = resident ? 0u : SCALE_PART_BYTES;                 // offset of the feature atoms behind the token atoms
    const uint32_t scale_atom_bytes = KIND == B2_KIND_NVFP4 ? token_part_bytes + uint32_t(args.scale_blocks) * SCALE_PART_BYTES : 0;
    const uint32_t scale_stage_bytes = kps * scale_atom_bytes;
    const uint32_t panel_base = base;
    const uint32_t panel_scale_base = panel_base + (resident ? uint32_t(args.num_kb) * A_TILE_BYTES : 0u);
    const uint32_t stage_base = panel_scale_base + (resident && KIND == B2_KIND_NVFP4 ? uint32_t(args.num_kb) * SCALE_PART_BYTES : 0u);
    const uint32_t scale_base = stage_base + uint32_t(args.stages) * stage_bytes;
    const uint32_t barrier_base = scale_base + uint32_t(args.stages) * scale_stage_bytes;
    const uint32_t full_bar = barrier_base;                       // [stages]
    const uint32_t empty_bar = barrier_base + 8 * MAX_STAGES;     // [stages]
    const uint32_t acc_full_bar = barrier_base + 16 * MAX_STAGES; // [2]
    const uint32_t acc_empty_bar = acc_full_bar + 16;             // [2]
    const uint32_t panel_bar = acc_empty_bar + 16;                // [MAX_RESIDENT_KB] token tile + scales of K stage kb landed
    const uint32_t tmem_slot = panel_bar + 8 * MAX_RESIDENT_KB;
    const uint32_t split_flag = tmem_slot + 8;                    // split-K: "this CTA drew the last ticket"
    const uint32_t compact_table = tmem_slot + 16;                // 2 * (gelu_hi - gelu_lo) bf16 entries

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&act_map);
        tma_prefetch_descriptor(&weight_map);
        for (int s = 0; s < args.stages; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar + 8 * b, 1);
            mbar_init(acc_empty_bar + 8 * b, epilogue_warps(EPI));
        }
        for (int kb = 0; kb < MAX_RESIDENT_KB; ++kb) mbar_init(panel_bar + 8 * kb, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLUMNS);
        tmem_relinquish();
    }
    if (USES_TABLE) fill_compact_gelu(args, compact_table, int(threadIdx.x), gemm_threads(EPI));
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");
    // Everything above is this launch's own set-up (the GELU table is a constant of the model); operands, scales,
    // bias and residual may come from the launch before this one.
    pdl_wait();

    bool failed = false;
    const int num_kb = args.num_kb;
    const int last_kb_mmas = ((args.k_bytes - (num_kb - 1) * STAGE_K_BYTES) + 31) / 32;

    // ------------------------------------------------------------- TMA producer
    // (all lanes run the loop; one elected lane issues the copies; like the MMA role it is specialised
    // on the launch-wide choices and entered once)
    // Launches whose CTAs have a single tile each are bound by how fast this one warp issues the copies of a stage
    // (a few hundred cycles for the barrier handling and the copy instructions), so they skip the L2 prefetches.
    const bool prefetch_ahead = args.splits == 1 && args.total_tiles > int(gridDim.x);
    auto producer_role = [&](auto resident_tag, auto prefetch_tag) {
            constexpr bool RESIDENT = decltype(resident_tag)::value, PREFETCH = decltype(prefetch_tag)::value;
            int stage = 0;
            uint32_t phase = 0;
            uint32_t filled = 0, fill_parity = 0;     // per stage: ever filled / phase of the last fill
            // L2 prefetch cursor, PREFETCH_DISTANCE K stages ahead of the loads.  Shared memory holds about
            // 2500 cycles' worth of loads at the tensor pipe's rate while a first touch of HBM takes about as
            // long to arrive, so loads that miss the L2 leave the pipe waiting; weights prefetched into the L2
            // a few thousand cycles earlier arrive in a third of that.  The token tiles sharing a weight slab
            // run side by side, so they take turns issuing its prefetches.
            TileWalk pf(args);
            int pf_kb = 0;
            for (int i = 0; i < PREFETCH_DISTANCE; ++i)
                if (++pf_kb == num_kb) { pf_kb = 0; pf.next(args); }
            int pf_f0 = 0, pf_turn = 0, pf_seen = -1;      // feature row of the cursor's tile; stages until this CTA's turn
            TileWalk walk(args);
            const bool panel_loaded = RESIDENT && walk.valid(args);
            if (panel_loaded) {
                // the token tile for all of K, and its scale atoms, once
                if (elect_one()) {
                    const uint8_t* token_scales = KIND == B2_KIND_NVFP4
                        ? args.act_scales + int64_t(walk.m_tile) * args.scale_column_tiles * SCALE_ATOM_BYTES : nullptr;
                    for (int kb = 0; kb < num_kb; ++kb) {
                        const uint32_t bar = panel_bar + 8 * kb;
                        const int atoms = min(SCALE_ATOMS_PER_STAGE, args.scale_column_tiles - kb * SCALE_ATOMS_PER_STAGE);
                        mbar_expect_tx(bar, A_TILE_BYTES + (KIND == B2_KIND_NVFP4 ? uint32_t(atoms) * SCALE_ATOM_BYTES : 0u));
                        tma_load_2d(panel_base + uint32_t(kb) * A_TILE_BYTES, &act_map, bar, kb * STAGE_K_BYTES, walk.m_tile * TILE_TOKENS);
                        if (KIND == B2_KIND_NVFP4)
                            bulk_load(panel_scale_base + uint32_t(kb) * SCALE_PART_BYTES,
                                      token_scales + int64_t(kb) * SCALE_PART_BYTES, uint32_t(atoms) * SCALE_ATOM_BYTES, bar);
                    }
                }
                __syncwarp();
            }
            for (; walk.valid(args); walk.next(args)) {
                const int n_tile = walk.n_tile;
                const int m_tile = walk.m_tile;
                const int m0 = m_tile * TILE_TOKENS;
                const int f0 = n_tile * features_per_tile;
                // weight rows whose scales this tile needs: up to two 128-row blocks
                int scale_row_block[2];
                int scale_blocks;
                if (GEGLU && (args.flags & B2_LINEAR_PAIRED_GATE_UP_SCALES)) {
                    scale_row_block[0] = n_tile;            // 64 gate rows + 64 up rows of this tile form one block
                    scale_row_block[1] = n_tile;
                    scale_blocks = 1;
                } else if (GEGLU) {
                    scale_row_block[0] = f0 >> 7;
                    scale_row_block[1] = (args.up_row_offset + f0) >> 7;
                    scale_blocks = 2;
                } else {
                    scale_row_block[0] = f0 >> 7;
                    scale_row_block[1] = scale_row_block[0] + 1;
                    scale_blocks = ((f0 + BN - 1) >> 7) - scale_row_block[0] + 1;
                }
                // Everything a K stage needs is fixed per tile except the K offset: source pointers of the
                // scale atoms, which of the two feature-scale blocks exist, and the byte count of a full stage.
                const uint8_t* token_scales = nullptr;
                const uint8_t* feature_scales[2] = {nullptr, nullptr};
                int live = 0;
                if (KIND == B2_KIND_NVFP4) {
                    token_scales = args.act_scales + int64_t(m_tile) * args.scale_column_tiles * SCALE_ATOM_BYTES;
                    live = RESIDENT ? 0 : 1;
                    for (int i = 0; i < scale_blocks; ++i)
                        if (scale_row_block[i] < args.weight_row_blocks) {
                            feature_scales[i] = args.weight_scales + int64_t(scale_row_block[i]) * args.scale_column_tiles * SCALE_ATOM_BYTES;
                            ++live;
                        }
                }
                const int tail_atoms = args.scale_column_tiles - (num_kb - 1) * SCALE_ATOMS_PER_STAGE;
                for (int kb = walk.kb_begin; kb < walk.kb_end; kb += int(kps)) {
                    mbar_wait(empty_bar + 8 * stage, phase ^ 1u, failed, args.status, STATUS_WAIT_PRODUCER);
                    __syncwarp();
                    filled |= 1u << stage;
                    fill_parity = (fill_parity & ~(1u << stage)) | (phase << stage);
                    if (elect_one()) {
                        const uint32_t bar = full_bar + 8 * stage;
                        const int atoms = min(int(kps), walk.kb_end - kb);
                        // bytes of the slot: full atoms, except that the last K atom of the matrix may have fewer scale atoms
                        uint32_t bytes = uint32_t(atoms) * atom_bytes;
                        if (KIND == B2_KIND_NVFP4)
                            bytes += uint32_t(live) * SCALE_ATOM_BYTES *
                                     uint32_t(atoms * SCALE_ATOMS_PER_STAGE - (kb + atoms == num_kb ? SCALE_ATOMS_PER_STAGE - tail_atoms : 0));
                        mbar_expect_tx(bar, bytes);
                        for (int k = 0; k < atoms; ++k) {
                            const uint32_t a_smem = stage_base + uint32_t(stage) * stage_bytes + uint32_t(k) * atom_bytes;
                            const uint32_t b_smem = a_smem + a_stage_bytes;
                            const int k0 = (kb + k) * STAGE_K_BYTES;
                            if (!RESIDENT) tma_load_2d(a_smem, &act_map, bar, k0, m0);
                            // gated: the map is three-dimensional (plane 0 = gate rows, plane 1 = up rows), one instruction
                            // brings both halves of the tile ([gate | up] in shared memory)
                            if (GEGLU) tma_load_3d(b_smem, &weight_map, bar, k0, f0, 0);
                            else tma_load_2d(b_smem, &weight_map, bar, k0, f0);
                            if (KIND == B2_KIND_NVFP4) {
                                const uint32_t copy_bytes = uint32_t(kb + k == num_kb - 1 ? tail_atoms : SCALE_ATOMS_PER_STAGE) * SCALE_ATOM_BYTES;
                                const uint32_t s_smem = scale_base + uint32_t(stage) * scale_stage_bytes + uint32_t(k) * scale_atom_bytes;
                                const int64_t offset = int64_t(kb + k) * (SCALE_ATOMS_PER_STAGE * SCALE_ATOM_BYTES);
                                if (!RESIDENT) bulk_load(s_smem, token_scales + offset, copy_bytes, bar);
                                if (feature_scales[0] != nullptr)
                                    bulk_load(s_smem + token_part_bytes, feature_scales[0] + offset, copy_bytes, bar);
                                if (feature_scales[1] != nullptr)
                                    bulk_load(s_smem + token_part_bytes + SCALE_PART_BYTES, feature_scales[1] + offset, copy_bytes, bar);
                            }
                        }
                    }
                    if (PREFETCH && pf.valid(args)) {
                        if (pf.n_tile != pf_seen) {
                            pf_f0 = pf.n_tile * features_per_tile;
                            pf_turn = (pf.m_tile + args.num_m_tiles - pf_kb % args.num_m_tiles) % args.num_m_tiles;
                            pf_seen = pf.n_tile;
                        }
                        if (pf_turn == 0) {
                            if (elect_one()) {
                                if (GEGLU) tma_prefetch_l2_3d(&weight_map, pf_kb * STAGE_K_BYTES, pf_f0, 0);
                                else tma_prefetch_l2_2d(&weight_map, pf_kb * STAGE_K_BYTES, pf_f0);
                            }
                            pf_turn = args.num_m_tiles;
                        }
                        --pf_turn;
                        if (++pf_kb == num_kb) { pf_kb = 0; pf.next(args); }
                    }
                    __syncwarp();
                    if (++stage == args.stages) { stage = 0; phase ^= 1u; }
                }
            }
            // Do not leave while a copy of this CTA is still in flight: wait (bounded) for the
            // last fill of every stage.  On the normal path these have all completed already.
            bool drain_failed = false;
            for (int s = 0; s < args.stages; ++s)
                if (filled & (1u << s))
                    mbar_wait(full_bar + 8 * s, (fill_parity >> s) & 1u, drain_failed, args.status, STATUS_WAIT_DRAIN);
            if (panel_loaded)
                for (int kb = 0; kb < num_kb; ++kb) mbar_wait(panel_bar + 8 * kb, 0u, drain_failed, args.status, STATUS_WAIT_DRAIN);
        };
    using Yes = std::true_type;
    using No = std::false_type;
    if (warp == 0) {
        // (split K ranges are a few stages long: nothing to prefetch ahead of; nor is there when every CTA has a
        // single tile: its loads are all issued within a few stages anyway, and each prefetch is one more
        // instruction on the warp whose issue rate bounds the small launches)
        if (resident) { if (prefetch_ahead) producer_role(Yes{}, Yes{}); else producer_role(Yes{}, No{}); }
        else { if (prefetch_ahead) producer_role(No{}, Yes{}); else producer_role(No{}, No{}); }
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer
        // (all lanes run the loop; one elected lane issues the tcgen05 instructions)
        // The launch-wide choices (resident token tile, one or two feature-scale blocks, split halves) are
        // compile-time tags of the role: it is entered once through the dispatch below, and the unrolled
        // copies and MMAs of its stage loop carry no branches.
        auto mma_role = [&](auto resident_tag, auto two_blocks_tag, auto split_tag) {
            constexpr bool RESIDENT = decltype(resident_tag)::value, TWO = decltype(two_blocks_tag)::value;
            constexpr bool SPLIT = decltype(split_tag)::value;
            // Descriptors are a constant high word plus (address >> 4), and everything that depends only
            // on the tile is computed once per tile.
            const uint32_t idesc = KIND == B2_KIND_NVFP4 ? idesc_nvf4(TILE_TOKENS, BN) : idesc_f8(TILE_TOKENS, BN);
            const uint32_t idesc_half = idesc_nvf4(TILE_TOKENS, 64);
            const uint64_t operand_desc = smem_desc_sw128(0);        // + (address >> 4)
            const uint32_t operand_low = uint32_t(operand_desc), operand_high = uint32_t(operand_desc >> 32);
            const bool paired_scales = GEGLU && (args.flags & B2_LINEAR_PAIRED_GATE_UP_SCALES) != 0;
            int stage = 0;
            uint32_t phase = 0;
            int local_tile = 0;
            // Scale factors: tcgen05.cp (shared memory -> TMEM) is ordered before a later tcgen05.mma of the
            // same thread, so this thread issues the copies of a K stage right before its MMAs (about 50
            // cycles per 512-byte atom, overlapping the MMAs already queued).  The reverse order is not
            // guaranteed: before a set of columns is overwritten, the MMAs that last read it (scale_sets
            // stages ago) must have completed, which their commit to that stage's `empty` barrier reports.
            // With one set per ring stage (the usual case) no such wait is needed: the stage's `full` barrier completed
            // again only after the producer had seen the `empty` barrier of its last use.
            const bool lag = args.scale_sets < args.stages * args.kps;     // the host keeps kps == 1 in that case
            int set = 0, lag_stage = 0, issued = 0;
            uint32_t lag_phase = 0;
            const uint32_t set_columns = uint32_t((RESIDENT ? 0 : TMEM_SFA_COLUMNS) + 16 * args.scale_blocks);
            const uint64_t scale_desc = smem_desc_scale_atom(0);
            const uint32_t scale_desc_high = uint32_t(scale_desc >> 32);
            // resident order: the token scales of all K stages sit in TMEM right after the accumulators
            const uint32_t resident_sfa = tmem_base + uint32_t(args.accumulators * args.accumulator_stride);
            TileWalk walk(args);
            if (RESIDENT && KIND == B2_KIND_NVFP4 && walk.valid(args)) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    mbar_wait(panel_bar + 8 * kb, 0u, failed, args.status, STATUS_WAIT_MMA_FULL);
                    tc_fence_after_sync();
                    __syncwarp();
                    if (elect_one()) {
                        const uint32_t atom_low = (panel_scale_base + uint32_t(kb) * SCALE_PART_BYTES) >> 4;
                        const int atoms = min(SCALE_ATOMS_PER_STAGE, args.scale_column_tiles - kb * SCALE_ATOMS_PER_STAGE);
                        for (int j = 0; j < atoms; ++j)
                            tc_copy_32x128b_x4(resident_sfa + uint32_t(kb * TMEM_SFA_COLUMNS + j * 4),
                                               desc_from_words(atom_low + uint32_t(j) * (SCALE_ATOM_BYTES >> 4), scale_desc_high));
                    }
                    __syncwarp();
                }
            }
            for (; walk.valid(args); walk.next(args), ++local_tile) {
                const int n_tile = walk.n_tile;
                const int f0 = n_tile * features_per_tile;
                // column of the feature-scale block the MMA starts reading at (a tile that starts 64 features
                // into a 128-row block starts at column 2)
                const uint32_t scale_column = (paired_scales || (GEGLU && BN == 256)) ? 0u : uint32_t((f0 & 127) >> 5);
                const int buffer = local_tile % args.accumulators;
                const uint32_t use = uint32_t(local_tile / args.accumulators);
                mbar_wait(acc_empty_bar + 8 * buffer, (use & 1u) ^ 1u, failed, args.status, STATUS_WAIT_MMA_TMEM);
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + uint32_t(buffer * args.accumulator_stride);
                for (int kb = walk.kb_begin; kb < walk.kb_end; kb += int(kps)) {
                    mbar_wait(full_bar + 8 * stage, phase, failed, args.status, STATUS_WAIT_MMA_FULL);
                    tc_fence_after_sync();
                    if (RESIDENT && local_tile == 0) {       // first pass over K: the token tile may still be landing (one atom per slot)
                        mbar_wait(panel_bar + 8 * kb, 0u, failed, args.status, STATUS_WAIT_MMA_FULL);
                        tc_fence_after_sync();
                    }
                    const uint32_t stage_smem = stage_base + uint32_t(stage) * stage_bytes;
                    if (KIND == B2_KIND_NVFP4 && lag) {      // (one atom per slot)
                        if (issued >= args.scale_sets) {
                            mbar_wait(empty_bar + 8 * lag_stage, lag_phase, failed, args.status, STATUS_WAIT_MMA_TMEM);
                            tc_fence_after_sync();
                            if (++lag_stage == args.stages) { lag_stage = 0; lag_phase ^= 1u; }
                        }
                        ++issued;
                    }
                    __syncwarp();
                    if (elect_one()) {
                        constexpr uint32_t ATOM = SCALE_ATOM_BYTES >> 4, PART = SCALE_ATOMS_PER_STAGE * ATOM;
                        const int atoms = min(int(kps), walk.kb_end - kb);
                        // one K atom of the slot: `count` MMAs of 32 bytes of K each with their scale copies in front;
                        // `count` is a literal on the full-atom path, only a ragged last K atom takes the generic one
                        auto issue = [&](const int k, const int count) {
                            const int atom_kb = kb + k;
                            const uint32_t atom_smem = stage_smem + uint32_t(k) * atom_bytes;
                            const uint32_t a_low = operand_low + ((RESIDENT ? panel_base + uint32_t(atom_kb) * A_TILE_BYTES : atom_smem) >> 4);
                            const uint32_t b_low = operand_low + ((atom_smem + a_stage_bytes) >> 4);
                            const uint32_t set_tmem = tmem_base + uint32_t(TMEM_COLUMNS) - set_columns * uint32_t((lag ? set : stage * int(kps) + k) + 1);
                            const uint32_t sfa_tmem = RESIDENT ? resident_sfa + uint32_t(atom_kb * TMEM_SFA_COLUMNS) : set_tmem;
                            const uint32_t sfb_tmem = RESIDENT ? set_tmem : set_tmem + TMEM_SFA_COLUMNS;
                            // shared memory per atom: [token atoms x4 | first feature block x4 | second feature block x4], 512 B each
                            const uint32_t atom_low = (scale_base + uint32_t(stage) * scale_stage_bytes + uint32_t(k) * scale_atom_bytes) >> 4;
                            const uint32_t feature_low = atom_low + (RESIDENT ? 0u : PART);   // no token atoms when they are resident
                            const uint32_t first_accumulate = atom_kb != walk.kb_begin;
                            if (KIND == B2_KIND_NVFP4) {
#pragma unroll
                                for (int j = 0; j < SCALE_ATOMS_PER_STAGE; ++j) {
                                    if (j < count) {
                                        if (!RESIDENT) tc_copy_32x128b_x4(sfa_tmem + j * 4, desc_from_words(atom_low + j * ATOM, scale_desc_high));
                                        tc_copy_32x128b_x4(sfb_tmem + j * (TWO ? 8 : 4), desc_from_words(feature_low + j * ATOM, scale_desc_high));
                                        if (TWO)
                                            tc_copy_32x128b_x4(sfb_tmem + j * 8 + 4, desc_from_words(feature_low + PART + j * ATOM, scale_desc_high));
                                    }
                                }
                            }
#pragma unroll
                            for (int j = 0; j < SCALE_ATOMS_PER_STAGE; ++j) {
                                if (j < count) {
                                    const uint32_t accumulate = j == 0 ? first_accumulate : 1u;
                                    const uint64_t a_desc = desc_from_words(a_low + 2 * j, operand_high);
                                    const uint64_t b_desc = desc_from_words(b_low + 2 * j, operand_high);
                                    if (KIND != B2_KIND_NVFP4) {
                                        mma_f8f6f4(d_tmem, a_desc, b_desc, idesc, accumulate);
                                    } else if (SPLIT) {
                                        // 64 gate + 64 up features sit in the same two columns of two different scale
                                        // blocks, and a copy can only land on a multiple of four columns: the blocks stay
                                        // apart and each half gets its own MMA (gate -> columns [0,64), up -> [64,128)).
                                        mma_nvf4(d_tmem, a_desc, b_desc, idesc_half, sfa_tmem + j * 4,
                                                 sfb_tmem + j * 8 + scale_column, accumulate);
                                        mma_nvf4(d_tmem + 64, a_desc, desc_from_words(b_low + ((64 * STAGE_K_BYTES) >> 4) + 2 * j, operand_high), idesc_half,
                                                 sfa_tmem + j * 4, sfb_tmem + j * 8 + 4 + scale_column, accumulate);
                                    } else {
                                        mma_nvf4(d_tmem, a_desc, b_desc, idesc, sfa_tmem + j * 4,
                                                 sfb_tmem + j * (TWO ? 8 : 4) + scale_column, accumulate);
                                    }
                                }
                            }
                        };
                        for (int k = 0; k < atoms; ++k) {
                            if (kb + k == num_kb - 1 && last_kb_mmas != SCALE_ATOMS_PER_STAGE) issue(k, last_kb_mmas);
                            else issue(k, SCALE_ATOMS_PER_STAGE);
                        }
                        tc_commit(empty_bar + 8 * stage);
                    }
                    __syncwarp();
                    if (KIND == B2_KIND_NVFP4 && ++set == args.scale_sets) set = 0;
                    if (++stage == args.stages) { stage = 0; phase ^= 1u; }
                }
                if (elect_one()) tc_commit(acc_full_bar + 8 * buffer);
                __syncwarp();
            }
        };
        using Yes = std::true_type;
        using No = std::false_type;
        const bool two_blocks = args.scale_blocks == 2;
        const bool split_halves = KIND == B2_KIND_NVFP4 && GEGLU && BN == 128 && !(args.flags & B2_LINEAR_PAIRED_GATE_UP_SCALES);
        if (KIND != B2_KIND_NVFP4) { if (resident) mma_role(Yes{}, No{}, No{}); else mma_role(No{}, No{}, No{}); }
        else if (split_halves) { if (resident) mma_role(Yes{}, Yes{}, Yes{}); else mma_role(No{}, Yes{}, Yes{}); }
        else if (two_blocks) { if (resident) mma_role(Yes{}, Yes{}, No{}); else mma_role(No{}, Yes{}, No{}); }
        else { if (resident) mma_role(Yes{}, No{}, No{}); else mma_role(No{}, No{}, No{}); }
    } else {
        // ------------------------------------------------------------- epilogue
        const int quarter = warp & 3;                      // the TMEM lane partition this warp may read
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
        const int part = (warp - FIRST_EPILOGUE_WARP) >> 2;     // 0 .. WARPS_PER_QUARTER-1
        int local_tile = 0;
        for (TileWalk walk(args); walk.valid(args); walk.next(args), ++local_tile) {
            const int n_tile = walk.n_tile;
            const int m_tile = walk.m_tile;
            const int token = m_tile * TILE_TOKENS + quarter * 32 + lane;
            const int f0 = n_tile * features_per_tile;
            const int buffer = local_tile % args.accumulators;
            const uint32_t use = uint32_t(local_tile / args.accumulators);
            mbar_wait(acc_full_bar + 8 * buffer, use & 1u, failed, args.status, STATUS_WAIT_EPILOGUE);
            tc_fence_after_sync();
            const uint32_t lane_address = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(buffer * args.accumulator_stride);
            const bool warp_has_tokens = m_tile * TILE_TOKENS + quarter * 32 < args.tokens;   // else: padding rows only
            // Split K: every CTA of a tile leaves its partial sums (fp32, valid token rows only) in its slot of
            // the workspace and takes a ticket; the CTA that draws the last ticket adds the slots in split order
            // (so the result does not depend on which CTA that is) and runs the epilogue on the sums.  No CTA
            // waits for another.
            const float* sums = nullptr;
            if (SPLIT_K) {
                const int64_t slot_floats = int64_t(TILE_TOKENS) * BN;
                float* slot = args.partials + (int64_t(walk.tile) * args.splits + walk.split) * slot_floats +
                              int64_t(quarter * 32 + lane) * BN;
                for (int chunk = part; chunk < BN / 32 && warp_has_tokens; chunk += WARPS_PER_QUARTER) {
                    uint32_t v[32];
                    tmem_load_32x32(lane_address + chunk * 32, v);
                    tmem_load_wait();
                    if (token < args.tokens) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            __stcg(reinterpret_cast<uint4*>(slot + chunk * 32) + i, make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar + 8 * buffer);
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"r"(32 * epilogue_warps(EPI)) : "memory");
                if (threadIdx.x == 32 * FIRST_EPILOGUE_WARP) {
                    const unsigned int ticket = atomicAdd(args.tickets + walk.tile, 1u);
                    const unsigned int last = ticket == unsigned(args.splits - 1);
                    if (last) args.tickets[walk.tile] = 0u;              // ready for the next launch
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(split_flag), "r"(last) : "memory");
                }
                asm volatile("bar.sync 1, %0;" ::"r"(32 * epilogue_warps(EPI)) : "memory");
                unsigned int last;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(last) : "r"(split_flag) : "memory");
                if (!last) continue;
                __threadfence();
                sums = args.partials + int64_t(walk.tile) * args.splits * slot_floats + int64_t(quarter * 32 + lane) * BN;
            }
            // 16 (or 32) accumulator columns of this lane's token from the split-K slots: the loads of up to four
            // splits of a 16-column group are issued together (one L2 round trip), then added in split order
            auto load_columns = [&](int column, uint32_t* values, int count) {
                const int64_t slot_floats = int64_t(TILE_TOKENS) * BN;
                for (int base = 0; base < count; base += 16) {
                    float4 total[4];
                    for (int first_split = 0; first_split < args.splits; first_split += 4) {
                        float4 part[4][4];
#pragma unroll
                        for (int s = 0; s < 4; ++s)
                            if (first_split + s < args.splits) {
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    part[s][j] = __ldcg(reinterpret_cast<const float4*>(sums + (first_split + s) * slot_floats + column + base) + j);
                            }
#pragma unroll
                        for (int s = 0; s < 4; ++s)
                            if (first_split + s < args.splits) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    if (first_split + s == 0) {
                                        total[j] = part[s][j];
                                    } else {
                                        total[j].x = __fadd_rn(total[j].x, part[s][j].x); total[j].y = __fadd_rn(total[j].y, part[s][j].y);
                                        total[j].z = __fadd_rn(total[j].z, part[s][j].z); total[j].w = __fadd_rn(total[j].w, part[s][j].w);
                                    }
                                }
                            }
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        values[base + 4 * j] = __float_as_uint(total[j].x); values[base + 4 * j + 1] = __float_as_uint(total[j].y);
                        values[base + 4 * j + 2] = __float_as_uint(total[j].z); values[base + 4 * j + 3] = __float_as_uint(total[j].w);
                    }
                }
            };
            const bool lane_has_token = token < args.tokens;
            if (GEGLU) {
                const int units = features_per_tile / 16;
                for (int unit = part; unit < units && warp_has_tokens; unit += WARPS_PER_QUARTER) {
                    uint32_t first[16], second[16];
                    if (SPLIT_K) {
                        if (lane_has_token) {
                            load_columns(unit * 16, first, 16);
                            load_columns(BN / 2 + unit * 16, second, 16);
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) first[i] = second[i] = 0u;
                        }
                    } else {
                        tmem_load_32x16(lane_address + unit * 16, first);
                        tmem_load_32x16(lane_address + BN / 2 + unit * 16, second);
                        tmem_load_wait();
                    }
                    epilogue_geglu_unit<GEGLU ? EPI : EPI_GEGLU_BF16>(first, second, args, compact_table, scale, scale_up,
                                                                     round_scale, out_scale, by_global, out_scale_rcp,
                                                                     true_div, token, f0 + unit * 16);
                }
            } else {
                const int chunks = features_per_tile / 32;
                for (int chunk = part; chunk < chunks && warp_has_tokens; chunk += WARPS_PER_QUARTER) {
                    uint32_t first[32];
                    if (SPLIT_K) {
                        if (lane_has_token) {
                            load_columns(chunk * 32, first, 32);
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) first[i] = 0u;
                        }
                    } else {
                        tmem_load_32x32(lane_address + chunk * 32, first);
                        tmem_load_wait();
                    }
                    epilogue_linear_chunk<GEGLU ? EPI_LINEAR : EPI>(first, args, scale, round_scale, token, f0 + chunk * 32, compact_table,
                                                                    out_scale, out_scale_rcp, true_div);
                }
            }
            if (!SPLIT_K) {                        // (split K released the accumulator right after the dump)
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar + 8 * buffer);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLUMNS);
    }
}

// ---------------------------------------------------------------------------
// host side

EncodeTiledFn encode_tiled_entry() {
    static EncodeTiledFn entry = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* pointer = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &pointer, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            entry = reinterpret_cast<EncodeTiledFn>(pointer);
    });
    return entry;
}

// Row-major byte matrix [rows, row_bytes] viewed as tiles of box_rows x 128 bytes, 128-byte swizzle.
// Rows and bytes beyond the matrix read as zero.
bool make_operand_map(CUtensorMap* map, const void* pointer, int64_t rows, int64_t row_bytes, int box_rows) {
    EncodeTiledFn encode = encode_tiled_entry();
    if (encode == nullptr) return false;
    const cuuint64_t dims[2] = {cuuint64_t(row_bytes), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(row_bytes)};
    const cuuint32_t box[2] = {cuuint32_t(STAGE_K_BYTES), cuuint32_t(box_rows)};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(pointer), dims, strides, box,
                  element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The packed [gate; up] weight ([2 * features, row_bytes]) as [2 planes][features][row_bytes]: one box of
// box_rows x 128 bytes x 2 planes lands as [gate rows | up rows].
bool make_gated_map(CUtensorMap* map, const void* pointer, int64_t features, int64_t row_bytes, int box_rows) {
    EncodeTiledFn encode = encode_tiled_entry();
    if (encode == nullptr) return false;
    const cuuint64_t dims[3] = {cuuint64_t(row_bytes), cuuint64_t(features), 2};
    const cuuint64_t strides[2] = {cuuint64_t(row_bytes), cuuint64_t(row_bytes) * cuuint64_t(features)};
    const cuuint32_t box[3] = {cuuint32_t(STAGE_K_BYTES), cuuint32_t(box_rows), 2};
    const cuuint32_t element_strides[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(pointer), dims, strides, box,
                  element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
    static int counts[64] = {0};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64) device = 0;
    if (counts[device] == 0) {
        int value = 0;
        cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device);
        counts[device] = value > 0 ? value : 148;
    }
    return counts[device];
}

bool pdl_enabled() {
    static const bool enabled = [] {
        const char* value = std::getenv("B2_PDL");
        return value != nullptr ? (value[0] != '\0' && value[0] != '0') : PDL_DEFAULT;
    }();
    return enabled;
}

// Two accumulators fit (beside the NVFP4 scale columns)?
static bool can_double_buffer(int kind, int tile_n, int scale_blocks = 2) {
    return 2 * tile_n <= (kind == B2_KIND_NVFP4 ? TMEM_COLUMNS - 2 * (TMEM_SFA_COLUMNS + 16 * scale_blocks) : TMEM_COLUMNS);
}

// LINEAR: 64, 128, 192 or 256 features per tile, FP8 also 32.  GEGLU: 64 or 128 features (128 or 256 columns).
// (NVFP4 stops at 64: the feature scales of a tile are read from the column of their 128-row block that the tile
// starts in, and the block-scaled MMA takes that column only on a multiple of two -- an odd one is a misaligned
// address.)
static bool tile_allowed(int kind, bool geglu, int features_per_tile) {
    if (geglu) return features_per_tile == 64 || features_per_tile == 128;
    if (features_per_tile == 32) return kind != B2_KIND_NVFP4;
    return features_per_tile == 64 || features_per_tile == 128 || features_per_tile == 192 || features_per_tile == 256;
}

constexpr int64_t TICKET_BYTES = 1024;     // fixed, so that launches of different shapes sharing a workspace find it zero
constexpr int MAX_SPLITS = 8;

// Features per tile and K splits, chosen together from a cycle estimate:
//   a K stage moves 128 token rows + `columns` weight rows through shared memory, which is what its time follows
//   (~2.9 cycles per row, measured); a work item (tile x split) adds ~2,500 cycles of pipeline fill and epilogue,
//   more when the accumulator is not double-buffered; a split launch adds the fix-up (partial sums through the
//   L2, ticket, fixed-order sum).  Splits are considered only when the launch stays within one wave.
//   A launch with a single token tile loads only the token rows it has, and with few CTAs each of them is bound by
//   what one SM takes in (~32 bytes per cycle measured: 4 cycles per 128-byte row, not below ~130 cycles per K atom):
//   1024 features at 64 per tile are 16 CTAs walking all of K, so such a launch may go down to 32 features per tile.
static void choose_tile_and_splits(int kind, bool geglu, int forced_tile, int features, int tokens, int m_tiles, int num_kb,
                                   bool allow_split, int* tile_out, int* splits_out) {
    const int sms = sm_count();
    double best_cost = 0.0;
    *tile_out = 0;
    *splits_out = 1;
    const int token_rows = (tokens + 7) / 8 * 8;
    for (int tile = 256; tile >= 32; tile -= tile > 64 ? 64 : 32) {
        if (!tile_allowed(kind, geglu, tile) || (forced_tile > 0 && tile != forced_tile)) continue;
        if (tile == 32 && forced_tile != 32 && m_tiles != 1) continue;
        const int columns = geglu ? 2 * tile : tile;
        const int64_t tiles = int64_t((features + tile - 1) / tile) * m_tiles;
        double stage = 2.9 * (128.0 + columns);
        if (m_tiles == 1) {
            stage = 4.0 * (token_rows + columns);
            if (stage < 130.0) stage = 130.0;
        }
        const double fixed = 2500.0 + (can_double_buffer(kind, columns) ? 0.0 : 10.0 * columns);
        for (int splits = 1; splits <= MAX_SPLITS; ++splits) {
            if (splits > 1 && (!allow_split || tiles * splits > sms || num_kb / splits < 4 || tiles * 4 > TICKET_BYTES)) break;
            const int64_t waves = (tiles * splits + sms - 1) / sms;
            const int kb_item = (num_kb + splits - 1) / splits;
            // fix-up as measured (560x2048x16384 in 2-3 splits of 192-256 columns: ~35 k cycles): it pays only for very long K
            const double cost = double(waves) * (kb_item * stage + fixed) + (splits > 1 ? 12000.0 + 45.0 * columns * splits : 0.0);
            if (*tile_out == 0 || cost < best_cost) { *tile_out = tile; *splits_out = splits; best_cost = cost; }
        }
    }
}

template <int KIND, int EPI, int SPLIT_MODE>
static int launch_linear_variant(const CUtensorMap& act_map, const CUtensorMap& weight_map, const KernelArgs& args,
                         int shared_bytes, cudaStream_t stream) {
    static bool configured[64] = {false};
    static std::mutex lock;
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64) {
        std::lock_guard<std::mutex> guard(lock);
        if (!configured[device]) {
            const cudaError_t error = cudaFuncSetAttribute(linear_kernel<KIND, EPI, SPLIT_MODE>,
                                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
            if (error != cudaSuccess) return int(error);
            configured[device] = true;
        }
    }
    const int items = args.total_tiles * args.splits;
    const int grid = items < sm_count() ? items : sm_count();
    return launch_kernel(linear_kernel<KIND, EPI, SPLIT_MODE>, dim3(unsigned(grid)), dim3(unsigned(gemm_threads(EPI))),
                         size_t(shared_bytes), stream, act_map, weight_map, args);
}

template <int KIND, int EPI>
static int launch_linear(const CUtensorMap& act_map, const CUtensorMap& weight_map, const KernelArgs& args,
                         int shared_bytes, cudaStream_t stream) {
    // only the plain epilogue has a split-K variant (the table epilogues would spill registers in the fix-up,
    // and `run_linear` never asks them to split)
    if constexpr (EPI == EPI_LINEAR) {
        if (args.splits > 1) return launch_linear_variant<KIND, EPI, SPLIT_GLOBAL>(act_map, weight_map, args, shared_bytes, stream);
    }
    return launch_linear_variant<KIND, EPI, SPLIT_NONE>(act_map, weight_map, args, shared_bytes, stream);
}

static bool aligned16(const void* pointer) { return (reinterpret_cast<uintptr_t>(pointer) & 15u) == 0; }

// `workspace_need` != nullptr: report the split-K scratch this launch could use and return without launching
// (pointer fields are then not required).
int run_linear(const b2_linear_desc* d, cudaStream_t stream, int64_t* workspace_need) {
    if (d == nullptr) return B2_E_INVALID;
    const bool planning = workspace_need != nullptr;
    if (d->kind != B2_KIND_FP8 && d->kind != B2_KIND_NVFP4) return B2_E_UNSUPPORTED;
    if (d->epilogue != B2_EPI_LINEAR && d->epilogue != B2_EPI_GEGLU && d->epilogue != B2_EPI_GELU) return B2_E_UNSUPPORTED;
    if (d->tokens <= 0 || d->features <= 0 || d->width <= 0) return B2_E_INVALID;
    constexpr int KNOWN_FLAGS = B2_LINEAR_ROUND_SCALE_BF16 | B2_LINEAR_PAIRED_GATE_UP_SCALES | B2_LINEAR_STREAM_TOKENS |
                                B2_LINEAR_SINGLE_CTA | B2_LINEAR_PAIRS | B2_LINEAR_CLUSTER | B2_GEGLU_TRUE_DIV;
    if (d->flags & ~KNOWN_FLAGS) return B2_E_INVALID;
    if (!planning) {
        if (d->act == nullptr || d->weight == nullptr || d->act_scale == nullptr || d->weight_scale == nullptr ||
            (d->out == nullptr && d->rope == nullptr))
            return B2_E_INVALID;
        if (!aligned16(d->act) || !aligned16(d->weight) || !aligned16(d->out)) return B2_E_INVALID;
    }
    if ((d->bias != nullptr && !aligned16(d->bias)) || (d->residual != nullptr && !aligned16(d->residual)))
        return B2_E_INVALID;
    const bool nvfp4 = d->kind == B2_KIND_NVFP4;
    if (d->width % (nvfp4 ? 64 : 16) != 0) return B2_E_UNSUPPORTED;
    if (!planning && nvfp4 && (d->act_scales == nullptr || d->weight_scales == nullptr || !aligned16(d->act_scales) ||
                               !aligned16(d->weight_scales)))
        return B2_E_INVALID;
    const bool geglu = d->epilogue == B2_EPI_GEGLU;
    int epilogue = EPI_LINEAR;
    if (geglu) {
        if ((!planning && d->gelu_table == nullptr) || d->bias != nullptr || d->residual != nullptr) return B2_E_INVALID;
        if (d->out_format == B2_OUT_BF16) epilogue = EPI_GEGLU_BF16;
        else if (d->out_format == B2_OUT_FP8) epilogue = EPI_GEGLU_FP8;
        else if (d->out_format == B2_OUT_NVFP4) epilogue = EPI_GEGLU_NVFP4;
        else return B2_E_UNSUPPORTED;
        if (!planning && epilogue != EPI_GEGLU_BF16 && d->out_scale == nullptr) return B2_E_INVALID;
        if (d->features % 16 != 0) return B2_E_UNSUPPORTED;            // whole output vectors / blocks
        if (nvfp4 && d->features % 128 != 0) return B2_E_UNSUPPORTED;   // the up rows must start a scale block
    } else if (d->epilogue == B2_EPI_GELU) {
        if ((!planning && d->gelu_table == nullptr) || d->residual != nullptr) return B2_E_INVALID;
        if (d->out_format == B2_OUT_BF16) epilogue = EPI_GELU_BF16;
        else if (d->out_format == B2_OUT_FP8) epilogue = EPI_GELU_FP8;
        else return B2_E_UNSUPPORTED;
        if (!planning && epilogue == EPI_GELU_FP8 && d->out_scale == nullptr) return B2_E_INVALID;
        if (d->features % 8 != 0) return B2_E_UNSUPPORTED;
    } else {
        if (d->out_format != B2_OUT_BF16) return B2_E_UNSUPPORTED;
        if (d->features % 8 != 0) return B2_E_UNSUPPORTED;             // 16-byte output vectors
    }

    // More than one 128-token tile: two CTAs share every weight tile (gemm_pair.cu), unless the caller asks for the
    // single-CTA schedule or passes a scale layout only that schedule reads.
    {
        const bool workspace_given = d->workspace != nullptr && aligned16(d->workspace);
        PairPlan plan = pair_plan(d, geglu, planning || workspace_given);
        if (!planning && plan.splits > 1 && d->workspace_bytes < plan.workspace_need)   // too small: decide again without splitting
            plan = pair_plan(d, geglu, false);
        if (plan.columns != 0) {
            if (planning) {
                *workspace_need = plan.workspace_need;
                return B2_OK;
            }
            return run_linear_pair(d, epilogue, plan, stream);
        }
    }

    // At most 128 tokens: the weight becomes the "A" operand and a cluster shares the K of a feature tile (gemm_skinny.cu).
    // Only that schedule has the attention preparation (d->rope) as an epilogue.
    if (d->rope != nullptr) {
        if (!skinny_rope_supported(d)) return B2_E_UNSUPPORTED;
        epilogue = EPI_ROPE;
    }
    {
        const SkinnyPlan plan = skinny_plan(d, geglu);
        if (d->rope != nullptr && plan.splits == 0) return B2_E_UNSUPPORTED;
        if (plan.splits != 0) {
            if (planning) {
                *workspace_need = 0;
                return B2_OK;
            }
            return run_linear_skinny(d, epilogue, plan, stream);
        }
    }

    KernelArgs args{};
    args.tokens = d->tokens;
    args.features = d->features;
    args.k_bytes = nvfp4 ? d->width / 2 : d->width;
    args.num_kb = (args.k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES;
    args.num_m_tiles = (d->tokens + TILE_TOKENS - 1) / TILE_TOKENS;
    const bool paired = (d->flags & B2_LINEAR_PAIRED_GATE_UP_SCALES) != 0;
    if (paired && !(geglu && nvfp4)) return B2_E_INVALID;
    if (paired && d->feature_tile != 0 && d->feature_tile != 64) return B2_E_UNSUPPORTED;
    if (d->feature_tile > 0 && !tile_allowed(d->kind, geglu, d->feature_tile)) return B2_E_UNSUPPORTED;
    // K is split only into a caller-provided workspace; when the one given is too small the choice is repeated
    // without splitting
    bool allow_split = d->epilogue == B2_EPI_LINEAR && (planning || (d->workspace != nullptr && aligned16(d->workspace)));
    int feature_tile = 0, splits = 1;
    for (int attempt = 0; attempt < 2; ++attempt) {
        choose_tile_and_splits(d->kind, geglu, paired ? 64 : d->feature_tile, d->features, d->tokens, args.num_m_tiles, args.num_kb,
                               allow_split, &feature_tile, &splits);
        if (feature_tile == 0) return B2_E_UNSUPPORTED;
        const int64_t tiles = int64_t((d->features + feature_tile - 1) / feature_tile) * args.num_m_tiles;
        const int64_t need = splits > 1 ? TICKET_BYTES + tiles * splits * TILE_TOKENS * (geglu ? 2 : 1) * feature_tile * 4 : 0;
        if (planning) {
            *workspace_need = need;
            return B2_OK;
        }
        if (splits == 1 || d->workspace_bytes >= need) break;
        allow_split = false;
    }
    args.tile_n = geglu ? 2 * feature_tile : feature_tile;
    args.num_n_tiles = (d->features + feature_tile - 1) / feature_tile;
    args.total_tiles = args.num_m_tiles * args.num_n_tiles;
    args.scale_blocks = paired ? 1 : (geglu || args.tile_n > 128) ? 2 : 1;   // 128-row blocks of feature scales per tile
    args.accumulators = can_double_buffer(d->kind, args.tile_n, args.scale_blocks) ? 2 : 1;
    args.accumulator_stride = nvfp4 ? args.tile_n : 256;     // the second accumulator starts on a multiple of the tile width
    args.up_row_offset = d->features;
    args.scale_column_tiles = nvfp4 ? (d->width / 16 + 3) / 4 : 0;
    args.act_row_blocks = (d->tokens + 127) / 128;
    const int weight_rows = (geglu ? 2 : 1) * d->features;
    args.weight_row_blocks = (weight_rows + 127) / 128;
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

    constexpr int SCALE_PART_BYTES = SCALE_ATOMS_PER_STAGE * SCALE_ATOM_BYTES;
    // A launch with one token tile loads only the token rows it has (rounded up to the 8-row swizzle atom): a K stage
    // is then mostly weights, more stages fit, and more of a long K is in flight at once.  The MMA still reads 128
    // rows, so the stage ring is followed by padding that keeps those reads inside the allocation.
    const int box_rows = args.num_m_tiles == 1 ? (d->tokens + 7) / 8 * 8 : TILE_TOKENS;
    args.a_box_bytes = box_rows * STAGE_K_BYTES;
    const int ring_padding = A_TILE_BYTES - args.a_box_bytes;
    int stage_bytes = args.a_box_bytes + args.tile_n * STAGE_K_BYTES;
    int scale_stage_bytes = nvfp4 ? (1 + args.scale_blocks) * SCALE_PART_BYTES : 0;
    args.gelu_lo = args.gelu_hi = 0;
    if (epilogue != EPI_LINEAR && d->gelu_lo >= 0x80 && d->gelu_hi > d->gelu_lo && d->gelu_hi <= 0x7f80 &&
        d->gelu_hi - d->gelu_lo <= MAX_COMPACT_GELU) {
        args.gelu_lo = d->gelu_lo;
        args.gelu_hi = d->gelu_hi;
    }
    const int fixed_bytes = 1024 /* alignment slack */ + 16 * MAX_STAGES + 8 * MAX_RESIDENT_KB + 128 + 4 * (args.gelu_hi - args.gelu_lo) + ring_padding;
    // Resident order (TileWalk): worth it when a CTA computes several feature tiles of its token tile and the
    // token tile of all K, the weight stages and (NVFP4) the token scales in TMEM all fit.
    int panel_bytes = 0;
    args.resident = 0;
    {
        const int grid = args.total_tiles < sm_count() ? args.total_tiles : sm_count();
        const int resident_panel = args.num_kb * (A_TILE_BYTES + (nvfp4 ? SCALE_PART_BYTES : 0));
        const int resident_stage = args.tile_n * STAGE_K_BYTES + (nvfp4 ? args.scale_blocks * SCALE_PART_BYTES : 0);
        const int resident_stages = (SMEM_LIMIT - fixed_bytes - resident_panel) / resident_stage;
        const int free_columns = TMEM_COLUMNS - args.accumulators * args.accumulator_stride - (nvfp4 ? args.num_kb * TMEM_SFA_COLUMNS : 0);
        const bool columns_fit = !nvfp4 || free_columns >= 2 * 16 * args.scale_blocks;
        if (splits == 1 && box_rows == TILE_TOKENS && !(d->flags & B2_LINEAR_STREAM_TOKENS) && args.num_kb <= MAX_RESIDENT_KB && args.num_m_tiles <= grid &&
            int64_t(args.num_n_tiles) * args.num_m_tiles >= 2 * int64_t(grid) && resident_stages >= 3 && columns_fit) {
            args.resident = 1;
            panel_bytes = resident_panel;
            stage_bytes = args.tile_n * STAGE_K_BYTES;
            scale_stage_bytes = nvfp4 ? args.scale_blocks * SCALE_PART_BYTES : 0;
        }
    }
    const int free_columns = TMEM_COLUMNS - args.accumulators * args.accumulator_stride - (args.resident ? args.num_kb * TMEM_SFA_COLUMNS : 0);
    const int sets_available = nvfp4 ? free_columns / ((args.resident ? 0 : TMEM_SFA_COLUMNS) + 16 * args.scale_blocks) : 0;
    // K atoms per ring slot.  A launch whose CTAs have one tile each and a long K (the expert's M = 10..80 projections:
    // 16 CTAs walking 32 atoms) is bound by what the MMA warp spends per slot around the MMAs -- two barrier waits, the
    // election, the commit, some 400 cycles against 70 of tensor work per atom at 64 columns -- so a slot carries four
    // atoms (two when K is shorter), as long as three such slots fit and (NVFP4) tensor memory has a scale set per atom.
    args.kps = 1;
    {
        const int grid = args.total_tiles < sm_count() ? args.total_tiles : sm_count();
        const int ring_bytes = SMEM_LIMIT - fixed_bytes - panel_bytes;
        if (!args.resident && splits == 1 && args.total_tiles <= grid && args.num_kb >= 8) {
            for (int kps = args.num_kb >= 16 ? 4 : 2; kps > 1; kps /= 2) {
                int slots = ring_bytes / (kps * (stage_bytes + scale_stage_bytes));
                if (nvfp4 && slots > sets_available / kps) slots = sets_available / kps;
                if (slots >= 3) {
                    args.kps = kps;
                    break;
                }
            }
        }
    }
    stage_bytes *= args.kps;
    scale_stage_bytes *= args.kps;
    int stages = (SMEM_LIMIT - fixed_bytes - panel_bytes) / (stage_bytes + scale_stage_bytes);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (args.kps > 1 && nvfp4 && stages > sets_available / args.kps) stages = sets_available / args.kps;
    if (stages < 2) return B2_E_UNSUPPORTED;
    args.stages = stages;
    args.scale_sets = 1;
    if (nvfp4) {
        args.scale_sets = sets_available;
        if (args.scale_sets > stages * args.kps) args.scale_sets = stages * args.kps;
        if (args.scale_sets < 2) return B2_E_UNSUPPORTED;
    }
    int shared_bytes = fixed_bytes + panel_bytes + stages * (stage_bytes + scale_stage_bytes);
    if (shared_bytes < SMEM_MINIMUM) shared_bytes = SMEM_MINIMUM;

    args.splits = splits;
    args.tickets = nullptr;
    args.partials = nullptr;
    if (splits > 1) {
        args.tickets = static_cast<unsigned int*>(d->workspace);
        args.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(d->workspace) + TICKET_BYTES);
    }

    CUtensorMap act_map, weight_map;
    if (!make_operand_map(&act_map, d->act, d->tokens, args.k_bytes, box_rows)) return B2_E_DRIVER;
    if (geglu ? !make_gated_map(&weight_map, d->weight, d->features, args.k_bytes, feature_tile)
              : !make_operand_map(&weight_map, d->weight, weight_rows, args.k_bytes, feature_tile))
        return B2_E_DRIVER;

    if (nvfp4) {
        switch (epilogue) {
            case EPI_LINEAR: return launch_linear<B2_KIND_NVFP4, EPI_LINEAR>(act_map, weight_map, args, shared_bytes, stream);
            case EPI_GEGLU_BF16: return launch_linear<B2_KIND_NVFP4, EPI_GEGLU_BF16>(act_map, weight_map, args, shared_bytes, stream);
            case EPI_GEGLU_FP8: return launch_linear<B2_KIND_NVFP4, EPI_GEGLU_FP8>(act_map, weight_map, args, shared_bytes, stream);
            case EPI_GELU_BF16: return launch_linear<B2_KIND_NVFP4, EPI_GELU_BF16>(act_map, weight_map, args, shared_bytes, stream);
            case EPI_GELU_FP8: return launch_linear<B2_KIND_NVFP4, EPI_GELU_FP8>(act_map, weight_map, args, shared_bytes, stream);
            default: return launch_linear<B2_KIND_NVFP4, EPI_GEGLU_NVFP4>(act_map, weight_map, args, shared_bytes, stream);
        }
    }
    switch (epilogue) {
        case EPI_LINEAR: return launch_linear<B2_KIND_FP8, EPI_LINEAR>(act_map, weight_map, args, shared_bytes, stream);
        case EPI_GEGLU_BF16: return launch_linear<B2_KIND_FP8, EPI_GEGLU_BF16>(act_map, weight_map, args, shared_bytes, stream);
        case EPI_GEGLU_FP8: return launch_linear<B2_KIND_FP8, EPI_GEGLU_FP8>(act_map, weight_map, args, shared_bytes, stream);
        case EPI_GELU_BF16: return launch_linear<B2_KIND_FP8, EPI_GELU_BF16>(act_map, weight_map, args, shared_bytes, stream);
        case EPI_GELU_FP8: return launch_linear<B2_KIND_FP8, EPI_GELU_FP8>(act_map, weight_map, args, shared_bytes, stream);
        default: return launch_linear<B2_KIND_FP8, EPI_GEGLU_NVFP4>(act_map, weight_map, args, shared_bytes, stream);
    }
}

}  // namespace b2
