// FP8 / MXFP8 / MXFP4 GEMM on CTA pairs (tcgen05 cta_group::2): a cluster of two CTAs computes one 256 x BLOCK_N tile.
// Dense, grouped (tiles never cross a group; 256-row tiles per group) and variable-K forms, as in gemm_fp8.cu.
// Included by gemm_fp8.cu (uses its GemmParams, GemmMode and epilogue_store_block).
//
// Why pairs: with one CTA per tile every tcgen05.mma reads its whole A (128 x 32 B) and B (BLOCK_N x 32 B) slice from
// that CTA's shared memory while TMA writes the next stages into it, and the 128 B/clk shared-memory port, not the
// tensor core, bounds the main loop.  In a pair each CTA stores only half of the B tile, so per CTA and K step the
// shared-memory traffic drops from 48 KB + 48 KB to 32 KB + 32 KB at the same number of MMA cycles.
//
//   both CTAs    warp 0: TMA producer for its own A rows and its own half of the B rows; every copy counts its bytes
//                on the leader's (rank 0) full barrier
//   leader       warp 1: issues the cta_group::2 MMAs; tcgen05.commit multicasts the arrivals to both CTAs
//                (stage free -> both producers, accumulator full -> both epilogues)
//   both CTAs    warps 2-5 (FP4: 2-9): epilogue of the CTA's own 128 accumulator rows.  FP4 uses two warps per TMEM
//                lane quarter, each taking half of the columns: at FP4 rates and short K the write-out is as long as
//                the main loop (grouped FP4 forward +5 %), while for FP8 the extra staging memory costs a pipeline
//                stage.  They hand the TMEM buffer back by arriving on the leader's barrier
// No TMA multicast is used.  Every wait is bounded exactly as in the single-CTA kernel.
#pragma once

namespace ptb {

// F4: packed e2m1 operands, 256 elements per 128-byte stage row = two 128-element scale blocks per stage (kSfPerStage)
template <int BLOCK_N, bool MX, bool F4 = false> struct PairCfg {
    static constexpr int kEpiWarps = F4 ? 8 : 4;
    static constexpr int kThreads = 32 * (2 + kEpiWarps);
    static constexpr int kHalfN = BLOCK_N / 2;
    static constexpr int kSfbBlocks = (BLOCK_N + 127) / 128;
    static constexpr int kSfPerStage = F4 ? 2 : 1;
    static constexpr int kSfColsHalf = 4 + 4 * kSfbBlocks;        // SFA block + SFB blocks of one 128-element scale block
    static constexpr int kSfColsOne = kSfColsHalf * kSfPerStage;  // ... of one stage
    static constexpr int kSfCols = MX ? 2 * kSfColsOne : 0;       // double buffered
    static constexpr int kAccStages = (2 * BLOCK_N + kSfCols <= 512) ? 2 : 1;
    static constexpr int kTmemCols = 512;
    static constexpr int kABytes = BLOCK_M * BLOCK_K;
    static constexpr int kBBytes = kHalfN * BLOCK_K;
    static constexpr int kSfBytes = MX ? 512 * (1 + kSfbBlocks) * kSfPerStage : 0;  // own A blocks + every B block of the tile
    static constexpr int kStageBytes = kABytes + kBBytes + kSfBytes;
    static constexpr int kEpiBytes = kEpiWarps * 32 * kStagePitchMax;
    static constexpr int kBarBytes = 1024;
    static constexpr int kSmemBudget = 227 * 1024 - 1024 /* alignment slack */ - 9216 /* static shared: group tables */;
    static constexpr int kStages = std::min(8, (kSmemBudget - kEpiBytes - kBarBytes) / kStageBytes);
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarBytes + 1024;
    static_assert(kStages >= 3, "not enough shared memory for a 3-stage ring");
    static_assert(BLOCK_N % 32 == 0 && BLOCK_N <= 256, "pair tile: N must be a multiple of 32 (16 B-tile rows per CTA)");
    static_assert(kBBytes % 1024 == 0, "B stage must keep 1024-byte alignment");
    static_assert(kAccStages * BLOCK_N + kSfCols <= 512, "accumulators and scales do not fit the tensor memory");
};

template <int BLOCK_N, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__((PairCfg<BLOCK_N, mode_is_mx(MODE), MODE == GEMM_MXF4>::kThreads), 1)
    gemm_fp8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_sf, GemmParams p) {
    constexpr bool MX = mode_is_mx(MODE);
    constexpr bool F4 = MODE == GEMM_MXF4;
    using Cfg = PairCfg<BLOCK_N, MX, F4>;
    constexpr int kSfP = Cfg::kSfPerStage;
    constexpr int kStages = Cfg::kStages;
    constexpr int kAccStages = Cfg::kAccStages;
    constexpr int kTileM = 2 * BLOCK_M;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem_a + kStages * Cfg::kABytes;
    uint8_t *smem_sf = smem_b + kStages * Cfg::kBBytes;
    uint8_t *smem_epi = smem_sf + kStages * Cfg::kSfBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_epi + Cfg::kEpiBytes);
    uint64_t *full_bar = bars;                     // [kStages]    used in the leader: bytes of both CTAs
    uint64_t *empty_bar = bars + kStages;          // [kStages]    one multicast commit arrival per use, in each CTA
    uint64_t *tmem_full_bar = bars + 2 * kStages;  // [kAccStages] one multicast commit arrival per tile, in each CTA
    uint64_t *tmem_empty_bar = tmem_full_bar + kAccStages;  // used in the leader: epilogue warps of both CTAs
    uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(tmem_empty_bar + kAccStages);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_base_slot + 1);
    __shared__ int s_tile_start[kMaxGroups + 1];    // running count of 256-row tiles (x column blocks) over the groups
    __shared__ int s_blk128_start[kMaxGroups + 1];  // running count of 128-row blocks: index of a group's first A scale block

    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const uint32_t rank = cluster_ctarank();
    const int num_n_blocks = (p.N + BLOCK_N - 1) / BLOCK_N;
    const int num_k_blocks = (p.K + BLOCK_K - 1) / BLOCK_K;
    const int G = p.G;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < kAccStages; ++s) {
            mbar_init(&tmem_full_bar[s], 1);
            mbar_init(&tmem_empty_bar[s], 2 * Cfg::kEpiWarps);
        }
        fence_barrier_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        if constexpr (MX) prefetch_tmap(&tmap_sf);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_base_slot, Cfg::kTmemCols);
        tmem_relinquish_pair();
    }
    // everything above is private to this launch; from here on memory written by earlier kernels is read
    grid_dep_wait();
    if (threadIdx.x == 0) {
        int tiles = 0, blks = 0;
        s_tile_start[0] = 0;
        s_blk128_start[0] = 0;
        for (int g = 0; g < G; ++g) {
            const int64_t len = (p.offs_write && !p.koffs) ? (p.offs_write[g + 1] - p.offs_write[g]) : p.M;
            tiles += (int) ((len + kTileM - 1) / kTileM) * num_n_blocks;
            blks += (int) ((len + BLOCK_M - 1) / BLOCK_M);
            s_tile_start[g + 1] = tiles;
            s_blk128_start[g + 1] = blks;
        }
    }
    tc_fence_before_sync();
    __syncwarp();
    cluster_sync_all();  // barriers of both CTAs are initialised before any remote arrival or copy
    tc_fence_after_sync();
    grid_dep_launch();
    const uint32_t tmem_base = *tmem_base_slot;
    const uint32_t tmem_sfa = tmem_base + kAccStages * BLOCK_N;
    const uint32_t tmem_sfb = tmem_sfa + 4;

    TileWalk walk{s_tile_start, G, num_n_blocks, 0, max(1, p.raster_m / 2)};
    bool ok = true;
    int gi, m_blk, n_blk;
    auto k_range = [&](int g, int &kb_begin, int &kb_count) {
        if (p.koffs) {  // offsets count elements; a stage holds 128 (fp8), 256 (packed fp4) or 64 (16-bit) of them
            constexpr int kElemsPerStage = F4 ? 2 * BLOCK_K : (MODE == GEMM_HP ? BLOCK_K / 2 : BLOCK_K);
            kb_begin = (int) (p.koffs[g] / kElemsPerStage);
            kb_count = (int) ((p.koffs[g + 1] - p.koffs[g]) / kElemsPerStage);
        } else {
            kb_begin = 0;
            kb_count = num_k_blocks;
        }
    };

    if (warp == 0) {
        // ================================================================ TMA producer (both CTAs)
        if (elect_one()) {
            uint32_t stage = 0, phase = 0;
            const uint64_t keep = l2_policy_evict_last();
            for (int t = pair; ok && walk.locate(t, gi, m_blk, n_blk); t += num_pairs) {
                const int a_row0 = (int) (((p.offs_read && !p.koffs) ? p.offs_read[gi] : 0) + (int64_t) m_blk * kTileM) + (int) rank * BLOCK_M;
                const int b_row0 = (int) ((p.koffs ? 0 : (int64_t) gi * p.b_group_rows) + (int64_t) n_blk * BLOCK_N) + (int) rank * Cfg::kHalfN;
                int kb_begin, kb_count;
                k_range(gi, kb_begin, kb_count);
                // 512-byte scale blocks as rows of four 128-byte lines: A block of this CTA's rows, all B blocks of the tile
                // (kSfP blocks per K step; one box fetches the kSfP consecutive blocks of a step).  A 256-row tile that
                // ends a group with an odd number of 128-row blocks reads the next block's scales for rows that are
                // never stored.
                const int64_t a_rb = (p.koffs ? 0 : s_blk128_start[gi]) + 2 * m_blk + (int) rank;
                const int64_t b_rb = ((p.koffs ? 0 : (int64_t) gi * num_n_blocks) + n_blk) * Cfg::kSfbBlocks;
                const int64_t sfa_line0 = (a_rb * num_k_blocks + kb_begin) * kSfP * 4;
                const int64_t sfb_line0 = p.sfb_line0 + (b_rb * num_k_blocks + kb_begin) * kSfP * 4;
                for (int kb = 0; kb < kb_count; ++kb) {
                    if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) break;
                    const uint32_t full_leader = map_to_rank(&full_bar[stage], 0);
                    if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::kStageBytes);
                    const int k0 = (kb_begin + kb) * BLOCK_K;
                    // MN-major operands (dense tensorwise / rowwise): 128 row indices x 128 contraction rows per CTA
                    if (!MX && p.a_mn) tma_load_2d_pair_hint(smem_a + stage * Cfg::kABytes, &tmap_a, full_leader, a_row0, k0, keep);
                    else tma_load_2d_pair_hint(smem_a + stage * Cfg::kABytes, &tmap_a, full_leader, k0, a_row0, keep);
                    if (!MX && p.b_mn) tma_load_2d_pair_hint(smem_b + stage * Cfg::kBBytes, &tmap_b, full_leader, b_row0, k0, keep);
                    else tma_load_2d_pair_hint(smem_b + stage * Cfg::kBBytes, &tmap_b, full_leader, k0, b_row0, keep);
                    if constexpr (MX) {
                        uint8_t *sf = smem_sf + stage * Cfg::kSfBytes;
                        tma_load_2d_pair(sf, &tmap_sf, full_leader, 0, (int) (sfa_line0 + 4 * kSfP * kb));
#pragma unroll
                        for (int j = 0; j < Cfg::kSfbBlocks; ++j)
                            tma_load_2d_pair(sf + kSfP * 512 * (1 + j), &tmap_sf, full_leader, 0,
                                             (int) (sfb_line0 + ((int64_t) j * num_k_blocks + kb) * kSfP * 4));
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ================================================================ MMA issuer (leader CTA only)
        if (rank == 0 && elect_one()) {
            const uint32_t idesc = F4 ? idesc_block_scaled(1, 1, kTileM, BLOCK_N)  // kind::mxf4: format code 1 = e2m1
                                   : MX ? idesc_block_scaled(p.a_fmt, p.b_fmt, kTileM, BLOCK_N)
                                        : (idesc_f8(p.a_fmt, p.b_fmt, kTileM, BLOCK_N) | ((uint32_t) (p.a_mn != 0) << 15) | ((uint32_t) (p.b_mn != 0) << 16));
            const bool a_mn = !MX && MODE != GEMM_HP && p.a_mn, b_mn = !MX && MODE != GEMM_HP && p.b_mn;
            const uint64_t a_kstep = a_mn ? (uint64_t) ((UMMA_K * 128) >> 4) : (uint64_t) (UMMA_K >> 4);
            const uint64_t b_kstep = b_mn ? (uint64_t) ((UMMA_K * 128) >> 4) : (uint64_t) (UMMA_K >> 4);
            uint32_t stage = 0, phase = 0, acc_stage = 0, acc_phase = 0, sf_buf = 0;
            for (int t = pair; ok && walk.locate(t, gi, m_blk, n_blk); t += num_pairs) {
                int kb_begin, kb_count;
                k_range(gi, kb_begin, kb_count);
                if (kb_count == 0) continue;  // empty contraction range: the epilogues write zeros on their own
                if (!(ok = mbar_wait(&tmem_empty_bar[acc_stage], acc_phase ^ 1, abort_flag))) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc_stage * BLOCK_N;
                for (int kb = 0; kb < kb_count; ++kb) {
                    if (!(ok = mbar_wait(&full_bar[stage], phase, abort_flag))) break;
                    tc_fence_after_sync();
                    const uint32_t sfa_cur = tmem_sfa + sf_buf * Cfg::kSfColsOne;
                    const uint32_t sfb_cur = tmem_sfb + sf_buf * Cfg::kSfColsOne;
                    if constexpr (MX) {
                        const uint32_t sf_addr = smem_u32(smem_sf + stage * Cfg::kSfBytes);
#pragma unroll
                        for (int h = 0; h < kSfP; ++h) {
                            tc_cp_sf_pair(sfa_cur + h * Cfg::kSfColsHalf, smem_desc_sf(sf_addr + 512 * h));
#pragma unroll
                            for (int j = 0; j < Cfg::kSfbBlocks; ++j)
                                tc_cp_sf_pair(sfb_cur + h * Cfg::kSfColsHalf + 4 * j, smem_desc_sf(sf_addr + kSfP * 512 * (1 + j) + 512 * h));
                        }
                        sf_buf ^= 1;
                    }
                    const uint32_t a_addr = smem_u32(smem_a + stage * Cfg::kABytes), b_addr = smem_u32(smem_b + stage * Cfg::kBBytes);
                    const uint64_t a_desc = a_mn ? smem_desc_sw128_mn(a_addr, 16384) : smem_desc_sw128(a_addr);
                    const uint64_t b_desc = b_mn ? smem_desc_sw128_mn(b_addr, 16384) : smem_desc_sw128(b_addr);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t adv = (uint64_t) ((k * UMMA_K) >> 4);
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        if constexpr (F4)  // 64 elements, two scales per row: scale block k / 2, bytes (k % 2) * 2 .. +1
                            mma_mxf4_pair(d_tmem, a_desc + adv, b_desc + adv, idesc_sf_ids(idesc, (k & 1) * 2, (k & 1) * 2),
                                          sfa_cur + (k >> 1) * Cfg::kSfColsHalf, sfb_cur + (k >> 1) * Cfg::kSfColsHalf, accumulate);
                        else if constexpr (MX) mma_mxf8_pair(d_tmem, a_desc + adv, b_desc + adv, idesc_sf_ids(idesc, k, k), sfa_cur, sfb_cur, accumulate);
                        else if constexpr (MODE == GEMM_HP) mma_f16_pair(d_tmem, a_desc + adv, b_desc + adv, idesc, accumulate);
                        else mma_f8_pair(d_tmem, a_desc + k * a_kstep, b_desc + k * b_kstep, idesc, accumulate);
                    }
                    tc_commit_pair(&empty_bar[stage], 3);  // frees the ring slot in both CTAs
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc_commit_pair(&tmem_full_bar[acc_stage], 3);
                if (++acc_stage == kAccStages) { acc_stage = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ================================================================ epilogue (both CTAs, own 128 rows)
        const int q = warp & 3;                      // TMEM lane quarter this warp may read
        const int half = (warp - kEpiWarp0) >> 2;    // with eight warps: which share of the tile's 32-column chunks
        constexpr int kChunks = (BLOCK_N + 31) / 32;
        const int c_begin = (Cfg::kEpiWarps == 8 && half) ? kChunks / 2 : 0;
        const int c_end = (Cfg::kEpiWarps == 8 && !half) ? kChunks / 2 : kChunks;
        uint8_t *stg = smem_epi + (warp - kEpiWarp0) * 32 * kStagePitchMax;
        uint32_t acc_stage = 0, acc_phase = 0;
        for (int t = pair; ok && walk.locate(t, gi, m_blk, n_blk); t += num_pairs) {
            const int64_t c_row_base = p.koffs ? (int64_t) gi * p.M : (p.offs_write ? p.offs_write[gi] : 0);
            const int64_t c_row_end = p.koffs ? c_row_base + p.M : (p.offs_write ? p.offs_write[gi + 1] : p.M);
            int kb_begin, kb_count;
            k_range(gi, kb_begin, kb_count);
            const bool have_acc = kb_count > 0;
            const int64_t tile_row0 = c_row_base + (int64_t) m_blk * kTileM + (int64_t) rank * BLOCK_M + q * 32;
            const int n0 = n_blk * BLOCK_N;
            if (have_acc && !(ok = mbar_wait_warp(&tmem_full_bar[acc_stage], acc_phase, abort_flag))) break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t) (q * 32) << 16) + acc_stage * BLOCK_N;
            const uint32_t release_addr = map_to_rank(&tmem_empty_bar[acc_stage], 0);
            epilogue_store_block<BLOCK_N, MODE>(p, taddr, have_acc, tile_row0, c_row_end, n0, gi, stg, lane, c_begin, c_end,
                                                [&]() { mbar_arrive_cluster(release_addr); });
            if (have_acc && ++acc_stage == kAccStages) { acc_stage = 0; acc_phase ^= 1; }
        }
    }

    // ---- teardown: both CTAs leave together (the leader's MMAs read the peer's shared and tensor memory)
    if (!ok || *abort_flag) {
        if (p.status && lane == 0) atomicExch(p.status, (int) PT_ERR_TIMEOUT);
        __nanosleep(200000);
    }
    tc_fence_before_sync();
    __syncwarp();  // the cluster barrier is warp-aligned: role branches above may have split the warp
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    }
}

}  // namespace ptb
