// CTA-pair form of the block-scaled FP8 GEMM (included by gemm_fp8_blockwise.cu): two CTAs of a cluster share a
// 256 x 256 tile, each holding its own 128 rows of A and one half of the B tile, and the leader issues
// tcgen05.mma.cta_group::2 for both.  Shared memory then carries 32 KiB per K step and CTA instead of 48, which is what
// limits the single-CTA kernel.  Everything else is that kernel's pipeline, run in both CTAs: 128 x 256 partial sums
// per CTA in its own tensor memory, promotion warps, scale rings (per CTA; here the promotion warps wait for and
// release their scale slots themselves, since only the leader has an MMA issuer).
#pragma once

// (inside namespace ptb, after the single-CTA kernel and its helpers)

template <int SBM, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kBwThreads, 1)
    gemm_fp8_blockwise_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                              const __grid_constant__ CUtensorMap tmap_c, BwParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem_a + kBwStages * kBwABytes;
    uint8_t *smem_epi = smem_b + kBwStages * kBwBBytes;
    float *smem_slab = reinterpret_cast<float *>(smem_epi + kBwEpiBytes);  // [kBwSlabRing][256] B column scales
    float *smem_scale = smem_slab + kBwSlabRing * (kBwSlabBytes / 4);      // [kBwSlabRing][kBwScaleSlot] row / tile scales
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_scale + kBwSlabRing * kBwScaleSlot);
    uint64_t *full_bar = bars;
    uint64_t *empty_bar = bars + kBwStages;
    uint64_t *part_full_bar = bars + 2 * kBwStages;  // [2]
    uint64_t *part_empty_bar = part_full_bar + 2;    // [2]
    uint64_t *slab_full_bar = part_empty_bar + 2;    // [kBwSlabRing]
    uint64_t *scale_full_bar = slab_full_bar + kBwSlabRing;    // [kBwSlabRing]
    uint64_t *scale_empty_bar = scale_full_bar + kBwSlabRing;  // [kBwSlabRing]
    uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(scale_empty_bar + kBwSlabRing);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_base_slot + 1);
    __shared__ int s_tile_start[kMaxGroups + 1];

    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int num_n_blocks = (p.N + BW_BLOCK_N - 1) / BW_BLOCK_N;
    const int num_k_blocks = (p.K + BLOCK_K - 1) / BLOCK_K;
    const int G = p.G;
    constexpr int kTileM = 2 * BLOCK_M;  // rows of a pair's tile; this CTA owns rows [rank * 128, rank * 128 + 128) of it
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        int acc = 0;
        s_tile_start[0] = 0;
        for (int g = 0; g < G; ++g) {
            const int64_t len = p.koffs ? p.M : (p.offs_write ? (p.offs_write[g + 1] - p.offs_write[g]) : p.M);
            acc += (int) ((len + kTileM - 1) / kTileM) * num_n_blocks;
            s_tile_start[g + 1] = acc;
        }
        *abort_flag = 0;
        for (int s = 0; s < kBwStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&part_full_bar[s], 1);                   // one multicast commit per K step, in each CTA
            mbar_init(&part_empty_bar[s], 2 * kBwPromoWarps);  // used in the leader: promotion warps of both CTAs
        }
        for (int s = 0; s < kBwSlabRing; ++s) {
            mbar_init(&slab_full_bar[s], 1);
            mbar_init(&scale_full_bar[s], 64);  // one deferred arrival per loader thread
            mbar_init(&scale_empty_bar[s], kBwPromoWarps);  // every promotion warp hands the slot back itself
        }
        fence_barrier_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_base_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncwarp();
    cluster_sync_all();  // barriers of both CTAs are initialised before any remote arrival or copy
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;

    TileWalk walk{s_tile_start, G, num_n_blocks, 0, max(1, p.raster_m / 2)};
    int gi, m_blk, n_blk;
    bool ok = true;

    // K steps of group g: all of K, or the group's contraction range in the variable-K form
    auto k_range = [&](int g, int &kb_begin, int &kb_count) {
        if (p.koffs) {
            kb_begin = (int) (p.koffs[g] / BLOCK_K);
            kb_count = (int) ((p.koffs[g + 1] - p.koffs[g]) / BLOCK_K);
        } else {
            kb_begin = 0;
            kb_count = num_k_blocks;
        }
    };

    if (warp < kBwPromoWarp0) {
    // the first warpgroup (producer, MMA issuer, scale loaders) gives registers to the promotion warps
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
        // ================================================================ TMA producer
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, step = 0;
            for (int t = pair; ok && walk.locate(t, gi, m_blk, n_blk); t += num_pairs) {
                const int64_t a_row0 = (p.koffs ? 0 : (p.offs_read ? p.offs_read[gi] : 0)) + (int64_t) m_blk * kTileM + rank * BLOCK_M;
                // this CTA stages its own half of the B tile: rows (K-major) or columns (MN-major) [rank * 128, +128)
                const int64_t b_row0 = (p.koffs ? 0 : (int64_t) gi * p.b_group_rows) + (int64_t) n_blk * BW_BLOCK_N + rank * (BW_BLOCK_N / 2);
                int kb_begin, kb_count;
                k_range(gi, kb_begin, kb_count);
                const int n0 = n_blk * BW_BLOCK_N;
                const int slab_cols = min(BW_BLOCK_N, p.N - n0);
                for (int kb = 0; kb < kb_count; ++kb, ++step) {
                    if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) break;
                    // the leader's barrier counts the bytes of both CTAs: A 128 x 128 and half of B each
                    const uint32_t full_leader = map_to_rank(&full_bar[stage], 0);
                    if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * (kBwABytes + kBwBBytes / 2));
                    const int k0 = (kb_begin + kb) * BLOCK_K;
                    uint8_t *sa = smem_a + stage * kBwABytes, *sb = smem_b + stage * kBwBBytes;
                    if (p.a_mn) tma_load_2d_pair(sa, &tmap_a, full_leader, (int) a_row0, k0);
                    else tma_load_2d_pair(sa, &tmap_a, full_leader, k0, (int) a_row0);
                    if (p.b_mn) {
                        // one 128-wide box per CTA; contraction rows of group g start at g * b_group_kstride
                        const int kr = (int) ((p.koffs ? 0 : (int64_t) gi * p.b_group_kstride) + k0);
                        tma_load_2d_pair(sb, &tmap_b, full_leader, n0 + (int) rank * (BW_BLOCK_N / 2), kr);
                    } else {
                        tma_load_2d_pair(sb, &tmap_b, full_leader, k0, (int) b_row0);
                    }
                    if constexpr (SBM == SB_SLAB) {
                        // per-column B scales of this K step: one contiguous run of `slab_cols` floats.  Ring slot
                        // step % 8 is free: the producer runs at most 4 stages + 2 partial buffers ahead of the readers.
                        const uint32_t slot = step % kBwSlabRing;
                        const float *src = p.sb.base + (int64_t) gi * p.sb.group_stride + (int64_t) (kb_begin + kb) * p.sb.kb_stride + n0;
                        mbar_arrive_expect_tx(&slab_full_bar[slot], (uint32_t) slab_cols * 4);
                        bulk_load(smem_slab + slot * (kBwSlabBytes / 4), src, (uint32_t) slab_cols * 4, &slab_full_bar[slot]);
                    }
                    if (++stage == kBwStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp >= 2) {
        // ================================================================ scale loader (warps 2-3)
        // Stages the fp32 scales of each K step into an 8-slot ring with asynchronous 4-byte copies: two A rows
        // per thread, and the two per-tile B scales.  The promotion warps then read their scales from shared
        // memory and never wait on a global load.  A slot is refilled once the MMA issuer has released it.
        const int lt = threadIdx.x - 64;  // 0..63
        constexpr bool sb_uniform = SBM == SB_TILE;
        const int64_t sa_last = p.a_rows_total - 1;
        uint32_t step = 0;
        for (int t = pair; ok && walk.locate(t, gi, m_blk, n_blk); t += num_pairs) {
            const int64_t a_row0 = (p.koffs ? 0 : (p.offs_read ? p.offs_read[gi] : 0)) + (int64_t) m_blk * kTileM + rank * BLOCK_M;
            int kb_begin, kb_count;
            k_range(gi, kb_begin, kb_count);
            // rows past the end of the operand are never stored; their scale reads are clamped to the last row
            const float *src0 = p.sa.base + (min(a_row0 + lt, sa_last) >> p.sa.shift) * p.sa.row_stride + (int64_t) kb_begin * p.sa.kb_stride;
            const float *src1 = p.sa.base + (min(a_row0 + lt + 64, sa_last) >> p.sa.shift) * p.sa.row_stride + (int64_t) kb_begin * p.sa.kb_stride;
            const int nb = min(n_blk * BW_BLOCK_N + 128 * (lt & 1), p.N - 1) >> 7;
            const float *srcb = p.sb.base + (int64_t) gi * p.sb.group_stride + (int64_t) kb_begin * p.sb.kb_stride + (int64_t) nb * p.sb.row_stride;
            for (int kb = 0; kb < kb_count; ++kb, ++step) {
                const uint32_t slot = step % kBwSlabRing;
                if (!(ok = mbar_wait_warp(&scale_empty_bar[slot], ((step / kBwSlabRing) & 1u) ^ 1u, abort_flag))) break;
                float *slot_ptr = smem_scale + slot * kBwScaleSlot;
                cp_async_4(slot_ptr + lt, src0 + (int64_t) kb * p.sa.kb_stride);
                cp_async_4(slot_ptr + lt + 64, src1 + (int64_t) kb * p.sa.kb_stride);
                if (sb_uniform && lt < 2) cp_async_4(slot_ptr + 128 + lt, srcb + (int64_t) kb * p.sb.kb_stride);
                cp_async_arrive_noinc(&scale_full_bar[slot]);
            }
        }
    } else if (warp == 1) {
        // ================================================================ MMA issuer
        if (rank == 0 && elect_one()) {  // the leader issues for both CTAs
            const uint32_t idesc = idesc_f8(p.a_fmt, p.b_fmt, kTileM, BW_BLOCK_N) | ((uint32_t) (p.a_mn != 0) << 15) |
                                   ((uint32_t) (p.b_mn != 0) << 16);
            uint32_t stage = 0, phase = 0, pb = 0, pphase = 0, step = 0;
            for (int t = pair; ok && walk.locate(t, gi, m_blk, n_blk); t += num_pairs) {
                int kb_begin, kb_count;
                k_range(gi, kb_begin, kb_count);
                for (int kb = 0; kb < kb_count; ++kb, ++step) {
                    // the scale rings are per CTA here: the promotion warps wait for their own slots
                    if (!(ok = mbar_wait(&full_bar[stage], phase, abort_flag))) break;
                    const uint32_t d_tmem = tmem_base + pb * BW_BLOCK_N;
                    const uint32_t a_addr = smem_u32(smem_a + stage * kBwABytes), b_addr = smem_u32(smem_b + stage * kBwBBytes);
                    const uint64_t a_desc = p.a_mn ? smem_desc_sw128_mn(a_addr, 16384) : smem_desc_sw128(a_addr);
                    const uint64_t b_desc = p.b_mn ? smem_desc_sw128_mn(b_addr, 16384) : smem_desc_sw128(b_addr);
                    if (!(ok = mbar_wait(&part_empty_bar[pb], pphase ^ 1, abort_flag))) break;
                    tc_fence_after_sync();
                    // one instruction consumes 32 contraction indices: 32 bytes along a K-major row, or 32 rows of
                    // 128 bytes in an MN-major tile
                    const uint64_t a_step = p.a_mn ? (uint64_t) ((UMMA_K * 128) >> 4) : (uint64_t) (UMMA_K >> 4);
                    const uint64_t b_step = p.b_mn ? (uint64_t) ((UMMA_K * 128) >> 4) : (uint64_t) (UMMA_K >> 4);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                        mma_f8_pair(d_tmem, a_desc + k * a_step, b_desc + k * b_step, idesc, k > 0 ? 1u : 0u);
                    tc_commit_pair(&empty_bar[stage], 3);    // frees the ring slot in both CTAs
                    tc_commit_pair(&part_full_bar[pb], 3);   // announces the partial sum in both CTAs
                    if (++stage == kBwStages) { stage = 0; phase ^= 1; }
                    if (++pb == 2) { pb = 0; pphase ^= 1; }
                }
                if (!ok) break;
            }
        }
    }
    } else {
        // ================================================================ promotion + epilogue
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        const int pw = warp - kBwPromoWarp0;
        const int q = warp & 3;       // TMEM lane quarter of this warp
        const int half = pw >> 2;     // which 128 columns of the 256-wide tile
        uint8_t *stg = smem_epi + pw * kBwEpiWarpBytes;
        uint32_t pb = 0, pphase = 0, step = 0;
        for (int t = pair; ok && walk.locate(t, gi, m_blk, n_blk); t += num_pairs) {
            const int64_t c_row_base = p.koffs ? (int64_t) gi * p.M : (p.offs_write ? p.offs_write[gi] : 0);
            const int64_t c_row_end = p.koffs ? c_row_base + p.M : (p.offs_write ? p.offs_write[gi + 1] : p.M);
            const int64_t a_row_base = p.koffs ? 0 : (p.offs_read ? p.offs_read[gi] : 0);
            int kb_begin, kb_count;
            k_range(gi, kb_begin, kb_count);
            const int row_in_tile = q * 32 + lane;  // row of this CTA's 128
            const int64_t my_c_row = c_row_base + (int64_t) m_blk * kTileM + rank * BLOCK_M + row_in_tile;
            const int64_t my_a_row = a_row_base + (int64_t) m_blk * kTileM + rank * BLOCK_M + row_in_tile;
            const bool row_ok = my_c_row < c_row_end;
            const int n0 = n_blk * BW_BLOCK_N + half * 128;
            const int n_end = min(p.N, n0 + 128);
            const float *sb_base = p.sb.base + (int64_t) gi * p.sb.group_stride + (int64_t) kb_begin * p.sb.kb_stride;
            constexpr bool sb_uniform = SBM == SB_TILE;

            __align__(8) float acc[128];
#pragma unroll
            for (int i = 0; i < 128; ++i) acc[i] = 0.f;

            for (int kb = 0; kb < kb_count; ++kb, ++step) {
                // scales (and the B slab) of this K step, staged by this CTA's loader warps / producer
                if (!(ok = mbar_wait_warp(&scale_full_bar[step % kBwSlabRing], (step / kBwSlabRing) & 1u, abort_flag))) break;
                if constexpr (SBM == SB_SLAB)
                    if (!(ok = mbar_wait_warp(&slab_full_bar[step % kBwSlabRing], (step / kBwSlabRing) & 1u, abort_flag))) break;
                if (!(ok = mbar_wait_warp(&part_full_bar[pb], pphase, abort_flag))) break;
                tc_fence_after_sync();
                const uint32_t taddr = tmem_base + ((uint32_t) (q * 32) << 16) + pb * BW_BLOCK_N + half * 128;
                // TMEM reads are issued one chunk ahead of the FMAs that consume them
                uint32_t r0[32], r1[32];
                tmem_ld32(taddr, r0);
                // the scales of this K step landed in the ring before the partial sum was announced
                const float *sc_slot = smem_scale + (step % kBwSlabRing) * kBwScaleSlot;
                const float sa_cur = sc_slot[row_in_tile], sbu_cur = sc_slot[128 + half];
                // acc[32 c ..] += partial chunk c * scales
                auto add_chunk = [&](int c, const uint32_t(&r)[32]) {
                    if constexpr (sb_uniform) {
                        const float sc = sa_cur * sbu_cur;  // one scale for the whole 32 x 128 block of this warp
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(__uint_as_float(r[i]), sc, acc[c * 32 + i]);
                    } else if constexpr (SBM == SB_SLAB) {
                        // the slab of this K step landed before the partial sum was announced (see the MMA issuer)
                        const float4 *sl =
                            reinterpret_cast<const float4 *>(smem_slab + (step % kBwSlabRing) * (kBwSlabBytes / 4) + half * 128);
                        // two elements per instruction (mul.f32x2 / fma.f32x2): this path does two operations per
                        // element and is bound by instruction issue
                        uint64_t sa2;
                        asm("mov.b64 %0, {%1, %1};" : "=l"(sa2) : "f"(sa_cur));
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 sv = sl[c * 8 + i];  // same address in every lane: a broadcast read
                            scaled_fma2(*reinterpret_cast<uint64_t *>(&acc[c * 32 + 4 * i + 0]), r[4 * i + 0], r[4 * i + 1], sv.x, sv.y, sa2);
                            scaled_fma2(*reinterpret_cast<uint64_t *>(&acc[c * 32 + 4 * i + 2]), r[4 * i + 2], r[4 * i + 3], sv.z, sv.w, sa2);
                        }
                    } else {
                        // general per-row B scales read from global memory (no reference path needs this to be fast)
                        const float *sbk = sb_base + (int64_t) kb * p.sb.kb_stride;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int n = n0 + c * 32 + i;
                            const float sbv = n < n_end ? __ldg(sbk + (int64_t) (n >> p.sb.shift) * p.sb.row_stride) : 0.f;
                            acc[c * 32 + i] = fmaf(__uint_as_float(r[i]) * sbv, sa_cur, acc[c * 32 + i]);
                        }
                    }
                };
                // Two TMEM loads are kept in flight, so the step has two load latencies on its critical path instead
                // of four; the partial buffer goes back to the MMA issuer as soon as the last load has landed.
                tmem_ld32(taddr + 32, r1);
                tmem_ld_wait();
                add_chunk(0, r0);
                tmem_ld32(taddr + 64, r0);
                add_chunk(1, r1);
                tmem_ld32(taddr + 96, r1);
                tmem_ld_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {  // the leader's MMA issuer owns the buffers
                    if (rank == 0) mbar_arrive(&part_empty_bar[pb]);
                    else mbar_arrive_cluster(map_to_rank(&part_empty_bar[pb], 0));
                }
                add_chunk(2, r0);
                add_chunk(3, r1);
                __syncwarp();
                if (lane == 0) mbar_arrive(&scale_empty_bar[step % kBwSlabRing]);  // this warp has read the slot (and slab) of the step
                if (++pb == 2) { pb = 0; pphase ^= 1; }
            }
            if (!ok) break;

            // ---- write-out through the per-warp staging buffer
            const int64_t tile_row0 = c_row_base + (int64_t) m_blk * kTileM + rank * BLOCK_M + q * 32;
            // whole blocks (or blocks cut only by the end of the matrix, which the TMA unit clips) take the bulk path
            if (p.c_tma && tile_row0 < c_row_end && n0 < p.N && (tile_row0 + 32 <= c_row_end || c_row_end == p.c_rows_total)) {
                bw_store_tile_bulk<OutT>(acc, stg, lane, tile_row0, n0, p.N, &tmap_c);
                continue;
            }
            if (p.c_tma) {  // the staging area may still be read by an earlier bulk store
                if (lane == 0) bulk_wait_read_all();
                __syncwarp();
            }
            bw_store_tile<OutT>(acc, stg, lane, tile_row0, c_row_end, n0, n_end, p);
        }
        // bulk stores still in flight read this CTA's shared memory
        if (p.c_tma && lane == 0) bulk_wait_all();
    }

    if (!ok || *abort_flag) {
        if (p.status && lane == 0) atomicExch(p.status, (int) PT_ERR_TIMEOUT);
        __nanosleep(200000);
    }
    // both CTAs leave together: the leader's MMAs read the peer's shared and tensor memory
    tc_fence_before_sync();
    __syncwarp();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
}


