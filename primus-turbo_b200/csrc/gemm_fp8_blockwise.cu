// FP8 GEMM with fp32 block scales (128-element blocks along K), dense and grouped:
//   C[m, n] = sum over K blocks kb of ( sum_{k in kb} A[m, k] * B[n, k] ) * sa(m, kb) * sb(n, kb)
// which is the accumulation order of the reference kernel
// (primus_turbo/triton/gemm/gemm_fp8_kernel.py:872-1013; grouped:
// primus_turbo/triton/grouped_gemm/grouped_gemm_fp8_kernel.py:1407-1556, 1661-1802).
//
// The tensor core has no fp32 block scaling, so accumulation is done on two levels: tcgen05.mma sums one
// 128-wide K block into a TMEM buffer (two buffers, ping-pong), and eight "promotion" warps read each finished
// block out of TMEM, multiply by the two scales and add into fp32 register accumulators while the tensor core
// is already working on the next block.  Tile 128 x 256: each promotion warp owns 32 rows x 128 columns.
//
//   warp 0       TMA producer (A 128 x 128 B, B 256 x 128 B per stage, 128-byte swizzle; B column-scale slabs)
//   warp 1       MMA issuer, owns TMEM (512 columns = 2 partial buffers x 256)
//   warps 2-3    scale loaders: stage the fp32 scales of each K step into a shared-memory ring (cp.async)
//   warps 4-11   promotion + epilogue, 232 registers each (128 fp32 accumulators per thread)
//
// Operand layouts: each operand may be K-major ([rows, K], the contraction index contiguous) or MN-major
// ([K, rows], the row index contiguous), selected per operand in the instruction descriptor.  MN-major tiles are
// loaded as 128-byte x 128-row TMA boxes and described to the tensor core with SBO = 1024 bytes (eight contraction
// rows) and LBO = 16 KiB (next 128-wide box); this is what lets dgrad (weight stored [N, K], contraction over N)
// and wgrad (both operands stored token-major, contraction over tokens) run without transposed copies.
// Variable-K form (grouped wgrad): every group g produces a full [rows_a, N] output block from the contraction
// range [koffs[g], koffs[g+1]) of both (MN-major) operands.
//
// Scales are addressed through a small descriptor so that every layout the reference produces is read in
// place: s(row, kb) = base[(row >> shift) * row_stride + kb * kb_stride]  (shift 0: per row, shift 7: per 128 rows).
#include <algorithm>
#include <cstdio>

#include "gemm_common.cuh"

namespace ptb {
using namespace sm100;

constexpr int BW_BLOCK_N = 256;
constexpr int kBwPromoWarps = 8;
constexpr int kBwPromoWarp0 = 4;  // warps 0-3 form the first warpgroup: producer, MMA issuer, two scale loaders
constexpr int kBwThreads = 32 * (kBwPromoWarp0 + kBwPromoWarps);
constexpr int kBwSlabRing = 8;    // ring of per-K-step B column-scale slabs (256 floats each)
constexpr int kBwSlabBytes = BW_BLOCK_N * 4;
constexpr int kBwScaleSlot = 136;  // floats per scale-ring slot: 128 A row scales, 2 B tile scales, padding
constexpr int kBwStagePitch = 64;  // staging row: 32 x 16-bit or 16 x fp32 columns; 16-byte chunks XOR-swizzled by row
constexpr int kBwABytes = BLOCK_M * BLOCK_K;
constexpr int kBwBBytes = BW_BLOCK_N * BLOCK_K;
constexpr int kBwStages = 3;
constexpr int kBwEpiWarpBytes = 8192;  // per promotion warp: two 32-row x 128-byte boxes of the bulk-store path
constexpr int kBwEpiBytes = kBwPromoWarps * kBwEpiWarpBytes;
constexpr int kBwSmemBytes =
    kBwStages * (kBwABytes + kBwBBytes) + kBwEpiBytes + kBwSlabRing * (kBwSlabBytes + kBwScaleSlot * 4) + 1024 + 1024;

struct ScaleDesc {
    const float *base;
    int shift;            // 0: one scale per row, 7: one per 128 rows
    int64_t row_stride;   // elements
    int64_t kb_stride;    // elements between consecutive K blocks
    int64_t group_stride; // elements between groups (B side of grouped GEMMs), else 0
};

struct BwParams {
    int64_t M;
    int N, K;
    void *C;
    int64_t ldc;
    int c_dtype, vec_store_ok;
    int c_tma;                 // C has a tensor map: whole 32-row blocks leave through bulk tensor stores
    int64_t c_rows_total;
    float beta;
    ScaleDesc sa, sb;
    int a_fmt, b_fmt;
    const int64_t *offs_read, *offs_write;
    int G;
    int64_t b_group_rows;
    int64_t a_rows_total;
    int *status;
    int raster_m;
    int a_mn, b_mn;            // operand is MN-major (stored [contraction, rows])
    int sb_slab;               // B scales are per column and contiguous along the columns: staged through shared memory
    const int64_t *koffs;      // variable-K: contraction row range of each group (multiples of 128), else null
    int64_t b_group_kstride;   // MN-major B of a grouped GEMM: contraction rows per group
};

// c (two adjacent fp32 accumulators viewed as one 64-bit register pair) += ((a0, a1) * (s0, s1)) * (t, t) with packed
// fp32 instructions; each product and sum rounds like the scalar sequence fmaf(a * s, t, c).
__device__ __forceinline__ void scaled_fma2(uint64_t &c, uint32_t a0, uint32_t a1, float s0, float s1, uint64_t t2) {
    asm("{\n\t.reg .b64 aa, ss;\n\t"
        "mov.b64 aa, {%1, %2};\n\t"
        "mov.b64 ss, {%3, %4};\n\t"
        "mul.rn.f32x2 aa, aa, ss;\n\t"
        "fma.rn.f32x2 %0, aa, %5, %0;\n\t}"
        : "+l"(c)
        : "r"(a0), "r"(a1), "f"(s0), "f"(s1), "l"(t2));
}

// Writes one warp's 32 x 128 fp32 accumulators (one row per lane) to C through a padded staging buffer so
// that global stores are 64-byte row segments; rows / columns outside the group or the matrix are skipped.
template <typename OutT>
__device__ __forceinline__ void bw_store_tile(const float (&acc)[128], uint8_t *stg, int lane, int64_t tile_row0,
                                              int64_t c_row_end, int n0, int n_end, const BwParams &p) {
    constexpr int esize = sizeof(OutT);
    constexpr int cols = 64 / esize;  // columns per staged row: 32 (16-bit) or 16 (fp32)
    constexpr int elems16 = 16 / esize;
    uint8_t *my = stg + lane * kBwStagePitch;
    const int sub = lane & 3;
    const int wsw = (lane >> 1) & 3;  // chunk swizzle of this lane's row: conflict-free writes and reads
#pragma unroll
    for (int c = 0; c < 128 / cols; ++c) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if constexpr (esize == 4) {
                *reinterpret_cast<float4 *>(my + 16 * (i ^ wsw)) =
                    make_float4(acc[c * 16 + 4 * i], acc[c * 16 + 4 * i + 1], acc[c * 16 + 4 * i + 2], acc[c * 16 + 4 * i + 3]);
            } else {
                const float *f = &acc[c * 32 + 8 * i];
                *reinterpret_cast<uint4 *>(my + 16 * (i ^ wsw)) =
                    make_uint4(pack2<OutT>(f[0], f[1]), pack2<OutT>(f[2], f[3]), pack2<OutT>(f[4], f[5]), pack2<OutT>(f[6], f[7]));
            }
        }
        __syncwarp();
#pragma unroll 1
        for (int pass = 0; pass < 32; pass += 8) {
            const int rr = pass + (lane >> 2);
            const int64_t grow = tile_row0 + rr;
            const int gcol = n0 + c * cols + sub * elems16;
            if (grow < c_row_end && gcol < n_end) {
                const uint4 val = *reinterpret_cast<const uint4 *>(stg + rr * kBwStagePitch + (sub ^ ((rr >> 1) & 3)) * 16);
                OutT *dst = reinterpret_cast<OutT *>(p.C) + grow * p.ldc + gcol;
                if (p.vec_store_ok && gcol + elems16 <= n_end && p.beta == 0.f) {
                    *reinterpret_cast<uint4 *>(dst) = val;
                } else {
                    const OutT *src = reinterpret_cast<const OutT *>(&val);
                    for (int e = 0; e < elems16 && gcol + e < n_end; ++e) {
                        float nv = static_cast<float>(src[e]);
                        if (p.beta != 0.f) nv += static_cast<float>(dst[e]);
                        dst[e] = static_cast<OutT>(nv);
                    }
                }
            }
        }
        __syncwarp();
    }
}

// Write-out of one warp's 32 x 128 block through bulk tensor stores: the block is converted into 128-byte-swizzled
// boxes of 32 rows x 128 bytes in the warp's staging area, and one lane hands them to the TMA unit, which clips
// rows / columns beyond the matrix.  The warp does not wait for the stores; the staging area is reclaimed at the
// next write-out (bulk_wait_read_all).
template <typename OutT>
__device__ __forceinline__ void bw_store_tile_bulk(const float (&acc)[128], uint8_t *stg, int lane, int64_t tile_row0, int n0,
                                                   int N, const CUtensorMap *tmap_c) {
    constexpr int esize = sizeof(OutT);
    constexpr int box_cols = 128 / esize;        // 64 (16-bit) or 32 (fp32) columns per box
    constexpr int rounds = 128 / (2 * box_cols);  // two boxes fit the staging area: 1 round (16-bit), 2 rounds (fp32)
    uint8_t *my = stg + lane * 128;
#pragma unroll
    for (int rd = 0; rd < rounds; ++rd) {
        if (lane == 0) bulk_wait_read_all();
        __syncwarp();
#pragma unroll
        for (int b = 0; b < 2; ++b) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float *f = &acc[(rd * 2 + b) * box_cols + j * (16 / esize)];
                uint4 v;
                if constexpr (esize == 4) v = make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
                else v = make_uint4(pack2<OutT>(f[0], f[1]), pack2<OutT>(f[2], f[3]), pack2<OutT>(f[4], f[5]), pack2<OutT>(f[6], f[7]));
                *reinterpret_cast<uint4 *>(my + b * 4096 + ((j ^ (lane & 7)) * 16)) = v;
            }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            const uint64_t leave = l2_policy_evict_first();   // the output is not read again by this kernel
#pragma unroll
            for (int b = 0; b < 2; ++b)
                if (n0 + (rd * 2 + b) * box_cols < N)  // boxes that start past the last column are dropped
                    tma_store_2d_hint(tmap_c, stg + b * 4096, (n0 + (rd * 2 + b) * box_cols) * esize, (int) tile_row0, leave);
            bulk_commit_group();
        }
    }
}

// SBM selects how the B scales reach the promotion warps (one kernel per mode keeps each K loop small):
//   SB_TILE   one scale per 128 columns (weights quantised in 128 x 128 blocks): staged with the A scales
//   SB_SLAB   one scale per column, contiguous along the columns: 256-float slabs through shared memory
//   SB_GLOBAL any other per-row layout, read from global memory
enum { SB_TILE = 0, SB_SLAB = 1, SB_GLOBAL = 2 };

template <int SBM, typename OutT>
__global__ void __launch_bounds__(kBwThreads, 1)
    gemm_fp8_blockwise_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
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

    if (threadIdx.x == 0) {
        int acc = 0;
        s_tile_start[0] = 0;
        for (int g = 0; g < G; ++g) {
            const int64_t len = p.koffs ? p.M : (p.offs_write ? (p.offs_write[g + 1] - p.offs_write[g]) : p.M);
            acc += (int) ((len + BLOCK_M - 1) / BLOCK_M) * num_n_blocks;
            s_tile_start[g + 1] = acc;
        }
        *abort_flag = 0;
        for (int s = 0; s < kBwStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&part_full_bar[s], 1);
            mbar_init(&part_empty_bar[s], kBwPromoWarps);
        }
        for (int s = 0; s < kBwSlabRing; ++s) {
            mbar_init(&slab_full_bar[s], 1);
            mbar_init(&scale_full_bar[s], 64);  // one deferred arrival per loader thread
            mbar_init(&scale_empty_bar[s], 1);  // released by the MMA issuer on behalf of the promotion warps
        }
        fence_barrier_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_base_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;

    TileWalk walk{s_tile_start, G, num_n_blocks, 0, p.raster_m};
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
            const uint64_t keep = l2_policy_evict_last();
            for (int t = blockIdx.x; ok && walk.locate(t, gi, m_blk, n_blk); t += gridDim.x) {
                const int64_t a_row0 = (p.koffs ? 0 : (p.offs_read ? p.offs_read[gi] : 0)) + (int64_t) m_blk * BLOCK_M;
                const int64_t b_row0 = (p.koffs ? 0 : (int64_t) gi * p.b_group_rows) + (int64_t) n_blk * BW_BLOCK_N;
                int kb_begin, kb_count;
                k_range(gi, kb_begin, kb_count);
                const int n0 = n_blk * BW_BLOCK_N;
                const int slab_cols = min(BW_BLOCK_N, p.N - n0);
                for (int kb = 0; kb < kb_count; ++kb, ++step) {
                    if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) break;
                    mbar_arrive_expect_tx(&full_bar[stage], kBwABytes + kBwBBytes);
                    const int k0 = (kb_begin + kb) * BLOCK_K;
                    uint8_t *sa = smem_a + stage * kBwABytes, *sb = smem_b + stage * kBwBBytes;
                    if (p.a_mn) tma_load_2d_hint(sa, &tmap_a, &full_bar[stage], (int) a_row0, k0, keep);
                    else tma_load_2d_hint(sa, &tmap_a, &full_bar[stage], k0, (int) a_row0, keep);
                    if (p.b_mn) {
                        // two 128-wide boxes; contraction rows of group g start at g * b_group_kstride
                        const int kr = (int) ((p.koffs ? 0 : (int64_t) gi * p.b_group_kstride) + k0);
                        tma_load_2d_hint(sb, &tmap_b, &full_bar[stage], n0, kr, keep);
                        tma_load_2d_hint(sb + kBwBBytes / 2, &tmap_b, &full_bar[stage], n0 + 128, kr, keep);
                    } else {
                        tma_load_2d_hint(sb, &tmap_b, &full_bar[stage], k0, (int) b_row0, keep);
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
        for (int t = blockIdx.x; ok && walk.locate(t, gi, m_blk, n_blk); t += gridDim.x) {
            const int64_t a_row0 = (p.koffs ? 0 : (p.offs_read ? p.offs_read[gi] : 0)) + (int64_t) m_blk * BLOCK_M;
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
        if (elect_one()) {
            const uint32_t idesc = idesc_f8(p.a_fmt, p.b_fmt, BLOCK_M, BW_BLOCK_N) | ((uint32_t) (p.a_mn != 0) << 15) |
                                   ((uint32_t) (p.b_mn != 0) << 16);
            uint32_t stage = 0, phase = 0, pb = 0, pphase = 0, step = 0;
            for (int t = blockIdx.x; ok && walk.locate(t, gi, m_blk, n_blk); t += gridDim.x) {
                int kb_begin, kb_count;
                k_range(gi, kb_begin, kb_count);
                for (int kb = 0; kb < kb_count; ++kb, ++step) {
                    // The partial sum of this step is only announced once its scales (and B slab) have landed, so the
                    // promotion warps need no barrier of their own for the scale rings.  Operands and scales arrive long before
                    // the partial buffer is handed back; waiting for the buffer last keeps that hand-over short.
                    if (!(ok = mbar_wait(&scale_full_bar[step % kBwSlabRing], (step / kBwSlabRing) & 1u, abort_flag))) break;
                    if constexpr (SBM == SB_SLAB)
                        if (!(ok = mbar_wait(&slab_full_bar[step % kBwSlabRing], (step / kBwSlabRing) & 1u, abort_flag))) break;
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
                        mma_f8(d_tmem, a_desc + k * a_step, b_desc + k * b_step, idesc, k > 0 ? 1u : 0u);
                    tc_commit(&empty_bar[stage]);
                    tc_commit(&part_full_bar[pb]);
                    // the promotion warps are done with step - 2 (its buffer was just reused): its scale slot is free
                    if (step >= 2) mbar_arrive(&scale_empty_bar[(step - 2) % kBwSlabRing]);
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
        for (int t = blockIdx.x; ok && walk.locate(t, gi, m_blk, n_blk); t += gridDim.x) {
            const int64_t c_row_base = p.koffs ? (int64_t) gi * p.M : (p.offs_write ? p.offs_write[gi] : 0);
            const int64_t c_row_end = p.koffs ? c_row_base + p.M : (p.offs_write ? p.offs_write[gi + 1] : p.M);
            const int64_t a_row_base = p.koffs ? 0 : (p.offs_read ? p.offs_read[gi] : 0);
            int kb_begin, kb_count;
            k_range(gi, kb_begin, kb_count);
            const int row_in_tile = q * 32 + lane;
            const int64_t my_c_row = c_row_base + (int64_t) m_blk * BLOCK_M + row_in_tile;
            const int64_t my_a_row = a_row_base + (int64_t) m_blk * BLOCK_M + row_in_tile;
            const bool row_ok = my_c_row < c_row_end;
            const int n0 = n_blk * BW_BLOCK_N + half * 128;
            const int n_end = min(p.N, n0 + 128);
            const float *sb_base = p.sb.base + (int64_t) gi * p.sb.group_stride + (int64_t) kb_begin * p.sb.kb_stride;
            constexpr bool sb_uniform = SBM == SB_TILE;

            __align__(8) float acc[128];
#pragma unroll
            for (int i = 0; i < 128; ++i) acc[i] = 0.f;

            for (int kb = 0; kb < kb_count; ++kb, ++step) {
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
                        uint64_t sc2;
                        asm("mov.b64 %0, {%1, %1};" : "=l"(sc2) : "f"(sc));
#pragma unroll
                        for (int i = 0; i < 16; ++i)   // two accumulators per instruction; each rounds like fmaf(r, sc, acc)
                            asm("{\n\t.reg .b64 rr;\n\tmov.b64 rr, {%1, %2};\n\tfma.rn.f32x2 %0, rr, %3, %0;\n\t}"
                                : "+l"(*reinterpret_cast<uint64_t *>(&acc[c * 32 + 2 * i]))
                                : "r"(r[2 * i]), "r"(r[2 * i + 1]), "l"(sc2));
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
                if (lane == 0) mbar_arrive(&part_empty_bar[pb]);
                add_chunk(2, r0);
                add_chunk(3, r1);
                if (++pb == 2) { pb = 0; pphase ^= 1; }
            }
            if (!ok) break;

            // ---- write-out through the per-warp staging buffer
            const int64_t tile_row0 = c_row_base + (int64_t) m_blk * BLOCK_M + q * 32;
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
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

#include "gemm_fp8_blockwise_pair.cuh"

// Raises the dynamic shared-memory limit of one kernel instantiation (on every call: it is a cheap host-side
// attribute write and keeps the limit right on every device of the process) and launches it.
template <typename Kernel>
static int bw_launch(Kernel kernel, int grid, cudaStream_t stream, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc,
                     const BwParams &p) {
    PT_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwSmemBytes));
    kernel<<<grid, kBwThreads, kBwSmemBytes, stream>>>(ta, tb, tc, p);
    PT_LAUNCH_OK();
    return PT_OK;
}

// CTA-pair launch: grid = 2 x min(tiles, co-resident clusters of this device).  PT_ERR_CUDA (clusters cannot be
// launched here) sends the caller back to the single-CTA kernel.
template <typename Kernel>
static int bw_launch_pair(Kernel kernel, int64_t tiles, cudaStream_t stream, const CUtensorMap &ta, const CUtensorMap &tb,
                          const CUtensorMap &tc, const BwParams &p) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwSmemBytes) != cudaSuccess) {
        cudaGetLastError();
        return PT_ERR_CUDA;
    }
    static int max_clusters_dev[64] = {};  // per instantiation and device
    int &max_clusters = max_clusters_dev[current_device_slot()];
    if (max_clusters == 0) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(2 * (unsigned) sm_count());
        cfg.blockDim = dim3(kBwThreads);
        cfg.dynamicSmemBytes = kBwSmemBytes;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, (const void *) kernel, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            return PT_ERR_CUDA;
        }
        max_clusters = n;
    }
    const int pairs = (int) std::min<int64_t>(tiles, max_clusters);
    if (pairs <= 0) return PT_OK;
    kernel<<<2 * pairs, kBwThreads, kBwSmemBytes, stream>>>(ta, tb, tc, p);
    if (cudaGetLastError() != cudaSuccess) return PT_ERR_CUDA;
    return PT_OK;
}

// The CTA-pair form is correct but slower than the single-CTA kernel (B200, 8192 x 14336 x 4096: 1730-1800 against
// 2157-2162 TFLOP/s; 8192^3: 1600-1640 against 2020-2070): it halves the operand traffic per SM, but the promotion warps set
// the pace in both forms and the pair adds a cross-CTA hand-over of the partial-sum buffer per K step.  It therefore runs only when
// PT_BW_GEMM_PAIR=1 (read per call); PT_GEMM_PAIR=0 switches it off together with the other pair kernels.
static bool bw_pair_enabled() {
    const char *on = getenv("PT_BW_GEMM_PAIR");
    const char *all = getenv("PT_GEMM_PAIR");
    return on && on[0] == '1' && !(all && all[0] == '0');
}

}  // namespace ptb

using namespace ptb;

extern "C" {

int pt_grouped_gemm_fp8_blockwise(const void *a, int a_fmt, int a_mn, int64_t a_mem_rows, int64_t a_mem_cols, const float *sa,
                                  int sa_shift, int64_t sa_row_stride, int64_t sa_kb_stride, const void *b, int b_fmt, int b_mn,
                                  int64_t b_mem_rows, int64_t b_mem_cols, const float *sb, int sb_shift, int64_t sb_row_stride,
                                  int64_t sb_kb_stride, int64_t sb_group_stride, void *c, int c_dtype, int64_t c_rows, int64_t N,
                                  int64_t K, const int64_t *group_offs_read, const int64_t *group_offs_write,
                                  const int64_t *k_offs, int G, float beta, int max_ctas, int *status, void *stream) {
    PT_REQUIRE(c_rows >= 0 && N >= 0 && K >= 0 && G >= 1 && G <= kMaxGroups, "blockwise GEMM: bad shape");
    PT_REQUIRE((a_fmt == PT_E4M3 || a_fmt == PT_E5M2) && (b_fmt == PT_E4M3 || b_fmt == PT_E5M2), "blockwise GEMM: operands must be e4m3 / e5m2");
    PT_REQUIRE(c_dtype == PT_BF16 || c_dtype == PT_F16 || c_dtype == PT_F32, "blockwise GEMM: bad output dtype");
    PT_REQUIRE((sa_shift == 0 || sa_shift == 7) && (sb_shift == 0 || sb_shift == 7), "blockwise GEMM: scale granularity must be 1 or 128 rows");
    PT_REQUIRE(beta == 0.f || beta == 1.f, "blockwise GEMM: beta must be 0 or 1");
    PT_REQUIRE(!k_offs || (a_mn && b_mn && !group_offs_read && !group_offs_write),
               "blockwise GEMM: the variable-K form takes MN-major operands and no row offsets");
    if (c_rows == 0 || N == 0) return PT_OK;
    PT_REQUIRE(k_offs || (K > 0 && (K % 16 == 0 || (a_mn && b_mn))), "blockwise GEMM: K must be a positive multiple of 16 (got %lld)", (long long) K);
    PT_REQUIRE(a && b && c && sa && sb, "blockwise GEMM: null pointer");
    PT_REQUIRE(a_mem_cols % 16 == 0 && b_mem_cols % 16 == 0, "blockwise GEMM: operand row pitch must be a multiple of 16 bytes");
    PT_REQUIRE(N < (1 << 30) && K < (1 << 30) && a_mem_rows < (1ll << 31) && b_mem_rows < (1ll << 31) && a_mem_cols < (1ll << 31) &&
                   b_mem_cols < (1ll << 31), "blockwise GEMM: extent exceeds 32-bit tile coordinates");
    PT_REQUIRE(!(b_mn && G > 1 && !k_offs) || K % BLOCK_K == 0,
               "blockwise GEMM: an MN-major grouped B needs a contraction length that is a multiple of 128");
    BwParams p{};
    p.M = c_rows; p.N = (int) N; p.K = (int) K; p.C = c; p.ldc = N; p.c_dtype = c_dtype; p.beta = beta;
    const int esize = c_dtype == PT_F32 ? 4 : 2;
    p.vec_store_ok = aligned(c, 16) && (N * esize) % 16 == 0;
    p.sa = ScaleDesc{sa, sa_shift, sa_row_stride, sa_kb_stride, 0};
    p.sb = ScaleDesc{sb, sb_shift, sb_row_stride, sb_kb_stride, sb_group_stride};
    p.a_fmt = a_fmt; p.b_fmt = b_fmt;
    p.offs_write = group_offs_write; p.offs_read = group_offs_read ? group_offs_read : group_offs_write;
    p.G = G; p.b_group_rows = N; p.a_rows_total = a_mn ? a_mem_cols : a_mem_rows;
    if (!group_offs_read) p.a_rows_total = std::min<int64_t>(p.a_rows_total, c_rows);  // rows that have scales
    p.status = status;
    p.a_mn = a_mn; p.b_mn = b_mn; p.koffs = k_offs; p.b_group_kstride = K;
    p.sb_slab = sb_shift == 0 && sb_row_stride == 1 && sb_kb_stride % 4 == 0 && sb_group_stride % 4 == 0 && N % 4 == 0 && aligned(sb, 16);
    p.raster_m = raster_rows(a_mn ? a_mem_cols : a_mem_rows, a_mn ? a_mem_rows : a_mem_cols);
    CUtensorMap ta, tb;
    int rc;
    // K-major: box = 128 contraction bytes x tile rows; MN-major: box = 128 row indices x 128 contraction rows
    if ((rc = make_tmap_bytes(&ta, a, a_mem_rows, a_mem_cols, a_mem_cols, a_mn ? BLOCK_K : BLOCK_M)) != PT_OK) return rc;
    if ((rc = make_tmap_bytes(&tb, b, b_mem_rows, b_mem_cols, b_mem_cols, b_mn ? BLOCK_K : BW_BLOCK_N)) != PT_OK) return rc;
    const int64_t m_blocks = k_offs ? (int64_t) G * ceil_div(c_rows, BLOCK_M) : ceil_div(c_rows, BLOCK_M) + (group_offs_write ? G : 0);
    const int64_t tiles = m_blocks * ceil_div(N, BW_BLOCK_N);
    int grid = (int) std::min<int64_t>(tiles, sm_count());
    if (max_ctas > 0) grid = std::min(grid, max_ctas);
    // C as a byte tensor of 128-byte x 32-row boxes for the bulk-store write-out
    CUtensorMap tc{};
    p.c_rows_total = k_offs ? (int64_t) G * c_rows : c_rows;
    p.c_tma = p.vec_store_ok && beta == 0.f && N * esize < (1ll << 31) && p.c_rows_total < (1ll << 31);
    if (p.c_tma && (rc = make_tmap_bytes(&tc, c, p.c_rows_total, N * esize, N * esize, 32)) != PT_OK) return rc;
    const int sbm = sb_shift == 7 ? SB_TILE : (p.sb_slab ? SB_SLAB : SB_GLOBAL);
    // Large problems run on CTA pairs (256-row tiles).  Group lengths live on the device: the average rows per group
    // decide (short groups would waste up to 255 rows of work each).
    {
        const int64_t rows_per_group = k_offs ? c_rows : c_rows / G;
        const int64_t out_elems = (k_offs ? (int64_t) G : 1) * c_rows * N;
        if (max_ctas <= 0 && sbm != SB_GLOBAL && bw_pair_enabled() && rows_per_group >= 1024 && N >= 512 &&
            out_elems >= (int64_t) 4096 * 4096) {
            CUtensorMap tb_pair;
            if ((rc = make_tmap_bytes(&tb_pair, b, b_mem_rows, b_mem_cols, b_mem_cols, b_mn ? BLOCK_K : BW_BLOCK_N / 2)) != PT_OK) return rc;
            const int64_t m_tiles = k_offs ? (int64_t) G * ceil_div(c_rows, 2 * BLOCK_M) : ceil_div(c_rows, 2 * BLOCK_M) + (group_offs_write ? G : 0);
            const int64_t pair_tiles = m_tiles * ceil_div(N, BW_BLOCK_N);
            BwParams pp = p;
            int prc = PT_ERR_CUDA;
#define PT_BWP_CASE(SBM_, T_) prc = bw_launch_pair(gemm_fp8_blockwise_pair_kernel<SBM_, T_>, pair_tiles, (cudaStream_t) stream, ta, tb_pair, tc, pp)
#define PT_BWP_DTYPE(SBM_)                                                                                           \
            do {                                                                                                     \
                if (c_dtype == PT_F32) PT_BWP_CASE(SBM_, float);                                                     \
                else if (c_dtype == PT_BF16) PT_BWP_CASE(SBM_, __nv_bfloat16);                                       \
                else PT_BWP_CASE(SBM_, __half);                                                                      \
            } while (0)
            if (sbm == SB_TILE) PT_BWP_DTYPE(SB_TILE);
            else PT_BWP_DTYPE(SB_SLAB);
#undef PT_BWP_DTYPE
#undef PT_BWP_CASE
            if (prc != PT_ERR_CUDA) return prc;  // a device that cannot launch clusters falls through to single CTAs
        }
    }
#define PT_BW_CASE(SBM_, T_)                                                                                         \
    return bw_launch(gemm_fp8_blockwise_kernel<SBM_, T_>, grid, (cudaStream_t) stream, ta, tb, tc, p)
#define PT_BW_DTYPE(SBM_)                                                                                            \
    do {                                                                                                             \
        if (c_dtype == PT_F32) PT_BW_CASE(SBM_, float);                                                              \
        if (c_dtype == PT_BF16) PT_BW_CASE(SBM_, __nv_bfloat16);                                                     \
        PT_BW_CASE(SBM_, __half);                                                                                    \
    } while (0)
    if (sbm == SB_TILE) PT_BW_DTYPE(SB_TILE);
    if (sbm == SB_SLAB) PT_BW_DTYPE(SB_SLAB);
    PT_BW_DTYPE(SB_GLOBAL);
#undef PT_BW_DTYPE
#undef PT_BW_CASE
}

}  // extern "C"
