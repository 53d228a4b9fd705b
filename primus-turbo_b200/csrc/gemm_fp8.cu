// Dense and grouped FP8 / MXFP8 GEMM for sm_100a:  C[m, n] = sum_k A[m, k] * B[n, k]  (both operands
// K-major, "NT"), fp32 accumulation in tensor memory.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer: A (128 x 128 B) and B (BLOCK_N x 128 B) tiles, 128-byte swizzle, into a ring
//   warp 1      MMA issuer (one elected lane): tcgen05.mma kind::f8f6f4 or kind::mxf8f6f4.block_scale;
//               owns the TMEM allocation
//   warps 2-5   epilogue: TMEM -> registers -> (scales) -> staging in shared memory -> coalesced global stores
// MX scales: the quantizers emit raw row-major ue8m0 bytes [rows, K/32]; a small pre-pass (sf_retile_kernel)
// re-tiles them per 128-row block and 128-K step into the 32 x 16-byte block layout tcgen05.cp expects, so the
// producer can fetch each block with one bulk copy next to the operand tiles (gathering them with ordinary loads
// inside the GEMM cost 20 % of its throughput).
// The accumulator is double buffered in TMEM when 2 * BLOCK_N (+ scale columns) fits in 512 columns, so the
// epilogue of tile i overlaps the main loop of tile i + 1.
//
// Scaling modes (reference semantics: primus_turbo/triton/gemm/gemm_fp8_kernel.py:167-169,231,447-565;
// MX: hardware block scaling as in csrc/pytorch/gemm/hipblaslt_gemm.cpp:127-135):
//   TENSORWISE   C = acc * (sa[0] * sb[0])
//   ROWWISE      C = acc * sa[m] * sb[n]
//   MX_BLOCKWISE C = sum over 32-element K blocks of (a * 2^(sfa-127)) * (b * 2^(sfb-127))
// Grouped form: rows of A / C are split into G groups (group g uses B[g]); tiles never cross a group.
#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "gemm_common.cuh"

namespace ptb {
using namespace sm100;

constexpr int kNumEpiWarps = 4;
constexpr int kGemmThreads = 32 * (2 + kNumEpiWarps);
constexpr int kEpiWarp0 = 2;
constexpr int kStagePitchMax = 128;  // staging row pitch (bytes) of the epilogue, fp32 worst case

enum GemmMode { GEMM_TENSOR = 0, GEMM_ROW = 1, GEMM_MX = 3, GEMM_MXF4 = 4, GEMM_HP = 5 };  // HP: fp16 / bf16 operands, no scales
constexpr bool mode_is_mx(int m) { return m == GEMM_MX || m == GEMM_MXF4; }

struct GemmParams {
    int64_t M;             // rows of A / C (all groups)
    int N, K;              // K in elements, contraction length the tensor maps cover
    void *C;
    int64_t ldc;           // elements
    int c_dtype;
    int vec_store_ok;
    float beta;            // 0 or 1 (C += ...)
    const float *sa, *sb;  // fp32 scales (tensorwise / rowwise)
    const uint8_t *sfa_tiled, *sfb_tiled;  // MX scales re-tiled by sf_retile_kernel: 512-byte blocks [row block][K step]
    int a_fmt, b_fmt;      // 0 = e4m3, 1 = e5m2
    // grouping: null offsets = one group covering [0, M)
    const int64_t *offs_read;   // [G+1] first A row of each group (layout A was written in)
    const int64_t *offs_write;  // [G+1] first C row of each group; group length = difference
    int G;
    int64_t b_group_rows;       // rows between consecutive B[g] (N for [G, N, K])
    const int64_t *koffs;       // variable-K form: contraction range [koffs[g], koffs[g+1]) of group g (multiples of 128);
                                // every group then yields a full [M, N] block of C (C is [G, M, N]), A and B are shared
    int *status;                // device int: set to a PT_ERR_* code on a bounded-wait expiry
    int raster_m;               // row blocks per raster band
    int64_t sfb_line0;          // CTA-pair MX kernel: first 128-byte line of the re-tiled B scales in the scale buffer
    int a_mn, b_mn;             // tensorwise / rowwise, one group: the operand is stored [contraction, rows] (MN-major) and read in
                                // place: 128-byte x 128-row boxes, described to the tensor core as in gemm_fp8_blockwise.cu
};

// F4: packed e2m1 operands.  A 128-byte stage row then holds 256 elements = two 128-element scale blocks, so every
// scale quantity per stage doubles (kSfPerStage) and one tcgen05.mma consumes 64 elements with two scales per row.
template <int BLOCK_N, bool MX, bool F4 = false> struct GemmCfg {
    static constexpr int kSfbBlocks = (BLOCK_N + 127) / 128;
    static constexpr int kSfPerStage = F4 ? 2 : 1;
    static constexpr int kSfColsHalf = 4 + 4 * kSfbBlocks;          // SFA block + SFB blocks of one 128-element scale block
    static constexpr int kSfColsOne = kSfColsHalf * kSfPerStage;    // ... of one stage
    static constexpr int kSfCols = MX ? (F4 ? 1 : 2) * kSfColsOne : 0;  // fp8: double buffered (it fits); fp4: single
    static constexpr int kAccStages = (2 * BLOCK_N + kSfCols <= 512) ? 2 : 1;
    static constexpr int kTmemColsNeeded = kAccStages * BLOCK_N + kSfCols;
    static constexpr int kTmemCols = kTmemColsNeeded <= 32 ? 32 : kTmemColsNeeded <= 64 ? 64 : kTmemColsNeeded <= 128 ? 128
                                     : kTmemColsNeeded <= 256 ? 256 : 512;
    static constexpr int kABytes = BLOCK_M * BLOCK_K;
    static constexpr int kBBytes = BLOCK_N * BLOCK_K;
    static constexpr int kSfBytes = MX ? 512 * (1 + kSfbBlocks) * kSfPerStage : 0;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfBytes;
    static constexpr int kEpiBytes = kNumEpiWarps * 32 * kStagePitchMax;
    static constexpr int kBarBytes = 1024;
    static constexpr int kSmemBudget = 227 * 1024 - 1024 /* alignment slack */ - 4608 /* static shared: tile table */;
    static constexpr int kStages = std::min(8, (kSmemBudget - kEpiBytes - kBarBytes) / kStageBytes);
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarBytes + 1024;
    static_assert(kStages >= 3, "not enough shared memory for a 3-stage ring");
    static_assert(BLOCK_N % 16 == 0 && BLOCK_N >= 16 && BLOCK_N <= 256, "invalid UMMA N");
    static_assert(kBBytes % 1024 == 0, "B stage must keep 1024-byte alignment");
};


// ------------------------------------------------------------------------------------------------ scale re-tiling
// Raw ue8m0 scales [rows, K/32] -> 512-byte blocks dst[(rb * num_kb + kb) * 512 + (r % 32) * 16 + (r / 32) * 4 + i],
// r = row inside row block rb, i = which 32-wide slice of K step kb.  Row blocks follow the GEMM's tiles:
//   A side (is_b == 0): group by group, block m of group g starts at offs_read[g] + 128 m;
//   B side (is_b == 1): tile (g, n) has `sfb_blocks` blocks starting at g * b_group_rows + n * block_n + 128 j.
struct RetileArgs {
    const uint8_t *src;
    uint8_t *dst;
    int64_t src_rows, sf_ld;  // rows of src, bytes per row (K / 32)
    int num_kb, is_b;         // num_kb: 512-byte blocks to produce per row block (those past sf_ld / 4 are zero)
    const int64_t *offs_read, *offs_write;
    int G;
    int64_t M;
    int block_n, sfb_blocks, num_n_blocks;
    int64_t b_group_rows;
    int64_t num_row_blocks;  // upper bound
};

// One launch re-tiles both operands: blocks [0, blocks_a) work on the A side, the rest on the B side.
__global__ void __launch_bounds__(128) sf_retile_kernel(RetileArgs args_a, RetileArgs args_b, int blocks_a) {
    __shared__ uint32_t s_words[128][33];
    __shared__ int s_start[kMaxGroups + 1];
    const bool side_b = (int) blockIdx.x >= blocks_a;
    const RetileArgs &a = side_b ? args_b : args_a;
    const int block_x = side_b ? (int) blockIdx.x - blocks_a : (int) blockIdx.x;
    const int grid_x = side_b ? (int) gridDim.x - blocks_a : blocks_a;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    grid_dep_wait();    // the scales come from the quantizer launched just before
    grid_dep_launch();  // the GEMM that follows may set up its barriers and TMEM meanwhile
    if (!a.is_b) {
        if (tid == 0) {
            int acc = 0;
            s_start[0] = 0;
            for (int g = 0; g < a.G; ++g) {
                const int64_t len = a.offs_write ? (a.offs_write[g + 1] - a.offs_write[g]) : a.M;
                acc += (int) ((len + BLOCK_M - 1) / BLOCK_M);
                s_start[g + 1] = acc;
            }
        }
        __syncthreads();
    }
    const int kb0 = blockIdx.y * 32;
    const int nkb = min(32, a.num_kb - kb0);
    int g = 0;
    for (int64_t rb = block_x; rb < a.num_row_blocks; rb += grid_x) {
        int64_t row_start;
        int rows_in_block = 128;
        if (a.is_b) {
            const int64_t tile = rb / a.sfb_blocks;
            const int j = (int) (rb % a.sfb_blocks);
            const int64_t gg = tile / a.num_n_blocks, n_blk = tile % a.num_n_blocks;
            row_start = gg * a.b_group_rows + n_blk * a.block_n + 128 * j;
            rows_in_block = min(128, a.block_n - 128 * j);
        } else {
            if (rb >= s_start[a.G]) break;
            while (rb >= s_start[g + 1]) ++g;
            row_start = (a.offs_read ? a.offs_read[g] : 0) + (rb - s_start[g]) * 128;
        }
        // coalesced read: one warp per row, lane = K step
        for (int r = warp; r < 128; r += 4) {
            const int64_t row = row_start + r;
            uint32_t w = 0;
            if (r < rows_in_block && row < a.src_rows && lane < nkb && (kb0 + lane) * 4 < a.sf_ld)
                w = __ldcg(reinterpret_cast<const uint32_t *>(a.src + row * a.sf_ld) + kb0 + lane);   // written by the kernel before: not the read-only path
            s_words[r][lane] = w;
        }
        __syncthreads();
        // each warp writes whole 512-byte blocks: lane l carries rows l, l+32, l+64, l+96
        for (int kb = warp; kb < nkb; kb += 4) {
            const uint4 v = make_uint4(s_words[lane][kb], s_words[lane + 32][kb], s_words[lane + 64][kb], s_words[lane + 96][kb]);
            *reinterpret_cast<uint4 *>(a.dst + (rb * a.num_kb + kb0 + kb) * 512 + lane * 16) = v;
        }
        __syncthreads();
    }
}

// Write-out of one epilogue warp's 32 x BLOCK_N block of a tile: TMEM -> registers -> scales -> XOR-swizzled staging
// rows in shared memory -> coalesced row-segment stores, masked at the end of the group / matrix.  `release` hands the
// accumulator buffer back to the MMA issuer as soon as the warp's last chunk is in registers.  The warp handles the
// 32-column chunks [c_begin, c_end) of the tile (all of them, or a share when several warps split a lane quarter).
template <int BLOCK_N, int MODE, typename Release>
__device__ __forceinline__ void epilogue_store_block(const GemmParams &p, uint32_t taddr, bool have_acc, int64_t tile_row0,
                                                     int64_t c_row_end, int n0, int gi, uint8_t *stg, int lane, int c_begin,
                                                     int c_end, Release release) {
    const int esize = p.c_dtype == PT_F32 ? 4 : 2;
    const int pitch = 32 * esize;  // unpadded rows; 16-byte chunks are XOR-swizzled by row so that neither the
                                   // row-per-lane writes nor the row-segment reads conflict on banks
    const int lanes_per_row = (32 * esize) / 16;      // 4 (16-bit) or 8 (fp32)
    const int rows_per_pass = 32 / lanes_per_row;     // 8 or 4
    float row_scale = 1.f;
    if (MODE == GEMM_TENSOR) row_scale = __ldcg(p.sa) * __ldcg(p.sb);   // scales may come from the kernel launched just before: no read-only path
    if (MODE == GEMM_ROW) row_scale = (tile_row0 + lane < c_row_end) ? __ldcg(p.sa + tile_row0 + lane) : 0.f;
    const int n_end = min(p.N, n0 + BLOCK_N);  // a last partial chunk reads past the tile; masked below
#pragma unroll 1
    for (int c = c_begin; c < c_end; ++c) {
        uint32_t r[32];
        if (have_acc) {
            tmem_ld32(taddr + c * 32, r);
            tmem_ld_wait();
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (have_acc && c == c_end - 1) {
            // whole accumulator is in registers / staged: hand the TMEM buffer back to the MMA warp
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) release();
        }
        const int col0 = n0 + c * 32;
        float f[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]) * row_scale;
        if (MODE == GEMM_ROW) {
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] *= (col0 + i < n_end) ? __ldcg(p.sb + (int64_t) gi * p.b_group_rows + col0 + i) : 0.f;
        }
        // stage this thread's row
        uint8_t *my = stg + lane * pitch;
        const int wsw = esize == 4 ? (lane & 7) : ((lane >> 1) & 3);  // chunk swizzle of this lane's row
        if (esize == 4) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                *reinterpret_cast<float4 *>(my + 16 * (i ^ wsw)) = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
        } else if (p.c_dtype == PT_BF16) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                *reinterpret_cast<uint4 *>(my + 16 * (i ^ wsw)) =
                    make_uint4(pack2<__nv_bfloat16>(f[8 * i], f[8 * i + 1]), pack2<__nv_bfloat16>(f[8 * i + 2], f[8 * i + 3]),
                               pack2<__nv_bfloat16>(f[8 * i + 4], f[8 * i + 5]), pack2<__nv_bfloat16>(f[8 * i + 6], f[8 * i + 7]));
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                *reinterpret_cast<uint4 *>(my + 16 * (i ^ wsw)) =
                    make_uint4(pack2<__half>(f[8 * i], f[8 * i + 1]), pack2<__half>(f[8 * i + 2], f[8 * i + 3]),
                               pack2<__half>(f[8 * i + 4], f[8 * i + 5]), pack2<__half>(f[8 * i + 6], f[8 * i + 7]));
        }
        __syncwarp();
        // coalesced write-out: lanes_per_row lanes cover one staged row
        const int sub = lane % lanes_per_row;
        const int elems16 = 16 / esize;
#pragma unroll 1
        for (int pass = 0; pass < 32; pass += rows_per_pass) {
            const int rr = pass + lane / lanes_per_row;
            const int64_t grow = tile_row0 + rr;
            const int gcol = col0 + sub * elems16;
            if (grow < c_row_end && gcol < n_end) {
                const int rsw = esize == 4 ? (rr & 7) : ((rr >> 1) & 3);
                const uint4 val = *reinterpret_cast<const uint4 *>(stg + rr * pitch + (sub ^ rsw) * 16);
                uint8_t *dst = reinterpret_cast<uint8_t *>(p.C) + (grow * p.ldc + gcol) * esize;
                if (p.vec_store_ok && gcol + elems16 <= n_end && p.beta == 0.f) {
                    // written once and not read by this kernel: streaming store, so that C leaves L2 before the operand
                    // panels that other CTAs are about to re-read
                    __stcs(reinterpret_cast<uint4 *>(dst), val);
                } else {
                    const uint8_t *src = reinterpret_cast<const uint8_t *>(&val);
                    for (int e = 0; e < elems16 && gcol + e < n_end; ++e) {
                        if (esize == 4) {
                            float nv = reinterpret_cast<const float *>(src)[e];
                            if (p.beta != 0.f) nv += reinterpret_cast<float *>(dst)[e];
                            reinterpret_cast<float *>(dst)[e] = nv;
                        } else if (p.c_dtype == PT_BF16) {
                            __nv_bfloat16 nv = reinterpret_cast<const __nv_bfloat16 *>(src)[e];
                            if (p.beta != 0.f) nv = __float2bfloat16_rn(__bfloat162float(nv) + __bfloat162float(reinterpret_cast<__nv_bfloat16 *>(dst)[e]));
                            reinterpret_cast<__nv_bfloat16 *>(dst)[e] = nv;
                        } else {
                            __half nv = reinterpret_cast<const __half *>(src)[e];
                            if (p.beta != 0.f) nv = __float2half_rn(__half2float(nv) + __half2float(reinterpret_cast<__half *>(dst)[e]));
                            reinterpret_cast<__half *>(dst)[e] = nv;
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
}

template <int BLOCK_N, int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmParams p) {
    constexpr bool MX = mode_is_mx(MODE);
    constexpr bool F4 = MODE == GEMM_MXF4;
    using Cfg = GemmCfg<BLOCK_N, MX, F4>;
    constexpr int kSfP = Cfg::kSfPerStage;
    constexpr int kStages = Cfg::kStages;
    constexpr int kAccStages = Cfg::kAccStages;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem_a + kStages * Cfg::kABytes;
    uint8_t *smem_sf = smem_b + kStages * Cfg::kBBytes;
    uint8_t *smem_epi = smem_sf + kStages * Cfg::kSfBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_epi + Cfg::kEpiBytes);
    uint64_t *full_bar = bars;                        // [kStages]
    uint64_t *empty_bar = bars + kStages;             // [kStages]
    uint64_t *tmem_full_bar = bars + 2 * kStages;     // [kAccStages]
    uint64_t *tmem_empty_bar = tmem_full_bar + kAccStages;
    uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(tmem_empty_bar + kAccStages);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_base_slot + 1);
    __shared__ int s_tile_start[kMaxGroups + 1];

    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int num_n_blocks = (p.N + BLOCK_N - 1) / BLOCK_N;
    const int num_k_blocks = (p.K + BLOCK_K - 1) / BLOCK_K;
    const int G = p.G;

    // ---- prologue: barriers, TMEM, then (after the earlier kernels of the stream are done) the tile table
    grid_dep_wait();
    if (threadIdx.x == 0) {
        int acc = 0;
        s_tile_start[0] = 0;
        for (int g = 0; g < G; ++g) {
            const int64_t len = (p.offs_write && !p.koffs) ? (p.offs_write[g + 1] - p.offs_write[g]) : p.M;
            acc += (int) ((len + BLOCK_M - 1) / BLOCK_M) * num_n_blocks;
            s_tile_start[g + 1] = acc;
        }
        *abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < kAccStages; ++s) {
            mbar_init(&tmem_full_bar[s], 1);
            mbar_init(&tmem_empty_bar[s], kNumEpiWarps);
        }
        fence_barrier_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_base_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    grid_dep_launch();
    const uint32_t tmem_base = *tmem_base_slot;
    const uint32_t tmem_sfa = tmem_base + kAccStages * BLOCK_N;
    const uint32_t tmem_sfb = tmem_sfa + 4;

    TileWalk walk{s_tile_start, G, num_n_blocks, 0, p.raster_m};
    int gi, m_blk, n_blk;
    bool ok = true;
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
        // ================================================================ TMA producer
        if (elect_one()) {
            uint32_t stage = 0, phase = 0;
            const uint64_t keep = l2_policy_evict_last();
            for (int t = blockIdx.x; ok && walk.locate(t, gi, m_blk, n_blk); t += gridDim.x) {
                const int64_t a_row0 = ((p.offs_read && !p.koffs) ? p.offs_read[gi] : 0) + (int64_t) m_blk * BLOCK_M;
                const int64_t b_row0 = (p.koffs ? 0 : (int64_t) gi * p.b_group_rows) + (int64_t) n_blk * BLOCK_N;
                int kb_begin, kb_count;
                k_range(gi, kb_begin, kb_count);
                // scale blocks of this tile: A row block = running count of 128-row blocks over the groups
                const uint8_t *sfa_blk = nullptr, *sfb_blk = nullptr;
                if constexpr (MX) {
                    const int64_t a_rb = p.koffs ? m_blk : s_tile_start[gi] / num_n_blocks + m_blk;
                    const int64_t b_rb = ((p.koffs ? 0 : (int64_t) gi * num_n_blocks) + n_blk) * Cfg::kSfbBlocks;
                    sfa_blk = p.sfa_tiled + (a_rb * num_k_blocks + kb_begin) * kSfP * 512;
                    sfb_blk = p.sfb_tiled + (b_rb * num_k_blocks + kb_begin) * kSfP * 512;
                }
                for (int kb = 0; kb < kb_count; ++kb) {
                    if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) break;
                    mbar_arrive_expect_tx(&full_bar[stage], Cfg::kABytes + Cfg::kBBytes + Cfg::kSfBytes);
                    const int k0 = (kb_begin + kb) * BLOCK_K;
                    if (!MX && p.a_mn) tma_load_2d_hint(smem_a + stage * Cfg::kABytes, &tmap_a, &full_bar[stage], (int) a_row0, k0, keep);
                    else tma_load_2d_hint(smem_a + stage * Cfg::kABytes, &tmap_a, &full_bar[stage], k0, (int) a_row0, keep);
                    if (!MX && p.b_mn) {   // one 128-wide box per 128 columns of the tile, 16 KiB apart
#pragma unroll
                        for (int j = 0; j < (BLOCK_N + 127) / 128; ++j)
                            tma_load_2d_hint(smem_b + stage * Cfg::kBBytes + j * 16384, &tmap_b, &full_bar[stage], (int) b_row0 + 128 * j, k0, keep);
                    } else {
                        tma_load_2d_hint(smem_b + stage * Cfg::kBBytes, &tmap_b, &full_bar[stage], k0, (int) b_row0, keep);
                    }
                    if constexpr (MX) {
                        // per stage: kSfP consecutive 512-byte blocks of A (one copy), and of each 128-row block of B
                        uint8_t *sf = smem_sf + stage * Cfg::kSfBytes;
                        bulk_load(sf, sfa_blk + (int64_t) kb * kSfP * 512, kSfP * 512, &full_bar[stage]);
#pragma unroll
                        for (int j = 0; j < Cfg::kSfbBlocks; ++j)
                            bulk_load(sf + kSfP * 512 * (1 + j), sfb_blk + ((int64_t) j * num_k_blocks + kb) * kSfP * 512, kSfP * 512,
                                      &full_bar[stage]);
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ================================================================ MMA issuer
        if (elect_one()) {
            constexpr uint32_t kIdescPlainShape = 0;
            (void) kIdescPlainShape;
            const bool a_mn = !MX && MODE != GEMM_HP && p.a_mn, b_mn = !MX && MODE != GEMM_HP && p.b_mn;
            const uint32_t idesc = F4 ? idesc_block_scaled(1, 1, BLOCK_M, BLOCK_N)   // kind::mxf4: format code 1 = e2m1
                                   : MX ? idesc_block_scaled(p.a_fmt, p.b_fmt, BLOCK_M, BLOCK_N)
                                        : (idesc_f8(p.a_fmt, p.b_fmt, BLOCK_M, BLOCK_N) | ((uint32_t) a_mn << 15) | ((uint32_t) b_mn << 16));
            // one instruction consumes 32 contraction indices: 32 bytes along a K-major row, or 32 rows of 128 bytes of an
            // MN-major tile
            const uint64_t a_kstep = a_mn ? (uint64_t) ((UMMA_K * 128) >> 4) : (uint64_t) (UMMA_K >> 4);
            const uint64_t b_kstep = b_mn ? (uint64_t) ((UMMA_K * 128) >> 4) : (uint64_t) (UMMA_K >> 4);
            uint32_t stage = 0, phase = 0, acc_stage = 0, acc_phase = 0, sf_buf = 0;
            for (int t = blockIdx.x; ok && walk.locate(t, gi, m_blk, n_blk); t += gridDim.x) {
                int kb_begin, kb_count;
                k_range(gi, kb_begin, kb_count);
                if (kb_count == 0) continue;  // empty contraction range: the epilogue writes zeros on its own
                if (!(ok = mbar_wait(&tmem_empty_bar[acc_stage], acc_phase ^ 1, abort_flag))) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc_stage * BLOCK_N;
                for (int kb = 0; kb < kb_count; ++kb) {
                    if (!(ok = mbar_wait(&full_bar[stage], phase, abort_flag))) break;
                    tc_fence_after_sync();
                    const uint32_t sfa_cur = tmem_sfa + sf_buf * Cfg::kSfColsOne;
                    const uint32_t sfb_cur = tmem_sfb + sf_buf * Cfg::kSfColsOne;
                    if constexpr (MX) {
                        // shared memory per stage: [A: kSfP blocks][B block 0: kSfP blocks][B block 1: ...];
                        // TMEM per stage: for each scale block h: [A 4 cols][B 4 cols per 128 rows]
                        const uint32_t sf_addr = smem_u32(smem_sf + stage * Cfg::kSfBytes);
#pragma unroll
                        for (int h = 0; h < kSfP; ++h) {
                            tc_cp_sf(sfa_cur + h * Cfg::kSfColsHalf, smem_desc_sf(sf_addr + 512 * h));
#pragma unroll
                            for (int j = 0; j < Cfg::kSfbBlocks; ++j)
                                tc_cp_sf(sfb_cur + h * Cfg::kSfColsHalf + 4 * j, smem_desc_sf(sf_addr + kSfP * 512 * (1 + j) + 512 * h));
                        }
                        if constexpr (!F4) sf_buf ^= 1;
                    }
                    const uint32_t a_addr = smem_u32(smem_a + stage * Cfg::kABytes), b_addr = smem_u32(smem_b + stage * Cfg::kBBytes);
                    const uint64_t a_desc = a_mn ? smem_desc_sw128_mn(a_addr, 16384) : smem_desc_sw128(a_addr);
                    const uint64_t b_desc = b_mn ? smem_desc_sw128_mn(b_addr, 16384) : smem_desc_sw128(b_addr);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t adv = (uint64_t) ((k * UMMA_K) >> 4);
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        if constexpr (F4)  // 64 elements, two scales per row: scale block k / 2, bytes (k % 2) * 2 .. +1
                            mma_mxf4(d_tmem, a_desc + adv, b_desc + adv, idesc_sf_ids(idesc, (k & 1) * 2, (k & 1) * 2),
                                     sfa_cur + (k >> 1) * Cfg::kSfColsHalf, sfb_cur + (k >> 1) * Cfg::kSfColsHalf, accumulate);
                        else if constexpr (MX)
                            mma_mxf8(d_tmem, a_desc + adv, b_desc + adv, idesc_sf_ids(idesc, k, k), sfa_cur, sfb_cur, accumulate);
                        else if constexpr (MODE == GEMM_HP)
                            mma_f16(d_tmem, a_desc + adv, b_desc + adv, idesc, accumulate);
                        else
                            mma_f8(d_tmem, a_desc + k * a_kstep, b_desc + k * b_kstep, idesc, accumulate);
                    }
                    tc_commit(&empty_bar[stage]);  // frees the ring slot once these MMAs have read it
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc_commit(&tmem_full_bar[acc_stage]);
                if (++acc_stage == kAccStages) { acc_stage = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ================================================================ epilogue
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        uint8_t *stg = smem_epi + (warp - kEpiWarp0) * 32 * kStagePitchMax;
        uint32_t acc_stage = 0, acc_phase = 0;
        for (int t = blockIdx.x; ok && walk.locate(t, gi, m_blk, n_blk); t += gridDim.x) {
            const int64_t c_row_base = p.koffs ? (int64_t) gi * p.M : (p.offs_write ? p.offs_write[gi] : 0);
            const int64_t c_row_end = p.koffs ? c_row_base + p.M : (p.offs_write ? p.offs_write[gi + 1] : p.M);
            int kb_begin, kb_count;
            k_range(gi, kb_begin, kb_count);
            const bool have_acc = kb_count > 0;
            const int64_t tile_row0 = c_row_base + (int64_t) m_blk * BLOCK_M + q * 32;
            const int n0 = n_blk * BLOCK_N;
            if (have_acc && !(ok = mbar_wait_warp(&tmem_full_bar[acc_stage], acc_phase, abort_flag))) break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t) (q * 32) << 16) + acc_stage * BLOCK_N;
            epilogue_store_block<BLOCK_N, MODE>(p, taddr, have_acc, tile_row0, c_row_end, n0, gi, stg, lane, 0, (BLOCK_N + 31) / 32,
                                                [&]() { mbar_arrive(&tmem_empty_bar[acc_stage]); });
            if (have_acc && ++acc_stage == kAccStages) { acc_stage = 0; acc_phase ^= 1; }
        }
    }

    // ---- teardown
    if (!ok || *abort_flag) {
        if (p.status && lane == 0) atomicExch(p.status, (int) PT_ERR_TIMEOUT);
        __nanosleep(200000);  // let any TMA copy still in flight land before the shared memory is released
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

}  // namespace ptb

#include "gemm_fp8_pair.cuh"

namespace ptb {

// ------------------------------------------------------------------------------------------------ host side
struct MxScales {
    const uint8_t *sfa, *sfb;  // raw [rows, K/32]
    int64_t sf_ld;             // bytes per scale row
    void *workspace;
    size_t workspace_bytes;
};

static size_t mx_workspace_bytes(int64_t c_rows, int64_t N, int64_t K, int G, bool grouped, int block_n) {
    const int64_t num_kb = ceil_div(K, BLOCK_K);
    const int64_t ra = ceil_div(c_rows, BLOCK_M) + (grouped ? G : 0);
    const int64_t rb = (int64_t) G * ceil_div(N, block_n) * ceil_div(block_n, 128);
    return (size_t) ((ra + rb) * num_kb * 512);
}

// Re-tiles the raw MX scales of both operands into the workspace ([A row blocks][B tile blocks], 512-byte blocks) and
// records where they are.  `block_n` is the tile width the B blocks follow.
static int prepare_mx_scales(GemmParams &p, const MxScales &mx, int64_t a_rows, int64_t b_rows, int block_n, int sfb_blocks,
                             int sf_per_stage, cudaStream_t st) {
    const bool grouped = p.offs_write != nullptr && !p.koffs;
    const int sf_groups = p.koffs ? 1 : p.G;  // variable-K: one shared A and one shared B
    const size_t need = mx_workspace_bytes(p.M, p.N, p.K, sf_groups, grouped, block_n) * sf_per_stage;
    PT_REQUIRE(mx.workspace && mx.workspace_bytes >= need && aligned(mx.workspace, 16),
               "MX GEMM: workspace of %zu bytes (16-byte aligned) required, got %zu", need, mx.workspace_bytes);
    const int num_kb = (int) ceil_div(p.K, BLOCK_K) * sf_per_stage;  // scale blocks per row block
    RetileArgs ra{};
    ra.src = mx.sfa; ra.dst = (uint8_t *) mx.workspace; ra.src_rows = a_rows; ra.sf_ld = mx.sf_ld; ra.num_kb = num_kb;
    ra.is_b = 0; ra.offs_read = grouped ? p.offs_read : nullptr; ra.offs_write = grouped ? p.offs_write : nullptr;
    ra.G = sf_groups; ra.M = p.M;
    ra.num_row_blocks = ceil_div(p.M, BLOCK_M) + (grouped ? p.G : 0);
    RetileArgs rb = ra;
    rb.src = mx.sfb; rb.dst = ra.dst + ra.num_row_blocks * num_kb * 512; rb.src_rows = b_rows; rb.is_b = 1;
    rb.block_n = block_n; rb.sfb_blocks = sfb_blocks; rb.num_n_blocks = (int) ceil_div(p.N, block_n);
    rb.b_group_rows = p.b_group_rows; rb.G = sf_groups; rb.num_row_blocks = (int64_t) sf_groups * rb.num_n_blocks * sfb_blocks;
    const int max_blocks = sm_count() * 8;
    const int blocks_a = (int) std::min<int64_t>(ra.num_row_blocks, max_blocks);
    const int blocks_b = (int) std::min<int64_t>(rb.num_row_blocks, max_blocks);
    dim3 grid((unsigned) (blocks_a + blocks_b), (unsigned) ceil_div(num_kb, 32));
    PT_CUDA_OK(launch_overlapped(sf_retile_kernel, grid, dim3(128), 0, st, ra, rb, blocks_a));
    p.sfa_tiled = ra.dst;
    p.sfb_tiled = rb.dst;
    p.sfb_line0 = (rb.dst - ra.dst) / 128;
    return PT_OK;
}

template <int BLOCK_N, int MODE>
static int launch_gemm(const void *a, int64_t a_rows, const void *b, int64_t b_rows, GemmParams p, const MxScales &mx,
                       int max_ctas, int64_t max_tiles, cudaStream_t st) {
    using Cfg = GemmCfg<BLOCK_N, mode_is_mx(MODE), MODE == GEMM_MXF4>;
    if constexpr (mode_is_mx(MODE)) {
        int rc0 = prepare_mx_scales(p, mx, a_rows, b_rows, BLOCK_N, Cfg::kSfbBlocks, Cfg::kSfPerStage, st);
        if (rc0 != PT_OK) return rc0;
    }
    CUtensorMap ta, tb;
    int rc;
    // K-major: box = 128 contraction bytes x tile rows; MN-major: box = 128 row indices x 128 contraction rows
    if ((rc = p.a_mn ? make_tmap_bytes(&ta, a, p.K, a_rows, a_rows, BLOCK_K) : make_tmap_bytes(&ta, a, a_rows, p.K, p.K, BLOCK_M)) != PT_OK) return rc;
    if ((rc = p.b_mn ? make_tmap_bytes(&tb, b, p.K, b_rows, b_rows, BLOCK_K) : make_tmap_bytes(&tb, b, b_rows, p.K, p.K, BLOCK_N)) != PT_OK) return rc;
    auto kern = gemm_fp8_kernel<BLOCK_N, MODE>;
    static bool attr_set[64] = {};  // per instantiation and device
    const int dev = current_device_slot();
    if (!attr_set[dev]) {
        PT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_set[dev] = true;
    }
    int grid = (int) std::min<int64_t>(max_tiles, sm_count());
    if (max_ctas > 0) grid = std::min(grid, max_ctas);
    if (grid <= 0) return PT_OK;
    PT_CUDA_OK(launch_overlapped(kern, dim3(grid), dim3(kGemmThreads), Cfg::kSmemBytes, st, ta, tb, p));
    return PT_OK;
}

// Devices on which a cluster launch was refused: the pair form is not tried again there.
static bool g_pair_refused[64] = {};

// CTA-pair launch: grid = 2 x min(tiles, co-resident clusters).  Returns PT_ERR_UNSUPPORTED (no message, CUDA's
// last-error cleared) only when the cluster launch itself is refused; every other failure is reported as it is.
template <int BLOCK_N, int MODE>
static int launch_gemm_pair(const void *a, int64_t a_rows, const void *b, int64_t b_rows, GemmParams p, const MxScales &mx,
                            cudaStream_t st) {
    using Cfg = PairCfg<BLOCK_N, mode_is_mx(MODE), MODE == GEMM_MXF4>;
    CUtensorMap ta, tb, tsf;
    int rc;
    if constexpr (mode_is_mx(MODE)) {
        if ((rc = prepare_mx_scales(p, mx, a_rows, b_rows, BLOCK_N, Cfg::kSfbBlocks, Cfg::kSfPerStage, st)) != PT_OK) return rc;
        const bool grouped = p.offs_write != nullptr && !p.koffs;
        const int64_t lines = (int64_t) mx_workspace_bytes(p.M, p.N, p.K, p.koffs ? 1 : p.G, grouped, BLOCK_N) * Cfg::kSfPerStage / 128;
        if ((rc = make_tmap_lines(&tsf, p.sfa_tiled, lines, 4 * Cfg::kSfPerStage)) != PT_OK) return rc;
    }
    if ((rc = p.a_mn ? make_tmap_bytes(&ta, a, p.K, a_rows, a_rows, BLOCK_K) : make_tmap_bytes(&ta, a, a_rows, p.K, p.K, BLOCK_M)) != PT_OK) return rc;
    if ((rc = p.b_mn ? make_tmap_bytes(&tb, b, p.K, b_rows, b_rows, BLOCK_K) : make_tmap_bytes(&tb, b, b_rows, p.K, p.K, Cfg::kHalfN)) != PT_OK) return rc;
    if constexpr (!mode_is_mx(MODE)) tsf = ta;
    auto kern = gemm_fp8_pair_kernel<BLOCK_N, MODE>;
    PT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    // upper bound on tiles: every group may add one partial 256-row tile
    const int64_t m_tiles = p.koffs ? (int64_t) p.G * ceil_div(p.M, 2 * BLOCK_M) : ceil_div(p.M, 2 * BLOCK_M) + (p.offs_write ? p.G : 0);
    const int64_t tiles = m_tiles * ceil_div(p.N, BLOCK_N);
    static int max_clusters_dev[64] = {};  // co-resident pairs, per instantiation and device
    int &max_clusters = max_clusters_dev[current_device_slot()];
    if (max_clusters == 0) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(2 * (unsigned) sm_count());
        cfg.blockDim = dim3(Cfg::kThreads);
        cfg.dynamicSmemBytes = Cfg::kSmemBytes;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, (const void *) kern, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = sm_count() / 2;
        }
        max_clusters = n;
    }
    const int pairs = (int) std::min<int64_t>(tiles, max_clusters);
    if (pairs <= 0) return PT_OK;
    const cudaError_t le = launch_overlapped(kern, dim3(2 * pairs), dim3(Cfg::kThreads), Cfg::kSmemBytes, st, ta, tb, tsf, p);
    if (le != cudaSuccess) {
        cudaGetLastError();  // the refusal must not surface in a later, unrelated call
        if (le == cudaErrorInvalidClusterSize || le == cudaErrorLaunchOutOfResources || le == cudaErrorInvalidConfiguration ||
            le == cudaErrorNotSupported) {
            g_pair_refused[current_device_slot()] = true;
            return PT_ERR_UNSUPPORTED;
        }
        return set_error(PT_ERR_CUDA, "CTA-pair GEMM launch failed: %s", cudaGetErrorString(le));
    }
    return PT_OK;
}

static bool pair_enabled() {
    const char *e = getenv("PT_GEMM_PAIR");  // PT_GEMM_PAIR=0 keeps every problem on the single-CTA kernel
    return !e || atoi(e) != 0;
}

static int default_block_n(int mode, int64_t N) { return N <= 128 ? 128 : (mode_is_mx(mode) ? 240 : 256); }

template <int MODE>
static int dispatch_block_n(int block_n, const void *a, int64_t a_rows, const void *b, int64_t b_rows, const GemmParams &p,
                            const MxScales &mx, int max_ctas, cudaStream_t st) {
    // upper bound on tiles: every group may add one partial row block
    const int64_t m_blocks_bound = p.koffs ? (int64_t) p.G * ceil_div(p.M, BLOCK_M) : ceil_div(p.M, BLOCK_M) + (p.offs_write ? p.G : 0);
    {
        // Large problems run on CTA pairs (256-row tiles, half of the B tile per CTA).  Group lengths live on the
        // device; the average rows per group decide (short groups would waste up to 128 rows of work each).
        const int64_t rows_per_group = p.koffs ? p.M : p.M / p.G;
        const int64_t out_elems = (p.koffs ? (int64_t) p.G : 1) * p.M * (int64_t) p.N;
        const bool grouped = p.offs_write != nullptr && !p.koffs;
        if (block_n == 0 && max_ctas <= 0 && pair_enabled() && !g_pair_refused[current_device_slot()] && rows_per_group >= 1024 && p.N >= 512 &&
            out_elems >= (int64_t) 4096 * 4096 && (!mode_is_mx(MODE) || aligned(mx.workspace, 128))) {
            if constexpr (mode_is_mx(MODE)) {
                constexpr int kSfP = MODE == GEMM_MXF4 ? 2 : 1;
                if (mx.workspace_bytes >= mx_workspace_bytes(p.M, p.N, p.K, p.koffs ? 1 : p.G, grouped, 224) * kSfP) {
                    const int rc = launch_gemm_pair<224, MODE>(a, a_rows, b, b_rows, p, mx, st);
                    if (rc != PT_ERR_UNSUPPORTED) return rc;  // a device that cannot launch clusters falls through to single CTAs
                }
            } else {
                const int rc = launch_gemm_pair<256, MODE>(a, a_rows, b, b_rows, p, mx, st);
                if (rc != PT_ERR_UNSUPPORTED) return rc;
            }
        }
    }
    if (block_n == 0) block_n = default_block_n(MODE, p.N);
    const int64_t tiles = m_blocks_bound * ceil_div(p.N, block_n);
    switch (block_n) {
    case 128: return launch_gemm<128, MODE>(a, a_rows, b, b_rows, p, mx, max_ctas, tiles, st);
    case 240: return launch_gemm<240, MODE>(a, a_rows, b, b_rows, p, mx, max_ctas, tiles, st);
    case 256: return launch_gemm<256, MODE>(a, a_rows, b, b_rows, p, mx, max_ctas, tiles, st);
    default: return set_error(PT_ERR_INVALID, "GEMM: BLOCK_N %d is not built (128, 240, 256)", block_n);
    }
}

int gemm_fp8_host(const void *a, const void *a_scale, int a_fmt, const void *b, const void *b_scale, int b_fmt, void *c,
                  int c_dtype, int64_t ldc, int granularity, int64_t M, int64_t N, int64_t K, float beta,
                  const int64_t *offs_read, const int64_t *offs_write, const int64_t *k_offs, int G, int64_t a_rows_total,
                  int block_n, int max_ctas, void *workspace, size_t workspace_bytes, int *status, void *stream, int a_mn = 0,
                  int b_mn = 0) {
    PT_REQUIRE(M >= 0 && N >= 0 && K >= 0 && G >= 1 && G <= kMaxGroups, "GEMM: bad shape (M=%lld N=%lld K=%lld G=%d)",
               (long long) M, (long long) N, (long long) K, G);
    const bool fp4 = a_fmt == PT_E2M1 || b_fmt == PT_E2M1;
    if (a_mn || b_mn) {
        PT_REQUIRE(G == 1 && !offs_read && !offs_write && !k_offs && (granularity == PT_TENSORWISE || granularity == PT_ROWWISE),
                   "GEMM: MN-major operands are taken by the dense tensorwise / rowwise form");
        PT_REQUIRE((!a_mn || M % 16 == 0) && (!b_mn || N % 16 == 0), "GEMM: an MN-major operand needs a row count that is a multiple of 16");
        PT_REQUIRE(block_n == 0 || block_n == 128 || block_n == 256, "GEMM: MN-major operands take 128- or 256-column tiles");
    }
    PT_REQUIRE(!fp4 || (a_fmt == PT_E2M1 && b_fmt == PT_E2M1 && granularity == PT_MX_BLOCKWISE),
               "GEMM: e2m1 operands go together and take MX_BLOCKWISE scales");
    PT_REQUIRE(fp4 || a_fmt == PT_E4M3 || a_fmt == PT_E5M2, "GEMM: A format must be e4m3, e5m2 or e2m1");
    PT_REQUIRE(fp4 || b_fmt == PT_E4M3 || b_fmt == PT_E5M2, "GEMM: B format must be e4m3, e5m2 or e2m1");
    PT_REQUIRE(c_dtype == PT_BF16 || c_dtype == PT_F16 || c_dtype == PT_F32, "GEMM: bad output dtype");
    PT_REQUIRE(beta == 0.f || beta == 1.f, "GEMM: beta must be 0 or 1");
    PT_REQUIRE((offs_read == nullptr) == (offs_write == nullptr) || offs_write, "GEMM: write offsets required with read offsets");
    if (M == 0 || N == 0) return PT_OK;
    PT_REQUIRE(K > 0 && (K % 16 == 0 || (a_mn && b_mn)), "GEMM: K must be a positive multiple of 16 (got %lld)", (long long) K);
    PT_REQUIRE(a && b && c && a_scale && b_scale, "GEMM: null pointer");
    PT_REQUIRE(N < (1 << 30) && K < (1 << 30) && a_rows_total < (1ll << 31) && (int64_t) G * N < (1ll << 31),
               "GEMM: extent exceeds 32-bit tile coordinates");
    GemmParams p{};
    p.a_mn = a_mn; p.b_mn = b_mn;
    p.M = M; p.N = (int) N; p.K = (int) K; p.C = c; p.ldc = ldc; p.c_dtype = c_dtype; p.beta = beta;
    const int esize = c_dtype == PT_F32 ? 4 : 2;
    p.vec_store_ok = aligned(c, 16) && (ldc * esize) % 16 == 0;
    p.a_fmt = a_fmt; p.b_fmt = b_fmt;
    p.offs_read = offs_read ? offs_read : offs_write; p.offs_write = offs_write; p.G = G; p.b_group_rows = N;
    p.koffs = k_offs;
    PT_REQUIRE(!k_offs || (!offs_read && !offs_write), "GEMM: the variable-K form takes no row offsets");
    p.status = status;
    p.raster_m = raster_rows(a_rows_total, K);
    cudaStream_t st = (cudaStream_t) stream;
    const int64_t b_rows = k_offs ? N : (int64_t) G * N;
    MxScales mx{nullptr, nullptr, 0, workspace, workspace_bytes};
    switch (granularity) {
    case PT_TENSORWISE:
        p.sa = (const float *) a_scale; p.sb = (const float *) b_scale;
        return dispatch_block_n<GEMM_TENSOR>(block_n, a, a_rows_total, b, b_rows, p, mx, max_ctas, st);
    case PT_ROWWISE:
        p.sa = (const float *) a_scale; p.sb = (const float *) b_scale;
        return dispatch_block_n<GEMM_ROW>(block_n, a, a_rows_total, b, b_rows, p, mx, max_ctas, st);
    case PT_MX_BLOCKWISE:
        PT_REQUIRE(K % 128 == 0, "MX GEMM: K must be padded to a multiple of 128 (got %lld)", (long long) K);
        mx.sfa = (const uint8_t *) a_scale; mx.sfb = (const uint8_t *) b_scale; mx.sf_ld = K / 32;
        PT_REQUIRE(aligned(a_scale, 4) && aligned(b_scale, 4), "MX GEMM: scale pointers must be 4-byte aligned");
        if (a_fmt == PT_E2M1) {
            // packed e2m1: the kernel's contraction extent is in bytes (two elements each)
            p.K = (int) (K / 2);
            return dispatch_block_n<GEMM_MXF4>(block_n, a, a_rows_total, b, b_rows, p, mx, max_ctas, st);
        }
        return dispatch_block_n<GEMM_MX>(block_n, a, a_rows_total, b, b_rows, p, mx, max_ctas, st);
    default:
        return set_error(PT_ERR_UNSUPPORTED, "GEMM: granularity %d is not handled by this kernel", granularity);
    }
}

// fp16 / bf16 operands on the same kernels (kind::f16, no scales): the kernels count the contraction in bytes
int gemm_hp_host(const void *a, const void *b, int ab_dtype, void *c, int c_dtype, int64_t M, int64_t N, int64_t K, float beta,
                 const int64_t *offs, const int64_t *k_offs, int G, int64_t a_rows_total, int max_ctas, int *status, void *stream) {
    PT_REQUIRE(M >= 0 && N >= 0 && K >= 0 && G >= 1 && G <= kMaxGroups, "GEMM: bad shape (M=%lld N=%lld K=%lld G=%d)",
               (long long) M, (long long) N, (long long) K, G);
    PT_REQUIRE(ab_dtype == PT_BF16 || ab_dtype == PT_F16, "GEMM: operands must be bf16 or fp16");
    PT_REQUIRE(c_dtype == PT_BF16 || c_dtype == PT_F16 || c_dtype == PT_F32, "GEMM: bad output dtype");
    PT_REQUIRE(beta == 0.f || beta == 1.f, "GEMM: beta must be 0 or 1");
    PT_REQUIRE(!k_offs || !offs, "GEMM: the variable-K form takes no row offsets");
    if (M == 0 || N == 0) return PT_OK;
    PT_REQUIRE(K > 0 && K % 8 == 0, "GEMM: K must be a positive multiple of 8 for 16-bit operands (got %lld)", (long long) K);
    PT_REQUIRE(a && b && c, "GEMM: null pointer");
    PT_REQUIRE(N < (1 << 30) && K < (1 << 29) && a_rows_total < (1ll << 31) && (int64_t) G * N < (1ll << 31),
               "GEMM: extent exceeds 32-bit tile coordinates");
    GemmParams p{};
    p.M = M; p.N = (int) N; p.K = (int) (2 * K); p.C = c; p.ldc = N; p.c_dtype = c_dtype; p.beta = beta;
    const int esize = c_dtype == PT_F32 ? 4 : 2;
    p.vec_store_ok = aligned(c, 16) && (N * esize) % 16 == 0;
    p.a_fmt = p.b_fmt = ab_dtype == PT_BF16 ? 1 : 0;
    p.offs_read = offs; p.offs_write = offs; p.G = G; p.b_group_rows = N;
    p.koffs = k_offs;
    p.status = status;
    p.raster_m = raster_rows(a_rows_total, 2 * K);
    const int64_t b_rows = k_offs ? N : (int64_t) G * N;
    MxScales mx{nullptr, nullptr, 0, nullptr, 0};
    return dispatch_block_n<GEMM_HP>(0, a, a_rows_total, b, b_rows, p, mx, max_ctas, (cudaStream_t) stream);
}

}  // namespace ptb

using namespace ptb;

extern "C" {

int pt_gemm(const void *a, const void *b, int ab_dtype, void *c, int c_dtype, int64_t M, int64_t N, int64_t K, float beta, int *status,
            void *stream) {
    return gemm_hp_host(a, b, ab_dtype, c, c_dtype, M, N, K, beta, nullptr, nullptr, 1, M, 0, status, stream);
}

int pt_grouped_gemm(const void *a, const void *b, int ab_dtype, void *c, int c_dtype, int64_t a_rows, int64_t N, int64_t K,
                    const int64_t *group_offs, int G, float beta, int max_ctas, int *status, void *stream) {
    PT_REQUIRE(group_offs, "grouped GEMM: group offsets required");
    return gemm_hp_host(a, b, ab_dtype, c, c_dtype, a_rows, N, K, beta, group_offs, nullptr, G, a_rows, max_ctas, status, stream);
}

int pt_grouped_gemm_variable_k(const void *a, const void *b, int ab_dtype, void *c, int c_dtype, int64_t M, int64_t N, int64_t K_total,
                               const int64_t *k_offs, int G, float beta, int max_ctas, int *status, void *stream) {
    PT_REQUIRE(k_offs, "variable-K GEMM: contraction offsets required");
    return gemm_hp_host(a, b, ab_dtype, c, c_dtype, M, N, K_total, beta, nullptr, k_offs, G, M, max_ctas, status, stream);
}

size_t pt_gemm_fp4_workspace_bytes(int64_t c_rows, int64_t N, int64_t K, int G, int grouped, int block_n) {
    if (c_rows <= 0 || N <= 0 || K <= 0 || G < 1) return 0;
    const bool auto_n = block_n == 0;
    if (block_n == 0) block_n = default_block_n(GEMM_MXF4, N);
    // K / 2 bytes per row -> ceil(K / 256) stages, two 512-byte scale blocks each
    if (grouped == 2)
        return 2 * std::max(mx_workspace_bytes(c_rows, N, K / 2, 1, false, block_n),
                            auto_n ? mx_workspace_bytes(c_rows, N, K / 2, 1, false, 224) : (size_t) 0);
    size_t need = 2 * mx_workspace_bytes(c_rows, N, K / 2, G, grouped != 0, block_n);
    if (auto_n) need = std::max(need, 2 * mx_workspace_bytes(c_rows, N, K / 2, G, grouped != 0, 224));  // CTA-pair tiles
    return need;
}

size_t pt_gemm_fp8_workspace_bytes(int granularity, int64_t c_rows, int64_t N, int64_t K, int G, int grouped, int block_n) {
    if (granularity != PT_MX_BLOCKWISE || c_rows <= 0 || N <= 0 || K <= 0 || G < 1) return 0;
    const bool auto_n = block_n == 0;
    if (block_n == 0) block_n = default_block_n(GEMM_MX, N);
    if (grouped == 2)  // variable-K: shared A and B
        return std::max(mx_workspace_bytes(c_rows, N, K, 1, false, block_n), auto_n ? mx_workspace_bytes(c_rows, N, K, 1, false, 224) : (size_t) 0);
    size_t need = mx_workspace_bytes(c_rows, N, K, G, grouped != 0, block_n);
    if (auto_n) need = std::max(need, mx_workspace_bytes(c_rows, N, K, G, grouped != 0, 224));  // CTA-pair tiles
    return need;
}

int pt_gemm_fp8(const void *a, const void *a_scale, int a_fmt, const void *b, const void *b_scale, int b_fmt, void *c,
                int c_dtype, int granularity, int64_t M, int64_t N, int64_t K, float beta, int block_n, void *workspace,
                size_t workspace_bytes, int *status, void *stream) {
    return gemm_fp8_host(a, a_scale, a_fmt, b, b_scale, b_fmt, c, c_dtype, N, granularity, M, N, K, beta, nullptr, nullptr,
                         nullptr, 1, M, block_n, 0, workspace, workspace_bytes, status, stream);
}

int pt_gemm_fp8_mn(const void *a, const void *a_scale, int a_fmt, int a_mn, const void *b, const void *b_scale, int b_fmt, int b_mn, void *c,
                   int c_dtype, int granularity, int64_t M, int64_t N, int64_t K, float beta, int *status, void *stream) {
    return gemm_fp8_host(a, a_scale, a_fmt, b, b_scale, b_fmt, c, c_dtype, N, granularity, M, N, K, beta, nullptr, nullptr, nullptr, 1, M, 0, 0,
                         nullptr, 0, status, stream, a_mn, b_mn);
}

int pt_grouped_gemm_fp8(const void *a, const void *a_scale, int a_fmt, const void *b, const void *b_scale, int b_fmt,
                        void *c, int c_dtype, int granularity, int64_t a_rows, int64_t c_rows, int64_t N, int64_t K,
                        const int64_t *group_offs_read, const int64_t *group_offs_write, int G, float beta, int block_n,
                        int max_ctas, void *workspace, size_t workspace_bytes, int *status, void *stream) {
    PT_REQUIRE(group_offs_write, "grouped GEMM: group offsets required");
    return gemm_fp8_host(a, a_scale, a_fmt, b, b_scale, b_fmt, c, c_dtype, N, granularity, c_rows, N, K, beta,
                         group_offs_read, group_offs_write, nullptr, G, a_rows, block_n, max_ctas, workspace, workspace_bytes,
                         status, stream);
}

int pt_gemm_fp4(const void *a, const void *a_scale, const void *b, const void *b_scale, void *c, int c_dtype, int64_t M, int64_t N,
                int64_t K, float beta, int block_n, void *workspace, size_t workspace_bytes, int *status, void *stream) {
    return gemm_fp8_host(a, a_scale, PT_E2M1, b, b_scale, PT_E2M1, c, c_dtype, N, PT_MX_BLOCKWISE, M, N, K, beta, nullptr, nullptr,
                         nullptr, 1, M, block_n, 0, workspace, workspace_bytes, status, stream);
}

int pt_grouped_gemm_fp4(const void *a, const void *a_scale, const void *b, const void *b_scale, void *c, int c_dtype, int64_t a_rows,
                        int64_t c_rows, int64_t N, int64_t K, const int64_t *group_offs_read, const int64_t *group_offs_write, int G,
                        float beta, int block_n, int max_ctas, void *workspace, size_t workspace_bytes, int *status, void *stream) {
    PT_REQUIRE(group_offs_write, "grouped FP4 GEMM: group offsets required");
    return gemm_fp8_host(a, a_scale, PT_E2M1, b, b_scale, PT_E2M1, c, c_dtype, N, PT_MX_BLOCKWISE, c_rows, N, K, beta,
                         group_offs_read, group_offs_write, nullptr, G, a_rows, block_n, max_ctas, workspace, workspace_bytes,
                         status, stream);
}

int pt_grouped_gemm_fp4_variable_k(const void *a, const void *a_scale, const void *b, const void *b_scale, void *c, int c_dtype,
                                   int64_t M, int64_t N, int64_t K_total, const int64_t *k_offs, int G, float beta, int block_n,
                                   int max_ctas, void *workspace, size_t workspace_bytes, int *status, void *stream) {
    PT_REQUIRE(k_offs, "variable-K FP4 GEMM: contraction offsets required");
    return gemm_fp8_host(a, a_scale, PT_E2M1, b, b_scale, PT_E2M1, c, c_dtype, N, PT_MX_BLOCKWISE, M, N, K_total, beta, nullptr,
                         nullptr, k_offs, G, M, block_n, max_ctas, workspace, workspace_bytes, status, stream);
}

int pt_grouped_gemm_fp8_variable_k(const void *a, const void *a_scale, int a_fmt, const void *b, const void *b_scale, int b_fmt,
                                   void *c, int c_dtype, int granularity, int64_t M, int64_t N, int64_t K_total,
                                   const int64_t *k_offs, int G, float beta, int block_n, int max_ctas, void *workspace,
                                   size_t workspace_bytes, int *status, void *stream) {
    PT_REQUIRE(k_offs, "variable-K GEMM: contraction offsets required");
    return gemm_fp8_host(a, a_scale, a_fmt, b, b_scale, b_fmt, c, c_dtype, N, granularity, M, N, K_total, beta, nullptr, nullptr,
                         k_offs, G, M, block_n, max_ctas, workspace, workspace_bytes, status, stream);
}

}  // extern "C"
