// 128-blockwise FP8 quantization: one CTA per 128 x 128 tile, the tile held in registers so that the
// row-wise (1 x 128), column-wise (128 x 1), dual, per-tile (weight) and grouped segment-M variants all
// read their input exactly once.
//
// Arithmetic follows primus_turbo/triton/quantization/quant_blockwise.py:11-18 and
// csrc/kernels/quantization/quantization_blockwise.cu:60-334 of the reference:
//   scale = qmax / fmaxf(amax, 1e-4f); q = fp8_rne(clamp(x * scale, +-qmax)); stored scale = 1.0f / scale.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "gemm_common.cuh"
#include "sm100_ptx.cuh"
#include "tile_sched.cuh"

namespace ptb {

constexpr int kBlk = 128;
constexpr int kTileThreads = 256;
constexpr int kPack = 8;
constexpr int kLanesPerRow = kBlk / kPack;             // 16
constexpr int kRowsPerRound = kTileThreads / kLanesPerRow;  // 16
constexpr int kRounds = kBlk / kRowsPerRound;          // 8
constexpr float kEpsBlock = 1e-4f;

enum TileMode { MODE_ROW = 1, MODE_COL = 2, MODE_DUAL = 3, MODE_WEIGHT = 4, MODE_SEGMENT = 7 };

template <typename T>
__device__ __forceinline__ void load_row8(const T *row_ptr, int64_t gn, int64_t N, bool valid, bool vec_ok,
                                          float (&v)[kPack]) {
    if (valid && vec_ok && gn + kPack <= N) {
        load8(row_ptr + gn, v);
    } else {
#pragma unroll
        for (int i = 0; i < kPack; ++i) v[i] = (valid && gn + i < N) ? load1(row_ptr + gn + i) : 0.f;
    }
}

template <int FMT>
__device__ __forceinline__ void store_row8(uint8_t *row_ptr, int64_t gn, int64_t N, bool vec_ok, const float (&v)[kPack]) {
    if (vec_ok && gn + kPack <= N) {
        uint2 o;
        o.x = cvt4_fp8<FMT>(v[0], v[1], v[2], v[3]);
        o.y = cvt4_fp8<FMT>(v[4], v[5], v[6], v[7]);
        *reinterpret_cast<uint2 *>(row_ptr + gn) = o;
    } else {
#pragma unroll
        for (int i = 0; i < kPack; ++i)
            if (gn + i < N) row_ptr[gn + i] = cvt1_fp8<FMT>(v[i]);
    }
}

struct SegmentArgs {
    const int64_t *group_offs;
    const int64_t *padded_offs;
    int num_groups;
};

// grid: (N tiles, M tiles, batch). For MODE_SEGMENT the M tiles run over the padded row space.
template <typename T, int FMT, int MODE>
__global__ void __launch_bounds__(kTileThreads)
    blockwise_tile_kernel(const T *__restrict__ x, int64_t M, int64_t N, int vec_ok, uint8_t *__restrict__ q_row,
                          float *__restrict__ s_row, uint8_t *__restrict__ q_col, float *__restrict__ s_col,
                          SegmentArgs seg) {
    constexpr bool kRow = (MODE & 1) != 0 && MODE != MODE_WEIGHT;
    constexpr bool kCol = (MODE & 2) != 0 && MODE != MODE_WEIGHT;
    constexpr bool kSeg = MODE == MODE_SEGMENT;
    constexpr bool kWeight = MODE == MODE_WEIGHT;

    const int tid = threadIdx.x;
    const int lane16 = tid % kLanesPerRow;
    const int row_base = tid / kLanesPerRow;
    const int64_t col_blk = blockIdx.x;
    const int64_t pid_m = blockIdx.y;
    const int64_t batch = blockIdx.z;
    const int64_t n_blocks = (N + kBlk - 1) / kBlk;
    const int64_t m_blocks = (M + kBlk - 1) / kBlk;
    const int64_t gn = col_blk * kBlk + lane16 * kPack;

    x += batch * M * N;

    // row mapping: plain tiles start at pid_m * 128; segment tiles live in padded row space
    int64_t in_row0 = pid_m * kBlk, in_lo = 0, in_hi = M, out_row0 = pid_m * kBlk;
    if constexpr (kSeg) {
        const int64_t m_padded = seg.padded_offs[seg.num_groups];
        if (out_row0 >= m_padded) return;
        int lo = 0, hi = seg.num_groups - 1;  // last group g with padded_offs[g] <= out_row0 (empty groups skipped)
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (seg.padded_offs[mid] <= out_row0) lo = mid; else hi = mid - 1;
        }
        in_lo = seg.group_offs[lo];
        in_hi = min(seg.group_offs[lo + 1], M);
        in_row0 = in_lo + (out_row0 - seg.padded_offs[lo]);
    }

    __shared__ float s_part[kRowsPerRound][kBlk];
    __shared__ float s_scale[kBlk];

    float vals[kRounds][kPack];
    float col_amax[kPack];
#pragma unroll
    for (int i = 0; i < kPack; ++i) col_amax[i] = 0.f;
    float tile_amax = 0.f;

#pragma unroll
    for (int r = 0; r < kRounds; ++r) {
        const int local_m = row_base + r * kRowsPerRound;
        const int64_t in_m = in_row0 + local_m;
        const bool valid = in_m >= in_lo && in_m < in_hi;
        load_row8(x + in_m * N, gn, N, valid, vec_ok != 0, vals[r]);
        float row_amax = 0.f;
#pragma unroll
        for (int i = 0; i < kPack; ++i) {
            const float av = fabsf(vals[r][i]);
            row_amax = fmaxf(row_amax, av);
            col_amax[i] = fmaxf(col_amax[i], av);
        }
        if constexpr (kWeight) tile_amax = fmaxf(tile_amax, row_amax);
        if constexpr (kRow) {
#pragma unroll
            for (int off = kLanesPerRow >> 1; off > 0; off >>= 1)
                row_amax = fmaxf(row_amax, __shfl_xor_sync(0xffffffffu, row_amax, off, kLanesPerRow));
            const float scale = scale_from_amax<FMT>(row_amax, kEpsBlock);
            if (valid) {
                float o[kPack];
#pragma unroll
                for (int i = 0; i < kPack; ++i) o[i] = mul_sat<FMT>(vals[r][i], scale);
                store_row8<FMT>(q_row + (batch * M + in_m) * N, gn, N, vec_ok != 0, o);
                if (lane16 == 0) {
                    const float inv = __fdiv_rn(1.0f, scale);
                    if constexpr (kSeg) s_row[col_blk * M + in_m] = inv;  // transposed [N blocks, M]
                    else s_row[(batch * M + in_m) * n_blocks + col_blk] = inv;
                }
            }
        }
    }

    if constexpr (kWeight) {
        tile_amax = warp_max(tile_amax);
        if ((tid & 31) == 0) s_part[0][tid >> 5] = tile_amax;
        __syncthreads();
        float m = 0.f;
#pragma unroll
        for (int w = 0; w < kTileThreads / 32; ++w) m = fmaxf(m, s_part[0][w]);
        const float scale = scale_from_amax<FMT>(m, kEpsBlock);
        if (tid == 0) s_row[(batch * m_blocks + pid_m) * n_blocks + col_blk] = __fdiv_rn(1.0f, scale);
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
            const int64_t in_m = in_row0 + row_base + r * kRowsPerRound;
            if (in_m < M) {
                float o[kPack];
#pragma unroll
                for (int i = 0; i < kPack; ++i) o[i] = mul_sat<FMT>(vals[r][i], scale);
                store_row8<FMT>(q_row + (batch * M + in_m) * N, gn, N, vec_ok != 0, o);
            }
        }
    }

    if constexpr (kCol) {
#pragma unroll
        for (int i = 0; i < kPack; ++i) s_part[row_base][lane16 * kPack + i] = col_amax[i];
        __syncthreads();
        if (tid < kBlk) {
            float m = 0.f;
#pragma unroll
            for (int rs = 0; rs < kRowsPerRound; ++rs) m = fmaxf(m, s_part[rs][tid]);
            const float scale = scale_from_amax<FMT>(m, kEpsBlock);
            s_scale[tid] = scale;
            const int64_t c = col_blk * kBlk + tid;
            if (c < N) s_col[(batch * (kSeg ? 0 : m_blocks) + pid_m) * N + c] = __fdiv_rn(1.0f, scale);
        }
        __syncthreads();
        float sc[kPack];
#pragma unroll
        for (int i = 0; i < kPack; ++i) sc[i] = s_scale[lane16 * kPack + i];
        const int64_t out_rows = kSeg ? seg.padded_offs[seg.num_groups] : M;
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
            const int64_t out_m = out_row0 + row_base + r * kRowsPerRound;
            if (out_m < out_rows) {
                float o[kPack];
#pragma unroll
                for (int i = 0; i < kPack; ++i) o[i] = mul_sat<FMT>(vals[r][i], sc[i]);  // invalid rows hold 0
                store_row8<FMT>(q_col + (batch * (kSeg ? 0 : M) + out_m) * N, gn, N, vec_ok != 0, o);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// Persistent, TMA-pipelined form of the tile kernel for 16-bit inputs with N % 16 == 0.
//
// One producer warp streams 128 x 128 tiles (two 128-row x 128-byte boxes of a 3-D tensor map, 128-byte swizzle)
// through a ring of shared-memory stages; eight consumer warps quantize a tile while the next ones are in flight.
//   row pass   8 lanes share one row: each lane owns 16 consecutive elements (two 16-byte chunks), the 128-wide
//              row amax is three shuffles, and a warp store writes four full 128-byte output rows
//   col pass   a warp owns 16 rows, a lane four adjacent columns; the 128-row column amax goes through a 2 KiB
//              shared-memory exchange (one named barrier per tile), and a warp store writes one 128-byte row
// amax is taken on packed 16-bit pairs (two elements per instruction); the scale / clamp / convert arithmetic is
// the same as in blockwise_tile_kernel, so both forms produce identical bytes.
constexpr int kBqStages = 3;
constexpr int kBqCtasPerSm = 2;
constexpr int kBqTileBytes = kBlk * kBlk * 2;
constexpr int kBqConsumerWarps = 8;
constexpr int kBqThreads = 32 * (1 + kBqConsumerWarps);
constexpr int kBqSmemBytes = kBqStages * kBqTileBytes + 1024 + 256;
constexpr int kBqMaxGroups = 256;  // segment form: offset tables of up to this many groups are held in shared memory

struct BqArgs {
    int64_t M, N;
    int tiles_n, tiles_m;      // tiles per row of tiles / per matrix (segment: over the padded row space)
    int64_t total_tiles;
    uint8_t *q_row, *q_col;
    float *s_row, *s_col;
    SegmentArgs seg;
    int *status;               // receives PT_ERR_TIMEOUT if a bounded wait gives up (may be null)
    int sched_slot;            // dynamic tile schedule: counter slot (tile_sched.cuh), or -1 for the static schedule
};

// what the producer hands over with each tile (col_blk < 0: no more tiles)
struct BqTileDesc {
    int batch, pid_m, col_blk, in_row0, n_valid, pad0, pad1, pad2;
};

template <typename T, int FMT, int MODE>
__global__ void __launch_bounds__(kBqThreads, kBqCtasPerSm)
    blockwise_tma_kernel(const __grid_constant__ CUtensorMap tmap, BqArgs a) {
    using namespace sm100;
    constexpr bool kRow = (MODE & 1) != 0 && MODE != MODE_WEIGHT;
    constexpr bool kCol = (MODE & 2) != 0 && MODE != MODE_WEIGHT;
    constexpr bool kSeg = MODE == MODE_SEGMENT;
    constexpr bool kWeight = MODE == MODE_WEIGHT;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + kBqStages * kBqTileBytes);
    uint64_t *empty_bar = full_bar + kBqStages;
    __shared__ uint2 s_cmax[2][kBqConsumerWarps][32];  // packed column maxima of each 16-row band
    __shared__ float s_wmax[2][kBqConsumerWarps];
    __shared__ __align__(16) BqTileDesc s_desc[kBqStages];
    __shared__ int s_abort;
    volatile int *abort_flag = &s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < kBqStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kBqConsumerWarps);
        }
        fence_barrier_init();
        prefetch_tmap(&tmap);
    }
    __syncthreads();
    grid_dep_wait();    // the input (and the group offsets) may come from the kernel launched just before
    grid_dep_launch();
    bool ok = true;
    const uint32_t per_b = (uint32_t) a.tiles_n * (uint32_t) a.tiles_m;
    const int64_t m_blocks = (a.M + kBlk - 1) / kBlk;
    const int64_t n_blocks = a.tiles_n;
    const int64_t m_padded = kSeg ? a.seg.padded_offs[a.seg.num_groups] : 0;
    // segment form: both offset tables are copied to shared memory first (a search through global memory would cost
    // each tile several dependent round trips)
    __shared__ int s_gtab[kSeg ? 2 * (kBqMaxGroups + 1) : 1];
    if constexpr (kSeg) {
        for (int i = threadIdx.x; i <= a.seg.num_groups; i += blockDim.x) {
            s_gtab[i] = (int) a.seg.padded_offs[i];
            s_gtab[(kBqMaxGroups + 1) + i] = (int) a.seg.group_offs[i];
        }
        __syncthreads();
    }

    // tile t -> batch, row block (segment: block of the padded row space), column block; and for the segment form
    // the input rows it covers: [in_row0, in_row0 + n_valid), written at padded rows out_row0 ...
    auto locate = [&](uint32_t t, int64_t &batch, int64_t &pid_m, int64_t &col_blk, int64_t &in_row0, int &n_valid) -> bool {
        const uint32_t b = t / per_b, rem = t - b * per_b;
        const uint32_t tm = rem / (uint32_t) a.tiles_n;
        batch = b; pid_m = tm; col_blk = rem - tm * (uint32_t) a.tiles_n;
        in_row0 = pid_m * kBlk;
        n_valid = kBlk;
        if constexpr (kSeg) {
            const int64_t out_row0 = pid_m * kBlk;
            if (out_row0 >= m_padded) return false;
            const int *poffs = s_gtab, *goffs = s_gtab + (kBqMaxGroups + 1);
            int lo = 0, hi = a.seg.num_groups - 1;  // last group g with padded_offs[g] <= out_row0 (empty groups skipped)
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (poffs[mid] <= out_row0) lo = mid; else hi = mid - 1;
            }
            in_row0 = goffs[lo] + (out_row0 - poffs[lo]);
            const int64_t in_hi = min((int64_t) goffs[lo + 1], a.M);
            n_valid = (int) max((int64_t) 0, min((int64_t) kBlk, in_hi - in_row0));
        }
        return true;
    };

    if (warp == 0) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            // the producer resolves every tile once (coordinates, and in the segment form its group) and hands the result
            // over in shared memory next to the data; tiles come from the dynamic schedule when a counter slot was given
            for (uint32_t t = blockIdx.x; t < (uint32_t) a.total_tiles; t = tile_sched_next(a.sched_slot, t)) {
                int64_t batch, pid_m, col_blk, in_row0;
                int n_valid;
                if (!locate(t, batch, pid_m, col_blk, in_row0, n_valid)) continue;
                if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) break;
                s_desc[stage] = BqTileDesc{(int) batch, (int) pid_m, (int) col_blk, (int) in_row0, n_valid, 0, 0, 0};
                mbar_arrive_expect_tx(&full_bar[stage], kBqTileBytes);
                uint8_t *dst = smem + stage * kBqTileBytes;
                tma_load_3d(dst, &tmap, &full_bar[stage], (int) (col_blk * kBlk), (int) in_row0, (int) batch);
                tma_load_3d(dst + kBqTileBytes / 2, &tmap, &full_bar[stage], (int) (col_blk * kBlk + 64), (int) in_row0, (int) batch);
                if (++stage == kBqStages) { stage = 0; phase ^= 1; }
            }
            if (ok && (ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) {   // the terminal descriptor
                s_desc[stage].col_blk = -1;
                mbar_arrive(&full_bar[stage]);
            }
            tile_sched_done(a.sched_slot);
        }
    } else {
        const int cw = warp - 1;
        // row pass: 8 lanes per row; lane l8 owns elements [16 l8, 16 l8 + 16) = chunks 2m, 2m + 1 of box l8 / 4.
        // Lanes of box 0 read their even chunk first, lanes of box 1 their odd chunk: the eight 16-byte reads of a
        // row then fall on eight different swizzled chunk positions (the two boxes share banks).
        const int l8 = lane & 7, r_box = l8 >> 2, r_m = l8 & 3, r_sub = lane >> 3;
        // col pass: lane = column quad of the 128-wide tile row, warp = band of 16 rows
        const int c_box = lane >> 4, c_chunk = (lane & 15) >> 1, c_off = (lane & 1) << 3;
        uint32_t stage = 0, phase = 0, tile_count = 0;
        while (true) {
            if (!(ok = mbar_wait_warp(&full_bar[stage], phase, abort_flag))) break;
            const int4 d0 = *reinterpret_cast<const int4 *>(&s_desc[stage]);
            if (d0.z < 0) break;
            const int64_t batch = d0.x, pid_m = d0.y, col_blk = d0.z, in_row0 = d0.w;
            const int n_valid = s_desc[stage].n_valid;
            const uint8_t *tile = smem + stage * kBqTileBytes;
            const int buf = tile_count & 1;
            ++tile_count;
            const int64_t n0 = col_blk * kBlk;
            const int64_t out_row0 = pid_m * kBlk;

            // ---- loads: everything this thread needs from the tile goes to registers, then the stage is released
            uint4 rc[4][2];  // row pass / weight: 4 rows x 2 chunks
            if constexpr (kRow || kWeight) {
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const int row = cw * 16 + it * 4 + r_sub;
                    const uint8_t *rp = tile + r_box * (kBqTileBytes / 2) + row * 128;
                    const int first = 2 * r_m + r_box, second = 2 * r_m + (r_box ^ 1);
                    const uint4 x0 = *reinterpret_cast<const uint4 *>(rp + ((first ^ (row & 7)) << 4));
                    const uint4 x1 = *reinterpret_cast<const uint4 *>(rp + ((second ^ (row & 7)) << 4));
                    rc[it][0] = r_box ? x1 : x0;  // chunk 2m
                    rc[it][1] = r_box ? x0 : x1;  // chunk 2m + 1
                }
            }
            uint2 cc[16];  // col pass: 16 rows x 4 columns
            if constexpr (kCol) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int row = cw * 16 + i;
                    cc[i] = *reinterpret_cast<const uint2 *>(tile + c_box * (kBqTileBytes / 2) + row * 128 +
                                                             ((c_chunk ^ (row & 7)) << 4) + c_off);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);  // this warp no longer reads the stage
            if (++stage == kBqStages) { stage = 0; phase ^= 1; }

            // ---- column maxima (and the tile maximum of the weight form) go through shared memory
            if constexpr (kCol) {
                uint32_t m01 = 0u, m23 = 0u;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (!kSeg || cw * 16 + i < n_valid) {  // rows past the group end belong to the next group
                        m01 = absmax2<T>(m01, cc[i].x);
                        m23 = absmax2<T>(m23, cc[i].y);
                    }
                }
                s_cmax[buf][cw][lane] = make_uint2(m01, m23);
            }
            float w_amax = 0.f;
            if constexpr (kWeight) {
                uint32_t m = 0u;
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const uint32_t w[8] = {rc[it][0].x, rc[it][0].y, rc[it][0].z, rc[it][0].w, rc[it][1].x, rc[it][1].y, rc[it][1].z, rc[it][1].w};
#pragma unroll
                    for (int k = 0; k < 8; ++k) m = absmax2<T>(m, w[k]);
                }
                m = absmax2_done(m);
                w_amax = warp_max(fmaxf(lo_f32<T>(m), hi_f32<T>(m)));
                if (lane == 0) s_wmax[buf][cw] = w_amax;
            }
            if constexpr (kCol || kWeight) sm100::named_barrier<1, kBqConsumerWarps * 32>();

            // ---- row pass
            if constexpr (kRow || kWeight) {
                float w_scale = 0.f;
                if constexpr (kWeight) {
                    float m = 0.f;
#pragma unroll
                    for (int w = 0; w < kBqConsumerWarps; ++w) m = fmaxf(m, s_wmax[buf][w]);
                    w_scale = scale_from_amax<FMT>(m, kEpsBlock);
                    if (cw == 0 && lane == 0) a.s_row[(batch * m_blocks + pid_m) * n_blocks + col_blk] = __fdiv_rn(1.0f, w_scale);
                }
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const int row = cw * 16 + it * 4 + r_sub;
                    const uint32_t w[8] = {rc[it][0].x, rc[it][0].y, rc[it][0].z, rc[it][0].w, rc[it][1].x, rc[it][1].y, rc[it][1].z, rc[it][1].w};
                    float scale = w_scale;
                    if constexpr (kRow) {
                        uint32_t m = 0u;
#pragma unroll
                        for (int k = 0; k < 8; ++k) m = absmax2<T>(m, w[k]);
                        m = absmax2_done(m);
                        float am = fmaxf(lo_f32<T>(m), hi_f32<T>(m));
                        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
                        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
                        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 4));
                        scale = scale_from_amax<FMT>(am, kEpsBlock);
                    }
                    const int64_t in_m = in_row0 + row;
                    const int64_t gn = n0 + l8 * 16;
                    if (row < n_valid && in_m < a.M && gn < a.N) {
                        uint32_t o[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            o[k] = cvt4_fp8<FMT>(mul_sat<FMT>(lo_f32<T>(w[2 * k]), scale), mul_sat<FMT>(hi_f32<T>(w[2 * k]), scale),
                                                 mul_sat<FMT>(lo_f32<T>(w[2 * k + 1]), scale), mul_sat<FMT>(hi_f32<T>(w[2 * k + 1]), scale));
                        *reinterpret_cast<uint4 *>(a.q_row + (batch * a.M + in_m) * a.N + gn) = make_uint4(o[0], o[1], o[2], o[3]);
                        if (kRow && l8 == 0) {
                            const float inv = __fdiv_rn(1.0f, scale);
                            if constexpr (kSeg) a.s_row[col_blk * a.M + in_m] = inv;  // transposed [N blocks, M]
                            else a.s_row[(batch * a.M + in_m) * n_blocks + col_blk] = inv;
                        }
                    }
                }
            }

            // ---- col pass
            if constexpr (kCol) {
                uint32_t m01 = 0u, m23 = 0u;
#pragma unroll
                for (int w = 0; w < kBqConsumerWarps; ++w) {
                    const uint2 v = s_cmax[buf][w][lane];
                    m01 = absmax2<T>(m01, v.x);
                    m23 = absmax2<T>(m23, v.y);
                }
                m01 = absmax2_done(m01);
                m23 = absmax2_done(m23);
                const float sc0 = scale_from_amax<FMT>(lo_f32<T>(m01), kEpsBlock), sc1 = scale_from_amax<FMT>(hi_f32<T>(m01), kEpsBlock);
                const float sc2 = scale_from_amax<FMT>(lo_f32<T>(m23), kEpsBlock), sc3 = scale_from_amax<FMT>(hi_f32<T>(m23), kEpsBlock);
                const int64_t gc = n0 + 4 * lane;
                if (gc < a.N) {
                    if (cw == 0)
                        *reinterpret_cast<float4 *>(a.s_col + (batch * (kSeg ? 0 : m_blocks) + pid_m) * a.N + gc) =
                            make_float4(__fdiv_rn(1.0f, sc0), __fdiv_rn(1.0f, sc1), __fdiv_rn(1.0f, sc2), __fdiv_rn(1.0f, sc3));
                    const int64_t out_rows = kSeg ? m_padded : a.M;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int row = cw * 16 + i;
                        const int64_t out_m = out_row0 + row;
                        if (out_m < out_rows) {
                            const bool live = !kSeg || row < n_valid;  // padding rows of a group are written as zeros
                            const uint32_t x01 = live ? cc[i].x : 0u, x23 = live ? cc[i].y : 0u;
                            const uint32_t o = cvt4_fp8<FMT>(mul_sat<FMT>(lo_f32<T>(x01), sc0), mul_sat<FMT>(hi_f32<T>(x01), sc1),
                                                             mul_sat<FMT>(lo_f32<T>(x23), sc2), mul_sat<FMT>(hi_f32<T>(x23), sc3));
                            *reinterpret_cast<uint32_t *>(a.q_col + (batch * (kSeg ? 0 : a.M) + out_m) * a.N + gc) = o;
                        }
                    }
                }
            }
        }
    }
    if (!ok || *abort_flag) {
        if (a.status && lane == 0) atomicExch(a.status, (int) PT_ERR_TIMEOUT);
        __nanosleep(100000);  // let a copy still in flight land before the shared memory is released
    }
}

// ------------------------------------------------------------------------------------------------ warp-split form
// Dual (row-wise + column-wise) and segment-M quantization of 16-bit inputs.  Same tiles, TMA ring, tile descriptors and
// dynamic schedule as blockwise_tma_kernel, but the eight consumer warps are split by output so that no shuffle and no
// CTA-wide barrier is needed:
//   * four warps produce the row-wise copy, one thread per tile row: the 128 elements of the row are read as sixteen
//     16-byte chunks (conflict-free under the 128-byte swizzle), the row maximum is local to the thread, the 128 output
//     bytes go to a swizzled staging tile that one bulk tensor store writes (whole tiles; a tile cut by a group's end
//     is stored row by row);
//   * four warps produce the column-wise copy, one thread per column pair and 64-row band: 64 rows x 2 columns in
//     registers, the two bands of a column meet through 512 bytes of shared memory (one named barrier among these four
//     warps), the output bytes are staged row-major and written by one bulk tensor store.
// Arithmetic is that of blockwise_tile_kernel (same scale, clamp and convert), so all three forms write the same bytes.
constexpr int kBsStages = 2;
constexpr int kBsCtasPerSm = 2;
constexpr int kBsGroupThreads = 128;
constexpr int kBsThreads = 32 + 2 * kBsGroupThreads;
constexpr int kBsStageOutBytes = kBlk * kBlk;   // one staged fp8 tile
constexpr int kBsSmemBytes = kBsStages * kBqTileBytes + 2 * kBsStageOutBytes + 1024 + 256;

template <typename T, int FMT, bool SEG>
__global__ void __launch_bounds__(kBsThreads, kBsCtasPerSm)
    blockwise_split_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap_qrow,
                           const __grid_constant__ CUtensorMap tmap_qcol, BqArgs a) {
    using namespace sm100;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *row_stage = smem + kBsStages * kBqTileBytes;
    uint8_t *col_stage = row_stage + kBsStageOutBytes;
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(col_stage + kBsStageOutBytes);
    uint64_t *empty_bar = full_bar + kBsStages;
    __shared__ uint32_t s_cmax[2][kBsGroupThreads];   // packed |max| of each (64-row band, column pair): index 64 band + pair
    __shared__ __align__(16) BqTileDesc s_desc[kBsStages];
    __shared__ int s_abort;
    volatile int *abort_flag = &s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int st = 0; st < kBsStages; ++st) {
            mbar_init(&full_bar[st], 1);
            mbar_init(&empty_bar[st], 2 * kBsGroupThreads / 32);
        }
        fence_barrier_init();
        prefetch_tmap(&tmap);
        prefetch_tmap(&tmap_qrow);
        prefetch_tmap(&tmap_qcol);
    }
    __shared__ int s_gtab[SEG ? 2 * (kBqMaxGroups + 1) : 1];
    __syncthreads();
    grid_dep_wait();    // the input (and the group offsets) may come from the kernel launched just before
    grid_dep_launch();
    if constexpr (SEG) {
        for (int i = threadIdx.x; i <= a.seg.num_groups; i += blockDim.x) {
            s_gtab[i] = (int) a.seg.padded_offs[i];
            s_gtab[(kBqMaxGroups + 1) + i] = (int) a.seg.group_offs[i];
        }
        __syncthreads();
    }
    bool ok = true;
    const int64_t n_blocks = a.tiles_n;
    const int64_t m_blocks = (a.M + kBlk - 1) / kBlk;

    if (warp == 0) {
        // ================================================================ producer: tile coordinates + TMA loads
        if (lane == 0) {
            const int64_t m_padded = SEG ? s_gtab[a.seg.num_groups] : 0;
            uint32_t stage = 0, phase = 0;
            for (uint32_t t = blockIdx.x; t < (uint32_t) a.total_tiles; t = tile_sched_next(a.sched_slot, t)) {
                const uint32_t tm = t / (uint32_t) a.tiles_n;
                BqTileDesc d{0, (int) tm, (int) (t - tm * (uint32_t) a.tiles_n), (int) tm * kBlk, kBlk, 0, 0, 0};
                if constexpr (SEG) {
                    const int64_t out_row0 = (int64_t) tm * kBlk;
                    if (out_row0 >= m_padded) continue;
                    const int *poffs = s_gtab, *goffs = s_gtab + (kBqMaxGroups + 1);
                    int lo = 0, hi = a.seg.num_groups - 1;  // last group g with padded_offs[g] <= out_row0 (empty groups skipped)
                    while (lo < hi) {
                        const int mid = (lo + hi + 1) >> 1;
                        if (poffs[mid] <= out_row0) lo = mid; else hi = mid - 1;
                    }
                    d.in_row0 = goffs[lo] + (int) (out_row0 - poffs[lo]);
                    d.n_valid = (int) max((int64_t) 0, min((int64_t) kBlk, min((int64_t) goffs[lo + 1], a.M) - d.in_row0));
                }
                if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) break;
                s_desc[stage] = d;
                mbar_arrive_expect_tx(&full_bar[stage], kBqTileBytes);
                uint8_t *dst = smem + stage * kBqTileBytes;
                tma_load_3d(dst, &tmap, &full_bar[stage], d.col_blk * kBlk, d.in_row0, 0);
                tma_load_3d(dst + kBqTileBytes / 2, &tmap, &full_bar[stage], d.col_blk * kBlk + 64, d.in_row0, 0);
                if (++stage == kBsStages) { stage = 0; phase ^= 1; }
            }
            if (ok && (ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) {   // the terminal descriptor
                s_desc[stage].col_blk = -1;
                mbar_arrive(&full_bar[stage]);
            }
            tile_sched_done(a.sched_slot);
        }
    } else if (warp <= kBsGroupThreads / 32) {
        // ================================================================ row-wise copy: thread = tile row
        const int row = threadIdx.x - 32;
        uint32_t stage = 0, phase = 0;
        while (true) {
            if (!(ok = mbar_wait_warp(&full_bar[stage], phase, abort_flag))) break;
            const int4 d0 = *reinterpret_cast<const int4 *>(&s_desc[stage]);
            if (d0.z < 0) break;
            const int pid_m = d0.y, col_blk = d0.z, in_row0 = d0.w;
            const int n_valid = SEG ? s_desc[stage].n_valid : kBlk;
            uint32_t w[64];
            {
                const uint8_t *rp = smem + stage * kBqTileBytes + row * 128;
#pragma unroll
                for (int b = 0; b < 2; ++b)
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint4 v = *reinterpret_cast<const uint4 *>(rp + b * (kBqTileBytes / 2) + ((c ^ (row & 7)) << 4));
                        w[32 * b + 4 * c] = v.x; w[32 * b + 4 * c + 1] = v.y; w[32 * b + 4 * c + 2] = v.z; w[32 * b + 4 * c + 3] = v.w;
                    }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);  // this warp no longer reads the stage
            if (++stage == kBsStages) { stage = 0; phase ^= 1; }
            uint32_t m2 = 0u;
#pragma unroll
            for (int k = 0; k < 64; ++k) m2 = absmax2<T>(m2, w[k]);
            m2 = absmax2_done(m2);
            const float scale = scale_from_amax<FMT>(fmaxf(lo_f32<T>(m2), hi_f32<T>(m2)), kEpsBlock);
            const int64_t in_m = (int64_t) in_row0 + row;
            const int64_t n0 = (int64_t) col_blk * kBlk;
            const bool live = row < n_valid && in_m < a.M;
            if (live) {
                const float inv = __fdiv_rn(1.0f, scale);
                if constexpr (SEG) a.s_row[(int64_t) col_blk * a.M + in_m] = inv;  // transposed [N blocks, M]
                else a.s_row[in_m * n_blocks + col_blk] = inv;
            }
            // a whole tile leaves through the staging tile and one bulk store; one cut by the end of a group (the rows
            // after it belong to other tiles) is stored row by row
            const bool whole = !SEG || n_valid == kBlk;
            if (whole) {
                if (row == 0) bulk_wait_read_all();   // the previous tile's store has read the staging tile
                sm100::named_barrier<1, kBsGroupThreads>();
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t x0 = w[8 * j + 2 * k], x1 = w[8 * j + 2 * k + 1];
                    o[k] = cvt4_fp8<FMT>(mul_sat<FMT>(lo_f32<T>(x0), scale), mul_sat<FMT>(hi_f32<T>(x0), scale), mul_sat<FMT>(lo_f32<T>(x1), scale),
                                         mul_sat<FMT>(hi_f32<T>(x1), scale));
                }
                if (whole) *reinterpret_cast<uint4 *>(row_stage + row * 128 + ((j ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                else if (live && n0 + 16 * j < a.N) *reinterpret_cast<uint4 *>(a.q_row + in_m * a.N + n0 + 16 * j) = make_uint4(o[0], o[1], o[2], o[3]);
            }
            if (whole) {
                fence_proxy_async_smem();
                sm100::named_barrier<1, kBsGroupThreads>();
                if (row == 0) {
                    tma_store_2d(&tmap_qrow, row_stage, (int) n0, in_row0);   // clipped at the matrix edges
                    bulk_commit_group();
                }
            }
        }
        if (row == 0) bulk_wait_read_all();
    } else {
        // ================================================================ column-wise copy: thread = (64-row band, column pair)
        const int ct = threadIdx.x - 32 - kBsGroupThreads;
        const int band = ct >> 6, pair = ct & 63;
        const int box = pair >> 5, chunk = (pair & 31) >> 2, sub = (pair & 3) << 2;
        uint32_t stage = 0, phase = 0, tile_i = 0;
        while (true) {
            if (!(ok = mbar_wait_warp(&full_bar[stage], phase, abort_flag))) break;
            const int4 d0 = *reinterpret_cast<const int4 *>(&s_desc[stage]);
            if (d0.z < 0) break;
            const int pid_m = d0.y, col_blk = d0.z;
            const int n_valid = SEG ? s_desc[stage].n_valid : kBlk;
            uint32_t w[64];
            {
                const uint8_t *cp = smem + stage * kBqTileBytes + box * (kBqTileBytes / 2) + band * 64 * 128 + sub;
#pragma unroll
                for (int r = 0; r < 64; ++r) {   // (64 band + r) % 8 == r % 8; a warp reads one 128-byte box row: no bank conflict
                    const uint32_t v = *reinterpret_cast<const uint32_t *>(cp + r * 128 + ((chunk ^ (r & 7)) << 4));
                    w[r] = (!SEG || band * 64 + r < n_valid) ? v : 0u;   // rows past the group's end count (and are written) as zeros
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);
            if (++stage == kBsStages) { stage = 0; phase ^= 1; }
            const int buf = tile_i & 1;
            ++tile_i;
            uint32_t m2 = 0u;
#pragma unroll
            for (int r = 0; r < 64; ++r) m2 = absmax2<T>(m2, w[r]);
            s_cmax[buf][ct] = m2;   // [band][pair] flattened: ct = 64 band + pair
            if (ct == 0) bulk_wait_read_all();   // the previous tile's store has read the staging tile
            sm100::named_barrier<2, kBsGroupThreads>();
            m2 = absmax2_done(absmax2<T>(m2, s_cmax[buf][ct ^ 64]));
            const float sc0 = scale_from_amax<FMT>(lo_f32<T>(m2), kEpsBlock), sc1 = scale_from_amax<FMT>(hi_f32<T>(m2), kEpsBlock);
            const int64_t n0 = (int64_t) col_blk * kBlk;
            const int64_t gc = n0 + 2 * pair;
            if (band == 0 && gc < a.N)
                *reinterpret_cast<float2 *>(a.s_col + (int64_t) pid_m * a.N + gc) = make_float2(__fdiv_rn(1.0f, sc0), __fdiv_rn(1.0f, sc1));
            // staged row-major: byte (row, column c) at row * 128 + swizzled chunk c / 16 + c % 16
            {
                const int c = 2 * pair;
                uint8_t *sp = col_stage + band * 64 * 128 + (c & 15);
                const int oc = c >> 4;
#pragma unroll
                for (int r = 0; r < 64; ++r) {
                    const uint16_t o = cvt2_fp8<FMT>(mul_sat<FMT>(lo_f32<T>(w[r]), sc0), mul_sat<FMT>(hi_f32<T>(w[r]), sc1));
                    *reinterpret_cast<uint16_t *>(sp + r * 128 + ((oc ^ (r & 7)) << 4)) = o;
                }
            }
            fence_proxy_async_smem();
            sm100::named_barrier<2, kBsGroupThreads>();
            if (ct == 0) {
                tma_store_2d(&tmap_qcol, col_stage, (int) n0, pid_m * kBlk);
                bulk_commit_group();
            }
        }
        if (ct == 0) bulk_wait_read_all();
    }
    if (!ok || *abort_flag) {
        if (a.status && lane == 0) atomicExch(a.status, (int) PT_ERR_TIMEOUT);
        __nanosleep(100000);  // let a copy still in flight land before the shared memory is released
    }
}

// y = float(q) * s for the three block-scale layouts
template <typename T, int FMT>
__global__ void __launch_bounds__(256) dequant_blockwise_kernel(const uint8_t *__restrict__ q,
                                                               const float *__restrict__ s, int kind, int64_t M,
                                                               int64_t N, int64_t total, T *__restrict__ y);

template <int FMT> __device__ __forceinline__ float decode8(uint8_t c) {
    if constexpr (FMT == PT_E5M2) return __half2float(__ushort_as_half((uint16_t) c << 8));
    // e4m3fn -> float: sign | exp(4) | man(3), bias 7
    const uint32_t sign = (uint32_t) (c & 0x80) << 24;
    const uint32_t e = (c >> 3) & 0xF, m = c & 7;
    if (e == 0) return __uint_as_float(sign | __float_as_uint((float) m * 0.001953125f));  // m * 2^-9
    if (e == 15 && m == 7) return __uint_as_float(sign | 0x7FC00000u);
    return __uint_as_float(sign | ((e + 120) << 23) | (m << 20));
}
template <typename T> __device__ __forceinline__ void put(T *p, float v);
template <> __device__ __forceinline__ void put<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void put<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void put<__half>(__half *p, float v) { *p = __float2half_rn(v); }

template <typename T, int FMT>
__global__ void __launch_bounds__(256) dequant_blockwise_kernel(const uint8_t *__restrict__ q,
                                                               const float *__restrict__ s, int kind, int64_t M,
                                                               int64_t N, int64_t total, T *__restrict__ y) {
    const int64_t nb = (N + kBlk - 1) / kBlk, mb = (M + kBlk - 1) / kBlk;
    const int64_t stride = (int64_t) gridDim.x * blockDim.x;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t b = i / (M * N), rem = i % (M * N), m = rem / N, n = rem % N;
        int64_t si;
        if (kind == 0) si = (b * M + m) * nb + n / kBlk;
        else if (kind == 1) si = (b * mb + m / kBlk) * N + n;
        else si = (b * mb + m / kBlk) * nb + n / kBlk;
        put(y + i, decode8<FMT>(q[i]) * __ldg(s + si));
    }
}

// offs[i+1] = sum_{j<=i} ceil_to(lens[j], align); one block, G <= 4096
__global__ void __launch_bounds__(1024) group_offs_kernel(const int64_t *__restrict__ lens, int G, int64_t align,
                                                          int64_t *__restrict__ plens, int64_t *__restrict__ offs) {
    __shared__ int64_t s[1024];
    __shared__ int64_t carry;
    if (threadIdx.x == 0) { carry = 0; offs[0] = 0; }
    __syncthreads();
    for (int base = 0; base < G; base += 1024) {
        const int i = base + threadIdx.x;
        int64_t v = 0;
        if (i < G) {
            v = lens[i];
            if (align > 1) v = (v + align - 1) / align * align;
            if (plens) plens[i] = v;
        }
        s[threadIdx.x] = v;
        __syncthreads();
        for (int d = 1; d < 1024; d <<= 1) {
            const int64_t t = threadIdx.x >= d ? s[threadIdx.x - d] : 0;
            __syncthreads();
            s[threadIdx.x] += t;
            __syncthreads();
        }
        if (i < G) offs[i + 1] = carry + s[threadIdx.x];
        __syncthreads();
        if (threadIdx.x == 1023) carry += s[1023];
        __syncthreads();
    }
}

// zero-fill of rows [*first_row, rows), 4-byte words, grid-stride; nothing to do in the usual case *first_row == rows
__global__ void __launch_bounds__(256) zero_rows_from_kernel(uint32_t *__restrict__ buf, int64_t rows, int64_t row_words,
                                                            const int64_t *__restrict__ first_row) {
    const int64_t begin = min(max(*first_row, (int64_t) 0), rows) * row_words, end = rows * row_words;
    const int64_t stride = (int64_t) gridDim.x * blockDim.x;
    for (int64_t i = begin + (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < end; i += stride) buf[i] = 0u;
}

// tiled transpose of 1/2/4-byte elements; blockIdx.z walks a batch of [M, N] matrices
template <typename E>
__global__ void __launch_bounds__(256) transpose_kernel(const E *__restrict__ x, int64_t M, int64_t N, E *__restrict__ y) {
    __shared__ E tile[64][64 + (sizeof(E) == 1 ? 4 : (sizeof(E) == 2 ? 2 : 1))];
    x += (int64_t) blockIdx.z * M * N;
    y += (int64_t) blockIdx.z * M * N;
    const int64_t m0 = (int64_t) blockIdx.y * 64, n0 = (int64_t) blockIdx.x * 64;
    const int tx = threadIdx.x % 64, ty = threadIdx.x / 64;
    for (int r = ty; r < 64; r += 4)
        if (m0 + r < M && n0 + tx < N) tile[r][tx] = x[(m0 + r) * N + n0 + tx];
    __syncthreads();
    for (int r = ty; r < 64; r += 4)
        if (n0 + r < N && m0 + tx < M) y[(n0 + r) * M + m0 + tx] = tile[tx][r];
}

// Grouped transpose with segment padding of a byte matrix: x [M, C] holds G groups of rows (group g = rows
// offs[g] .. offs[g+1]); y [C, T] receives group g's rows as columns poffs[g] .. poffs[g] + len_g, the rest of each
// 128-aligned segment and everything from poffs[G] on as zero bytes.  A block moves 64 padded columns x 64 source
// columns; segments start on multiples of 128, so the 64 padded columns of a block belong to one group.
// Shared-memory layout: row r keeps its four 16-byte chunks at chunk index (chunk ^ (r >> 4)), which spreads the
// transposed byte reads of the four thread quarters over different banks.
__global__ void __launch_bounds__(256)
    grouped_transpose_pad_kernel(const uint8_t *__restrict__ x, int64_t C, int vec_ok, const int64_t *__restrict__ offs,
                                 const int64_t *__restrict__ poffs, int G, uint8_t *__restrict__ y, int64_t T) {
    __shared__ __align__(16) uint8_t tile[64][80];
    __shared__ int64_t s_src;
    __shared__ int s_valid;
    const int64_t t0 = (int64_t) blockIdx.y * 64, c0 = (int64_t) blockIdx.x * 64;
    if (threadIdx.x == 0) {
        int valid = 0;
        int64_t src = 0;
        if (G > 0 && t0 < poffs[G]) {
            int lo = 0, hi = G - 1;  // last group whose segment starts at or before t0
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (poffs[mid] <= t0) lo = mid;
                else hi = mid - 1;
            }
            const int64_t in_seg = t0 - poffs[lo];
            const int64_t left = offs[lo + 1] - offs[lo] - in_seg;
            valid = (int) max((int64_t) 0, min((int64_t) 64, left));
            src = offs[lo] + in_seg;
        }
        s_valid = valid;
        s_src = src;
    }
    __syncthreads();
    const int valid = s_valid;
    const int r = threadIdx.x >> 2, part = threadIdx.x & 3;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < valid) {
        const int64_t col = c0 + part * 16;
        const uint8_t *p = x + (s_src + r) * C + col;
        if (vec_ok && col + 16 <= C) {
            v = *reinterpret_cast<const uint4 *>(p);
        } else {
            uint8_t b[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) b[k] = col + k < C ? p[k] : (uint8_t) 0;
            v = *reinterpret_cast<uint4 *>(b);
        }
    }
    *reinterpret_cast<uint4 *>(&tile[r][(part ^ (r >> 4)) * 16]) = v;
    __syncthreads();
    const int c = threadIdx.x >> 2;  // output row inside the tile; this thread writes padded columns part*16 .. +15
    if (c0 + c < C) {
        __align__(16) uint8_t b[16];
        const int pos = (((c >> 4) ^ part) << 4) | (c & 15);
#pragma unroll
        for (int k = 0; k < 16; ++k) b[k] = tile[part * 16 + k][pos];
        *reinterpret_cast<uint4 *>(y + (c0 + c) * T + t0 + part * 16) = *reinterpret_cast<uint4 *>(b);
    }
}

// The same for 2-byte elements (bf16 / fp16 operands of the 16-bit variable-K GEMM): 64 padded columns x 64 source
// columns per block through a padded shared-memory tile.
__global__ void __launch_bounds__(256)
    grouped_transpose_pad16_kernel(const uint16_t *__restrict__ x, int64_t C, const int64_t *__restrict__ offs,
                                   const int64_t *__restrict__ poffs, int G, uint16_t *__restrict__ y, int64_t T) {
    __shared__ uint16_t tile[64][64 + 2];
    __shared__ int64_t s_src;
    __shared__ int s_valid;
    const int64_t t0 = (int64_t) blockIdx.y * 64, c0 = (int64_t) blockIdx.x * 64;
    if (threadIdx.x == 0) {
        int valid = 0;
        int64_t src = 0;
        if (G > 0 && t0 < poffs[G]) {
            int lo = 0, hi = G - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (poffs[mid] <= t0) lo = mid;
                else hi = mid - 1;
            }
            const int64_t in_seg = t0 - poffs[lo];
            valid = (int) max((int64_t) 0, min((int64_t) 64, offs[lo + 1] - offs[lo] - in_seg));
            src = offs[lo] + in_seg;
        }
        s_valid = valid;
        s_src = src;
    }
    __syncthreads();
    const int valid = s_valid;
    const int tx = threadIdx.x % 64, ty = threadIdx.x / 64;
    for (int r = ty; r < 64; r += 4)
        tile[r][tx] = (r < valid && c0 + tx < C) ? x[(s_src + r) * C + c0 + tx] : (uint16_t) 0;
    __syncthreads();
    for (int r = ty; r < 64; r += 4)
        if (c0 + r < C) y[(c0 + r) * T + t0 + tx] = tile[tx][r];
}

}  // namespace ptb

using namespace ptb;

template <int MODE>
static int launch_tile(const void *x, int x_dtype, int64_t B, int64_t m_tiles, int64_t M, int64_t N, int fmt,
                       void *q_row, float *s_row, void *q_col, float *s_col, SegmentArgs seg, void *stream) {
    PT_REQUIRE(B <= 65535 && m_tiles <= 65535, "blockwise: too many tiles along M or batch");
    dim3 grid((unsigned) ceil_div(N, kBlk), (unsigned) m_tiles, (unsigned) B);
    const int64_t tiles_n = ceil_div(N, kBlk), total_tiles = tiles_n * m_tiles * B;
    // persistent TMA form: 16-bit input, 16-byte vectors on every output row
    const bool tma_ok = x_dtype != PT_F32 && N % 16 == 0 && aligned(x, 16) && (!q_row || aligned(q_row, 16)) &&
                        (!q_col || aligned(q_col, 16)) && (!s_col || aligned(s_col, 16)) && M < (1ll << 31) && N < (1ll << 31) &&
                        total_tiles < (1ll << 31) && getenv("PT_BW_QUANT_NO_TMA") == nullptr &&
                        seg.num_groups <= kBqMaxGroups && m_tiles * kBlk < (1ll << 31);
    if (tma_ok) {
        CUtensorMap tmap;
        int rc = make_tmap_u16_3d(&tmap, x, B, M, N, kBlk);
        if (rc != PT_OK) return rc;
        if constexpr (MODE == MODE_DUAL || MODE == MODE_SEGMENT) {
            // both copies of a 16-bit input: the warp-split kernel (PT_BW_QUANT_NO_SPLIT=1 keeps the older form)
            if (B == 1 && aligned(s_col, 8) && getenv("PT_BW_QUANT_NO_SPLIT") == nullptr) {
                constexpr bool kSegK = MODE == MODE_SEGMENT;
                CUtensorMap trow, tcol;
                if ((rc = make_tmap_bytes(&trow, q_row, M, N, N, kBlk)) != PT_OK) return rc;
                if ((rc = make_tmap_bytes(&tcol, q_col, kSegK ? m_tiles * kBlk : M, N, N, kBlk)) != PT_OK) return rc;
                BqArgs a{M, N, (int) tiles_n, (int) m_tiles, total_tiles, (uint8_t *) q_row, (uint8_t *) q_col, s_row, s_col, seg, default_status(),
                         tile_sched_acquire((cudaStream_t) stream)};
                const int sgrid = (int) std::min<int64_t>(total_tiles, (int64_t) sm_count() * kBsCtasPerSm);
#define PT_BS_LAUNCH(T_)                                                                                           \
                PT_SWITCH_FP8(fmt, F, {                                                                            \
                    auto kern = blockwise_split_kernel<T_, F, kSegK>;                                              \
                    PT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBsSmemBytes)); \
                    PT_CUDA_OK(launch_overlapped(kern, dim3(sgrid), dim3(kBsThreads), kBsSmemBytes, (cudaStream_t) stream, tmap, trow, tcol, a)); \
                })
                if (x_dtype == PT_BF16) { PT_BS_LAUNCH(__nv_bfloat16); } else { PT_BS_LAUNCH(__half); }
#undef PT_BS_LAUNCH
                PT_LAUNCH_OK();
                tile_sched_release(a.sched_slot, (cudaStream_t) stream);
                return PT_OK;
            }
        }
        BqArgs a{M, N, (int) tiles_n, (int) m_tiles, total_tiles, (uint8_t *) q_row, (uint8_t *) q_col, s_row, s_col, seg, default_status(), tile_sched_acquire((cudaStream_t) stream)};
        const int tma_grid = (int) std::min<int64_t>(total_tiles, (int64_t) sm_count() * kBqCtasPerSm);
#define PT_BQ_LAUNCH(T_)                                                                                           \
        PT_SWITCH_FP8(fmt, F, {                                                                                    \
            auto kern = blockwise_tma_kernel<T_, F, MODE>;                                                         \
            PT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBqSmemBytes));     \
            PT_CUDA_OK(launch_overlapped(kern, dim3(tma_grid), dim3(kBqThreads), kBqSmemBytes, (cudaStream_t) stream, tmap, a)); \
        })
        if (x_dtype == PT_BF16) { PT_BQ_LAUNCH(__nv_bfloat16); } else { PT_BQ_LAUNCH(__half); }
#undef PT_BQ_LAUNCH
        PT_LAUNCH_OK();
        tile_sched_release(a.sched_slot, (cudaStream_t) stream);
        return PT_OK;
    }
    PT_SWITCH_SRC(x_dtype, T, {
        const int vec_ok = aligned(x, 16) && (N % 8 == 0) && (!q_row || aligned(q_row, 8)) && (!q_col || aligned(q_col, 8));
        PT_SWITCH_FP8(fmt, F, {
            blockwise_tile_kernel<T, F, MODE><<<grid, kTileThreads, 0, (cudaStream_t) stream>>>(
                (const T *) x, M, N, vec_ok, (uint8_t *) q_row, s_row, (uint8_t *) q_col, s_col, seg);
        });
        PT_LAUNCH_OK();
    });
    return PT_OK;
}

extern "C" {

int pt_quantize_fp8_blockwise(const void *x, int x_dtype, int64_t M, int64_t N, int fmt, void *q_row, float *s_row,
                              void *q_col, float *s_col, void *stream) {
    PT_REQUIRE(M >= 0 && N >= 0, "blockwise: negative shape");
    const bool row = q_row != nullptr, col = q_col != nullptr;
    PT_REQUIRE(row || col, "blockwise: no output requested");
    PT_REQUIRE((!row || s_row) && (!col || s_col), "blockwise: missing scale output");
    if (M * N == 0) return PT_OK;
    PT_REQUIRE(x, "blockwise: null input");
    SegmentArgs seg{nullptr, nullptr, 0};
    const int64_t mt = ceil_div(M, kBlk);
    if (row && col) return launch_tile<MODE_DUAL>(x, x_dtype, 1, mt, M, N, fmt, q_row, s_row, q_col, s_col, seg, stream);
    if (row) return launch_tile<MODE_ROW>(x, x_dtype, 1, mt, M, N, fmt, q_row, s_row, nullptr, nullptr, seg, stream);
    return launch_tile<MODE_COL>(x, x_dtype, 1, mt, M, N, fmt, nullptr, nullptr, q_col, s_col, seg, stream);
}

int pt_quantize_fp8_blockwise_weight(const void *w, int x_dtype, int64_t B, int64_t M, int64_t N, int fmt, void *q,
                                     float *s, void *stream) {
    PT_REQUIRE(B >= 0 && M >= 0 && N >= 0, "blockwise weight: negative shape");
    if (B * M * N == 0) return PT_OK;
    PT_REQUIRE(w && q && s, "blockwise weight: null pointer");
    SegmentArgs seg{nullptr, nullptr, 0};
    return launch_tile<MODE_WEIGHT>(w, x_dtype, B, ceil_div(M, kBlk), M, N, fmt, q, s, nullptr, nullptr, seg, stream);
}

int pt_quantize_fp8_blockwise_segment_m(const void *x, int x_dtype, int64_t M, int64_t N, int G,
                                        const int64_t *group_offs, const int64_t *padded_offs, int fmt, void *q_row,
                                        float *s_row, void *q_col, float *s_col, void *stream) {
    PT_REQUIRE(M >= 0 && N >= 0 && G >= 1, "segment-M: bad shape");
    PT_REQUIRE(group_offs && padded_offs && q_row && s_row && q_col && s_col, "segment-M: null pointer");
    if (N == 0) return PT_OK;
    SegmentArgs seg{group_offs, padded_offs, G};
    const int64_t m_alloc = M + (int64_t) G * kBlk;
    return launch_tile<MODE_SEGMENT>(x, x_dtype, 1, ceil_div(m_alloc, kBlk), M, N, fmt, q_row, s_row, q_col, s_col, seg,
                                     stream);
}

int pt_dequantize_fp8_blockwise(const void *q, int fmt, const float *s, int kind, int64_t B, int64_t M, int64_t N,
                                void *y, int y_dtype, void *stream) {
    const int64_t total = B * M * N;
    PT_REQUIRE(total >= 0 && kind >= 0 && kind <= 2, "blockwise dequantize: bad arguments");
    if (total == 0) return PT_OK;
    PT_REQUIRE(q && s && y, "blockwise dequantize: null pointer");
    const int blocks = (int) std::min<int64_t>(ceil_div(total, 256), (int64_t) sm_count() * 16);
    PT_SWITCH_SRC(y_dtype, T, {
        PT_SWITCH_FP8(fmt, F, {
            dequant_blockwise_kernel<T, F><<<blocks, 256, 0, (cudaStream_t) stream>>>((const uint8_t *) q, s, kind, M, N,
                                                                                      total, (T *) y);
        });
        PT_LAUNCH_OK();
    });
    return PT_OK;
}

int pt_compute_group_offs(const int64_t *lens, int G, int64_t *offs, void *stream) {
    PT_REQUIRE(lens && offs && G >= 0 && G <= 4096, "group offsets: bad arguments");
    group_offs_kernel<<<1, 1024, 0, (cudaStream_t) stream>>>(lens, G, 1, nullptr, offs);
    PT_LAUNCH_OK();
    return PT_OK;
}

int pt_compute_padded_group_offs(const int64_t *lens, int G, int64_t align, int64_t *plens, int64_t *poffs,
                                 void *stream) {
    PT_REQUIRE(lens && poffs && G >= 0 && G <= 4096 && align >= 1, "padded group offsets: bad arguments");
    group_offs_kernel<<<1, 1024, 0, (cudaStream_t) stream>>>(lens, G, align, plens, poffs);
    PT_LAUNCH_OK();
    return PT_OK;
}

int pt_zero_rows_from(void *buf, int64_t rows, int64_t row_bytes, const int64_t *first_row, void *stream) {
    PT_REQUIRE(rows >= 0 && row_bytes >= 0 && row_bytes % 4 == 0, "zero rows: bad extents");
    if (rows == 0 || row_bytes == 0) return PT_OK;
    PT_REQUIRE(buf && first_row && aligned(buf, 4), "zero rows: null or unaligned pointer");
    // the tail is normally empty or a few rows: a small fixed grid is enough
    zero_rows_from_kernel<<<sm_count() * 4, 256, 0, (cudaStream_t) stream>>>((uint32_t *) buf, rows, row_bytes / 4, first_row);
    PT_LAUNCH_OK();
    return PT_OK;
}

int pt_grouped_transpose_pad(const void *x, int64_t M, int64_t C, int elem_bytes, const int64_t *group_offs,
                             const int64_t *padded_offs, int G, void *y, int64_t T, void *stream) {
    PT_REQUIRE(M >= 0 && C >= 0 && T >= 0 && G >= 0, "grouped transpose: negative extent");
    PT_REQUIRE(elem_bytes == 1 || elem_bytes == 2, "grouped transpose: 1- or 2-byte elements");
    if (C == 0 || T == 0) return PT_OK;
    PT_REQUIRE(y && group_offs && padded_offs && (x || M == 0), "grouped transpose: null pointer");
    PT_REQUIRE(T % 64 == 0 && aligned(y, 16), "grouped transpose: the padded token count must be a multiple of 64 and y 16-byte aligned");
    PT_REQUIRE(T / 64 <= 65535, "grouped transpose: too many tokens");
    const int vec_ok = C % 16 == 0 && aligned(x, 16);
    dim3 grid((unsigned) ceil_div(C, 64), (unsigned) (T / 64));
    if (elem_bytes == 2) {
        grouped_transpose_pad16_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>((const uint16_t *) x, C, group_offs, padded_offs, G,
                                                                                (uint16_t *) y, T);
        PT_LAUNCH_OK();
        return PT_OK;
    }
    grouped_transpose_pad_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>((const uint8_t *) x, C, vec_ok, group_offs, padded_offs, G,
                                                                          (uint8_t *) y, T);
    PT_LAUNCH_OK();
    return PT_OK;
}

int pt_transpose_2d(const void *x, int64_t M, int64_t N, int elem_bytes, void *y, void *stream) {
    return pt_transpose_batched(x, 1, M, N, elem_bytes, y, stream);
}

int pt_transpose_batched(const void *x, int64_t B, int64_t M, int64_t N, int elem_bytes, void *y, void *stream) {
    PT_REQUIRE(B >= 0 && M >= 0 && N >= 0, "transpose: negative shape");
    if (B * M * N == 0) return PT_OK;
    PT_REQUIRE(x && y, "transpose: null pointer");
    PT_REQUIRE(ceil_div(M, 64) <= 65535 && B <= 65535, "transpose: M or batch too large");
    dim3 grid((unsigned) ceil_div(N, 64), (unsigned) ceil_div(M, 64), (unsigned) B);
    cudaStream_t st = (cudaStream_t) stream;
    if (elem_bytes == 1) transpose_kernel<uint8_t><<<grid, 256, 0, st>>>((const uint8_t *) x, M, N, (uint8_t *) y);
    else if (elem_bytes == 2) transpose_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t *) x, M, N, (uint16_t *) y);
    else if (elem_bytes == 4) transpose_kernel<uint32_t><<<grid, 256, 0, st>>>((const uint32_t *) x, M, N, (uint32_t *) y);
    else return set_error(PT_ERR_INVALID, "transpose: element size %d not supported", elem_bytes);
    PT_LAUNCH_OK();
    return PT_OK;
}

}  // extern "C"
