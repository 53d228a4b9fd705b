// MX (32-element block, ue8m0 scale) quantization to e4m3 / e5m2 / e2m1 and the matching dequantize.
//
// One CTA owns a 128 (rows) x 64 (cols) tile of the bf16 / fp16 input.  The row-wise copy is produced
// straight from the registers the tile was loaded into (4 lanes x 8 elements per 32-block, amax by
// warp shuffle); the col-wise (transposed) copy is produced from a shared-memory image of the tile,
// one thread per (column, 32-row band).  The input is read from HBM once for both copies.
//
// Arithmetic follows csrc/kernels/quantization/quantization_mxfp8.cu:68-214 and
// quantization_mxfp4.cu:91-227 of the reference:
//   e    = (((bits(amax) + (1 << (22 - mbits))) >> 23) & 0x1FF) - 127 - emax_target, clamped to [-127, 128]
//   byte = e + 127, scale = 2^e
//   fp8:  q = rne(clamp(v, +-qmax * scale) / scale)  (a NaN becomes -qmax)        fp4: q = rne_sat(v / scale)
// A block whose scale byte is 0 (every |v| < 2^-118 or so) is written as zeros.
#include <algorithm>
#include <atomic>
#include <type_traits>

#include "common.cuh"
#include "gemm_common.cuh"
#include "sm100_ptx.cuh"
#include "act_math.cuh"
#include "tile_sched.cuh"

namespace ptb {

constexpr int kTileM = 128;
constexpr int kTileN = 64;
constexpr int kMxThreads = 256;
constexpr int kSmemStride = kTileN + 2;  // halfwords; keeps 4-byte alignment of pairs

template <int FMT> struct MxParams;
template <> struct MxParams<PT_E4M3> { static constexpr int mbits = 3, target = 8; static constexpr float qmax = 448.f; };
template <> struct MxParams<PT_E5M2> { static constexpr int mbits = 2, target = 15; static constexpr float qmax = 57344.f; };
template <> struct MxParams<PT_E2M1> { static constexpr int mbits = 1, target = 2; static constexpr float qmax = 6.f; };

struct MxScale {
    uint8_t byte;
    float native;  // 2^e as the reference builds it: (byte << 23) reinterpret; 0.0f for byte 0
    float inv;     // 2^-e, exact
};

template <int FMT> __device__ __forceinline__ MxScale mx_scale(float amax, bool zero_is_one) {
    const uint32_t bits = __float_as_uint(amax);
    int e = (int) (((bits + (1u << (22 - MxParams<FMT>::mbits))) >> 23) & 0x1FFu) - 127 - MxParams<FMT>::target;
    e = max(-127, min(128, e));
    MxScale s;
    if (zero_is_one && amax == 0.f) e = 0;  // grouped kernels: an all-zero block gets scale 1.0 (byte 127)
    s.byte = (uint8_t) (e + 127);
    s.native = __uint_as_float((uint32_t) s.byte << 23);
    if (e >= -126 && e <= 126) s.inv = __uint_as_float((uint32_t) (127 - e) << 23);
    else if (e == 127) s.inv = __uint_as_float(0x00400000u);  // 2^-127
    else s.inv = 0.f;                                         // byte 0 (data forced to 0) or byte 255
    return s;
}

// ---- stochastic rounding (e2m1 only).  The reference seeds every launch from a process-wide counter and hashes the
// seed with the thread index (quantization_mxfp4.cu:59-71, :518); its results are "unbiased, not bit-exact" by its own
// account.  Here: the same per-launch counter, a 32-bit mixer over (seed, position of the 4-element group), and the
// hardware's stochastic convert, which takes four floats and 32 random bits.
__device__ __forceinline__ uint32_t sr_mix(uint32_t x) {   // "lowbias32" integer hash
    x ^= x >> 16; x *= 0x7feb352du;
    x ^= x >> 15; x *= 0x846ca68bu;
    x ^= x >> 16;
    return x;
}
// four floats -> four e2m1 codes with stochastic rounding, a in the lowest nibble (the instruction puts its FIRST operand
// in the highest nibble)
__device__ __forceinline__ uint32_t cvt4_e2m1_sr(float a, float b, float c, float d, uint32_t rbits) {
    uint16_t r;
    asm("cvt.rs.satfinite.e2m1x4.f32 %0, {%1, %2, %3, %4}, %5;" : "=h"(r) : "f"(d), "f"(c), "f"(b), "f"(a), "r"(rbits));
    return r;
}
static inline uint32_t sr_seed_from(uint32_t n) {   // host: launch number -> seed (never 0)
    uint32_t x = n * 0x9e3779b9u + 0x85ebca6bu;
    x ^= x >> 16; x *= 0x7feb352du;
    x ^= x >> 15; x *= 0x846ca68bu;
    x ^= x >> 16;
    return x | 1u;
}
struct SrState {
    uint32_t key;   // 0: round to nearest even; else seed-derived key, advanced once per 4-element group
    __device__ __forceinline__ bool on() const { return key != 0u; }
    __device__ __forceinline__ uint32_t next() { key = sr_mix(key + 0x9e3779b9u); return key; }
};

// 8 scaled values -> 8 codes packed into 8 bytes (fp8) or 4 bytes (fp4)
template <int FMT> __device__ __forceinline__ uint2 mx_encode8(const float (&v)[8], const MxScale &s, SrState *sr = nullptr) {
    uint2 o = make_uint2(0u, 0u);
    if (s.byte == 0) return o;
    float t[8];
    if constexpr (FMT == PT_E2M1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) t[i] = v[i] * s.inv;
        if (sr != nullptr && sr->on()) {
            o.x = cvt4_e2m1_sr(t[0], t[1], t[2], t[3], sr->next()) | (cvt4_e2m1_sr(t[4], t[5], t[6], t[7], sr->next()) << 16);
            return o;
        }
        o.x = (uint32_t) cvt2_e2m1(t[0], t[1]) | ((uint32_t) cvt2_e2m1(t[2], t[3]) << 8) |
              ((uint32_t) cvt2_e2m1(t[4], t[5]) << 16) | ((uint32_t) cvt2_e2m1(t[6], t[7]) << 24);
    } else {
        // the reference clamps to +-qmax * scale first (fmin(fmax(v, -lim), lim)); the saturating convert below does
        // that for every non-NaN input, so only the half that decides what a NaN becomes is kept: fmax(NaN, -lim) = -lim
        const float nlim = -MxParams<FMT>::qmax * s.native;
#pragma unroll
        for (int i = 0; i < 8; ++i) t[i] = fmaxf(v[i], nlim) * s.inv;
        o.x = cvt4_fp8<FMT>(t[0], t[1], t[2], t[3]);
        o.y = cvt4_fp8<FMT>(t[4], t[5], t[6], t[7]);
    }
    return o;
}

// 16-point Hadamard over v[0..15] (four runs of 4), operation order of quantization_mxfp4.cu:91-136
__device__ __forceinline__ void rht16(float *v) {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        float *p = v + 4 * t;
        const float a0 = p[0] + p[1], a1 = p[0] - p[1], a2 = p[2] + p[3], a3 = p[2] - p[3];
        p[0] = a0 + a2; p[2] = a0 - a2; p[1] = a1 + a3; p[3] = a1 - a3;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // partner = run xor 1: odd run takes (partner - own), even (partner + own)
        const float r0 = v[i], r1 = v[4 + i], r2 = v[8 + i], r3 = v[12 + i];
        v[i] = r1 + r0; v[4 + i] = r0 - r1; v[8 + i] = r3 + r2; v[12 + i] = r2 - r3;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // partner = run xor 2
        const float r0 = v[i], r1 = v[4 + i], r2 = v[8 + i], r3 = v[12 + i];
        v[i] = (r2 + r0) * 0.25f; v[4 + i] = (r3 + r1) * 0.25f;
        v[8 + i] = (r0 - r2) * 0.25f; v[12 + i] = (r1 - r3) * 0.25f;
    }
}

struct MxArgs {
    const void *x;
    int64_t M, N, M_pad, N_pad;
    uint8_t *q_row, *s_row, *q_col, *s_col;
    int64_t x_gstride, qrow_gstride, srow_gstride, qcol_gstride, scol_gstride;  // per batch entry, in elements/bytes
    // grouped form: rows of x are split into groups; the tile grid runs over the 128-padded row space
    const int64_t *group_offs, *poffs_row, *poffs_col;
    int num_groups;
    uint32_t sr_seed;        // stochastic rounding (e2m1): per-launch seed, never 0 when one of the two flags is set
    int sr_row, sr_col;
    // fused prologue of the warp-split kernel (PRO != 0): the quantized tensor is f(x), computed tile by tile in shared memory
    int64_t x_cols;                 // row length of x when it differs from N (gated activations: 2 N), else 0
    const float *pro_rowvec;        // per input row: the routing probability (gated activations) or rstd (RMSNorm)
    const int64_t *pro_mask;        // gated activations, optional: rows with a zero entry quantize as zeros
    const void *pro_gamma;          // RMSNorm: gain [N], the input's type
    int pro_zero_centered;          // RMSNorm: gain is 1 + gamma
};

// grid: (N_pad / 64, M_pad / 128, G); GROUPED: (N_pad / 64, (M + groups * 128) / 128, 1)
// GROUPED (csrc/kernels/quantization/quantization_mxfp8.cu:979-1709 of the reference): every 128-row tile of the
// 128-padded row space belongs to one group; rows past the group's end read as zero; the col-wise copy is written
// in that padded space, the row-wise copy at the group's own (32-padded for fp8, tight for fp4) offset, real rows
// only; an all-zero block gets scale byte 127.
template <typename T, int FMT, bool ROW, bool COL, bool ROW2D, bool COL2D, bool ROWRHT, bool COLRHT, bool GROUPED = false>
__global__ void __launch_bounds__(kMxThreads) mx_quant_kernel(MxArgs a) {
    constexpr bool kFp4 = FMT == PT_E2M1;
    constexpr bool kNeed2D = (ROW && ROW2D) || (COL && COL2D);
    __shared__ __align__(16) uint16_t s_tile[COL ? kTileM : 1][kSmemStride];
    __shared__ unsigned s_amax2d[4][2];

    const int tid = threadIdx.x;
    const int64_t g = blockIdx.z;
    const int64_t m0 = (int64_t) blockIdx.y * kTileM;  // tile origin: input rows, or padded rows when GROUPED
    const int64_t n0 = (int64_t) blockIdx.x * kTileN;
    const T *x = reinterpret_cast<const T *>(a.x) + g * a.x_gstride;
    int64_t in_row0 = m0, in_end = a.M, row_out0 = m0;
    if constexpr (GROUPED) {
        if (m0 >= a.poffs_col[a.num_groups]) return;
        int lo = 0, hi = a.num_groups - 1;  // last group whose padded start is <= m0 (empty groups are skipped)
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (a.poffs_col[mid] <= m0) lo = mid; else hi = mid - 1;
        }
        const int64_t into = m0 - a.poffs_col[lo];
        in_row0 = a.group_offs[lo] + into;
        in_end = min(a.group_offs[lo + 1], a.M);
        row_out0 = a.poffs_row[lo] + into;
    }

    if constexpr (kNeed2D) {
        if (tid < 8) s_amax2d[tid >> 1][tid & 1] = 0u;
        __syncthreads();
    }

    // ---- load: iteration i covers rows 32 i .. 32 i + 31 (8 lanes x 8 elements per row)
    const int cvec = tid & 7;
    const int rsub = tid >> 3;
    const int64_t gn = n0 + cvec * 8;
    float v[4][8];
    float amax4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t gm = in_row0 + 32 * i + rsub;
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        if (gm < in_end && gn < a.N) {
            const uint4 r = __ldg(reinterpret_cast<const uint4 *>(x + gm * a.N + gn));
            w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            v[i][2 * k] = Src<T>::to_f32((uint16_t) (w[k] & 0xFFFF));
            v[i][2 * k + 1] = Src<T>::to_f32((uint16_t) (w[k] >> 16));
        }
        if constexpr (COL) {
            // keep the raw 16-bit pattern; re-expanded exactly when read back
            uint32_t *dst = reinterpret_cast<uint32_t *>(&s_tile[32 * i + rsub][cvec * 8]);
            dst[0] = w[0]; dst[1] = w[1]; dst[2] = w[2]; dst[3] = w[3];
        }
        if constexpr (kNeed2D) {
            float m = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) m = fmaxf(m, fabsf(v[i][k]));
            amax4[i] = m;
        }
    }
    if constexpr (kNeed2D) {
        // 32 x 32 tile amax: (band i, column half c) collects lanes with cvec / 4 == c
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float m = amax4[i];
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
            if ((tid & 27) == 0) atomicMax(&s_amax2d[i][(tid >> 2) & 1], __float_as_uint(m));
        }
    }
    if constexpr (COL || kNeed2D) __syncthreads();

    // ---- row-wise copy from registers
    if constexpr (ROW) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t gm = in_row0 + 32 * i + rsub;  // input row
            const int64_t go = row_out0 + 32 * i + rsub; // row of the row-wise copy
            float t[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) t[k] = v[i][k];
            if constexpr (ROWRHT) {
                // a 16-group spans two lanes: runs 0,1 in the even lane, runs 2,3 in the odd lane
                float full[16];
                const bool odd = cvec & 1;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float other = __shfl_xor_sync(0xffffffffu, t[k], 1);
                    full[k] = odd ? other : t[k];
                    full[8 + k] = odd ? t[k] : other;
                }
                rht16(full);
#pragma unroll
                for (int k = 0; k < 8; ++k) t[k] = odd ? full[8 + k] : full[k];
            }
            float m;
            if constexpr (ROW2D) {
                m = __uint_as_float(s_amax2d[i][cvec >> 2]);
            } else {
                m = 0.f;
#pragma unroll
                for (int k = 0; k < 8; ++k) m = fmaxf(m, fabsf(t[k]));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
            }
            const MxScale s = mx_scale<FMT>(m, GROUPED);
            SrState sr{a.sr_row ? sr_mix(a.sr_seed ^ (uint32_t) ((gm * a.N_pad + gn) >> 2)) | 1u : 0u};
            const uint2 o = mx_encode8<FMT>(t, s, &sr);
            if (gm < in_end && gn < a.N_pad) {
                uint8_t *qr = a.q_row + g * a.qrow_gstride;
                if constexpr (kFp4) *reinterpret_cast<uint32_t *>(qr + (go * a.N_pad + gn) / 2) = o.x;
                else *reinterpret_cast<uint2 *>(qr + go * a.N_pad + gn) = o;
                if ((cvec & 3) == 0) (a.s_row + g * a.srow_gstride)[go * (a.N_pad / 32) + gn / 32] = s.byte;
            }
        }
    }

    // ---- col-wise (transposed) copy from shared memory: thread = (column tid % 64, band tid / 64)
    if constexpr (COL) {
        const int col = tid & 63;
        const int band = tid >> 6;
        const int64_t gc = n0 + col;
        if (gc < a.N) {
            float c[32];
#pragma unroll
            for (int r = 0; r < 32; ++r) c[r] = Src<T>::to_f32(s_tile[band * 32 + r][col]);
            if constexpr (COLRHT) { rht16(c); rht16(c + 16); }
            float m;
            if constexpr (COL2D) {
                m = __uint_as_float(s_amax2d[band][col >> 5]);
            } else {
                m = 0.f;
#pragma unroll
                for (int r = 0; r < 32; ++r) m = fmaxf(m, fabsf(c[r]));
            }
            const MxScale s = mx_scale<FMT>(m, GROUPED);
            const int64_t gm = m0 + band * 32;
            uint8_t *qc = a.q_col + g * a.qcol_gstride;
            uint32_t w[8];
            SrState sr{a.sr_col ? sr_mix(~a.sr_seed ^ (uint32_t) ((gc * a.M_pad + gm) >> 2)) | 1u : 0u};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float t[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) t[k] = c[8 * j + k];
                const uint2 o = mx_encode8<FMT>(t, s, &sr);
                if constexpr (kFp4) w[j] = o.x; else { w[2 * j] = o.x; w[2 * j + 1] = o.y; }
            }
            if constexpr (kFp4) {
                *reinterpret_cast<uint4 *>(qc + (gc * a.M_pad + gm) / 2) = make_uint4(w[0], w[1], w[2], w[3]);
            } else {
                uint4 *dst = reinterpret_cast<uint4 *>(qc + gc * a.M_pad + gm);
                dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
            (a.s_col + g * a.scol_gstride)[gc * (a.M_pad / 32) + gm / 32] = s.byte;
        }
    }
}

// ------------------------------------------------------------------------------------------------ TMA-pipelined form
// Same arithmetic and outputs as mx_quant_kernel for the non-grouped case, restructured so that input loads are
// always in flight: persistent CTAs (three per SM), one producer thread streaming 128 x 64 tiles into a four-stage
// shared-memory ring with cp.async.bulk.tensor (3-D map [G, M, N]; rows past M and columns past N arrive as zeros),
// eight consumer warps quantizing one tile while the next three are on their way.  The first form issues its loads,
// waits, computes and stores in sequence inside each CTA and reached 44 % of the copy bandwidth; it stays in use
// for the grouped layout, whose row masking a plain TMA box cannot express.
constexpr int kQStages = 4;
constexpr int kQCtasPerSm = 3;
constexpr int kQTileBytes = kTileM * kTileN * 2;
constexpr int kQConsumerWarps = 8;
constexpr int kQThreads = 32 * (1 + kQConsumerWarps);
constexpr int kQSmemBytes = kQStages * kQTileBytes + 1024 + 1024;
constexpr int kQMaxGroups = 256;  // grouped form: offset tables of up to this many groups are held in shared memory

// 32 scaled values -> 32 fp8 codes (8 words) or 32 fp4 codes (4 words).  Of the reference's soft clamp to +-qmax*scale
// only fmax(v, -lim) is kept (it sends a NaN to -qmax as the reference does); the saturating convert does the rest.
template <int FMT> __device__ __forceinline__ void mx_encode32(const float (&v)[32], const MxScale &s, uint32_t (&w)[8], SrState *sr = nullptr) {
    if (s.byte == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = 0u;
        return;
    }
    if constexpr (FMT == PT_E2M1) {
        if (sr != nullptr && sr->on()) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float *t = &v[8 * i];
                w[i] = cvt4_e2m1_sr(t[0] * s.inv, t[1] * s.inv, t[2] * s.inv, t[3] * s.inv, sr->next()) |
                       (cvt4_e2m1_sr(t[4] * s.inv, t[5] * s.inv, t[6] * s.inv, t[7] * s.inv, sr->next()) << 16);
            }
            return;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float *t = &v[8 * i];
            w[i] = (uint32_t) cvt2_e2m1(t[0] * s.inv, t[1] * s.inv) | ((uint32_t) cvt2_e2m1(t[2] * s.inv, t[3] * s.inv) << 8) |
                   ((uint32_t) cvt2_e2m1(t[4] * s.inv, t[5] * s.inv) << 16) | ((uint32_t) cvt2_e2m1(t[6] * s.inv, t[7] * s.inv) << 24);
        }
    } else {
        const float nlim = -MxParams<FMT>::qmax * s.native;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            w[i] = cvt4_fp8<FMT>(fmaxf(v[4 * i], nlim) * s.inv, fmaxf(v[4 * i + 1], nlim) * s.inv,
                                 fmaxf(v[4 * i + 2], nlim) * s.inv, fmaxf(v[4 * i + 3], nlim) * s.inv);
    }
}

// Shared-memory tile as TMA writes it with the 128-byte swizzle: 128 rows of 128 bytes, the 16-byte chunk c of
// row r stored at chunk position c ^ (r % 8).
template <typename T> struct SwizzledTile {
    const uint8_t *base;
    __device__ __forceinline__ uint4 chunk(int row, int c) const {
        return *reinterpret_cast<const uint4 *>(base + row * 128 + ((c ^ (row & 7)) << 4));
    }
    __device__ __forceinline__ uint32_t pair(int row, int col_pair) const {  // elements 2*col_pair, 2*col_pair + 1
        const int c = col_pair >> 2;
        return *reinterpret_cast<const uint32_t *>(base + row * 128 + ((c ^ (row & 7)) << 4) + ((col_pair & 3) << 2));
    }
};

// GROUPED: the tile grid runs over the padded row space of the col-wise copy (see mx_quant_kernel): a tile maps to
// rows [in_row0, in_row0 + n_valid) of one group, later rows of the fetched box belong to the next group and are
// treated as zeros; the row-wise copy goes to the group's own row offset, real rows only.
template <typename T, int FMT, bool ROW, bool COL, bool ROW2D, bool COL2D, bool ROWRHT, bool COLRHT, bool GROUPED = false>
__global__ void __launch_bounds__(kQThreads, kQCtasPerSm)
    mx_quant_tma_kernel(const __grid_constant__ CUtensorMap tmap, MxArgs a, int tiles_n, int tiles_m, int64_t total_tiles, int *status) {
    using namespace sm100;
    constexpr bool kFp4 = FMT == PT_E2M1;
    constexpr bool kNeed2D = (ROW && ROW2D) || (COL && COL2D);
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + kQStages * kQTileBytes);
    uint64_t *empty_bar = full_bar + kQStages;
    __shared__ unsigned s_amax2d[3][4][2];
    __shared__ int s_abort;
    volatile int *abort_flag = &s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < kQStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kQConsumerWarps);
        }
        fence_barrier_init();
        prefetch_tmap(&tmap);
    }
    if (threadIdx.x < 24) (&s_amax2d[0][0][0])[threadIdx.x] = 0u;
    __syncthreads();
    sm100::grid_dep_wait();    // the input may come from the previous kernel, and a GEMM before it may still read the outputs
    sm100::grid_dep_launch();
    bool ok = true;
    // grouped: tile row block tm -> first input row, number of rows of the group in the tile, first row of the
    // row-wise copy; false for tiles past the padded end
    // (the three offset tables are copied to shared memory first: a search through global memory would cost each tile
    // several dependent round trips)
    __shared__ int s_gtab[GROUPED ? 3 * (kQMaxGroups + 1) : 1];
    if constexpr (GROUPED) {
        for (int i = threadIdx.x; i <= a.num_groups; i += blockDim.x) {
            s_gtab[i] = (int) a.poffs_col[i];
            s_gtab[(kQMaxGroups + 1) + i] = (int) a.group_offs[i];
            s_gtab[2 * (kQMaxGroups + 1) + i] = (int) a.poffs_row[i];
        }
        __syncthreads();
    }
    auto locate_group = [&](int tm, int64_t &in_row0, int &n_valid, int64_t &row_out0) -> bool {
        const int *pcol = s_gtab, *goffs = s_gtab + (kQMaxGroups + 1), *prow = s_gtab + 2 * (kQMaxGroups + 1);
        const int m0 = tm * kTileM;
        if (m0 >= pcol[a.num_groups]) return false;
        int lo = 0, hi = a.num_groups - 1;  // last group whose padded start is <= m0 (empty groups are skipped)
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (pcol[mid] <= m0) lo = mid; else hi = mid - 1;
        }
        const int into = m0 - pcol[lo];
        in_row0 = goffs[lo] + into;
        n_valid = max(0, min(kTileM, min(goffs[lo + 1], (int) a.M) - (int) in_row0));
        row_out0 = prow[lo] + into;
        return true;
    };

    if (warp == 0) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            // 32-bit tile arithmetic: 64-bit divisions cost more instructions than quantizing the tile
            const uint32_t per_g = (uint32_t) tiles_n * (uint32_t) tiles_m;
            for (uint32_t t = blockIdx.x; t < (uint32_t) total_tiles; t += gridDim.x) {
                const uint32_t g = t / per_g, rem = t - g * per_g;
                const int tm = (int) (rem / (uint32_t) tiles_n), tn = (int) (rem - (uint32_t) tm * tiles_n);
                int64_t in_row0 = (int64_t) tm * kTileM, row_out0 = 0;
                int n_valid = kTileM;
                if constexpr (GROUPED)
                    if (!locate_group(tm, in_row0, n_valid, row_out0)) continue;
                if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) break;
                mbar_arrive_expect_tx(&full_bar[stage], kQTileBytes);
                sm100::tma_load_3d(smem + stage * kQTileBytes, &tmap, &full_bar[stage], tn * kTileN, (int) in_row0, (int) g);
                if (++stage == kQStages) { stage = 0; phase ^= 1; }
            }
        }
    } else {
        const int tid = threadIdx.x - 32;
        // row-wise work item: one 32-element block per thread (row tid / 2, block tid % 2)
        const int r_row = tid >> 1, r_blk = tid & 1;
        // col-wise work item: two adjacent columns x 16 rows per thread; lanes 2i, 2i+1 share a 32-row block
        const int cw = warp - 1;
        // Two lane layouts.  kWide (no Hadamard transform): a warp owns four column pairs over all 128 rows, lane =
        // (band, half, pair); the eight (band, half) lanes of a column store 8 x 16 = 128 contiguous bytes of the
        // transposed output and its four scale bytes leave as one word.  Their rows are 16 apart (same swizzle phase,
        // same banks), so lane group k = lane / 4 walks its 16 rows in the order r ^ k: eight different phases, no
        // bank conflict; the bytes are put back in order after the convert.  Otherwise (the transform needs the rows in
        // order): a warp owns 16 column pairs of one 32-row band, lanes 2i, 2i+1 hold its two halves.
        constexpr bool kWide = !COLRHT;
        const int c_k = kWide ? (lane >> 2) : 0;                            // row-order key
        const int c_half = kWide ? ((lane >> 2) & 1) : (lane & 1);
        const int c_band = kWide ? (lane >> 3) : (cw >> 1);
        const int c_pair = kWide ? ((cw << 2) | (lane & 3)) : (((cw & 1) << 4) | (lane >> 1));
        const int c_chunk = (c_pair >> 2) ^ c_k;
        const uint32_t c_bsel = 0x3210u ^ (0x1111u * (uint32_t) (c_k & 1)) ^ (0x2222u * (uint32_t) ((c_k >> 1) & 1));
        uint32_t stage = 0, phase = 0, tile_count = 0;
        const uint32_t per_g = (uint32_t) tiles_n * (uint32_t) tiles_m;
        for (uint32_t t = blockIdx.x; t < (uint32_t) total_tiles; t += gridDim.x) {
            const uint32_t gq = t / per_g, rem = t - gq * per_g;
            const int tm = (int) (rem / (uint32_t) tiles_n), tn = (int) (rem - (uint32_t) tm * tiles_n);
            const int64_t g = gq;
            const int64_t m0 = (int64_t) tm * kTileM, n0 = (int64_t) tn * kTileN;
            int64_t in_row0 = m0, row_out0 = m0;
            int n_valid = kTileM;
            if constexpr (GROUPED)
                if (!locate_group(tm, in_row0, n_valid, row_out0)) continue;
            ++tile_count;
            if (!(ok = mbar_wait_warp(&full_bar[stage], phase, abort_flag))) break;
            const SwizzledTile<T> tile{smem + stage * kQTileBytes};
            unsigned(*amax2d)[2] = s_amax2d[tile_count % 3];

            // ---- this thread's row block: 64 bytes = chunks 4 * r_blk .. + 3 of row r_row
            float rv[32];
            float r_amax = 0.f;
            if constexpr (ROW || kNeed2D) {
                uint32_t pm = 0u;  // packed |max| of the 16 words: two elements per instruction
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 q = tile.chunk(r_row, 4 * r_blk + j);
                    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        rv[8 * j + 2 * k] = Src<T>::to_f32((uint16_t) (w[k] & 0xFFFF));
                        rv[8 * j + 2 * k + 1] = Src<T>::to_f32((uint16_t) (w[k] >> 16));
                        pm = absmax2<T>(pm, w[k]);
                    }
                }
                if constexpr (ROW && ROWRHT) {  // the scale follows the transformed values
                    rht16(rv); rht16(rv + 16);
#pragma unroll
                    for (int k = 0; k < 32; ++k) r_amax = fmaxf(r_amax, fabsf(rv[k]));
                } else {
                    pm = absmax2_done(pm);
                    r_amax = fmaxf(lo_f32<T>(pm), hi_f32<T>(pm));
                }
            }
            if constexpr (kNeed2D) {
                // 32 x 32 tile maxima through shared memory (of the untransformed values; RHT and 2-D are never combined).
                // The buffer of the tile after next is cleared here: every consumer has passed the previous tile's barrier.
                if (tid < 8) (&s_amax2d[(tile_count + 1) % 3][0][0])[tid] = 0u;
                float m = r_amax;  // lanes of a warp: 16 rows x 2 blocks; reduce over the rows (lane bits 1..4)
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
                if (lane < 2) atomicMax(&amax2d[r_row >> 5][r_blk], __float_as_uint(m));
                sm100::named_barrier<1, kQConsumerWarps * 32>();
            }

            if constexpr (ROW) {
                // row of the row-wise copy: the input row, or the group's own offset in the grouped form
                const int64_t gm = GROUPED ? row_out0 + r_row : m0 + r_row, gn = n0 + 32 * r_blk;
                const float m = ROW2D ? __uint_as_float(amax2d[r_row >> 5][r_blk]) : r_amax;
                const MxScale sc = mx_scale<FMT>(m, GROUPED);
                uint32_t w[8];
                SrState sr{a.sr_row ? sr_mix(a.sr_seed ^ (uint32_t) ((gm * a.N_pad + gn) >> 2)) | 1u : 0u};
                mx_encode32<FMT>(rv, sc, w, &sr);
                if ((GROUPED ? r_row < n_valid : gm < a.M) && gn < a.N_pad) {
                    uint8_t *qr = a.q_row + g * a.qrow_gstride;
                    if constexpr (kFp4) {
                        *reinterpret_cast<uint4 *>(qr + (gm * a.N_pad + gn) / 2) = make_uint4(w[0], w[1], w[2], w[3]);
                    } else {
                        uint8_t *dst = qr + gm * a.N_pad + gn;
                        if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
                            // one 32-byte store: lanes 2i, 2i+1 then cover a 64-byte row segment in one instruction
                            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(w[0]), "r"(w[1]),
                                         "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
                        } else {
                            reinterpret_cast<uint4 *>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            reinterpret_cast<uint4 *>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        }
                    }
                    (a.s_row + g * a.srow_gstride)[gm * (a.N_pad / 32) + gn / 32] = sc.byte;
                }
            }

            if constexpr (COL) {
                // columns 2 c_pair, 2 c_pair + 1; rows c_band * 32 + c_half * 16 .. + 15
                float c0[16], c1[16];
                uint32_t pmc = 0u;  // packed |max| of (column 2 c_pair, column 2 c_pair + 1)
                const uint8_t *cbase = tile.base + (c_band * 32 + c_half * 16) * 128 + ((c_pair & 3) << 2);
#pragma unroll
                for (int r = 0; r < 16; ++r) {
                    const int rr = r ^ c_k;  // row inside this thread's 16
                    const int row = c_band * 32 + c_half * 16 + rr;
                    // grouped: rows past the group's end hold the next group's data and count as zeros
                    const uint32_t w = (!GROUPED || row < n_valid)
                                           ? *reinterpret_cast<const uint32_t *>(cbase + rr * 128 + ((c_chunk ^ (r & 7)) << 4))
                                           : 0u;
                    c0[r] = Src<T>::to_f32((uint16_t) (w & 0xFFFF));
                    c1[r] = Src<T>::to_f32((uint16_t) (w >> 16));
                    pmc = absmax2<T>(pmc, w);
                }
                if constexpr (COLRHT) { rht16(c0); rht16(c1); }
                float m0c = 0.f, m1c = 0.f;
                if constexpr (COL2D) {
                    m0c = m1c = __uint_as_float(amax2d[c_band][c_pair >> 4]);
                } else {
                    if constexpr (COLRHT) {
#pragma unroll
                        for (int r = 0; r < 16; ++r) { m0c = fmaxf(m0c, fabsf(c0[r])); m1c = fmaxf(m1c, fabsf(c1[r])); }
                    } else {
                        pmc = absmax2_done(pmc);
                        m0c = lo_f32<T>(pmc);
                        m1c = hi_f32<T>(pmc);
                    }
                    m0c = fmaxf(m0c, __shfl_xor_sync(0xffffffffu, m0c, kWide ? 4 : 1));
                    m1c = fmaxf(m1c, __shfl_xor_sync(0xffffffffu, m1c, kWide ? 4 : 1));
                }
                const MxScale s0 = mx_scale<FMT>(m0c, GROUPED), s1 = mx_scale<FMT>(m1c, GROUPED);
                const int64_t gc = n0 + 2 * c_pair;
                const int64_t gm = m0 + c_band * 32 + c_half * 16;
                if (gc < a.N) {  // N is a multiple of 32: both columns are in or out together
                    uint8_t *qc = a.q_col + g * a.qcol_gstride;
                    uint8_t *scl = a.s_col + g * a.scol_gstride;
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const float(&cv)[16] = cc ? c1 : c0;
                        const MxScale &sc = cc ? s1 : s0;
                        float t0[8], t1[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) { t0[k] = cv[k]; t1[k] = cv[8 + k]; }
                        SrState sr{a.sr_col ? sr_mix(~a.sr_seed ^ (uint32_t) (((gc + cc) * a.M_pad + gm) >> 2)) | 1u : 0u};
                        uint2 o0 = mx_encode8<FMT>(t0, sc, &sr), o1 = mx_encode8<FMT>(t1, sc, &sr);
                        if constexpr (kWide) {  // value r holds row r ^ k: undo the permutation on the codes
                            if constexpr (kFp4) {   // 8 codes per word: nibble r of o?.x
                                if (c_k & 1) {
                                    o0.x = ((o0.x & 0x0F0F0F0Fu) << 4) | ((o0.x >> 4) & 0x0F0F0F0Fu);
                                    o1.x = ((o1.x & 0x0F0F0F0Fu) << 4) | ((o1.x >> 4) & 0x0F0F0F0Fu);
                                }
                                const uint32_t sel = 0x3210u ^ (0x1111u * (uint32_t) ((c_k >> 1) & 1)) ^ (0x2222u * (uint32_t) ((c_k >> 2) & 1));
                                o0.x = __byte_perm(o0.x, 0u, sel);
                                o1.x = __byte_perm(o1.x, 0u, sel);
                            } else {                // 4 codes per word: byte r % 4 of word r / 4
                                const bool sw = c_k & 4;
                                const uint32_t a0 = sw ? o0.y : o0.x, a1 = sw ? o0.x : o0.y;
                                const uint32_t b0 = sw ? o1.y : o1.x, b1 = sw ? o1.x : o1.y;
                                o0 = make_uint2(__byte_perm(a0, 0u, c_bsel), __byte_perm(a1, 0u, c_bsel));
                                o1 = make_uint2(__byte_perm(b0, 0u, c_bsel), __byte_perm(b1, 0u, c_bsel));
                            }
                        }
                        if constexpr (kFp4) *reinterpret_cast<uint2 *>(qc + ((gc + cc) * a.M_pad + gm) / 2) = make_uint2(o0.x, o1.x);
                        else *reinterpret_cast<uint4 *>(qc + (gc + cc) * a.M_pad + gm) = make_uint4(o0.x, o0.y, o1.x, o1.y);
                        if constexpr (kWide) {
                            // the four band scales of this column, gathered into the band-0 lane: one 4-byte store
                            uint32_t sb = sc.byte;
                            sb |= __shfl_down_sync(0xffffffffu, sb, 8) << 8;
                            sb |= __shfl_down_sync(0xffffffffu, sb, 16) << 16;
                            if (lane < 4) *reinterpret_cast<uint32_t *>(scl + (gc + cc) * (a.M_pad / 32) + m0 / 32) = sb;
                        } else {
                            if (c_half == 0) scl[(gc + cc) * (a.M_pad / 32) + gm / 32] = sc.byte;
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);  // this warp no longer reads the stage
            if (++stage == kQStages) { stage = 0; phase ^= 1; }
        }
    }
    if (!ok || *abort_flag) {
        if (status && lane == 0) atomicExch(status, (int) PT_ERR_TIMEOUT);
        __nanosleep(100000);  // let a copy still in flight land before the shared memory is released
    }
}

// ------------------------------------------------------------------------------------------------ warp-split form
// The form used for bf16 inputs, both copies, without the Hadamard option.  Same tiles and TMA input ring as
// mx_quant_tma_kernel, but the eight consumer warps are split by output and never synchronise with one another:
//   * four warps produce the row-wise copy, one thread per tile row (two 32-element blocks read as eight 16-byte
//     chunks); the dense FP8 copy is staged as a 128 x 64-byte tile and written with one bulk tensor store per tile
//     (grouped row copies, which need row masks, and fp4 use 32- / 16-byte stores from registers);
//   * four warps produce the transposed copy, one thread per column pair and 32-row band: a whole MX block of each of
//     its two columns, so rows are read in order, every lane of a warp in the same tile row (no bank conflict, no
//     exchange between threads); the 64 x 128-byte (fp4: 64-byte) transposed tile is staged in the swizzled layout and
//     written with one bulk tensor store, the four band scales of a column as one word.
// The two groups synchronise only among their own four warps (one named barrier per tile, around the double-buffered
// staging tile).  The producer thread also resolves each tile's coordinates (and, in the grouped form, its group) once
// and hands them over in shared memory next to the data; outside stream capture it draws tiles from a device counter,
// so CTAs that get ahead take more tiles and all SMs finish together.  (Per-warp stores of 32-byte wide pieces, which
// need no barrier, measured slower: four times as many store transactions.)  Scaling is exact in packed bf16 (the scale is a power of two), so one
// mul.bf16x2 scales two elements.  A block holding a NaN is found with the NaN-propagating packed maximum and patched
// with max.bf16x2(v, -qmax * scale), which is the half of the reference's clamp that decides what a NaN becomes; all
// other blocks skip the clamp (the saturating convert covers it).
constexpr int kSStages = 2;
constexpr int kSCtasPerSm = 3;
constexpr int kSGroupWarps = 4;                       // warps per output copy
constexpr int kSGroupThreads = 32 * kSGroupWarps;
constexpr int kSThreads = 32 * (1 + 2 * kSGroupWarps);
constexpr int kSStageOutBytes = 8192;                 // one staged output tile (fp8: 128 x 64 bytes either way round)


struct TileDesc {
    int tn, tm, g, in_row0, n_valid, row_out0, pad0, pad1;   // tn < 0: no more tiles
};

__device__ __forceinline__ uint32_t absmax2_nan_bf16(uint32_t m, uint32_t w) {
    uint32_t r;
    asm("max.NaN.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(m), "r"(w));
    return r;
}
// either half of a packed bf16 |max| is a NaN
__device__ __forceinline__ bool packed_bf16_has_nan(uint32_t pm) {
    const uint32_t a = pm & 0x7FFF7FFFu;
    return ((a & 0xFFFFu) > 0x7F80u) | ((a >> 16) > 0x7F80u);
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
// max(a, b) per half; a NaN half yields the other operand
__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t bf16_bits_x2(float lo, float hi) {
    return (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xFFFF0000u);
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
// four floats -> four fp8 codes, a in the lowest byte
template <int FMT> __device__ __forceinline__ uint32_t pack4_fp8(float a, float b, float c, float d) {
    uint32_t r;
    if constexpr (FMT == PT_E5M2)
        asm("{ .reg .b16 x, y; cvt.rn.satfinite.e5m2x2.f32 x, %2, %1; cvt.rn.satfinite.e5m2x2.f32 y, %4, %3; mov.b32 %0, {x, y}; }"
            : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d));
    else
        asm("{ .reg .b16 x, y; cvt.rn.satfinite.e4m3x2.f32 x, %2, %1; cvt.rn.satfinite.e4m3x2.f32 y, %4, %3; mov.b32 %0, {x, y}; }"
            : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d));
    return r;
}
// eight floats -> eight e2m1 codes, a in the lowest nibble
__device__ __forceinline__ uint32_t pack8_e2m1(float a, float b, float c, float d, float e, float f, float g, float h) {
    uint32_t r;
    asm("{ .reg .b8 x, y, z, w; cvt.rn.satfinite.e2m1x2.f32 x, %2, %1; cvt.rn.satfinite.e2m1x2.f32 y, %4, %3;"
        " cvt.rn.satfinite.e2m1x2.f32 z, %6, %5; cvt.rn.satfinite.e2m1x2.f32 w, %8, %7; mov.b32 %0, {x, y, z, w}; }"
        : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d), "f"(e), "f"(f), "f"(g), "f"(h));
    return r;
}
// 3-D tiled store shared -> global (bulk-group completion), cf. tma_store_2d
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *m, const void *smem_src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(reinterpret_cast<uint64_t>(m)),
                 "r"(sm100::smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}

// 16 packed words (one 32-element block of a row) -> 8 words of fp8 codes or 4 words of e2m1 codes
template <int FMT> __device__ __forceinline__ void encode_row_block(const uint32_t *x, uint32_t inv2, uint32_t *o) {
    if constexpr (FMT == PT_E2M1) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t s0 = mul_bf16x2(x[4 * k], inv2), s1 = mul_bf16x2(x[4 * k + 1], inv2);
            const uint32_t s2 = mul_bf16x2(x[4 * k + 2], inv2), s3 = mul_bf16x2(x[4 * k + 3], inv2);
            o[k] = pack8_e2m1(bf16_lo(s0), bf16_hi(s0), bf16_lo(s1), bf16_hi(s1), bf16_lo(s2), bf16_hi(s2), bf16_lo(s3), bf16_hi(s3));
        }
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t s0 = mul_bf16x2(x[2 * k], inv2), s1 = mul_bf16x2(x[2 * k + 1], inv2);
            o[k] = pack4_fp8<FMT>(bf16_lo(s0), bf16_hi(s0), bf16_lo(s1), bf16_hi(s1));
        }
    }
}

// Loads in kernels that are launched to overlap their predecessor (launch_overlapped) and read what it wrote: the grid
// exists before that data does, and the read-only path (ld.global.nc, __ldg, const __restrict__ kernel parameters) is
// defined for data that does not change during the grid's lifetime.  These kernels therefore read such data (row
// statistics, probabilities, gains, scales) with __ldcg.
//
// Fused prologues: what is quantized is f(x), computed once per tile in shared memory by all eight consumer warps before
// the two groups go their own ways.  The arithmetic is that of the stand-alone kernels (act_math.cuh), rounded to bf16
// as they round, so "activation kernel, then quantizer" and the fused kernel write the same bytes.
enum { PT_PRO_NONE = 0, PT_PRO_SWIGLU = 1, PT_PRO_GEGLU = 2, PT_PRO_RMSNORM = 3 };
constexpr bool pro_is_glu(int pro) { return pro == PT_PRO_SWIGLU || pro == PT_PRO_GEGLU; }
// a gated activation needs two input tiles per stage (the two halves of the row)
constexpr int split_stage_bytes(int pro) { return pro_is_glu(pro) ? 2 * kQTileBytes : kQTileBytes; }
constexpr int split_smem_bytes(int pro) { return kSStages * split_stage_bytes(pro) + 4 * kSStageOutBytes + 1024 + 1024; }
constexpr int split_ctas_per_sm(int pro) { return pro_is_glu(pro) ? 2 : kSCtasPerSm; }

// RMSNorm: thread t owns one 8-column chunk (its gains unpacked once) in rows t / 8 + {0, 32, 64, 96}; two packed fp32
// multiplies per pair of elements, each rounding like the scalar x * rstd * g of the stand-alone kernel.  (Fetching the
// gains and row statistics one tile ahead, off a barrier on the published descriptor, did not change the time: the
// prologue is bound by its instructions, not by these loads.)
struct RmsAux {
    uint4 gv;
    float rv[4];
};
__device__ __forceinline__ void split_prologue_rmsnorm(uint8_t *tile, int t, int in_row0, int tn, const MxArgs &a) {
    const int c = t & 7, r0 = t >> 3;
    RmsAux x;
    const int64_t n = (int64_t) tn * kTileN + c * 8;
    x.gv = make_uint4(0u, 0u, 0u, 0u);
    if (n < a.N) x.gv = __ldcg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(a.pro_gamma) + n));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int64_t grow = (int64_t) in_row0 + r0 + 32 * j;
        x.rv[j] = grow < a.M ? __ldcg(a.pro_rowvec + grow) : 0.f;
    }
    const uint32_t gw[4] = {x.gv.x, x.gv.y, x.gv.z, x.gv.w};
    const float zc = a.pro_zero_centered ? 1.0f : 0.0f;
    uint64_t g2[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) asm("mov.b64 %0, {%1, %2};" : "=l"(g2[k]) : "f"(bf16_lo(gw[k]) + zc), "f"(bf16_hi(gw[k]) + zc));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int row = r0 + 32 * j;
        if ((int64_t) in_row0 + row >= a.M) continue;   // zero-filled rows stay +0 (0 * rstd * negative gain would make them -0)
        uint8_t *pa = tile + row * 128 + ((c ^ (r0 & 7)) << 4);
        const uint4 av = *reinterpret_cast<const uint4 *>(pa);
        const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
        uint32_t ow[4];
        uint64_t r2;
        asm("mov.b64 %0, {%1, %1};" : "=l"(r2) : "f"(x.rv[j]));
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float lo, hi;
            asm("{\n\t.reg .b64 xx;\n\tmov.b64 xx, {%2, %3};\n\tmul.rn.f32x2 xx, xx, %4;\n\tmul.rn.f32x2 xx, xx, %5;\n\tmov.b64 {%0, %1}, xx;\n\t}"
                : "=f"(lo), "=f"(hi)
                : "f"(bf16_lo(aw[k])), "f"(bf16_hi(aw[k])), "l"(r2), "l"(g2[k]));
            const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
            ow[k] = *reinterpret_cast<const uint32_t *>(&r);
        }
        *reinterpret_cast<uint4 *>(pa) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    sm100::fence_proxy_async_smem();   // the next bulk load into this stage must order after these writes
    sm100::named_barrier<3, 2 * kSGroupThreads>();
}

// t: 0 .. 255 over the consumer threads; thread (row = t / 2, half = t % 2) transforms 32 elements of its row in place
template <int PRO>
__device__ __forceinline__ void split_prologue(uint8_t *tile, int t, int in_row0, int tn, const MxArgs &a) {
    static_assert(PRO != PT_PRO_RMSNORM, "the RMSNorm prologue is split_prologue_rmsnorm");
    const int row = t >> 1, half = t & 1;
    const int64_t grow = (int64_t) in_row0 + row;
    const bool in = grow < a.M;
    const float rv = in ? __ldcg(a.pro_rowvec + grow) : 0.f;
    bool masked = false;
    if constexpr (pro_is_glu(PRO)) masked = in && a.pro_mask != nullptr && __ldcg(a.pro_mask + grow) == 0;
    uint8_t *rp = tile + row * 128;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        if (!in) break;   // zero-filled rows stay +0 (0 * rstd * negative gain would make them -0)
        const int chunk = 4 * half + c;
        uint8_t *pa = rp + ((chunk ^ (row & 7)) << 4);
        const uint4 av = *reinterpret_cast<const uint4 *>(pa);
        const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
        uint32_t ow[4];
        if constexpr (pro_is_glu(PRO)) {
            constexpr int ACT = PRO == PT_PRO_SWIGLU ? PT_ACT_SILU : PT_ACT_GELU;
            const uint4 bv = *reinterpret_cast<const uint4 *>(pa + kQTileBytes);
            const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float lo = glu_value<ACT>(bf16_lo(aw[k]), bf16_lo(bw[k]), rv), hi = glu_value<ACT>(bf16_hi(aw[k]), bf16_hi(bw[k]), rv);
                const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
                ow[k] = masked ? 0u : *reinterpret_cast<const uint32_t *>(&r);
            }
        } else {
            const int64_t n = (int64_t) tn * kTileN + chunk * 8;
            uint4 gv = make_uint4(0u, 0u, 0u, 0u);
            if (n < a.N) gv = __ldcg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(a.pro_gamma) + n));
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
            const float zc = a.pro_zero_centered ? 1.0f : 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float lo = rmsnorm_value(bf16_lo(aw[k]), rv, bf16_lo(gw[k]) + zc), hi = rmsnorm_value(bf16_hi(aw[k]), rv, bf16_hi(gw[k]) + zc);
                const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
                ow[k] = *reinterpret_cast<const uint32_t *>(&r);
            }
        }
        *reinterpret_cast<uint4 *>(pa) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    sm100::fence_proxy_async_smem();   // the next bulk load into this stage must order after these writes
    sm100::named_barrier<3, 2 * kSGroupThreads>();
}

// The quantization of one 32-element block held by four neighbouring lanes, eight bf16 values (four packed words) each:
// |max| over the four lanes (NaN ignored), ue8m0 scale, codes.  Every lane of the warp must call it.  Returns the scale
// byte; `out` receives 8 fp8 codes (two words) or 8 e2m1 codes (one word).
template <int FMT>
__device__ __forceinline__ uint8_t mx_block_of_four_lanes(uint32_t (&y)[4], uint32_t (&out)[2]) {
    using T = __nv_bfloat16;
    constexpr bool kFp4 = FMT == PT_E2M1;
    uint32_t pm = 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i) pm = absmax2_nan_bf16(pm, y[i]);
    pm = absmax2_nan_bf16(pm, __shfl_xor_sync(0xffffffffu, pm, 1));
    pm = absmax2_nan_bf16(pm, __shfl_xor_sync(0xffffffffu, pm, 2));
    const bool has_nan = packed_bf16_has_nan(pm);
    if (__any_sync(0xffffffffu, has_nan)) {   // a NaN element takes no part in the maximum (rare: the whole warp redoes it)
        uint32_t pq = 0u;
#pragma unroll
        for (int i = 0; i < 4; ++i) pq = absmax2<T>(pq, y[i]);
        pq = absmax2<T>(pq, __shfl_xor_sync(0xffffffffu, pq, 1));
        pq = absmax2<T>(pq, __shfl_xor_sync(0xffffffffu, pq, 2));
        if (has_nan) pm = pq;
    }
    pm = absmax2_done(pm);
    const MxScale sc = mx_scale<FMT>(fmaxf(bf16_lo(pm), bf16_hi(pm)), false);
    if (has_nan && !kFp4) {
        const float nlim = -MxParams<FMT>::qmax * sc.native;
        const uint32_t nlim2 = bf16_bits_x2(nlim, nlim);
#pragma unroll
        for (int i = 0; i < 4; ++i) y[i] = max_bf16x2(y[i], nlim2);
    }
    const uint32_t inv2 = bf16_bits_x2(sc.inv, sc.inv);
    const uint32_t s0 = mul_bf16x2(y[0], inv2), s1 = mul_bf16x2(y[1], inv2), s2 = mul_bf16x2(y[2], inv2), s3 = mul_bf16x2(y[3], inv2);
    if constexpr (kFp4) {
        out[0] = pack8_e2m1(bf16_lo(s0), bf16_hi(s0), bf16_lo(s1), bf16_hi(s1), bf16_lo(s2), bf16_hi(s2), bf16_lo(s3), bf16_hi(s3));
        out[1] = 0u;
    } else {
        out[0] = pack4_fp8<FMT>(bf16_lo(s0), bf16_hi(s0), bf16_lo(s1), bf16_hi(s1));
        out[1] = pack4_fp8<FMT>(bf16_lo(s2), bf16_hi(s2), bf16_lo(s3), bf16_hi(s3));
    }
    if (sc.byte == 0) out[0] = out[1] = 0u;
    return sc.byte;
}

// RMSNorm and the row-wise MX copy in one pass over x (the forward-only / inference form: no transposed copy): a block
// reads a row into registers, forms rstd in the order of the stand-alone RMSNorm kernel (activation_norm.cu: per-thread
// sums over its vectors in turn, eight warp reductions, then the eight warp sums in turn), normalises with its
// arithmetic and rounding, and quantizes each 32-element block, which sits in four neighbouring threads (eight elements
// each): two shuffles give the block |max|.  The bytes are those of the RMSNorm kernel followed by the row-wise quantizer.
// ncu on 8192 x 4096: 24 thread instructions per element, issue slots 80 % busy: the kernel is bound by instruction issue
// (33.7 us; a one-warp-per-row form with sixteen loads in flight per lane was slower, 46 us).
constexpr int kRnThreads = 256, kRnKeep = 4;
// KEEP: 16-byte words per thread and row (2 for rows of up to 4096 elements: fewer registers, more CTAs per SM).  The next
// row of the block is requested before the current one is reduced, so its latency overlaps the two block-wide exchanges.
template <int FMT, int KEEP>
__global__ void __launch_bounds__(kRnThreads, KEEP == 2 ? 5 : 4) rmsnorm_mx_row_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ gamma,
                                                                    float eps, int zero_centered, int64_t rows, int64_t H, int64_t n_pad,
                                                                    uint8_t *__restrict__ q_row, uint8_t *__restrict__ s_row,
                                                                    float *__restrict__ rstd_out) {
    using T = __nv_bfloat16;
    constexpr bool kFp4 = FMT == PT_E2M1;
    __shared__ float s_red[kRnThreads / 32];
    const float zc = zero_centered ? 1.0f : 0.0f;
    auto fetch = [&](int64_t r, uint4(&v)[KEEP]) {
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int64_t h = ((int64_t) k * kRnThreads + threadIdx.x) * 8;
            v[k] = (h < H && r < rows) ? __ldg(reinterpret_cast<const uint4 *>(x + r * H + h)) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    // this thread's gains are the same for every row: converted once when they fit the registers (KEEP == 2)
    constexpr bool kGainsInRegs = KEEP == 2;
    [[maybe_unused]] float gp[kGainsInRegs ? KEEP : 1][8];
    if constexpr (kGainsInRegs) {
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int64_t h = ((int64_t) k * kRnThreads + threadIdx.x) * 8;
            uint4 gv = make_uint4(0u, 0u, 0u, 0u);
            if (h < H) gv = __ldg(reinterpret_cast<const uint4 *>(gamma + h));
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) { gp[k][2 * i] = bf16_lo(gw[i]) + zc; gp[k][2 * i + 1] = bf16_hi(gw[i]) + zc; }
        }
    }
    uint4 keep[KEEP], next[KEEP];
    fetch(blockIdx.x, keep);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        fetch(r + gridDim.x, next);
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int64_t h = ((int64_t) k * kRnThreads + threadIdx.x) * 8;
            if (h < H) {
                const uint32_t w[4] = {keep[k].x, keep[k].y, keep[k].z, keep[k].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float lo = bf16_lo(w[i]), hi = bf16_hi(w[i]);
                    ss += lo * lo;
                    ss += hi * hi;
                }
            }
        }
        float v = ss;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        __syncthreads();   // s_red may still be read for the previous row
        if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
        __syncthreads();
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kRnThreads / 32; ++w) total += s_red[w];
        const float rstd = rsqrtf(total / (float) H + eps);
        if (threadIdx.x == 0) rstd_out[r] = rstd;
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int64_t h = ((int64_t) k * kRnThreads + threadIdx.x) * 8;
            const bool live = h < n_pad;   // every lane takes part in the shuffles below; only the stores are conditional
            uint32_t y[4] = {0u, 0u, 0u, 0u};
            if (h < H) {
                const uint32_t xw[4] = {keep[k].x, keep[k].y, keep[k].z, keep[k].w};
                if constexpr (kGainsInRegs) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const __nv_bfloat162 t = __floats2bfloat162_rn(rmsnorm_value(bf16_lo(xw[i]), rstd, gp[k][2 * i]),
                                                                       rmsnorm_value(bf16_hi(xw[i]), rstd, gp[k][2 * i + 1]));
                        y[i] = *reinterpret_cast<const uint32_t *>(&t);
                    }
                } else {
                    const uint4 gv = __ldg(reinterpret_cast<const uint4 *>(gamma + h));
                    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const __nv_bfloat162 t = __floats2bfloat162_rn(rmsnorm_value(bf16_lo(xw[i]), rstd, bf16_lo(gw[i]) + zc),
                                                                       rmsnorm_value(bf16_hi(xw[i]), rstd, bf16_hi(gw[i]) + zc));
                        y[i] = *reinterpret_cast<const uint32_t *>(&t);
                    }
                }
            }
            uint32_t o[2];
            const uint8_t sbyte = mx_block_of_four_lanes<FMT>(y, o);   // every lane takes part
            if (live) {
                if constexpr (kFp4) *reinterpret_cast<uint32_t *>(q_row + (r * n_pad + h) / 2) = o[0];
                else *reinterpret_cast<uint2 *>(q_row + r * n_pad + h) = make_uint2(o[0], o[1]);
            }
            if (live && (threadIdx.x & 3) == 0) s_row[r * (n_pad / 32) + h / 32] = sbyte;
        }
#pragma unroll
        for (int k = 0; k < KEEP; ++k) keep[k] = next[k];
    }
}

// Gated activation and the row-wise MX copy in one pass (forward-only callers): out = act(x[:, :H]) * x[:, H:] * probs[row]
// with the stand-alone kernel's arithmetic and rounding (activation_norm.cu, act_math.cuh), quantized as the row-wise
// quantizer does; masked rows are zeros.  A block walks a row in steps of 2048 columns.  (Requesting the next step's inputs
// ahead made it slower, 4200 -> 3900 GB/s on 32768 x 2048: it is bound by its arithmetic, not by the loads.)
template <int FMT, int ACT>
__global__ void __launch_bounds__(kRnThreads) glu_mx_row_kernel(const __nv_bfloat16 *__restrict__ x, const float *__restrict__ probs,
                                                                const int64_t *__restrict__ row_mask, int64_t rows, int64_t H, int64_t n_pad,
                                                                uint8_t *__restrict__ q_row, uint8_t *__restrict__ s_row) {
    constexpr bool kFp4 = FMT == PT_E2M1;
    const int64_t steps = (n_pad + kRnThreads * 8 - 1) / (kRnThreads * 8);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const bool masked = row_mask != nullptr && row_mask[r] == 0;
        const float p = probs[r];
        const __nv_bfloat16 *a = x + r * 2 * H, *b = a + H;
        for (int64_t it = 0; it < steps; ++it) {
            const int64_t h = (it * kRnThreads + threadIdx.x) * 8;
            uint32_t y[4] = {0u, 0u, 0u, 0u};
            if (h < H && !masked) {
                const uint4 ar = __ldg(reinterpret_cast<const uint4 *>(a + h)), br = __ldg(reinterpret_cast<const uint4 *>(b + h));
                const uint32_t aw[4] = {ar.x, ar.y, ar.z, ar.w}, bw[4] = {br.x, br.y, br.z, br.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __nv_bfloat162 t = __floats2bfloat162_rn(glu_value<ACT>(bf16_lo(aw[i]), bf16_lo(bw[i]), p),
                                                                   glu_value<ACT>(bf16_hi(aw[i]), bf16_hi(bw[i]), p));
                    y[i] = *reinterpret_cast<const uint32_t *>(&t);
                }
            }
            uint32_t o[2];
            const uint8_t sbyte = mx_block_of_four_lanes<FMT>(y, o);   // every lane takes part
            if (h < n_pad) {
                if constexpr (kFp4) *reinterpret_cast<uint32_t *>(q_row + (r * n_pad + h) / 2) = o[0];
                else *reinterpret_cast<uint2 *>(q_row + r * n_pad + h) = make_uint2(o[0], o[1]);
                if ((threadIdx.x & 3) == 0) s_row[r * (n_pad / 32) + h / 32] = sbyte;
            }
        }
    }
}

// ROWSTAGE: the row-wise copy is staged and written by TMA (dense FP8); otherwise by 32-byte stores from registers.
// COLRHT (e2m1): the transposed copy is taken of the 16-point Hadamard transform of each run of 16 rows, in fp32 and in the
// operation order of mx_quant_tma_kernel's column pass (same bytes); the 64 fp32 values per thread cost a CTA per SM.
template <int FMT, bool ROW2D, bool COL2D, bool GROUPED, bool ROWSTAGE, int PRO = PT_PRO_NONE, bool COLRHT = false>
__global__ void __launch_bounds__(kSThreads, COLRHT ? 2 : split_ctas_per_sm(PRO))
    mx_quant_split_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap_qrow,
                          const __grid_constant__ CUtensorMap tmap_qcol, MxArgs a, int tiles_n, int tiles_m, int64_t total_tiles,
                          int sched_slot, int *status) {
    using namespace sm100;
    using T = __nv_bfloat16;
    constexpr bool kFp4 = FMT == PT_E2M1;
    constexpr int kStageBytes = split_stage_bytes(PRO);
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *col_stage = smem + kSStages * kStageBytes;            // 2 x 8 KiB
    uint8_t *row_stage = col_stage + 2 * kSStageOutBytes;          // 2 x 8 KiB
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(row_stage + 2 * kSStageOutBytes);
    uint64_t *empty_bar = full_bar + kSStages;
    __shared__ __align__(16) TileDesc s_desc[kSStages];
    __shared__ __align__(4) uint8_t s_colscale[2][kTileN][4];      // [buffer][column][band]
    __shared__ int s_abort;
    volatile int *abort_flag = &s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < kSStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 2 * kSGroupWarps);
        }
        fence_barrier_init();
        prefetch_tmap(&tmap);
        prefetch_tmap(&tmap_qcol);
        if (ROWSTAGE) prefetch_tmap(&tmap_qrow);
    }
    __shared__ int s_gtab[GROUPED ? 3 * (kQMaxGroups + 1) : 1];   // grouped: the three offset tables, read by the producer
    __syncthreads();
    sm100::grid_dep_wait();    // the input may come from the previous kernel, and a GEMM before it may still read the outputs
    sm100::grid_dep_launch();
    if constexpr (GROUPED) {
        for (int i = threadIdx.x; i <= a.num_groups; i += blockDim.x) {
            s_gtab[i] = (int) a.poffs_col[i];
            s_gtab[(kQMaxGroups + 1) + i] = (int) a.group_offs[i];
            s_gtab[2 * (kQMaxGroups + 1) + i] = (int) a.poffs_row[i];
        }
        __syncthreads();
    }
    bool ok = true;

    if (warp == 0) {
        // ================================================================ producer: tile coordinates + TMA loads
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            const uint32_t per_g = (uint32_t) tiles_n * (uint32_t) tiles_m;
            int grp = 0;   // grouped: tiles arrive in ascending row order, so the group index only moves forward
            // static schedule (sched_slot < 0): tiles blockIdx.x, + gridDim.x, ...; dynamic: the first tile is blockIdx.x,
            // every further one comes from the slot's counter (tile_sched.cuh)
            for (uint32_t t = blockIdx.x; t < (uint32_t) total_tiles; t = tile_sched_next(sched_slot, t)) {
                TileDesc d;
                d.g = (int) (t / per_g);
                const uint32_t rem = t - (uint32_t) d.g * per_g;
                d.tm = (int) (rem / (uint32_t) tiles_n);
                d.tn = (int) (rem - (uint32_t) d.tm * tiles_n);
                d.in_row0 = d.tm * kTileM; d.n_valid = kTileM; d.row_out0 = d.tm * kTileM; d.pad0 = d.pad1 = 0;
                if constexpr (GROUPED) {
                    const int *pcol = s_gtab, *goffs = s_gtab + (kQMaxGroups + 1), *prow = s_gtab + 2 * (kQMaxGroups + 1);
                    const int m0 = d.tm * kTileM;
                    if (m0 >= pcol[a.num_groups]) continue;   // past the padded end
                    while (grp + 1 < a.num_groups && pcol[grp + 1] <= m0) ++grp;   // last group starting at or before m0
                    const int into = m0 - pcol[grp];
                    d.in_row0 = goffs[grp] + into;
                    d.n_valid = max(0, min(kTileM, min(goffs[grp + 1], (int) a.M) - d.in_row0));
                    d.row_out0 = prow[grp] + into;
                }
                if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) break;
                s_desc[stage] = d;
                mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
                sm100::tma_load_3d(smem + stage * kStageBytes, &tmap, &full_bar[stage], d.tn * kTileN, d.in_row0, d.g);
                if constexpr (pro_is_glu(PRO))   // the gate half of the same rows: columns N .. 2N of x
                    sm100::tma_load_3d(smem + stage * kStageBytes + kQTileBytes, &tmap, &full_bar[stage], (int) a.N + d.tn * kTileN, d.in_row0, d.g);
                if (++stage == kSStages) { stage = 0; phase ^= 1; }
            }
            if (ok && (ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) {   // the terminal descriptor
                s_desc[stage].tn = -1;
                mbar_arrive(&full_bar[stage]);
            }
            tile_sched_done(sched_slot);
        }
    } else if (warp <= kSGroupWarps) {
        // ================================================================ row-wise copy: thread = tile row
        const int row = threadIdx.x - 32;
        uint32_t stage = 0, phase = 0, tile_i = 0;
        while (true) {
            if (!(ok = mbar_wait_warp(&full_bar[stage], phase, abort_flag))) break;
            const int4 d0 = *reinterpret_cast<const int4 *>(&s_desc[stage]);
            const int2 d1 = *reinterpret_cast<const int2 *>(&s_desc[stage].n_valid);
            const int tn = d0.x, tm = d0.y, n_valid = d1.x, row_out0 = d1.y;
            const int64_t g = d0.z;
            if (tn < 0) break;
            if constexpr (PRO == PT_PRO_RMSNORM) {
                split_prologue_rmsnorm(smem + stage * kStageBytes, threadIdx.x - 32, s_desc[stage].in_row0, tn, a);
            } else if constexpr (PRO != PT_PRO_NONE) {
                split_prologue<PRO>(smem + stage * kStageBytes, threadIdx.x - 32, s_desc[stage].in_row0, tn, a);
            }
            uint32_t w[32];
            {
                const uint8_t *rp = smem + stage * kStageBytes + row * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 q = *reinterpret_cast<const uint4 *>(rp + ((c ^ (row & 7)) << 4));
                    w[4 * c] = q.x; w[4 * c + 1] = q.y; w[4 * c + 2] = q.z; w[4 * c + 3] = q.w;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);  // this warp no longer reads the stage
            if (++stage == kSStages) { stage = 0; phase ^= 1; }
            const int buf = tile_i & 1;
            ++tile_i;
            const int64_t gm = (GROUPED ? row_out0 : tm * kTileM) + row;    // row of the row-wise copy
            const bool live = GROUPED ? row < n_valid : gm < a.M;
            const int64_t n0 = (int64_t) tn * kTileN;
            uint8_t sbyte[2];
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                uint32_t *x = &w[16 * b];
                uint32_t o[8];
                uint32_t pm = 0u;
#pragma unroll
                for (int k = 0; k < 16; ++k) pm = absmax2_nan_bf16(pm, x[k]);
                const bool has_nan = packed_bf16_has_nan(pm);
                if (has_nan) {  // a NaN element takes no part in the maximum
                    pm = 0u;
#pragma unroll
                    for (int k = 0; k < 16; ++k) pm = absmax2<T>(pm, x[k]);
                }
                pm = absmax2_done(pm);
                float m = fmaxf(bf16_lo(pm), bf16_hi(pm));
                if constexpr (ROW2D) m = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(m)));  // 32 rows = this warp
                const MxScale sc = mx_scale<FMT>(m, GROUPED);
                sbyte[b] = sc.byte;
                if (has_nan && !kFp4) {   // fmax(NaN, -qmax * scale) = -qmax * scale, exact in bf16 (1.75 * 2^k, or -inf)
                    const float nlim = -MxParams<FMT>::qmax * sc.native;
                    const uint32_t nlim2 = bf16_bits_x2(nlim, nlim);
#pragma unroll
                    for (int k = 0; k < 16; ++k) x[k] = max_bf16x2(x[k], nlim2);
                }
                bool sr_done = false;
                if constexpr (kFp4) {
                    if (a.sr_row) {   // stochastic rounding: 32 random bits per four elements from a hash of (seed, position)
                        const uint32_t inv2 = bf16_bits_x2(sc.inv, sc.inv);
                        SrState sr{sr_mix(a.sr_seed ^ (uint32_t) ((gm * a.N_pad + n0 + 32 * b) >> 2)) | 1u};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t v0 = mul_bf16x2(x[4 * k], inv2), v1 = mul_bf16x2(x[4 * k + 1], inv2);
                            const uint32_t v2 = mul_bf16x2(x[4 * k + 2], inv2), v3 = mul_bf16x2(x[4 * k + 3], inv2);
                            o[k] = cvt4_e2m1_sr(bf16_lo(v0), bf16_hi(v0), bf16_lo(v1), bf16_hi(v1), sr.next()) |
                                   (cvt4_e2m1_sr(bf16_lo(v2), bf16_hi(v2), bf16_lo(v3), bf16_hi(v3), sr.next()) << 16);
                        }
                        sr_done = true;
                    }
                }
                if (!sr_done) encode_row_block<FMT>(x, bf16_bits_x2(sc.inv, sc.inv), o);
                if (sc.byte == 0) {       // such a block is written as (positive) zeros
#pragma unroll
                    for (int k = 0; k < 8; ++k) o[k] = 0u;
                }
                if constexpr (ROWSTAGE) {
                    // staged tile of 64-byte rows, 64-byte swizzle: chunk c of row r sits at chunk c ^ ((r >> 1) & 3)
                    uint8_t *dst = row_stage + buf * kSStageOutBytes + row * 64;
                    const int sw = (row >> 1) & 3;
                    *reinterpret_cast<uint4 *>(dst + (((2 * b) ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4 *>(dst + (((2 * b + 1) ^ sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                } else if (live) {
                    uint8_t *qr = a.q_row + g * a.qrow_gstride;
                    if constexpr (kFp4) {
                        *reinterpret_cast<uint4 *>(qr + (gm * a.N_pad + n0) / 2 + 16 * b) = make_uint4(o[0], o[1], o[2], o[3]);
                    } else {
                        uint8_t *dst = qr + gm * a.N_pad + n0 + 32 * b;
                        if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
                            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(o[0]), "r"(o[1]),
                                         "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
                        } else {
                            reinterpret_cast<uint4 *>(dst)[0] = make_uint4(o[0], o[1], o[2], o[3]);
                            reinterpret_cast<uint4 *>(dst)[1] = make_uint4(o[4], o[5], o[6], o[7]);
                        }
                    }
                }
            }
            if constexpr (ROWSTAGE) {
                fence_proxy_async_smem();
                if (row == 0) bulk_wait_read_all();   // the store of the previous tile has read the other buffer
                sm100::named_barrier<1, kSGroupThreads>();
                if (row == 0) {
                    tma_store_3d(&tmap_qrow, row_stage + buf * kSStageOutBytes, (int) n0, tm * kTileM, (int) g);
                    bulk_commit_group();
                }
            }
            if (live) {   // the two scale bytes of this row (an even offset: one 16-bit store)
                uint8_t *sp = a.s_row + g * a.srow_gstride + gm * (a.N_pad / 32) + n0 / 32;
                *reinterpret_cast<uint16_t *>(sp) = (uint16_t) (sbyte[0] | ((uint16_t) sbyte[1] << 8));
            }
        }
        if (ROWSTAGE && row == 0) bulk_wait_read_all();
    } else {
        // ================================================================ transposed copy: thread = (32-row band, column pair)
        const int ct = threadIdx.x - 32 - kSGroupThreads;
        const int band = ct >> 5, pair = lane;
        const int chunk = pair >> 2;
        uint32_t stage = 0, phase = 0, tile_i = 0;
        while (true) {
            if (!(ok = mbar_wait_warp(&full_bar[stage], phase, abort_flag))) break;
            const int4 d0 = *reinterpret_cast<const int4 *>(&s_desc[stage]);
            const int tn = d0.x, tm = d0.y;
            const int64_t g = d0.z;
            if (tn < 0) break;
            if constexpr (PRO == PT_PRO_RMSNORM) {
                split_prologue_rmsnorm(smem + stage * kStageBytes, threadIdx.x - 32, s_desc[stage].in_row0, tn, a);
            } else if constexpr (PRO != PT_PRO_NONE) {
                split_prologue<PRO>(smem + stage * kStageBytes, threadIdx.x - 32, s_desc[stage].in_row0, tn, a);
            }
            const int n_valid = GROUPED ? s_desc[stage].n_valid : kTileM;
            uint32_t w[32];
            {
                const uint8_t *cp = smem + stage * kStageBytes + band * 32 * 128 + ((pair & 3) << 2);
#pragma unroll
                for (int r = 0; r < 32; ++r) {   // (32 band + r) % 8 == r % 8: every lane reads tile row r, no bank conflict
                    const uint32_t v = *reinterpret_cast<const uint32_t *>(cp + r * 128 + ((chunk ^ (r & 7)) << 4));
                    w[r] = (!GROUPED || band * 32 + r < n_valid) ? v : 0u;   // rows past the group's end count as zeros
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);
            if (++stage == kSStages) { stage = 0; phase ^= 1; }
            const int buf = tile_i & 1;
            ++tile_i;
            uint32_t o0[8], o1[8];   // 32 codes of column 2 pair and of column 2 pair + 1
            MxScale s0, s1;
            if constexpr (COLRHT) {
                static_assert(!COLRHT || FMT == PT_E2M1, "the Hadamard option is an e2m1 one");
                float c0[32], c1[32];
#pragma unroll
                for (int r = 0; r < 32; ++r) { c0[r] = bf16_lo(w[r]); c1[r] = bf16_hi(w[r]); }
                rht16(c0); rht16(c0 + 16); rht16(c1); rht16(c1 + 16);
                float m0c = 0.f, m1c = 0.f;
#pragma unroll
                for (int r = 0; r < 32; ++r) { m0c = fmaxf(m0c, fabsf(c0[r])); m1c = fmaxf(m1c, fabsf(c1[r])); }
                s0 = mx_scale<FMT>(m0c, GROUPED);
                s1 = mx_scale<FMT>(m1c, GROUPED);
                if (a.sr_col) {
                    const uint32_t pos = (uint32_t) ((((int64_t) tn * kTileN + 2 * pair) * a.M_pad + (int64_t) tm * kTileM + 32 * band) >> 2);
                    SrState r0{sr_mix(~a.sr_seed ^ pos) | 1u}, r1{sr_mix(~a.sr_seed ^ (pos + (uint32_t) (a.M_pad >> 2))) | 1u};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        o0[k] = cvt4_e2m1_sr(c0[8 * k] * s0.inv, c0[8 * k + 1] * s0.inv, c0[8 * k + 2] * s0.inv, c0[8 * k + 3] * s0.inv, r0.next()) |
                                (cvt4_e2m1_sr(c0[8 * k + 4] * s0.inv, c0[8 * k + 5] * s0.inv, c0[8 * k + 6] * s0.inv, c0[8 * k + 7] * s0.inv, r0.next()) << 16);
                        o1[k] = cvt4_e2m1_sr(c1[8 * k] * s1.inv, c1[8 * k + 1] * s1.inv, c1[8 * k + 2] * s1.inv, c1[8 * k + 3] * s1.inv, r1.next()) |
                                (cvt4_e2m1_sr(c1[8 * k + 4] * s1.inv, c1[8 * k + 5] * s1.inv, c1[8 * k + 6] * s1.inv, c1[8 * k + 7] * s1.inv, r1.next()) << 16);
                    }
                } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    o0[k] = pack8_e2m1(c0[8 * k] * s0.inv, c0[8 * k + 1] * s0.inv, c0[8 * k + 2] * s0.inv, c0[8 * k + 3] * s0.inv, c0[8 * k + 4] * s0.inv,
                                       c0[8 * k + 5] * s0.inv, c0[8 * k + 6] * s0.inv, c0[8 * k + 7] * s0.inv);
                    o1[k] = pack8_e2m1(c1[8 * k] * s1.inv, c1[8 * k + 1] * s1.inv, c1[8 * k + 2] * s1.inv, c1[8 * k + 3] * s1.inv, c1[8 * k + 4] * s1.inv,
                                       c1[8 * k + 5] * s1.inv, c1[8 * k + 6] * s1.inv, c1[8 * k + 7] * s1.inv);
                }
                }
            } else {
            uint32_t pm = 0u;
#pragma unroll
            for (int r = 0; r < 32; ++r) pm = absmax2_nan_bf16(pm, w[r]);
            const bool has_nan = packed_bf16_has_nan(pm);
            if (has_nan) {
                pm = 0u;
#pragma unroll
                for (int r = 0; r < 32; ++r) pm = absmax2<T>(pm, w[r]);
            }
            pm = absmax2_done(pm);
            float m0c = bf16_lo(pm), m1c = bf16_hi(pm);
            if constexpr (COL2D) {   // 32 x 32 tile: the 16 column pairs of this half warp
                float m = fmaxf(m0c, m1c);
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
                m0c = m1c = m;
            }
            s0 = mx_scale<FMT>(m0c, GROUPED);
            s1 = mx_scale<FMT>(m1c, GROUPED);
            if (has_nan && !kFp4) {
                const uint32_t nlim2 = bf16_bits_x2(-MxParams<FMT>::qmax * s0.native, -MxParams<FMT>::qmax * s1.native);
#pragma unroll
                for (int r = 0; r < 32; ++r) w[r] = max_bf16x2(w[r], nlim2);
            }
            const uint32_t inv2 = bf16_bits_x2(s0.inv, s1.inv);
#pragma unroll
            for (int r = 0; r < 32; ++r) w[r] = mul_bf16x2(w[r], inv2);
            if (kFp4 && a.sr_col) {
                const uint32_t pos = (uint32_t) ((((int64_t) tn * kTileN + 2 * pair) * a.M_pad + (int64_t) tm * kTileM + 32 * band) >> 2);
                SrState r0{sr_mix(~a.sr_seed ^ pos) | 1u}, r1{sr_mix(~a.sr_seed ^ (pos + (uint32_t) (a.M_pad >> 2))) | 1u};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    o0[k] = cvt4_e2m1_sr(bf16_lo(w[8 * k]), bf16_lo(w[8 * k + 1]), bf16_lo(w[8 * k + 2]), bf16_lo(w[8 * k + 3]), r0.next()) |
                            (cvt4_e2m1_sr(bf16_lo(w[8 * k + 4]), bf16_lo(w[8 * k + 5]), bf16_lo(w[8 * k + 6]), bf16_lo(w[8 * k + 7]), r0.next()) << 16);
                    o1[k] = cvt4_e2m1_sr(bf16_hi(w[8 * k]), bf16_hi(w[8 * k + 1]), bf16_hi(w[8 * k + 2]), bf16_hi(w[8 * k + 3]), r1.next()) |
                            (cvt4_e2m1_sr(bf16_hi(w[8 * k + 4]), bf16_hi(w[8 * k + 5]), bf16_hi(w[8 * k + 6]), bf16_hi(w[8 * k + 7]), r1.next()) << 16);
                }
            } else if constexpr (kFp4) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    o0[k] = pack8_e2m1(bf16_lo(w[8 * k]), bf16_lo(w[8 * k + 1]), bf16_lo(w[8 * k + 2]), bf16_lo(w[8 * k + 3]),
                                       bf16_lo(w[8 * k + 4]), bf16_lo(w[8 * k + 5]), bf16_lo(w[8 * k + 6]), bf16_lo(w[8 * k + 7]));
                    o1[k] = pack8_e2m1(bf16_hi(w[8 * k]), bf16_hi(w[8 * k + 1]), bf16_hi(w[8 * k + 2]), bf16_hi(w[8 * k + 3]),
                                       bf16_hi(w[8 * k + 4]), bf16_hi(w[8 * k + 5]), bf16_hi(w[8 * k + 6]), bf16_hi(w[8 * k + 7]));
                }
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    o0[k] = pack4_fp8<FMT>(bf16_lo(w[4 * k]), bf16_lo(w[4 * k + 1]), bf16_lo(w[4 * k + 2]), bf16_lo(w[4 * k + 3]));
                    o1[k] = pack4_fp8<FMT>(bf16_hi(w[4 * k]), bf16_hi(w[4 * k + 1]), bf16_hi(w[4 * k + 2]), bf16_hi(w[4 * k + 3]));
                }
            }
            }   // !COLRHT
            if (__any_sync(0xffffffffu, s0.byte == 0 || s1.byte == 0)) {   // such a column is written as (positive) zeros
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (s0.byte == 0) o0[k] = 0u;
                    if (s1.byte == 0) o1[k] = 0u;
                }
            }
            // staged transposed tile: row c = tile column c holds its 128 rows; this thread owns rows 32 band .. + 31
            uint8_t *cs = col_stage + buf * kSStageOutBytes;
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int c = 2 * pair + cc;
                const uint32_t *o = cc ? o1 : o0;
                if constexpr (kFp4) {   // 64-byte rows, 64-byte swizzle; 16 bytes = chunk `band`
                    *reinterpret_cast<uint4 *>(cs + c * 64 + ((band ^ ((c >> 1) & 3)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                } else {                // 128-byte rows, 128-byte swizzle; 32 bytes = chunks 2 band, 2 band + 1
                    *reinterpret_cast<uint4 *>(cs + c * 128 + (((2 * band) ^ (c & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4 *>(cs + c * 128 + (((2 * band + 1) ^ (c & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                }
                s_colscale[buf][c][band] = cc ? s1.byte : s0.byte;
            }
            fence_proxy_async_smem();
            if (ct == 0) bulk_wait_read_all();   // the store of the previous tile has read the other buffer
            sm100::named_barrier<2, kSGroupThreads>();
            const int64_t m0 = (int64_t) tm * kTileM, n0 = (int64_t) tn * kTileN;
            if (ct == 0) {
                tma_store_3d(&tmap_qcol, cs, (int) (kFp4 ? m0 / 2 : m0), (int) n0, (int) g);
                bulk_commit_group();
            }
            if (ct < kTileN && n0 + ct < a.N)   // the four band scales of column ct: one 32-bit store
                *reinterpret_cast<uint32_t *>(a.s_col + g * a.scol_gstride + (n0 + ct) * (a.M_pad / 32) + m0 / 32) =
                    *reinterpret_cast<const uint32_t *>(&s_colscale[buf][ct][0]);
        }
        if (ct == 0) bulk_wait_read_all();
    }
    if (!ok || *abort_flag) {
        if (status && lane == 0) atomicExch(status, (int) PT_ERR_TIMEOUT);
        __nanosleep(100000);  // let a copy still in flight land before the shared memory is released
    }
}

// ------------------------------------------------------------------------------------------------ dequantize
template <typename T> __device__ __forceinline__ void put_out(T *p, float v);
template <> __device__ __forceinline__ void put_out<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void put_out<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void put_out<__half>(__half *p, float v) { *p = __float2half_rn(v); }

__device__ __forceinline__ float decode_code(int fmt, uint8_t c) {
    if (fmt == PT_E5M2) return __half2float(__ushort_as_half((uint16_t) c << 8));
    if (fmt == PT_E4M3) {
        const uint32_t sign = (uint32_t) (c & 0x80) << 24, e = (c >> 3) & 0xF, m = c & 7;
        if (e == 0) return __uint_as_float(sign | __float_as_uint((float) m * 0.001953125f));
        if (e == 15 && m == 7) return __uint_as_float(sign | 0x7FC00000u);
        return __uint_as_float(sign | ((e + 120) << 23) | (m << 20));
    }
    const float tab[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    const float mag = tab[c & 7];
    return (c & 8) ? -mag : mag;
}

template <typename T>
__global__ void __launch_bounds__(256) mx_dequant_kernel(const uint8_t *__restrict__ q, int fmt,
                                                        const uint8_t *__restrict__ s, int64_t rows, int64_t cols,
                                                        int64_t cols_stored, int transpose_out, T *__restrict__ y) {
    const int64_t total = rows * cols;
    const int64_t stride = (int64_t) gridDim.x * blockDim.x;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / cols, c = i % cols;
        uint8_t code;
        if (fmt == PT_E2M1) {
            const uint8_t b = q[(r * cols_stored + c) >> 1];
            code = (c & 1) ? (b >> 4) : (b & 0xF);
        } else {
            code = q[r * cols_stored + c];
        }
        const int sb = s[r * (cols_stored / 32) + c / 32];
        // e8m0_to_scale of the reference (device/utils.cuh:124-126): byte << 23 reinterpreted; byte 0 is 0.0, byte 255 +inf
        const float sc = __uint_as_float((uint32_t) sb << 23);
        const float val = decode_code(fmt, code) * sc;
        put_out(y + (transpose_out ? c * rows + r : i), val);
    }
}

// 3-D tensor map over x [G, M, N] (16-bit elements), box 64 x 128 x 1, 128-byte swizzle
static int make_tmap_x(CUtensorMap *m, const void *base, int64_t G, int64_t M, int64_t N) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return set_error(PT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {(cuuint64_t) N, (cuuint64_t) M, (cuuint64_t) G};
    cuuint64_t strides[2] = {(cuuint64_t) N * 2, (cuuint64_t) M * N * 2};
    cuuint32_t box[3] = {(cuuint32_t) kTileN, (cuuint32_t) kTileM, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(PT_ERR_CUDA, "cuTensorMapEncodeTiled (quantize input) failed with code %d", (int) r);
    return PT_OK;
}

// 3-D byte tensor map [G, rows, row_bytes] for a staged output tile of box_bytes x box_rows (64- or 128-byte swizzle)
static int make_tmap_out(CUtensorMap *m, const void *base, int64_t G, int64_t rows, int64_t row_bytes, int box_bytes, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return set_error(PT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {(cuuint64_t) row_bytes, (cuuint64_t) rows, (cuuint64_t) G};
    cuuint64_t strides[2] = {(cuuint64_t) row_bytes, (cuuint64_t) rows * (cuuint64_t) row_bytes};
    cuuint32_t box[3] = {(cuuint32_t) box_bytes, (cuuint32_t) box_rows, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(PT_ERR_CUDA, "cuTensorMapEncodeTiled (quantize output) failed with code %d", (int) r);
    return PT_OK;
}

// The warp-split kernel covers bf16 inputs, both copies requested, no Hadamard transform, 16-byte aligned outputs.
// Returns PT_ERR_UNSUPPORTED (without setting an error message) when the call is outside that.
template <int FMT, bool GROUPED, int PRO = PT_PRO_NONE, bool COLRHT = false>
static int launch_mx_split(const MxArgs &a, int64_t G, int64_t m_tiles_rows, unsigned flags, cudaStream_t st) {
    if (PRO == PT_PRO_NONE && getenv("PT_MX_QUANT_NO_SPLIT") != nullptr) return PT_ERR_UNSUPPORTED;
    if (PRO != PT_PRO_NONE && (flags & (PT_MX_ROW_2D | PT_MX_COL_2D))) return PT_ERR_UNSUPPORTED;
    if (pro_is_glu(PRO) && a.N % kTileN != 0) return PT_ERR_UNSUPPORTED;   // the value tile's last columns would be gate columns
    const bool row = flags & PT_MX_ROW, col = flags & PT_MX_COL;
    if (!row || !col || (flags & PT_MX_ROW_RHT) || ((flags & PT_MX_COL_RHT) != 0) != COLRHT) return PT_ERR_UNSUPPORTED;
    if ((flags & (PT_MX_ROW_SR | PT_MX_COL_SR)) && (FMT != PT_E2M1 || PRO != PT_PRO_NONE)) return PT_ERR_UNSUPPORTED;
    if (COLRHT && (flags & (PT_MX_ROW_2D | PT_MX_COL_2D))) return PT_ERR_UNSUPPORTED;
    constexpr bool kFp4 = FMT == PT_E2M1;
    if (!aligned(a.x, 16) || !aligned(a.q_row, 16) || !aligned(a.q_col, 16) || !aligned(a.s_row, 2) || !aligned(a.s_col, 4)) return PT_ERR_UNSUPPORTED;
    if (a.M >= (1ll << 31) || m_tiles_rows >= (1ll << 31)) return PT_ERR_UNSUPPORTED;
    if (GROUPED && a.num_groups > kQMaxGroups) return PT_ERR_UNSUPPORTED;
    const int tiles_n = (int) (a.N_pad / kTileN), tiles_m = (int) (m_tiles_rows / kTileM);
    const int64_t total_tiles = (int64_t) tiles_n * tiles_m * G;
    PT_REQUIRE(total_tiles < (1ll << 31), "MX quantize: too many tiles");
    CUtensorMap tx, trow, tcol;
    int rc = make_tmap_x(&tx, a.x, G, a.M, a.x_cols ? a.x_cols : a.N);
    if (rc != PT_OK) return rc;
    constexpr bool kRowStage = !GROUPED && !kFp4;
    trow = tx;
    if (kRowStage && (rc = make_tmap_out(&trow, a.q_row, G, a.M, a.N_pad, 64, kTileM)) != PT_OK) return rc;
    if ((rc = make_tmap_out(&tcol, a.q_col, G, a.N, kFp4 ? a.M_pad / 2 : a.M_pad, kFp4 ? 64 : 128, kTileN)) != PT_OK) return rc;
    const int slot = tile_sched_acquire(st);
    const int grid = (int) std::min<int64_t>(total_tiles, (int64_t) sm_count() * (COLRHT ? 2 : split_ctas_per_sm(PRO)));
    constexpr int kSmem = split_smem_bytes(PRO);
    const bool r2d = flags & PT_MX_ROW_2D, c2d = flags & PT_MX_COL_2D;
#define PT_MXS_CASE(R2, C2)                                                                                       \
    if (r2d == R2 && c2d == C2) {                                                                                 \
        auto kern = mx_quant_split_kernel<FMT, R2, C2, GROUPED, kRowStage, PRO, COLRHT>;                          \
        static bool attr_set_dev[64] = {};                                                                        \
        bool &attr_set = attr_set_dev[current_device_slot()];                                                     \
        if (!attr_set) {                                                                                          \
            PT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));           \
            attr_set = true;                                                                                      \
        }                                                                                                         \
        PT_CUDA_OK(launch_overlapped(kern, dim3(grid), dim3(kSThreads), kSmem, st, tx, trow, tcol, a, tiles_n, tiles_m, total_tiles, slot, default_status())); \
        PT_LAUNCH_OK();                                                                                           \
        tile_sched_release(slot, st);                                                                             \
        return PT_OK;                                                                                             \
    }
    PT_MXS_CASE(false, false)
    if constexpr (!GROUPED && PRO == PT_PRO_NONE && !COLRHT) {
        PT_MXS_CASE(true, true)
        if constexpr (!kFp4) {
            PT_MXS_CASE(true, false)
            PT_MXS_CASE(false, true)
        }
    }
#undef PT_MXS_CASE
    return PT_ERR_UNSUPPORTED;
}

template <typename T, int FMT>
static int launch_mx(const MxArgs &a, int64_t G, unsigned flags, cudaStream_t st) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        int rc = launch_mx_split<FMT, false>(a, G, a.M_pad, flags, st);
        if constexpr (FMT == PT_E2M1)
            if (rc == PT_ERR_UNSUPPORTED) rc = launch_mx_split<FMT, false, PT_PRO_NONE, true>(a, G, a.M_pad, flags, st);
        if (rc != PT_ERR_UNSUPPORTED) return rc;
    }
    dim3 grid((unsigned) (a.N_pad / kTileN), (unsigned) (a.M_pad / kTileM), (unsigned) G);
    // TMA needs a 16-byte row pitch; N % 32 == 0 guarantees it for 16-bit elements
    const bool use_tma = getenv("PT_MX_QUANT_NO_TMA") == nullptr;
    CUtensorMap tmap;
    const int tiles_n = (int) (a.N_pad / kTileN), tiles_m = (int) (a.M_pad / kTileM);
    const int64_t total_tiles = (int64_t) tiles_n * tiles_m * G;
    int tma_grid = 0;
    if (use_tma) {
        int rc = make_tmap_x(&tmap, a.x, G, a.M, a.N);
        if (rc != PT_OK) return rc;
        PT_REQUIRE(total_tiles < (1ll << 31), "MX quantize: too many tiles");
        tma_grid = (int) std::min<int64_t>(total_tiles, (int64_t) sm_count() * kQCtasPerSm);
    }
    const bool row = flags & PT_MX_ROW, col = flags & PT_MX_COL;
    const bool r2d = flags & PT_MX_ROW_2D, c2d = flags & PT_MX_COL_2D;
    const bool rrht = flags & PT_MX_ROW_RHT, crht = flags & PT_MX_COL_RHT;
#define PT_MX_CASE(R, C, R2, C2, RR, CR)                                                                   \
    if (row == R && col == C && (!R || r2d == R2) && (!C || c2d == C2) && (!R || rrht == RR) && (!C || crht == CR)) { \
        if (use_tma) {                                                                                     \
            auto kern = mx_quant_tma_kernel<T, FMT, R, C, R2, C2, RR, CR>;                                 \
            static bool attr_set_dev[64] = {};                                                             \
            bool &attr_set = attr_set_dev[current_device_slot()];                                          \
            if (!attr_set) {                                                                               \
                PT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kQSmemBytes)); \
                attr_set = true;                                                                           \
            }                                                                                              \
            PT_CUDA_OK(launch_overlapped(kern, dim3(tma_grid), dim3(kQThreads), kQSmemBytes, st, tmap, a, tiles_n, tiles_m, total_tiles, default_status())); \
        } else {                                                                                           \
            mx_quant_kernel<T, FMT, R, C, R2, C2, RR, CR><<<grid, kMxThreads, 0, st>>>(a);                 \
        }                                                                                                  \
        PT_LAUNCH_OK();                                                                                    \
        return PT_OK;                                                                                      \
    }
    if constexpr (FMT == PT_E2M1) {
        PT_MX_CASE(true, false, false, false, false, false)
        PT_MX_CASE(true, false, true, false, false, false)
        PT_MX_CASE(true, false, false, false, true, false)
        PT_MX_CASE(false, true, false, false, false, false)
        PT_MX_CASE(false, true, false, true, false, false)
        PT_MX_CASE(false, true, false, false, false, true)
        PT_MX_CASE(true, true, false, false, false, false)
        PT_MX_CASE(true, true, true, true, false, false)
        PT_MX_CASE(true, true, false, false, false, true)
        PT_MX_CASE(true, true, false, false, true, true)
        PT_MX_CASE(true, true, false, false, true, false)
    } else {
        PT_MX_CASE(true, false, false, false, false, false)
        PT_MX_CASE(true, false, true, false, false, false)
        PT_MX_CASE(false, true, false, false, false, false)
        PT_MX_CASE(false, true, false, true, false, false)
        PT_MX_CASE(true, true, false, false, false, false)
        PT_MX_CASE(true, true, true, true, false, false)
        PT_MX_CASE(true, true, true, false, false, false)
        PT_MX_CASE(true, true, false, true, false, false)
    }
#undef PT_MX_CASE
    return set_error(PT_ERR_UNSUPPORTED, "MX quantize: flag combination 0x%x is not built for this format", flags);
}

template <typename T, int FMT>
static int launch_mx_grouped(const MxArgs &a, int64_t m_alloc, unsigned flags, cudaStream_t st) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        int rc = launch_mx_split<FMT, true>(a, 1, m_alloc, flags, st);
        if constexpr (FMT == PT_E2M1)
            if (rc == PT_ERR_UNSUPPORTED) rc = launch_mx_split<FMT, true, PT_PRO_NONE, true>(a, 1, m_alloc, flags, st);
        if (rc != PT_ERR_UNSUPPORTED) return rc;
    }
    dim3 grid((unsigned) (a.N_pad / kTileN), (unsigned) (m_alloc / kTileM), 1u);  // tiles past padded_offs_col[G] return at once
    const bool row = flags & PT_MX_ROW, col = flags & PT_MX_COL;
    const bool rrht = flags & PT_MX_ROW_RHT, crht = flags & PT_MX_COL_RHT;
    // persistent TMA form: needs a 16-byte row pitch and base (N % 32 == 0 gives the pitch for 16-bit elements)
    const bool use_tma = getenv("PT_MX_QUANT_NO_TMA") == nullptr && aligned(a.x, 16) && a.M < (1ll << 31) && m_alloc < (1ll << 31) &&
                         a.num_groups <= kQMaxGroups;
    CUtensorMap tmap;
    const int tiles_n = (int) (a.N_pad / kTileN), tiles_m = (int) (m_alloc / kTileM);
    const int64_t total_tiles = (int64_t) tiles_n * tiles_m;
    int tma_grid = 0;
    if (use_tma) {
        int rc = make_tmap_x(&tmap, a.x, 1, a.M, a.N);
        if (rc != PT_OK) return rc;
        PT_REQUIRE(total_tiles < (1ll << 31), "grouped MX quantize: too many tiles");
        tma_grid = (int) std::min<int64_t>(total_tiles, (int64_t) sm_count() * kQCtasPerSm);
    }
#define PT_MXG_CASE(R, C, RR, CR)                                                                     \
    if (row == R && col == C && (!R || rrht == RR) && (!C || crht == CR)) {                          \
        if (use_tma) {                                                                                \
            auto kern = mx_quant_tma_kernel<T, FMT, R, C, false, false, RR, CR, true>;               \
            PT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kQSmemBytes)); \
            PT_CUDA_OK(launch_overlapped(kern, dim3(tma_grid), dim3(kQThreads), kQSmemBytes, st, tmap, a, tiles_n, tiles_m, total_tiles, default_status())); \
        } else {                                                                                      \
            mx_quant_kernel<T, FMT, R, C, false, false, RR, CR, true><<<grid, kMxThreads, 0, st>>>(a); \
        }                                                                                             \
        PT_LAUNCH_OK();                                                                               \
        return PT_OK;                                                                                 \
    }
    PT_MXG_CASE(true, false, false, false)
    PT_MXG_CASE(false, true, false, false)
    PT_MXG_CASE(true, true, false, false)
    if constexpr (FMT == PT_E2M1) {
        PT_MXG_CASE(false, true, false, true)
        PT_MXG_CASE(true, true, false, true)
        PT_MXG_CASE(true, true, true, true)
        PT_MXG_CASE(true, false, true, false)
    }
#undef PT_MXG_CASE
    return set_error(PT_ERR_UNSUPPORTED, "grouped MX quantize: flag combination 0x%x is not built", flags);
}

// Every launch that rounds stochastically takes a fresh seed from a process-wide counter (as the reference does,
// quantization_mxfp4.cu:62,1141): two calls on the same input draw different bits.
static void set_sr(MxArgs &a, unsigned flags) {
    static std::atomic<uint32_t> counter{1};
    a.sr_row = (flags & PT_MX_ROW_SR) != 0;
    a.sr_col = (flags & PT_MX_COL_SR) != 0;
    a.sr_seed = (a.sr_row || a.sr_col) ? sr_seed_from(counter.fetch_add(1, std::memory_order_relaxed)) : 0u;
}


// Shared argument checks and MxArgs set-up of the fused entry points (dense when group_offs is null).
static int fused_args(MxArgs &a, const char *what, const void *x, int x_dtype, int64_t rows, int64_t H, int fmt, unsigned flags, void *q_row,
                      uint8_t *s_row, void *q_col, uint8_t *s_col, int G, const int64_t *group_offs, const int64_t *poffs_row,
                      const int64_t *poffs_col, int64_t col_alloc) {
    PT_REQUIRE(rows >= 0 && H >= 0, "%s: bad shape", what);
    PT_REQUIRE(x_dtype == PT_BF16, "%s: the fused kernels take bf16 input", what);
    PT_REQUIRE(H % 32 == 0, "%s: the quantized width must be divisible by 32 (got %lld)", what, (long long) H);
    PT_REQUIRE((flags & (PT_MX_ROW | PT_MX_COL)) == (PT_MX_ROW | PT_MX_COL) && !(flags & ~(unsigned) (PT_MX_ROW | PT_MX_COL | PT_MX_COL_RHT)),
               "%s: the fused kernels write both copies, with 1-D block scales and round-to-nearest (flags 0x%x)", what, flags);
    PT_REQUIRE(!(flags & PT_MX_COL_RHT) || fmt == PT_E2M1, "%s: the Hadamard transform of the transposed copy is an e2m1 option", what);
    PT_REQUIRE(fmt == PT_E4M3 || fmt == PT_E2M1, "%s: formats e4m3 and e2m1", what);
    PT_REQUIRE(q_row && s_row && q_col && s_col, "%s: outputs missing", what);
    a.x = x; a.M = rows; a.N = H; a.N_pad = ceil_to(H, 128);
    a.q_row = (uint8_t *) q_row; a.s_row = s_row; a.q_col = (uint8_t *) q_col; a.s_col = s_col;
    if (group_offs) {
        PT_REQUIRE(G >= 1 && poffs_row && poffs_col, "%s: group offsets required", what);
        PT_REQUIRE(col_alloc % 128 == 0 && col_alloc >= rows && col_alloc / kTileM <= 65535, "%s: col_alloc must be the 128-multiple width of the col-wise buffers", what);
        a.M_pad = col_alloc; a.group_offs = group_offs; a.poffs_row = poffs_row; a.poffs_col = poffs_col; a.num_groups = G;
    } else {
        const int div = fmt == PT_E2M1 ? 2 : 1;
        a.M_pad = ceil_to(rows, 128);
        a.qrow_gstride = rows * a.N_pad / div; a.srow_gstride = rows * (a.N_pad / 32);
        a.qcol_gstride = H * a.M_pad / div; a.scol_gstride = H * (a.M_pad / 32);
    }
    return PT_OK;
}

template <int PRO, bool GROUPED>
static int launch_fused(const MxArgs &a, const char *what, int fmt, unsigned flags, cudaStream_t st) {
    int rc = PT_ERR_UNSUPPORTED;
    if (fmt == PT_E4M3) rc = launch_mx_split<PT_E4M3, GROUPED, PRO>(a, 1, a.M_pad, flags, st);
    if (fmt == PT_E2M1) {
        if constexpr (pro_is_glu(PRO)) {
            rc = (flags & PT_MX_COL_RHT) ? launch_mx_split<PT_E2M1, GROUPED, PRO, true>(a, 1, a.M_pad, flags, st)
                                         : launch_mx_split<PT_E2M1, GROUPED, PRO>(a, 1, a.M_pad, flags, st);
        } else {
            rc = launch_mx_split<PT_E2M1, GROUPED, PRO>(a, 1, a.M_pad, flags, st);
        }
    }
    if (rc == PT_ERR_UNSUPPORTED)
        return set_error(PT_ERR_UNSUPPORTED, "%s: outside the fused kernel's range (16-byte aligned buffers, fewer than 2^31 rows, at most %d groups, "
                                             "width a multiple of 64 for the gated activations)", what, kQMaxGroups);
    return rc;
}

}  // namespace ptb

using namespace ptb;

extern "C" {

int pt_glu_quantize_mx(const void *x, int x_dtype, const float *probs, const int64_t *row_mask, int64_t rows, int64_t H, int act, int fmt,
                       unsigned flags, void *q_row, uint8_t *s_row, void *q_col, uint8_t *s_col, void *stream) {
    const char *what = "fused gated activation + MX quantize";
    MxArgs a{};
    int rc = fused_args(a, what, x, x_dtype, rows, H, fmt, flags, q_row, s_row, q_col, s_col, 0, nullptr, nullptr, nullptr, 0);
    if (rc != PT_OK) return rc;
    PT_REQUIRE(act == 0 || act == 1, "%s: act must be 0 (SiLU) or 1 (GELU)", what);
    if (rows == 0 || H == 0) return PT_OK;
    PT_REQUIRE(x && probs, "%s: null pointer", what);
    a.x_cols = 2 * H; a.pro_rowvec = probs; a.pro_mask = row_mask;
    return act == 0 ? launch_fused<PT_PRO_SWIGLU, false>(a, what, fmt, flags, (cudaStream_t) stream)
                    : launch_fused<PT_PRO_GEGLU, false>(a, what, fmt, flags, (cudaStream_t) stream);
}

int pt_grouped_glu_quantize_mx(const void *x, int x_dtype, const float *probs, const int64_t *row_mask, int64_t rows, int64_t H, int act, int G,
                               const int64_t *group_offs, const int64_t *padded_offs_row, const int64_t *padded_offs_col, int fmt, unsigned flags,
                               void *q_row, uint8_t *s_row, void *q_col, uint8_t *s_col, int64_t col_alloc, void *stream) {
    const char *what = "fused gated activation + grouped MX quantize";
    PT_REQUIRE(group_offs, "%s: group offsets required", what);
    MxArgs a{};
    int rc = fused_args(a, what, x, x_dtype, rows, H, fmt, flags, q_row, s_row, q_col, s_col, G, group_offs, padded_offs_row, padded_offs_col, col_alloc);
    if (rc != PT_OK) return rc;
    PT_REQUIRE(act == 0 || act == 1, "%s: act must be 0 (SiLU) or 1 (GELU)", what);
    if (H == 0) return PT_OK;
    PT_REQUIRE(rows == 0 || (x && probs), "%s: null pointer", what);
    a.x_cols = 2 * H; a.pro_rowvec = probs; a.pro_mask = row_mask;
    return act == 0 ? launch_fused<PT_PRO_SWIGLU, true>(a, what, fmt, flags, (cudaStream_t) stream)
                    : launch_fused<PT_PRO_GEGLU, true>(a, what, fmt, flags, (cudaStream_t) stream);
}

int pt_rmsnorm_quantize_mx(const void *x, int x_dtype, const float *rstd, const void *gamma, int zero_centered, int64_t rows, int64_t H, int fmt,
                           unsigned flags, void *q_row, uint8_t *s_row, void *q_col, uint8_t *s_col, void *stream) {
    const char *what = "fused RMSNorm + MX quantize";
    MxArgs a{};
    int rc = fused_args(a, what, x, x_dtype, rows, H, fmt, flags, q_row, s_row, q_col, s_col, 0, nullptr, nullptr, nullptr, 0);
    if (rc != PT_OK) return rc;
    if (rows == 0 || H == 0) return PT_OK;
    PT_REQUIRE(x && rstd && gamma && aligned(gamma, 16), "%s: null or unaligned pointer", what);
    a.pro_rowvec = rstd; a.pro_gamma = gamma; a.pro_zero_centered = zero_centered;
    return launch_fused<PT_PRO_RMSNORM, false>(a, what, fmt, flags, (cudaStream_t) stream);
}

int pt_glu_quantize_mx_row(const void *x, int x_dtype, const float *probs, const int64_t *row_mask, int64_t rows, int64_t H, int act, int fmt,
                           void *q_row, uint8_t *s_row, void *stream) {
    const char *what = "gated activation + row-wise MX quantize";
    PT_REQUIRE(rows >= 0 && H >= 0 && (act == 0 || act == 1), "%s: bad arguments", what);
    PT_REQUIRE(x_dtype == PT_BF16, "%s: bf16 input", what);
    PT_REQUIRE(fmt == PT_E4M3 || fmt == PT_E5M2 || fmt == PT_E2M1, "%s: formats e4m3, e5m2, e2m1", what);
    if (H % 32 != 0) return PT_ERR_UNSUPPORTED;   // the caller runs the two kernels
    if (rows == 0 || H == 0) return PT_OK;
    PT_REQUIRE(x && probs && q_row && s_row && aligned(x, 16) && aligned(q_row, 8), "%s: null or unaligned pointer", what);
    const int64_t n_pad = ceil_to(H, 128);
    cudaStream_t st = (cudaStream_t) stream;
#define PT_GR_LAUNCH(F_, A_)                                                                                        \
    do {                                                                                                            \
        auto kern = glu_mx_row_kernel<F_, A_>;                                                                      \
        int per_sm = 0;                                                                                             \
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kRnThreads, 0) != cudaSuccess || per_sm <= 0) { \
            cudaGetLastError();                                                                                     \
            per_sm = 2;                                                                                             \
        }                                                                                                           \
        const int64_t per_cta = std::max<int64_t>(1, ceil_div(rows, (int64_t) sm_count() * per_sm));               \
        kern<<<(int) ceil_div(rows, per_cta), kRnThreads, 0, st>>>((const __nv_bfloat16 *) x, probs, row_mask, rows, H, n_pad, \
                                                                   (uint8_t *) q_row, s_row);                      \
    } while (0)
#define PT_GR_FMT(A_)                                                                                               \
    do {                                                                                                            \
        if (fmt == PT_E4M3) PT_GR_LAUNCH(PT_E4M3, A_);                                                              \
        else if (fmt == PT_E5M2) PT_GR_LAUNCH(PT_E5M2, A_);                                                         \
        else PT_GR_LAUNCH(PT_E2M1, A_);                                                                             \
    } while (0)
    if (act == 0) PT_GR_FMT(PT_ACT_SILU);
    else PT_GR_FMT(PT_ACT_GELU);
#undef PT_GR_FMT
#undef PT_GR_LAUNCH
    PT_LAUNCH_OK();
    return PT_OK;
}

int pt_rmsnorm_quantize_mx_row(const void *x, int x_dtype, const void *gamma, float eps, int zero_centered, int64_t rows, int64_t H,
                               int fmt, void *q_row, uint8_t *s_row, float *rstd, void *stream) {
    const char *what = "RMSNorm + row-wise MX quantize";
    PT_REQUIRE(rows >= 0 && H >= 0, "%s: bad shape", what);
    PT_REQUIRE(x_dtype == PT_BF16, "%s: bf16 input", what);
    PT_REQUIRE(fmt == PT_E4M3 || fmt == PT_E5M2 || fmt == PT_E2M1, "%s: formats e4m3, e5m2, e2m1", what);
    if (H % 32 != 0 || ceil_to(H, 128) > (int64_t) kRnThreads * 8 * kRnKeep) return PT_ERR_UNSUPPORTED;   // the caller runs the two kernels
    if (rows == 0 || H == 0) return PT_OK;
    PT_REQUIRE(x && gamma && q_row && s_row && rstd && aligned(x, 16) && aligned(gamma, 16) && aligned(q_row, 8) && aligned(s_row, 4),
               "%s: null or unaligned pointer", what);
    cudaStream_t st = (cudaStream_t) stream;
    const int64_t n_pad = ceil_to(H, 128);
#define PT_RN_LAUNCH_K(F_, K_)                                                                                      \
    do {                                                                                                            \
        auto kern = rmsnorm_mx_row_kernel<F_, K_>;                                                                  \
        int per_sm = 0;                                                                                             \
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kRnThreads, 0) != cudaSuccess || per_sm <= 0) { \
            cudaGetLastError();                                                                                     \
            per_sm = 2;                                                                                             \
        }                                                                                                           \
        const int64_t per_cta = std::max<int64_t>(1, ceil_div(rows, (int64_t) sm_count() * per_sm));               \
        const int grid = (int) ceil_div(rows, per_cta);                                                             \
        kern<<<grid, kRnThreads, 0, st>>>((const __nv_bfloat16 *) x, (const __nv_bfloat16 *) gamma, eps, zero_centered, rows, H, n_pad, \
                                          (uint8_t *) q_row, s_row, rstd);                                          \
    } while (0)
#define PT_RN_LAUNCH(F_)                                                                                            \
    do {                                                                                                            \
        if (n_pad <= (int64_t) kRnThreads * 8 * 2) PT_RN_LAUNCH_K(F_, 2);                                           \
        else PT_RN_LAUNCH_K(F_, 4);                                                                                 \
    } while (0)
    if (fmt == PT_E4M3) PT_RN_LAUNCH(PT_E4M3);
    else if (fmt == PT_E5M2) PT_RN_LAUNCH(PT_E5M2);
    else PT_RN_LAUNCH(PT_E2M1);
#undef PT_RN_LAUNCH_K
#undef PT_RN_LAUNCH
    PT_LAUNCH_OK();
    return PT_OK;
}

int pt_grouped_quantize_mx(const void *x, int x_dtype, int64_t M, int64_t N, int G, const int64_t *group_offs,
                           const int64_t *padded_offs_row, const int64_t *padded_offs_col, int fmt, unsigned flags, void *q_row,
                           uint8_t *s_row, void *q_col, uint8_t *s_col, int64_t col_alloc, void *stream) {
    PT_REQUIRE(M >= 0 && N >= 0 && G >= 1, "grouped MX quantize: bad shape");
    PT_REQUIRE(N % 32 == 0, "grouped MX quantize: N must be divisible by 32 (got %lld)", (long long) N);
    PT_REQUIRE(x_dtype == PT_BF16 || x_dtype == PT_F16, "grouped MX quantize: input must be bf16 or fp16");
    PT_REQUIRE(flags & (PT_MX_ROW | PT_MX_COL), "grouped MX quantize: no output requested");
    PT_REQUIRE(!(flags & (PT_MX_ROW_2D | PT_MX_COL_2D)), "grouped MX quantize: 2-D block scales are a weight option, not a grouped one");
    PT_REQUIRE(group_offs && padded_offs_col, "grouped MX quantize: group offsets required");
    PT_REQUIRE(!(flags & PT_MX_ROW) || (q_row && s_row && padded_offs_row), "grouped MX quantize: row outputs missing");
    PT_REQUIRE(!(flags & PT_MX_COL) || (q_col && s_col), "grouped MX quantize: col outputs missing");
    PT_REQUIRE(col_alloc % 128 == 0 && col_alloc >= M, "grouped MX quantize: col_alloc must be the 128-multiple width of the col-wise buffers");
    PT_REQUIRE(fmt == PT_E2M1 || !(flags & (PT_MX_ROW_RHT | PT_MX_COL_RHT | PT_MX_ROW_SR | PT_MX_COL_SR)),
               "grouped MX quantize: RHT and stochastic rounding are e2m1 options");
    if (N == 0) return PT_OK;
    PT_REQUIRE(x == nullptr ? M == 0 : aligned(x, 16), "grouped MX quantize: input must be 16-byte aligned");
    MxArgs a{};
    a.x = x; a.M = M; a.N = N; a.M_pad = col_alloc; a.N_pad = ceil_to(N, 128);
    a.q_row = (uint8_t *) q_row; a.s_row = s_row; a.q_col = (uint8_t *) q_col; a.s_col = s_col;
    a.group_offs = group_offs; a.poffs_row = padded_offs_row; a.poffs_col = padded_offs_col; a.num_groups = G;
    set_sr(a, flags);
    const int64_t m_alloc = col_alloc;  // the padded row space never exceeds the width the caller allocated for it
    PT_REQUIRE(m_alloc / kTileM <= 65535, "grouped MX quantize: too many rows");
    cudaStream_t st = (cudaStream_t) stream;
    if (x_dtype == PT_BF16) {
        if (fmt == PT_E4M3) return launch_mx_grouped<__nv_bfloat16, PT_E4M3>(a, m_alloc, flags, st);
        if (fmt == PT_E5M2) return launch_mx_grouped<__nv_bfloat16, PT_E5M2>(a, m_alloc, flags, st);
        if (fmt == PT_E2M1) return launch_mx_grouped<__nv_bfloat16, PT_E2M1>(a, m_alloc, flags, st);
    } else {
        if (fmt == PT_E4M3) return launch_mx_grouped<__half, PT_E4M3>(a, m_alloc, flags, st);
        if (fmt == PT_E5M2) return launch_mx_grouped<__half, PT_E5M2>(a, m_alloc, flags, st);
        if (fmt == PT_E2M1) return launch_mx_grouped<__half, PT_E2M1>(a, m_alloc, flags, st);
    }
    return set_error(PT_ERR_INVALID, "grouped MX quantize: unknown format %d", fmt);
}

int pt_quantize_mx(const void *x, int x_dtype, int64_t G, int64_t M, int64_t N, int fmt, unsigned flags, void *q_row,
                   uint8_t *s_row, void *q_col, uint8_t *s_col, void *stream) {
    PT_REQUIRE(G >= 1 && M >= 0 && N >= 0, "MX quantize: bad shape");
    PT_REQUIRE(N % 32 == 0, "MX quantize: N must be divisible by 32 (got %lld)", (long long) N);
    PT_REQUIRE(x_dtype == PT_BF16 || x_dtype == PT_F16, "MX quantize: input must be bf16 or fp16");
    PT_REQUIRE(flags & (PT_MX_ROW | PT_MX_COL), "MX quantize: no output requested");
    PT_REQUIRE(!(flags & PT_MX_ROW) || (q_row && s_row), "MX quantize: row outputs missing");
    PT_REQUIRE(!(flags & PT_MX_COL) || (q_col && s_col), "MX quantize: col outputs missing");
    PT_REQUIRE(fmt == PT_E2M1 || !(flags & (PT_MX_ROW_RHT | PT_MX_COL_RHT | PT_MX_ROW_SR | PT_MX_COL_SR)),
               "MX quantize: RHT and stochastic rounding are e2m1 options");
    if (M == 0 || N == 0) return PT_OK;
    PT_REQUIRE(x && aligned(x, 16), "MX quantize: input must be 16-byte aligned");
    PT_REQUIRE(G <= 65535, "MX quantize: batch too large");
    MxArgs a{};
    a.x = x; a.M = M; a.N = N; a.M_pad = ceil_to(M, 128); a.N_pad = ceil_to(N, 128);
    PT_REQUIRE(a.M_pad / kTileM <= 65535, "MX quantize: M too large");
    a.q_row = (uint8_t *) q_row; a.s_row = s_row; a.q_col = (uint8_t *) q_col; a.s_col = s_col;
    const int div = fmt == PT_E2M1 ? 2 : 1;
    a.x_gstride = M * N;
    a.qrow_gstride = M * a.N_pad / div; a.srow_gstride = M * (a.N_pad / 32);
    a.qcol_gstride = N * a.M_pad / div; a.scol_gstride = N * (a.M_pad / 32);
    set_sr(a, flags);
    cudaStream_t st = (cudaStream_t) stream;
    if (x_dtype == PT_BF16) {
        if (fmt == PT_E4M3) return launch_mx<__nv_bfloat16, PT_E4M3>(a, G, flags, st);
        if (fmt == PT_E5M2) return launch_mx<__nv_bfloat16, PT_E5M2>(a, G, flags, st);
        if (fmt == PT_E2M1) return launch_mx<__nv_bfloat16, PT_E2M1>(a, G, flags, st);
    } else {
        if (fmt == PT_E4M3) return launch_mx<__half, PT_E4M3>(a, G, flags, st);
        if (fmt == PT_E5M2) return launch_mx<__half, PT_E5M2>(a, G, flags, st);
        if (fmt == PT_E2M1) return launch_mx<__half, PT_E2M1>(a, G, flags, st);
    }
    return set_error(PT_ERR_INVALID, "MX quantize: unknown format %d", fmt);
}

int pt_dequantize_mx(const void *q, int fmt, const uint8_t *s, int64_t rows, int64_t cols, int64_t cols_stored,
                     int transpose_out, void *y, int y_dtype, void *stream) {
    PT_REQUIRE(rows >= 0 && cols >= 0 && cols <= cols_stored && cols_stored % 32 == 0, "MX dequantize: bad shape");
    PT_REQUIRE(fmt == PT_E4M3 || fmt == PT_E5M2 || fmt == PT_E2M1, "MX dequantize: unknown format %d", fmt);
    if (rows * cols == 0) return PT_OK;
    PT_REQUIRE(q && s && y, "MX dequantize: null pointer");
    const int blocks = (int) std::min<int64_t>(ceil_div(rows * cols, 256), (int64_t) sm_count() * 16);
    PT_SWITCH_SRC(y_dtype, T, {
        mx_dequant_kernel<T><<<blocks, 256, 0, (cudaStream_t) stream>>>((const uint8_t *) q, fmt, s, rows, cols,
                                                                        cols_stored, transpose_out, (T *) y);
        PT_LAUNCH_OK();
    });
    return PT_OK;
}

}  // extern "C"
