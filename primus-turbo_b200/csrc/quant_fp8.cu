// Tensorwise and rowwise FP8 quantize / dequantize: HBM-bound streaming kernels.
//
// Arithmetic follows csrc/include/primus_turbo/device/quant_utils.cuh:33-74 of the reference:
//   scale = qmax / fmax(amax, 1e-12f), scale_inv = 1.0f / scale,
//   q = fp8_rne(fmax(fmin(float(x) * scale, qmax), -qmax)),
// the clamp being done by the saturating convert (mul_sat in common.cuh).
#include <cuda_fp8.h>
#include <stdarg.h>
#include <algorithm>
#include <mutex>
#include <stdio.h>

#include "common.cuh"

namespace ptb {

// ------------------------------------------------------------------------------------------------
// error plumbing
static thread_local char g_err[512] = "";
int set_error(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

constexpr int kThreads = 256;
constexpr float kEpsTensor = 1e-12f;

// ------------------------------------------------------------------------------------------------
// amax over a flat array: 8-element vectors, 4 in flight per thread, one atomicMax per block.
// Entry of a kernel launched with launch_overlapped(): wait until every earlier kernel of the stream has completed (its
// results are then visible), then let the next kernel of the stream begin its own launch.  Only the second kernel of a
// quantizer is launched that way: its grid exists before the first one has finished, so what the first one wrote (the
// amax words) is read with __ldcg, never through the read-only path; x was complete before the first kernel started.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Non-negative floats order like their bit patterns, so the running maximum is kept as uint32.
template <typename T>
__global__ void __launch_bounds__(kThreads) amax_flat_kernel(const T *__restrict__ x, int64_t n, int vec_ok,
                                                             unsigned *__restrict__ amax_bits) {
    pdl_enter();
    float m = 0.f;
    const int64_t tid = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nthreads = (int64_t) gridDim.x * blockDim.x;
    int64_t done = 0;
    if (vec_ok) {
        const int64_t nvec = n / 8;
        int64_t i = tid;
        for (; i + 3 * nthreads < nvec; i += 4 * nthreads) {
            float v[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) load8(x + (i + u * nthreads) * 8, v[u]);
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int k = 0; k < 8; ++k) m = fmaxf(m, fabsf(v[u][k]));
        }
        for (; i < nvec; i += nthreads) {
            float v[8];
            load8(x + i * 8, v);
#pragma unroll
            for (int k = 0; k < 8; ++k) m = fmaxf(m, fabsf(v[k]));
        }
        done = nvec * 8;
    }
    for (int64_t i = done + tid; i < n; i += nthreads) m = fmaxf(m, fabsf(load1(x + i)));

    m = warp_max(m);
    __shared__ float s[kThreads / 32];
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        float w = threadIdx.x < kThreads / 32 ? s[threadIdx.x] : 0.f;
        w = warp_max(w);
        if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_uint(w));
    }
}

// Flat cast with one scale read from device memory. 16 elements per thread per step.
template <typename T, int FMT>
__global__ void __launch_bounds__(kThreads)
    cast_flat_kernel(const T *__restrict__ x, int64_t n, int vec_ok, const unsigned *__restrict__ amax_bits,
                     const float *__restrict__ scale_opt, uint8_t *__restrict__ q, float *__restrict__ scale_inv) {
    pdl_enter();
    float scale;
    if (scale_opt != nullptr) scale = __ldcg(scale_opt);
    else scale = scale_from_amax<FMT>(__uint_as_float(__ldcg(amax_bits)), kEpsTensor);   // from the kernel before: not the read-only path
    const int64_t tid = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nthreads = (int64_t) gridDim.x * blockDim.x;
    if (tid == 0) *scale_inv = __fdiv_rn(1.0f, scale);
    int64_t done = 0;
    if (vec_ok) {
        const int64_t nvec = n / 16;
        for (int64_t i = tid; i < nvec; i += nthreads) {
            float a[8], b[8];
            load8(x + i * 16, a);
            load8(x + i * 16 + 8, b);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                a[k] = mul_sat<FMT>(a[k], scale);
                b[k] = mul_sat<FMT>(b[k], scale);
            }
            uint4 o;
            o.x = cvt4_fp8<FMT>(a[0], a[1], a[2], a[3]);
            o.y = cvt4_fp8<FMT>(a[4], a[5], a[6], a[7]);
            o.z = cvt4_fp8<FMT>(b[0], b[1], b[2], b[3]);
            o.w = cvt4_fp8<FMT>(b[4], b[5], b[6], b[7]);
            *reinterpret_cast<uint4 *>(q + i * 16) = o;
        }
        done = nvec * 16;
    }
    for (int64_t i = done + tid; i < n; i += nthreads) q[i] = cvt1_fp8<FMT>(mul_sat<FMT>(load1(x + i), scale));
}

// ------------------------------------------------------------------------------------------------
// Row-major rowwise: one block per row; the row is read twice (second read hits L1/L2).
template <typename T, int FMT>
__global__ void __launch_bounds__(kThreads)
    rowwise_last_axis_kernel(const T *__restrict__ x, int64_t rows, int64_t len, int vec_ok,
                             const float *__restrict__ scale_opt, uint8_t *__restrict__ q,
                             float *__restrict__ scale_inv) {
    __shared__ float s[kThreads / 32];
    __shared__ float s_scale;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T *xr = x + row * len;
        uint8_t *qr = q + row * len;
        float scale;
        if (scale_opt != nullptr) {
            scale = __ldg(scale_opt + row);
        } else {
            float m = 0.f;
            int64_t done = 0;
            if (vec_ok) {
                const int64_t nvec = len / 8;
                for (int64_t i = threadIdx.x; i < nvec; i += kThreads) {
                    float v[8];
                    load8(xr + i * 8, v);
#pragma unroll
                    for (int k = 0; k < 8; ++k) m = fmaxf(m, fabsf(v[k]));
                }
                done = nvec * 8;
            }
            for (int64_t i = done + threadIdx.x; i < len; i += kThreads) m = fmaxf(m, fabsf(load1(xr + i)));
            m = warp_max(m);
            if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
            __syncthreads();
            if (threadIdx.x < 32) {
                float w = threadIdx.x < kThreads / 32 ? s[threadIdx.x] : 0.f;
                w = warp_max(w);
                if (threadIdx.x == 0) s_scale = scale_from_amax<FMT>(w, kEpsTensor);
            }
            __syncthreads();
            scale = s_scale;
        }
        if (threadIdx.x == 0) scale_inv[row] = __fdiv_rn(1.0f, scale);
        int64_t done = 0;
        if (vec_ok) {
            const int64_t nvec = len / 8;
            for (int64_t i = threadIdx.x; i < nvec; i += kThreads) {
                float v[8];
                load8(xr + i * 8, v);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[k] = mul_sat<FMT>(v[k], scale);
                uint2 o;
                o.x = cvt4_fp8<FMT>(v[0], v[1], v[2], v[3]);
                o.y = cvt4_fp8<FMT>(v[4], v[5], v[6], v[7]);
                *reinterpret_cast<uint2 *>(qr + i * 8) = o;
            }
            done = nvec * 8;
        }
        for (int64_t i = done + threadIdx.x; i < len; i += kThreads)
            qr[i] = cvt1_fp8<FMT>(mul_sat<FMT>(load1(xr + i), scale));
        __syncthreads();  // s / s_scale are reused by the next row
    }
}

// Rows of 16-bit elements that fit the registers of one block (up to 4 x 16 bytes per thread = 8192 elements): the row
// is read once, its |max| is formed on packed pairs, one block-wide exchange gives the scale, and the kept words are
// scaled and converted.  Same arithmetic as rowwise_last_axis_kernel.
template <typename T, int FMT, int KEEP>
__global__ void __launch_bounds__(kThreads, KEEP == 2 ? 8 : 4) rowwise_row_in_regs_kernel(const T *__restrict__ x, int64_t rows, int64_t len,
                                                                                        uint8_t *__restrict__ q, float *__restrict__ scale_inv) {
    pdl_enter();
    constexpr int kKeep = KEEP;   // 16-byte words per thread: 2 (rows of up to 4096 elements, eight CTAs per SM) or 4
    __shared__ float s[kThreads / 32];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T *xr = x + row * len;
        uint4 keep[kKeep];
        uint32_t m2 = 0u;
#pragma unroll
        for (int k = 0; k < kKeep; ++k) {
            const int64_t i = ((int64_t) k * kThreads + threadIdx.x) * 8;
            if (i < len) {
                keep[k] = __ldg(reinterpret_cast<const uint4 *>(xr + i));
                m2 = absmax2<T>(absmax2<T>(absmax2<T>(absmax2<T>(m2, keep[k].x), keep[k].y), keep[k].z), keep[k].w);
            }
        }
        m2 = absmax2_done(m2);
        float m = warp_max(fmaxf(lo_f32<T>(m2), hi_f32<T>(m2)));
        __syncthreads();   // s may still be read for the previous row
        if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
        __syncthreads();
        m = 0.f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) m = fmaxf(m, s[w]);
        const float scale = scale_from_amax<FMT>(m, kEpsTensor);
        if (threadIdx.x == 0) scale_inv[row] = __fdiv_rn(1.0f, scale);
#pragma unroll
        for (int k = 0; k < kKeep; ++k) {
            const int64_t i = ((int64_t) k * kThreads + threadIdx.x) * 8;
            if (i < len) {
                const uint32_t w[4] = {keep[k].x, keep[k].y, keep[k].z, keep[k].w};
                uint2 o;
                o.x = cvt4_fp8<FMT>(mul_sat<FMT>(lo_f32<T>(w[0]), scale), mul_sat<FMT>(hi_f32<T>(w[0]), scale), mul_sat<FMT>(lo_f32<T>(w[1]), scale),
                                    mul_sat<FMT>(hi_f32<T>(w[1]), scale));
                o.y = cvt4_fp8<FMT>(mul_sat<FMT>(lo_f32<T>(w[2]), scale), mul_sat<FMT>(hi_f32<T>(w[2]), scale), mul_sat<FMT>(lo_f32<T>(w[3]), scale),
                                    mul_sat<FMT>(hi_f32<T>(w[3]), scale));
                *reinterpret_cast<uint2 *>(q + row * len + i) = o;
            }
        }
    }
}

// Column amax of x [B, M, N]: each block owns a (b, 64-row, 256-column) tile and folds it into
// amax_bits [B, N] with atomicMax.
template <typename T>
__global__ void __launch_bounds__(kThreads)
    amax_cols_kernel(const T *__restrict__ x, int64_t M, int64_t N, unsigned *__restrict__ amax_bits) {
    const int64_t b = blockIdx.z;
    const int64_t col = (int64_t) blockIdx.x * kThreads + threadIdx.x;
    if (col >= N) return;
    const int64_t r0 = (int64_t) blockIdx.y * 64;
    const int64_t r1 = min(M, r0 + 64);
    const T *p = x + (b * M) * N + col;
    float m = 0.f;
    for (int64_t r = r0; r < r1; ++r) m = fmaxf(m, fabsf(load1(p + r * N)));
    atomicMax(amax_bits + b * N + col, __float_as_uint(m));
}

// The same for 16-bit inputs with 16-byte aligned rows.  A CTA covers 256 rows x 256 columns: a warp reads 512 contiguous
// bytes of a row (eight columns per lane, |max| on packed pairs), the eight warps take 32 rows each in two batches of
// sixteen loads that are all in flight together, their partial maxima meet in shared memory and one atomic per column
// leaves the CTA.  (With 128 rows per CTA and the loads issued a few at a time the kernel read 3.7 TB/s.)
constexpr int kAmaxVecRows = 128, kAmaxVecCols = 256;   // tiling of the cast kernel
constexpr int kAmaxCtaRows = 256;                       // rows per CTA of the amax kernel
template <typename T>
__global__ void __launch_bounds__(kThreads, 4)
    amax_cols_vec_kernel(const T *__restrict__ x, int64_t M, int64_t N, unsigned *__restrict__ amax_bits) {
    pdl_enter();
    __shared__ uint32_t s_m[kThreads / 32][32][4];
    const int64_t b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t c0 = (int64_t) blockIdx.x * kAmaxVecCols + lane * 8;
    const int64_t r0 = (int64_t) blockIdx.y * kAmaxCtaRows + warp * (kAmaxCtaRows / (kThreads / 32));
    uint32_t m[4] = {0u, 0u, 0u, 0u};
    if (c0 < N) {
        const T *p = x + (b * M) * N + c0;
#pragma unroll 1
        for (int batch = 0; batch < kAmaxCtaRows / (kThreads / 32) / 16; ++batch) {
            uint4 v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int64_t r = r0 + batch * 16 + i;
                v[i] = r < M ? __ldg(reinterpret_cast<const uint4 *>(p + r * N)) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                m[0] = absmax2<T>(m[0], v[i].x); m[1] = absmax2<T>(m[1], v[i].y); m[2] = absmax2<T>(m[2], v[i].z); m[3] = absmax2<T>(m[3], v[i].w);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) s_m[warp][lane][k] = m[k];
    __syncthreads();
    // thread t < 128 finishes column pair t of the CTA's 256 columns
    if (threadIdx.x < 128) {
        const int l = threadIdx.x >> 2, k = threadIdx.x & 3;
        uint32_t w = 0u;
#pragma unroll
        for (int g = 0; g < kThreads / 32; ++g) w = absmax2<T>(w, s_m[g][l][k]);
        w = absmax2_done(w);
        const int64_t c = (int64_t) blockIdx.x * kAmaxVecCols + 2 * threadIdx.x;
        if (c < N) {
            atomicMax(amax_bits + b * N + c, __float_as_uint(lo_f32<T>(w)));
            atomicMax(amax_bits + b * N + c + 1, __float_as_uint(hi_f32<T>(w)));
        }
    }
}

// The cast for 16-bit inputs with 16-byte aligned rows, on the tiling of amax_cols_vec_kernel: a lane owns eight columns
// (their scales computed once), a warp 16 rows of them, all sixteen loads in flight.
template <typename T, int FMT>
__global__ void __launch_bounds__(kThreads)
    cast_cols_vec_kernel(const T *__restrict__ x, int64_t M, int64_t N, const unsigned *__restrict__ amax_bits, uint8_t *__restrict__ q,
                         float *__restrict__ scale_inv) {
    pdl_enter();
    const int64_t b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t c0 = (int64_t) blockIdx.x * kAmaxVecCols + lane * 8;
    if (c0 >= N) return;
    const int64_t r0 = (int64_t) blockIdx.y * kAmaxVecRows + warp * 16;
    float sc[8];
    {
        // written by the amax kernel this launch overlaps: not the read-only path
        const uint4 a0 = __ldcg(reinterpret_cast<const uint4 *>(amax_bits + b * N + c0)), a1 = __ldcg(reinterpret_cast<const uint4 *>(amax_bits + b * N + c0 + 4));
        const uint32_t ab[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) sc[k] = scale_from_amax<FMT>(__uint_as_float(ab[k]), kEpsTensor);
        if (blockIdx.y == 0 && warp == 0) {
            float4 i0, i1;
            i0.x = __fdiv_rn(1.0f, sc[0]); i0.y = __fdiv_rn(1.0f, sc[1]); i0.z = __fdiv_rn(1.0f, sc[2]); i0.w = __fdiv_rn(1.0f, sc[3]);
            i1.x = __fdiv_rn(1.0f, sc[4]); i1.y = __fdiv_rn(1.0f, sc[5]); i1.z = __fdiv_rn(1.0f, sc[6]); i1.w = __fdiv_rn(1.0f, sc[7]);
            *reinterpret_cast<float4 *>(scale_inv + b * N + c0) = i0;
            *reinterpret_cast<float4 *>(scale_inv + b * N + c0 + 4) = i1;
        }
    }
    uint4 v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
        if (r0 + i < M) v[i] = __ldg(reinterpret_cast<const uint4 *>(x + (b * M + r0 + i) * N + c0));
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        if (r0 + i < M) {
            uint2 o;
            o.x = cvt4_fp8<FMT>(mul_sat<FMT>(lo_f32<T>(v[i].x), sc[0]), mul_sat<FMT>(hi_f32<T>(v[i].x), sc[1]), mul_sat<FMT>(lo_f32<T>(v[i].y), sc[2]),
                                mul_sat<FMT>(hi_f32<T>(v[i].y), sc[3]));
            o.y = cvt4_fp8<FMT>(mul_sat<FMT>(lo_f32<T>(v[i].z), sc[4]), mul_sat<FMT>(hi_f32<T>(v[i].z), sc[5]), mul_sat<FMT>(lo_f32<T>(v[i].w), sc[6]),
                                mul_sat<FMT>(hi_f32<T>(v[i].w), sc[7]));
            *reinterpret_cast<uint2 *>(q + (b * M + r0 + i) * N + c0) = o;
        }
    }
}

// Cast of x [B, M, N] with one scale per (b, column). 8 columns per thread when aligned.
template <typename T, int FMT>
__global__ void __launch_bounds__(kThreads)
    cast_cols_kernel(const T *__restrict__ x, int64_t M, int64_t N, int vec_ok, const unsigned *__restrict__ amax_bits,
                     const float *__restrict__ scale_opt, uint8_t *__restrict__ q, float *__restrict__ scale_inv) {
    const int64_t b = blockIdx.z;
    const int64_t r0 = (int64_t) blockIdx.y * 32;
    const int64_t r1 = min(M, r0 + 32);
    const int W = vec_ok ? 8 : 1;
    const int64_t c0 = ((int64_t) blockIdx.x * kThreads + threadIdx.x) * W;
    if (c0 >= N) return;
    float sc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        if (k < W) {
            sc[k] = scale_opt ? __ldg(scale_opt + b * N + c0 + k)
                              : scale_from_amax<FMT>(__uint_as_float(amax_bits[b * N + c0 + k]), kEpsTensor);
            if (blockIdx.y == 0) scale_inv[b * N + c0 + k] = __fdiv_rn(1.0f, sc[k]);
        }
    }
    for (int64_t r = r0; r < r1; ++r) {
        const int64_t off = (b * M + r) * N + c0;
        if (vec_ok) {
            float v[8];
            load8(x + off, v);
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = mul_sat<FMT>(v[k], sc[k]);
            uint2 o;
            o.x = cvt4_fp8<FMT>(v[0], v[1], v[2], v[3]);
            o.y = cvt4_fp8<FMT>(v[4], v[5], v[6], v[7]);
            *reinterpret_cast<uint2 *>(q + off) = o;
        } else {
            q[off] = cvt1_fp8<FMT>(mul_sat<FMT>(load1(x + off), sc[0]));
        }
    }
}

// ------------------------------------------------------------------------------------------------
// dequantize: y = float(q) * scale_inv
template <int FMT> __device__ __forceinline__ float decode_fp8(uint8_t c) {
    if constexpr (FMT == PT_E4M3) {
        __half_raw h = __nv_cvt_fp8_to_halfraw(c, __NV_E4M3);
        return __half2float(__half(h));
    } else {
        return __half2float(__ushort_as_half((uint16_t) c << 8));  // e5m2 is the top byte of fp16
    }
}
template <typename T> __device__ __forceinline__ void store1(T *p, float v);
template <> __device__ __forceinline__ void store1<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void store1<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void store1<__half>(__half *p, float v) { *p = __float2half_rn(v); }

template <typename T, int FMT>
__global__ void __launch_bounds__(kThreads) dequant_kernel(const uint8_t *__restrict__ q, const float *__restrict__ s,
                                                           int kind, int64_t M, int64_t N, int64_t total,
                                                           T *__restrict__ y) {
    const int64_t stride = (int64_t) gridDim.x * blockDim.x;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int64_t si = 0;
        if (kind == 1) si = i / N;                             // per row
        else if (kind == 2) si = (i / (M * N)) * N + (i % N);  // per (batch, column)
        store1(y + i, decode_fp8<FMT>(q[i]) * __ldg(s + si));
    }
}

// ------------------------------------------------------------------------------------------------
// Scratch for pt_quantize_fp8_colscale_noalloc: the per-column running amax lives in this fixed array
// instead of caller-provided memory.  Every GPU that loads the library holds these 256 KiB until exit.
constexpr int64_t kNoAllocMaxColumns = 65536;
static __device__ __align__(256) unsigned g_noalloc_amax[kNoAllocMaxColumns];

// In host code `g_noalloc_amax` is only a stand-in for the symbol, not a device address; the address a
// kernel can use is looked up once per device (with that device current) and cached.
static int noalloc_scratch(unsigned **out) {
    static std::mutex mu;
    static unsigned *cached[64] = {nullptr};
    int dev = 0;
    PT_CUDA_OK(cudaGetDevice(&dev));
    PT_REQUIRE(dev >= 0 && dev < 64, "no-alloc quantize: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void *p = nullptr;
        PT_CUDA_OK(cudaGetSymbolAddress(&p, g_noalloc_amax));
        PT_REQUIRE(p != nullptr, "no-alloc quantize: the scratch symbol has no address on device %d", dev);
        cached[dev] = static_cast<unsigned *>(p);
    }
    *out = cached[dev];
    return PT_OK;
}

}  // namespace ptb

namespace ptb {
// Grid for a grid-stride loop over `items` units of work: no more CTAs than are resident at once, and every CTA the same
// number of units give or take one.  (A fixed "SMs x 16" grid gave the 8192-row rowwise quantizer 3.2 waves of CTAs of
// 3 or 4 rows each: the last wave ran a third full.)
template <typename Kernel> static int balanced_grid(Kernel kern, int threads, int64_t items) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, 0) != cudaSuccess || per_sm <= 0) {
        cudaGetLastError();
        per_sm = 4;
    }
    const int64_t resident = (int64_t) sm_count() * per_sm;
    const int64_t per_cta = std::max<int64_t>(1, ceil_div(items, resident));
    return (int) std::max<int64_t>(1, ceil_div(items, per_cta));
}

}  // namespace ptb

using namespace ptb;

extern "C" {

const char *pt_last_error(void) { return ptb::g_err; }

int pt_device_sm_count(void) {
    int dev = 0, n = 0;
    PT_CUDA_OK(cudaGetDevice(&dev));
    PT_CUDA_OK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    return n;
}

size_t pt_quantize_fp8_tensorwise_workspace_bytes(void) { return 256; }

int pt_quantize_fp8_tensorwise(const void *x, int x_dtype, int64_t n, int fmt, void *q, float *scale_inv,
                               const float *scale_opt, void *workspace, size_t workspace_bytes, void *stream) {
    PT_REQUIRE(n >= 0 && (n == 0 || (x && q)) && scale_inv, "tensorwise: null pointer or negative size");
    PT_REQUIRE(scale_opt || (workspace && workspace_bytes >= 4), "tensorwise: workspace of >= 4 bytes required");
    cudaStream_t st = (cudaStream_t) stream;
    unsigned *amax = (unsigned *) workspace;
    const int64_t max_blocks = (int64_t) sm_count() * 8;
    PT_SWITCH_SRC(x_dtype, T, {
        const int vec_ok = aligned(x, sizeof(T) == 4 ? 16 : 16) && aligned(q, 16);
        if (!scale_opt) {
            PT_CUDA_OK(cudaMemsetAsync(amax, 0, 4, st));
            const int blocks = vec_ok ? balanced_grid(amax_flat_kernel<T>, kThreads, ceil_div(n, (int64_t) kThreads * 8))
                                      : (int) std::max<int64_t>(1, std::min(max_blocks, ceil_div(n, (int64_t) kThreads * 32)));
            amax_flat_kernel<T><<<blocks, kThreads, 0, st>>>((const T *) x, n, vec_ok, amax);   // reads x through the read-only path: an ordinary launch
            PT_LAUNCH_OK();
        }
        PT_SWITCH_FP8(fmt, F, {
            const int blocks = vec_ok ? balanced_grid(cast_flat_kernel<T, F>, kThreads, ceil_div(n, (int64_t) kThreads * 16))
                                      : (int) std::max<int64_t>(1, std::min(max_blocks * 2, ceil_div(n, (int64_t) kThreads * 16)));
            PT_CUDA_OK(launch_overlapped(cast_flat_kernel<T, F>, dim3(blocks), dim3(kThreads), 0, st, (const T *) x, n, vec_ok, (const unsigned *) amax,
                                         scale_opt, (uint8_t *) q, scale_inv));
        });
        PT_LAUNCH_OK();
    });
    return PT_OK;
}

int pt_quantize_fp8_rowwise(const void *x, int x_dtype, int64_t B, int64_t M, int64_t N, int axis_is_last, int fmt,
                            void *q, float *scale_inv, const float *scale_opt, void *workspace,
                            size_t workspace_bytes, void *stream) {
    PT_REQUIRE(B >= 0 && M >= 0 && N >= 0 && scale_inv, "rowwise: bad shape or null scale_inv");
    if (B * M * N == 0) return PT_OK;
    PT_REQUIRE(x && q, "rowwise: null pointer");
    cudaStream_t st = (cudaStream_t) stream;
    if (axis_is_last) {
        const int64_t rows = B * M;
        PT_SWITCH_SRC(x_dtype, T, {
            const int vec_ok = aligned(x, 16) && aligned(q, 8) && (N % 8 == 0);
            const int blocks = (int) std::min<int64_t>(rows, (int64_t) sm_count() * 16);
            PT_SWITCH_FP8(fmt, F, {
                if constexpr (sizeof(T) == 2) {
                    if (vec_ok && !scale_opt && N <= (int64_t) kThreads * 8 * 4) {
                        if (N <= (int64_t) kThreads * 8 * 2) {
                            const int rblocks = balanced_grid(rowwise_row_in_regs_kernel<T, F, 2>, kThreads, rows);
                            rowwise_row_in_regs_kernel<T, F, 2><<<rblocks, kThreads, 0, st>>>((const T *) x, rows, N, (uint8_t *) q, scale_inv);
                        } else {
                            const int rblocks = balanced_grid(rowwise_row_in_regs_kernel<T, F, 4>, kThreads, rows);
                            rowwise_row_in_regs_kernel<T, F, 4><<<rblocks, kThreads, 0, st>>>((const T *) x, rows, N, (uint8_t *) q, scale_inv);
                        }
                        PT_LAUNCH_OK();
                        return PT_OK;
                    }
                }
                rowwise_last_axis_kernel<T, F><<<blocks, kThreads, 0, st>>>((const T *) x, rows, N, vec_ok, scale_opt,
                                                                            (uint8_t *) q, scale_inv);
            });
            PT_LAUNCH_OK();
        });
        return PT_OK;
    }
    PT_REQUIRE(B <= 65535, "rowwise: batch too large");
    // the column-scaled kernels put the 32-row blocks of M in grid.y
    PT_REQUIRE(M <= 65535ll * 32, "rowwise: the scaled axis has %lld rows, at most %lld are supported", (long long) M, 65535ll * 32);
    unsigned *amax = (unsigned *) workspace;
    if (!scale_opt) {
        PT_REQUIRE(workspace && workspace_bytes >= (size_t) (B * N) * 4, "rowwise: workspace of B*N floats required");
        PT_CUDA_OK(cudaMemsetAsync(amax, 0, (size_t) (B * N) * 4, st));
    }
    PT_SWITCH_SRC(x_dtype, T, {
        const int vec_ok = aligned(x, 16) && aligned(q, 8) && (N % 8 == 0);
        if (!scale_opt) {
            bool done = false;
            if constexpr (sizeof(T) == 2) {
                if (vec_ok) {
                    dim3 grid((unsigned) ceil_div(N, kAmaxVecCols), (unsigned) ceil_div(M, kAmaxCtaRows), (unsigned) B);
                    amax_cols_vec_kernel<T><<<grid, kThreads, 0, st>>>((const T *) x, M, N, amax);   // reads x through the read-only path: an ordinary launch
                    done = true;
                }
            }
            if (!done) {
                dim3 grid((unsigned) ceil_div(N, kThreads), (unsigned) ceil_div(M, 64), (unsigned) B);
                amax_cols_kernel<T><<<grid, kThreads, 0, st>>>((const T *) x, M, N, amax);
            }
            PT_LAUNCH_OK();
        }
        if constexpr (sizeof(T) == 2) {
            if (vec_ok && !scale_opt && aligned(amax, 16) && aligned(scale_inv, 16)) {
                dim3 vgrid((unsigned) ceil_div(N, kAmaxVecCols), (unsigned) ceil_div(M, kAmaxVecRows), (unsigned) B);
                PT_SWITCH_FP8(fmt, F, {
                    PT_CUDA_OK(launch_overlapped(cast_cols_vec_kernel<T, F>, vgrid, dim3(kThreads), 0, st, (const T *) x, M, N, (const unsigned *) amax,
                                                 (uint8_t *) q, scale_inv));
                });
                return PT_OK;
            }
        }
        dim3 grid((unsigned) ceil_div(N, kThreads * (vec_ok ? 8 : 1)), (unsigned) ceil_div(M, 32), (unsigned) B);
        PT_SWITCH_FP8(fmt, F, {
            cast_cols_kernel<T, F><<<grid, kThreads, 0, st>>>((const T *) x, M, N, vec_ok, amax, scale_opt,
                                                              (uint8_t *) q, scale_inv);
        });
        PT_LAUNCH_OK();
    });
    return PT_OK;
}

int pt_dequantize_fp8(const void *q, int fmt, const float *scale_inv, int scale_kind, int64_t B, int64_t M, int64_t N,
                      void *y, int y_dtype, void *stream) {
    const int64_t total = B * M * N;
    PT_REQUIRE(total >= 0 && scale_kind >= 0 && scale_kind <= 2, "dequantize: bad arguments");
    if (total == 0) return PT_OK;
    PT_REQUIRE(q && y && scale_inv, "dequantize: null pointer");
    const int blocks = (int) std::min<int64_t>(ceil_div(total, kThreads), (int64_t) sm_count() * 16);
    PT_SWITCH_SRC(y_dtype, T, {
        PT_SWITCH_FP8(fmt, F, {
            dequant_kernel<T, F><<<blocks, kThreads, 0, (cudaStream_t) stream>>>((const uint8_t *) q, scale_inv,
                                                                                 scale_kind, M, N, total, (T *) y);
        });
        PT_LAUNCH_OK();
    });
    return PT_OK;
}

int pt_quantize_fp8_colscale_noalloc(const void *x, int x_dtype, int64_t B, int64_t M, int64_t N, int fmt, void *q,
                                     float *scale_inv, void *stream) {
    PT_REQUIRE(B >= 0 && M >= 0 && N >= 0 && scale_inv, "no-alloc quantize: bad shape or null scale_inv");
    PT_REQUIRE(B * N <= kNoAllocMaxColumns,
               "no-alloc quantize: B * N = %lld columns exceed the built-in scratch of %lld; use pt_quantize_fp8_rowwise "
               "with a caller-provided workspace", (long long) (B * N), (long long) kNoAllocMaxColumns);
    if (B * M * N == 0) return PT_OK;
    PT_REQUIRE(x && q, "no-alloc quantize: null pointer");
    PT_REQUIRE(B <= 65535, "no-alloc quantize: batch too large");
    PT_REQUIRE(M <= 65535ll * 32, "no-alloc quantize: the scaled axis has %lld rows, at most %lld are supported", (long long) M,
               65535ll * 32);
    unsigned *amax = nullptr;
    int rc = noalloc_scratch(&amax);  // first call on a device resolves the scratch address
    if (rc != PT_OK) return rc;
    cudaStream_t st = (cudaStream_t) stream;
    // the array keeps the previous call's maxima: start this call's columns from zero
    PT_CUDA_OK(cudaMemsetAsync(amax, 0, (size_t) (B * N) * sizeof(unsigned), st));
    PT_SWITCH_SRC(x_dtype, T, {
        dim3 grid_a((unsigned) ceil_div(N, kThreads), (unsigned) ceil_div(M, 64), (unsigned) B);
        amax_cols_kernel<T><<<grid_a, kThreads, 0, st>>>((const T *) x, M, N, amax);
        PT_LAUNCH_OK();
        const int vec_ok = aligned(x, 16) && aligned(q, 8) && (N % 8 == 0);
        dim3 grid_c((unsigned) ceil_div(N, kThreads * (vec_ok ? 8 : 1)), (unsigned) ceil_div(M, 32), (unsigned) B);
        PT_SWITCH_FP8(fmt, F, {
            cast_cols_kernel<T, F><<<grid_c, kThreads, 0, st>>>((const T *) x, M, N, vec_ok, amax, nullptr, (uint8_t *) q,
                                                                scale_inv);
        });
        PT_LAUNCH_OK();
    });
    return PT_OK;
}

}  // extern "C"
