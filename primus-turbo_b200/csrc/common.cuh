// Shared device / host helpers for the sm_100a low-precision GEMM path.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/pt_b200.h"

namespace ptb {

// ---------------------------------------------------------------- error reporting
// Records a message for pt_last_error() and returns `code`.
int set_error(int code, const char *fmt, ...);

#define PT_REQUIRE(cond, ...)                                                                      \
    do {                                                                                           \
        if (!(cond)) return ::ptb::set_error(PT_ERR_INVALID, __VA_ARGS__);                         \
    } while (0)

#define PT_CUDA_OK(expr)                                                                           \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return ::ptb::set_error(PT_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                   \
                                    cudaGetErrorString(_e), __FILE__, __LINE__);                   \
    } while (0)

#define PT_LAUNCH_OK() PT_CUDA_OK(cudaGetLastError())

int sm_count();  // cached multiprocessor count of the current device
int *default_status();  // status word registered for the current device with pt_set_default_status, or null

// Index of the current device for the small per-device caches below (function attributes and occupancy are
// per-device state; a process may drive several GPUs).
inline int current_device_slot() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    return dev;
}

// Launch that may overlap the tail of the previous kernel on the stream (programmatic stream serialization): only for
// kernels that call sm100::grid_dep_wait() before touching memory an earlier kernel produces or reads.
// PT_NO_PDL=1 (read per call) launches the ordinary way, for A/B runs.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = getenv("PT_NO_PDL") == nullptr ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t ceil_to(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

// ---------------------------------------------------------------- element access
template <typename T> struct Src;
template <> struct Src<__nv_bfloat16> {
    static constexpr uint32_t kInfBits = 0x7F80u;
    static __device__ __forceinline__ float to_f32(uint16_t b) { return __uint_as_float((uint32_t) b << 16); }
};
template <> struct Src<__half> {
    static constexpr uint32_t kInfBits = 0x7C00u;
    static __device__ __forceinline__ float to_f32(uint16_t b) { return __half2float(__ushort_as_half(b)); }
};

// Loads 8 consecutive elements starting at p (16-byte aligned for 2-byte types, 32 for fp32).
template <typename T> __device__ __forceinline__ void load8(const T *p, float (&v)[8]) {
    const uint4 r = __ldg(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i]     = Src<T>::to_f32((uint16_t) (w[i] & 0xFFFF));
        v[2 * i + 1] = Src<T>::to_f32((uint16_t) (w[i] >> 16));
    }
}
template <> __device__ __forceinline__ void load8<float>(const float *p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p));
    const float4 b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <typename T> __device__ __forceinline__ float load1(const T *p) {
    return Src<T>::to_f32(*reinterpret_cast<const uint16_t *>(p));
}
template <> __device__ __forceinline__ float load1<float>(const float *p) { return *p; }

// ---------------------------------------------------------------- packed 16-bit helpers
// Running |max| over words holding two bf16 / fp16 elements, one instruction per word: max.xorsign.abs takes the
// magnitudes of both inputs itself (the sign it leaves in the result is meaningless and dropped by absmax2_done at
// the end); a NaN half is ignored, as by fmaxf.
template <typename T> __device__ __forceinline__ uint32_t absmax2(uint32_t m, uint32_t w);
template <> __device__ __forceinline__ uint32_t absmax2<__nv_bfloat16>(uint32_t m, uint32_t w) {
    uint32_t r;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(m), "r"(w));
    return r;
}
template <> __device__ __forceinline__ uint32_t absmax2<__half>(uint32_t m, uint32_t w) {
    uint32_t r;
    asm("max.xorsign.abs.f16x2 %0, %1, %2;" : "=r"(r) : "r"(m), "r"(w));
    return r;
}
__device__ __forceinline__ uint32_t absmax2_done(uint32_t m) { return m & 0x7FFF7FFFu; }
// The same with NaN propagation: a NaN half in any input leaves a NaN in that half of the running maximum, which is how
// the quantizers find the (rare) blocks that hold a NaN without a test per element.
template <typename T> __device__ __forceinline__ uint32_t absmax2_nan(uint32_t m, uint32_t w);
template <> __device__ __forceinline__ uint32_t absmax2_nan<__nv_bfloat16>(uint32_t m, uint32_t w) {
    uint32_t r;
    asm("max.NaN.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(m), "r"(w));
    return r;
}
template <> __device__ __forceinline__ uint32_t absmax2_nan<__half>(uint32_t m, uint32_t w) {
    uint32_t r;
    asm("max.NaN.xorsign.abs.f16x2 %0, %1, %2;" : "=r"(r) : "r"(m), "r"(w));
    return r;
}
// either half of a packed running maximum is a NaN
template <typename T> __device__ __forceinline__ bool packed_has_nan(uint32_t pm) {
    const uint32_t a = pm & 0x7FFF7FFFu;
    const uint32_t lim = Src<T>::kInfBits;
    return ((a & 0xFFFFu) > lim) | ((a >> 16) > lim);
}
template <typename T> __device__ __forceinline__ float lo_f32(uint32_t w) { return Src<T>::to_f32((uint16_t) (w & 0xFFFF)); }
template <typename T> __device__ __forceinline__ float hi_f32(uint32_t w) { return Src<T>::to_f32((uint16_t) (w >> 16)); }

// ---------------------------------------------------------------- fp32 -> fp8 / fp4 (RNE, saturate to finite)
// Two floats to two codes; `lo` lands in the low byte (lower address).
template <int FMT> __device__ __forceinline__ uint16_t cvt2_fp8(float lo, float hi) {
    uint16_t r;
    if constexpr (FMT == PT_E4M3)
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    else
        asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
template <int FMT> __device__ __forceinline__ uint32_t cvt4_fp8(float a, float b, float c, float d) {
    return (uint32_t) cvt2_fp8<FMT>(a, b) | ((uint32_t) cvt2_fp8<FMT>(c, d) << 16);
}
template <int FMT> __device__ __forceinline__ uint8_t cvt1_fp8(float a) {
    return (uint8_t) (cvt2_fp8<FMT>(a, 0.f) & 0xFF);
}
// Two floats to one byte of e2m1 codes; `lo` in the low nibble.
__device__ __forceinline__ uint8_t cvt2_e2m1(float lo, float hi) {
    uint16_t r;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(r) : "f"(hi), "f"(lo));
    return (uint8_t) r;
}

template <int FMT> struct FmtMax;
template <> struct FmtMax<PT_E4M3> { static constexpr float value = 448.f; };
template <> struct FmtMax<PT_E5M2> { static constexpr float value = 57344.f; };

// fmin(x * scale, qmax), to be fed to a saturating convert.  The reference clamps the product to +-qmax
// (fmax(fmin(x * scale, qmax), -qmax)); cvt.rn.satfinite clamps every non-NaN product itself, so only the half of the
// clamp that decides what a NaN becomes is kept: fmin(NaN, qmax) = qmax, as in the reference.
template <int FMT> __device__ __forceinline__ float mul_sat(float x, float scale) { return fminf(x * scale, FmtMax<FMT>::value); }
// scale = qmax / fmax(amax, eps), a true (correctly rounded) division
template <int FMT> __device__ __forceinline__ float scale_from_amax(float amax, float eps) {
    return __fdiv_rn(FmtMax<FMT>::value, fmaxf(amax, eps));
}

__device__ __forceinline__ float warp_max(float v) {
    return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v)));  // v >= 0
}

// ---------------------------------------------------------------- dispatch helpers (host)
#define PT_SWITCH_SRC(dtype, T, ...)                                                               \
    switch (dtype) {                                                                               \
    case PT_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;                                 \
    case PT_F16: { using T = __half; __VA_ARGS__; } break;                                         \
    case PT_F32: { using T = float; __VA_ARGS__; } break;                                          \
    default: return ::ptb::set_error(PT_ERR_INVALID, "unsupported source dtype %d", (int) dtype);  \
    }

#define PT_SWITCH_FP8(fmt, F, ...)                                                                 \
    switch (fmt) {                                                                                 \
    case PT_E4M3: { constexpr int F = PT_E4M3; __VA_ARGS__; } break;                               \
    case PT_E5M2: { constexpr int F = PT_E5M2; __VA_ARGS__; } break;                               \
    default: return ::ptb::set_error(PT_ERR_INVALID, "unsupported fp8 format %d", (int) fmt);      \
    }

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
template <typename T> constexpr size_t vec8_align() { return sizeof(T) == 4 ? 16 : 16; }

}  // namespace ptb
