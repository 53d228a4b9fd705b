// Pieces shared by the tcgen05 GEMM kernels: tile geometry, the group-aware tile walk, output packing
// and the host-side construction of TMA tensor maps.
#pragma once
#include <mutex>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ptb {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 128;  // bytes == fp8 elements per stage row
constexpr int UMMA_K = 32;    // fp8 elements per tcgen05.mma
constexpr int kMaxGroups = 1024;

// Tile walk shared by every role: tiles are numbered group by group.  Inside a group the order is the usual
// L2-friendly raster: bands of kRasterM row blocks, rows fastest inside a band, so that the ~148 tiles in flight
// cover a roughly square patch of C and re-read only ~2 * sqrt(148) operand panels from L2 / HBM.  When the whole
// A operand fits in L2 next to the streaming B panels, one band over all rows measured faster (B200: 2973 vs
// 2856 TFLOP/s at 8192 x 14336 x 4096), while an A operand larger than L2 needs the bands (2056 -> 2472 at
// 16384 x 28672 x 8192); raster_rows() picks between the two.
struct TileWalk {
    const int *tile_start;  // shared memory [G+1]
    int G, num_n_blocks;
    int g;
    int kRasterM;
    int cached_g = -1, cached_m_blocks = 0;  // row blocks of group `cached_g` (saves a division per tile)
    __device__ __forceinline__ bool locate(int t, int &g_out, int &m_blk, int &n_blk) {
        if (t >= tile_start[G]) return false;
        while (t >= tile_start[g + 1]) ++g;
        const int local = t - tile_start[g];
        if (g != cached_g) {
            cached_g = g;
            cached_m_blocks = (tile_start[g + 1] - tile_start[g]) / num_n_blocks;
        }
        const int m_blocks = cached_m_blocks;
        g_out = g;
        if (kRasterM >= m_blocks) {  // one band over all row blocks of the group
            n_blk = local / m_blocks;
            m_blk = local - n_blk * m_blocks;
            return true;
        }
        const int per_band = kRasterM * num_n_blocks;
        const int band = local / per_band;
        const int first_m = band * kRasterM;
        const int band_rows = min(kRasterM, m_blocks - first_m);
        const int in_band = local - band * per_band;
        n_blk = in_band / band_rows;
        m_blk = first_m + in_band - n_blk * band_rows;
        return true;
    }
};

template <typename OutT> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

inline int raster_rows(int64_t a_rows, int64_t k_bytes) {
    if (const char *e = getenv("PT_GEMM_RASTER_M")) {   // row blocks (of 128 rows) per band, for experiments
        const int v = atoi(e);
        if (v > 0) return v;
    }
    return a_rows * k_bytes <= (int64_t) 48 * 1024 * 1024 ? (1 << 20) : 16;
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    // The driver call needs a context bound to the calling thread.  A thread that has made no runtime call yet
    // (autograd's backward threads reach the quantizers this way) has none: cudaFree(nullptr) binds the device's
    // primary context; once per thread.
    thread_local bool bound = false;
    if (!bound) {
        cudaFree(nullptr);
        bound = true;
    }
    return fn;
}

// 2-D byte tensor [rows, row_bytes] (pitch `pitch_bytes`), box = 128 bytes x box_rows, 128-byte swizzle.
inline int make_tmap_bytes(CUtensorMap *m, const void *base, int64_t rows, int64_t row_bytes, int64_t pitch_bytes, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return set_error(PT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    PT_REQUIRE(aligned(base, 16) && pitch_bytes % 16 == 0, "GEMM operand base / row pitch must be 16-byte aligned");
    cuuint64_t dims[2] = {(cuuint64_t) row_bytes, (cuuint64_t) rows};
    cuuint64_t strides[1] = {(cuuint64_t) pitch_bytes};
    cuuint32_t box[2] = {128u, (cuuint32_t) box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(PT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int) r);
    return PT_OK;
}


// 2-D byte tensor of 128-byte lines without swizzle, box = 128 bytes x box_lines (bulk fetch of small contiguous blocks)
inline int make_tmap_lines(CUtensorMap *m, const void *base, int64_t lines, int box_lines) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return set_error(PT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    PT_REQUIRE(aligned(base, 128), "line tensor map: base must be 128-byte aligned");
    cuuint64_t dims[2] = {128u, (cuuint64_t) lines};
    cuuint64_t strides[1] = {128u};
    cuuint32_t box[2] = {128u, (cuuint32_t) box_lines};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(PT_ERR_CUDA, "cuTensorMapEncodeTiled (lines) failed with code %d", (int) r);
    return PT_OK;
}

// 3-D tensor map over a [G, M, N] array of 16-bit elements, box = 64 columns (128 bytes) x box_rows x 1,
// 128-byte swizzle; out-of-range rows / columns read as zero.
inline int make_tmap_u16_3d(CUtensorMap *m, const void *base, int64_t G, int64_t M, int64_t N, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return set_error(PT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    PT_REQUIRE(aligned(base, 16) && (N * 2) % 16 == 0, "tensor map: base / row pitch must be 16-byte aligned");
    cuuint64_t dims[3] = {(cuuint64_t) N, (cuuint64_t) M, (cuuint64_t) G};
    cuuint64_t strides[2] = {(cuuint64_t) N * 2, (cuuint64_t) M * N * 2};
    cuuint32_t box[3] = {64u, (cuuint32_t) box_rows, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(PT_ERR_CUDA, "cuTensorMapEncodeTiled (16-bit 3-D) failed with code %d", (int) r);
    return PT_OK;
}

}  // namespace ptb
