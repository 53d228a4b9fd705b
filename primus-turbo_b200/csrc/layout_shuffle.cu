// Pre-shuffled MX layouts: byte permutations of a ue8m0 scale matrix and of MXFP4 / MXFP8 codes into the tile orders the
// reference hands to its pre-shuffled GEMM back ends.  Definitions (reference: csrc/include/primus_turbo/device/shuffle.cuh
// :39-80, host side csrc/pytorch/shuffle/shuffle.cpp:16-92):
//
//   scale [M, N] -> [ceil(M, 256), ceil(N, 8)], zero padded: element (row, col) goes to
//       ((row / 32) * (N_pad / 8) + col / 8) * 256 + (col % 4) * 64 + (row % 16) * 4 + ((col % 8) / 4) * 2 + (row % 32) / 16
//   codes [M, Nb bytes], M % 16 == 0, Nb % 32 == 0 -> same shape: byte (row, col) goes to
//       (row / 16) * (Nb * 16) + (col / 32) * 512 + ((col % 32) / 16) * 256 + (row % 16) * 16 + col % 16
//
// Both kernels are written from the output side: a thread owns 4 (scale) or 16 (codes) consecutive output bytes, so stores
// are coalesced and every output byte, padding included, is written exactly once.
#include <algorithm>

#include "common.cuh"

namespace ptb {

// One thread per output word of four bytes: (i4, i1) = (0,0), (0,1), (1,0), (1,1) at fixed (tile, i5, i2).
__global__ void __launch_bounds__(256) shuffle_scale_kernel(const uint8_t *__restrict__ src, int64_t M, int64_t N, int64_t n_pad,
                                                            int64_t words, uint32_t *__restrict__ dst) {
    const int64_t tiles_n = n_pad >> 3;
    for (int64_t w = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; w < words; w += (int64_t) gridDim.x * blockDim.x) {
        const int64_t tile = w >> 6;
        const int in_tile = (int) (w & 63), i5 = in_tile >> 4, i2 = in_tile & 15;
        const int64_t row0 = (tile / tiles_n) * 32 + i2, col0 = (tile % tiles_n) * 8 + i5;
        uint32_t word = 0u;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int64_t row = row0 + 16 * (b & 1), col = col0 + 4 * (b >> 1);
            if (row < M && col < N) word |= (uint32_t) src[row * N + col] << (8 * b);
        }
        dst[w] = word;
    }
}

// One thread per 16 output bytes: a (16-row, 32-byte) tile becomes two 16 x 16-byte halves, first half then second.
__global__ void __launch_bounds__(256) shuffle_codes_kernel(const uint4 *__restrict__ src, int64_t row_chunks, int64_t chunks,
                                                            uint4 *__restrict__ dst) {
    for (int64_t c = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (int64_t) gridDim.x * blockDim.x) {
        // output chunk c = ((nb * k_blocks + kb) * 2 + sub) * 16 + r   (k_blocks = row_chunks / 2)
        const int r = (int) (c & 15), sub = (int) ((c >> 4) & 1);
        const int64_t tile = c >> 5, k_blocks = row_chunks >> 1;
        const int64_t nb = tile / k_blocks, kb = tile % k_blocks;
        dst[c] = src[(nb * 16 + r) * row_chunks + kb * 2 + sub];
    }
}

}  // namespace ptb

using namespace ptb;

extern "C" {

int pt_shuffle_e8m0_scale(const uint8_t *scale, int64_t M, int64_t N, uint8_t *out, void *stream) {
    PT_REQUIRE(M >= 0 && N >= 0, "shuffle_scale: bad shape");
    const int64_t m_pad = ceil_to(M, 256), n_pad = ceil_to(N, 8);
    const int64_t words = m_pad * n_pad / 4;
    if (words == 0) return PT_OK;
    PT_REQUIRE(out && (scale || M * N == 0) && aligned(out, 4), "shuffle_scale: null or unaligned pointer");
    const int grid = (int) std::min<int64_t>(ceil_div(words, 256), (int64_t) sm_count() * 8);
    shuffle_scale_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>(scale, M, N, n_pad, words, (uint32_t *) out);
    PT_LAUNCH_OK();
    return PT_OK;
}

int pt_shuffle_mx_codes(const void *codes, int64_t M, int64_t row_bytes, void *out, void *stream) {
    PT_REQUIRE(M >= 0 && row_bytes >= 0, "shuffle_weight: bad shape");
    PT_REQUIRE(M % 16 == 0, "shuffle_weight: the row count must be divisible by 16 (got %lld)", (long long) M);
    PT_REQUIRE(row_bytes % 32 == 0, "shuffle_weight: the row length must be divisible by 32 bytes (got %lld)", (long long) row_bytes);
    const int64_t chunks = M * row_bytes / 16;
    if (chunks == 0) return PT_OK;
    PT_REQUIRE(codes && out && aligned(codes, 16) && aligned(out, 16), "shuffle_weight: null or unaligned pointer");
    const int grid = (int) std::min<int64_t>(ceil_div(chunks, 256), (int64_t) sm_count() * 8);
    shuffle_codes_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>((const uint4 *) codes, row_bytes / 16, chunks, (uint4 *) out);
    PT_LAUNCH_OK();
    return PT_OK;
}

}  // extern "C"
