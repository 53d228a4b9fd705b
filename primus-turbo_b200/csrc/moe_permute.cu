// MoE token permutation (mask-map form): expert-major gather of token rows, its inverse with optional probability
// weighting, and the backward of the weighted inverse.
//
// Semantics follow the reference's fused token_permute / token_unpermute
// (primus_turbo/pytorch/ops/moe/permutation.py:26-286, primus_turbo/triton/moe/permutation.py): rows routed to expert 0
// come first, then expert 1, ...; inside an expert tokens keep their order.  row_id_map has the reference's layout
// [T, 2E + 1]: per token the destination rows of its routed experts (ascending expert), at column E the expert ids in the
// same order, in the last column their number.
//
// All kernels are HBM-bound copies / reductions over token rows: one CTA per token row, 16-byte accesses, the row read
// once and written (or summed from) its `n_routed` places.  The map is built by three launches without any wait between
// CTAs: a per-expert column scan (ranks), a scan over the expert counts, and a per-token compaction.
#include "common.cuh"

namespace ptb {

constexpr int kPermThreads = 256;

// ---------------------------------------------------------------------------------------------- row_id_map
// One CTA per expert: ranks[t, e] = number of tokens before t routed to e (or -1), counts[e] = their total.
template <typename MapT>
__global__ void __launch_bounds__(1024) moe_rank_kernel(const MapT *__restrict__ routing_map, int T, int E,
                                                        int *__restrict__ ranks, int64_t *__restrict__ counts) {
    const int e = blockIdx.x;
    __shared__ int s_warp[32];
    __shared__ int s_carry;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 0; base < T; base += blockDim.x) {
        const int t = base + threadIdx.x;
        const int v = (t < T && routing_map[(int64_t) t * E + e] != 0) ? 1 : 0;
        const unsigned ballot = __ballot_sync(0xffffffffu, v);
        const int in_warp = __popc(ballot & ((1u << lane) - 1u));
        if (lane == 0) s_warp[warp] = __popc(ballot);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < (int) (blockDim.x >> 5); ++w) {
            const int c = s_warp[w];
            if (w < warp) before += c;
            total += c;
        }
        const int carry = s_carry;
        if (t < T) ranks[(int64_t) t * E + e] = v ? carry + before + in_warp : -1;
        __syncthreads();
        if (threadIdx.x == 0) s_carry = carry + total;
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[e] = s_carry;
}

// One CTA: offs[e] = sum of counts[0 .. e)
__global__ void __launch_bounds__(1024) moe_offs_kernel(const int64_t *__restrict__ counts, int E, int *__restrict__ offs) {
    __shared__ int s[1024];
    int carry = 0;
    for (int base = 0; base < E; base += 1024) {
        const int i = base + threadIdx.x;
        const int v = i < E ? (int) counts[i] : 0;
        s[threadIdx.x] = v;
        __syncthreads();
        for (int d = 1; d < 1024; d <<= 1) {
            const int t = threadIdx.x >= d ? s[threadIdx.x - d] : 0;
            __syncthreads();
            s[threadIdx.x] += t;
            __syncthreads();
        }
        if (i < E) offs[i] = carry + s[threadIdx.x] - v;
        carry += s[1023];
        __syncthreads();
    }
}

// One warp per token: compacts its routed experts (ascending) into the reference's row layout.
__global__ void __launch_bounds__(256) moe_compact_kernel(const int *__restrict__ ranks, const int *__restrict__ offs, int T, int E,
                                                          int *__restrict__ row_id_map) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const int lane = threadIdx.x & 31;
    int *row = row_id_map + (int64_t) t * (2 * E + 1);
    int n = 0;
    for (int base = 0; base < E; base += 32) {
        const int e = base + lane;
        const int r = e < E ? ranks[(int64_t) t * E + e] : -1;
        const unsigned ballot = __ballot_sync(0xffffffffu, r >= 0);
        if (r >= 0) {
            const int pos = n + __popc(ballot & ((1u << lane) - 1u));
            row[pos] = offs[e] + r;
            row[E + pos] = e;
        }
        n += __popc(ballot);
    }
    // unused slots: -1 (the reference leaves them unspecified; a fixed value keeps the map comparable)
    for (int i = n + lane; i < E; i += 32) { row[i] = -1; row[E + i] = -1; }
    if (lane == 0) row[2 * E] = n;
}

// ---- the same map built from row-major passes (E <= 1024): thread = expert, so every access to the [T, E] routing map and
// every intermediate is contiguous across a warp.
//   1. per block of 32 tokens, the number of tokens routed to each expert;
//   2. per expert, the exclusive scan of those counts over the blocks (and the expert's total);
//   3. per block again: ranks of its 32 tokens (expert offset + block offset + running count) into shared memory, then one
//      warp per token compacts its routed experts into the row layout.
constexpr int kMapTokens = 32;

template <typename MapT>
__global__ void __launch_bounds__(1024) moe_block_count_kernel(const MapT *__restrict__ routing_map, int T, int E, int *__restrict__ block_counts) {
    const int e = threadIdx.x;
    if (e >= E) return;
    const int t0 = blockIdx.x * kMapTokens;
    int c = 0;
#pragma unroll 8
    for (int i = 0; i < kMapTokens; ++i)
        if (t0 + i < T) c += routing_map[(int64_t) (t0 + i) * E + e] != 0;
    block_counts[(int64_t) blockIdx.x * E + e] = c;
}

// grid: groups of 32 experts; block: (32 experts, 32 segments of consecutive blocks)
__global__ void __launch_bounds__(1024) moe_block_scan_kernel(int *__restrict__ block_counts, int nblocks, int E, int64_t *__restrict__ counts) {
    __shared__ int s_seg[32][33];
    const int e = blockIdx.x * 32 + threadIdx.x, seg = threadIdx.y;
    const int per = (nblocks + 31) / 32, b0 = seg * per, b1 = min(nblocks, b0 + per);
    int sum = 0;
    if (e < E)
        for (int b = b0; b < b1; ++b) sum += block_counts[(int64_t) b * E + e];
    s_seg[seg][threadIdx.x] = sum;
    __syncthreads();
    int before = 0, total = 0;
    for (int k = 0; k < 32; ++k) {
        const int v = s_seg[k][threadIdx.x];
        if (k < seg) before += v;
        total += v;
    }
    if (e < E) {
        int run = before;
        for (int b = b0; b < b1; ++b) {
            const int v = block_counts[(int64_t) b * E + e];
            block_counts[(int64_t) b * E + e] = run;   // exclusive prefix over the blocks, in place
            run += v;
        }
        if (seg == 0) counts[e] = total;
    }
}

template <typename MapT>
__global__ void __launch_bounds__(1024) moe_block_map_kernel(const MapT *__restrict__ routing_map, int T, int E, const int *__restrict__ block_offs,
                                                             const int64_t *__restrict__ counts, int *__restrict__ row_id_map) {
    extern __shared__ int s_rank[];   // [kMapTokens][E]
    __shared__ int s_warp[32];
    const int e = threadIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    // first destination row of every expert: exclusive scan of the totals over the experts
    const int cnt = e < E ? (int) counts[e] : 0;
    int incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; ++w) base += s_warp[w];
    const int t0 = blockIdx.x * kMapTokens;
    if (e < E) {
        int run = base + incl - cnt + block_offs[(int64_t) blockIdx.x * E + e];
#pragma unroll 8
        for (int i = 0; i < kMapTokens; ++i) {
            const bool v = t0 + i < T && routing_map[(int64_t) (t0 + i) * E + e] != 0;
            s_rank[i * E + e] = v ? run : -1;
            run += v;
        }
    }
    __syncthreads();
    for (int i = warp; i < kMapTokens && t0 + i < T; i += nwarps) {
        int *row = row_id_map + (int64_t) (t0 + i) * (2 * E + 1);
        int n = 0;
        for (int eb = 0; eb < E; eb += 32) {
            const int ee = eb + lane;
            const int r = ee < E ? s_rank[i * E + ee] : -1;
            const unsigned ballot = __ballot_sync(0xffffffffu, r >= 0);
            if (r >= 0) {
                const int pos = n + __popc(ballot & ((1u << lane) - 1u));
                row[pos] = r;
                row[E + pos] = ee;
            }
            n += __popc(ballot);
        }
        for (int k = n + lane; k < E; k += 32) { row[k] = -1; row[E + k] = -1; }   // unused slots, as moe_compact_kernel
        if (lane == 0) row[2 * E] = n;
    }
}

// ---------------------------------------------------------------------------------------------- permute
// One CTA per token: the row is read once (16-byte vectors) and written to each of its destinations.
__global__ void __launch_bounds__(kPermThreads) moe_permute_kernel(const uint4 *__restrict__ tokens, int64_t row_vecs, int T, int E,
                                                                   const int *__restrict__ row_id_map, const uint8_t *__restrict__ probs,
                                                                   int probs_bytes, int64_t num_out, uint4 *__restrict__ out,
                                                                   uint8_t *__restrict__ out_probs) {
    const int t = blockIdx.x;
    const int *row = row_id_map + (int64_t) t * (2 * E + 1);
    const int n = row[2 * E];
    if (probs != nullptr && threadIdx.x < n) {
        const int dst = row[threadIdx.x], e = row[E + threadIdx.x];
        if (dst >= 0 && dst < num_out)
            for (int b = 0; b < probs_bytes; ++b) out_probs[(int64_t) dst * probs_bytes + b] = probs[((int64_t) t * E + e) * probs_bytes + b];
    }
    for (int64_t v = threadIdx.x; v < row_vecs; v += kPermThreads) {
        const uint4 x = __ldg(tokens + (int64_t) t * row_vecs + v);
        for (int k = 0; k < n; ++k) {
            const int dst = row[k];
            if (dst >= 0 && dst < num_out) out[(int64_t) dst * row_vecs + v] = x;
        }
    }
}

// ---------------------------------------------------------------------------------------------- unpermute
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// out[t] = sum over the routed experts of (prob[t, e] *) in[dst], fp32 accumulation in expert order.
// PT: dtype of merging_probs.  Also (optional) scatters permuted_probs back to [T, E] (zeros elsewhere).
template <typename T, typename PT>
__global__ void __launch_bounds__(kPermThreads) moe_unpermute_kernel(const T *__restrict__ in, int64_t H, int Tn, int E,
                                                                     const int *__restrict__ row_id_map, const PT *__restrict__ merging_probs,
                                                                     const PT *__restrict__ permuted_probs, T *__restrict__ out,
                                                                     PT *__restrict__ unpermuted_probs) {
    const int t = blockIdx.x;
    const int *row = row_id_map + (int64_t) t * (2 * E + 1);
    const int n = row[2 * E];
    if (unpermuted_probs != nullptr) {
        for (int e = threadIdx.x; e < E; e += kPermThreads) unpermuted_probs[(int64_t) t * E + e] = from_f<PT>(0.f);
        __syncthreads();
        if (threadIdx.x < n && row[threadIdx.x] >= 0)
            unpermuted_probs[(int64_t) t * E + row[E + threadIdx.x]] = permuted_probs[row[threadIdx.x]];
    }
    if (out == nullptr) return;
    constexpr int V = 16 / sizeof(T);
    for (int64_t h = (int64_t) threadIdx.x * V; h < H; h += (int64_t) kPermThreads * V) {
        float acc[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = 0.f;
        for (int k = 0; k < n; ++k) {
            const int src = row[k];
            if (src < 0) continue;
            const float p = merging_probs ? to_f<PT>(merging_probs[(int64_t) t * E + row[E + k]]) : 1.f;
            const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(in + (int64_t) src * H + h));
            const T *x = reinterpret_cast<const T *>(&raw);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] += to_f<T>(x[i]) * p;
        }
        uint4 o;
        T *y = reinterpret_cast<T *>(&o);
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = from_f<T>(acc[i]);
        *reinterpret_cast<uint4 *>(out + (int64_t) t * H + h) = o;
    }
}

// Backward of the weighted unpermute: act_grad[dst] = grad_out[t] * prob[t, e]; probs_grad[t, e] = <grad_out[t], fwd_in[dst]>.
template <typename T, typename PT>
__global__ void __launch_bounds__(kPermThreads) moe_unpermute_bwd_kernel(const T *__restrict__ grad_out, const T *__restrict__ fwd_in, int64_t H,
                                                                         int Tn, int E, const int *__restrict__ row_id_map,
                                                                         const PT *__restrict__ merging_probs, T *__restrict__ act_grad,
                                                                         PT *__restrict__ probs_grad) {
    const int t = blockIdx.x;
    const int *row = row_id_map + (int64_t) t * (2 * E + 1);
    const int n = row[2 * E];
    __shared__ float s_red[kPermThreads / 32];
    for (int e = threadIdx.x; e < E; e += kPermThreads) probs_grad[(int64_t) t * E + e] = from_f<PT>(0.f);
    __syncthreads();
    constexpr int V = 16 / sizeof(T);
    for (int k = 0; k < n; ++k) {
        const int dst = row[k], e = row[E + k];
        if (dst < 0) continue;
        const float p = to_f<PT>(merging_probs[(int64_t) t * E + e]);
        float dot = 0.f;
        for (int64_t h = (int64_t) threadIdx.x * V; h < H; h += (int64_t) kPermThreads * V) {
            const uint4 g_raw = __ldg(reinterpret_cast<const uint4 *>(grad_out + (int64_t) t * H + h));
            const uint4 x_raw = __ldg(reinterpret_cast<const uint4 *>(fwd_in + (int64_t) dst * H + h));
            const T *g = reinterpret_cast<const T *>(&g_raw), *x = reinterpret_cast<const T *>(&x_raw);
            uint4 o;
            T *y = reinterpret_cast<T *>(&o);
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const float gf = to_f<T>(g[i]);
                y[i] = from_f<T>(gf * p);
                dot += gf * to_f<T>(x[i]);
            }
            *reinterpret_cast<uint4 *>(act_grad + (int64_t) dst * H + h) = o;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = dot;
        __syncthreads();
        if (threadIdx.x == 0) {
            float s = 0.f;
            for (int w = 0; w < kPermThreads / 32; ++w) s += s_red[w];
            probs_grad[(int64_t) t * E + e] = from_f<PT>(s);
        }
        __syncthreads();
    }
}

}  // namespace ptb

using namespace ptb;

extern "C" {

size_t pt_moe_row_id_map_workspace_bytes(int64_t T, int E) { return (size_t) ((int64_t) T * E + E) * sizeof(int); }

int pt_moe_make_row_id_map(const void *routing_map, int map_elem_bytes, int64_t T, int E, int *row_id_map, int64_t *tokens_per_expert,
                           void *workspace, size_t workspace_bytes, void *stream) {
    PT_REQUIRE(T >= 0 && E >= 1 && T < (1ll << 31), "moe row_id_map: bad shape");
    PT_REQUIRE(map_elem_bytes == 1 || map_elem_bytes == 4 || map_elem_bytes == 8, "moe row_id_map: routing_map must be bool / int32 / int64");
    PT_REQUIRE(tokens_per_expert && (T == 0 || (routing_map && row_id_map)), "moe row_id_map: null pointer");
    PT_REQUIRE(workspace && workspace_bytes >= pt_moe_row_id_map_workspace_bytes(T, E), "moe row_id_map: workspace too small");
    cudaStream_t st = (cudaStream_t) stream;
    if (E <= 1024 && T > 0) {   // row-major passes, thread = expert
        int *block_counts = (int *) workspace;   // [ceil(T / 32), E] <= T * E ints
        const int nblocks = (int) ceil_div(T, kMapTokens), threads = (int) ceil_to(E, 32);
        const int smem = kMapTokens * E * (int) sizeof(int);
#define PT_MOE_MAP(MapT_)                                                                                                             \
        do {                                                                                                                          \
            moe_block_count_kernel<MapT_><<<nblocks, threads, 0, st>>>((const MapT_ *) routing_map, (int) T, E, block_counts);            \
            PT_LAUNCH_OK();                                                                                                           \
            moe_block_scan_kernel<<<(unsigned) ceil_div(E, 32), dim3(32, 32), 0, st>>>(block_counts, nblocks, E, tokens_per_expert);     \
            PT_LAUNCH_OK();                                                                                                           \
            auto kern = moe_block_map_kernel<MapT_>;                                                                                  \
            if (smem > 48 * 1024) PT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));            \
            kern<<<nblocks, threads, smem, st>>>((const MapT_ *) routing_map, (int) T, E, block_counts, tokens_per_expert, row_id_map);  \
            PT_LAUNCH_OK();                                                                                                           \
        } while (0)
        if (map_elem_bytes == 1) PT_MOE_MAP(uint8_t);
        else if (map_elem_bytes == 4) PT_MOE_MAP(int);
        else PT_MOE_MAP(int64_t);
#undef PT_MOE_MAP
        return PT_OK;
    }
    int *ranks = (int *) workspace, *offs = ranks + (int64_t) T * E;
    if (map_elem_bytes == 1) moe_rank_kernel<uint8_t><<<E, 1024, 0, st>>>((const uint8_t *) routing_map, (int) T, E, ranks, tokens_per_expert);
    else if (map_elem_bytes == 4) moe_rank_kernel<int><<<E, 1024, 0, st>>>((const int *) routing_map, (int) T, E, ranks, tokens_per_expert);
    else moe_rank_kernel<int64_t><<<E, 1024, 0, st>>>((const int64_t *) routing_map, (int) T, E, ranks, tokens_per_expert);
    PT_LAUNCH_OK();
    if (T == 0) return PT_OK;
    moe_offs_kernel<<<1, 1024, 0, st>>>(tokens_per_expert, E, offs);
    PT_LAUNCH_OK();
    moe_compact_kernel<<<(unsigned) ceil_div(T, 8), 256, 0, st>>>(ranks, offs, (int) T, E, row_id_map);
    PT_LAUNCH_OK();
    return PT_OK;
}

int pt_moe_permute(const void *tokens, int64_t T, int64_t row_bytes, int E, const int *row_id_map, const void *probs, int probs_elem_bytes,
                   int64_t num_out_tokens, void *out, void *out_probs, void *stream) {
    PT_REQUIRE(T >= 0 && E >= 1 && row_bytes >= 0 && num_out_tokens >= 0, "moe permute: bad shape");
    if (T == 0 || row_bytes == 0) return PT_OK;
    PT_REQUIRE(tokens && row_id_map && out, "moe permute: null pointer");
    PT_REQUIRE(row_bytes % 16 == 0 && aligned(tokens, 16) && aligned(out, 16), "moe permute: rows must be multiples of 16 bytes, 16-byte aligned");
    PT_REQUIRE((probs == nullptr) == (out_probs == nullptr), "moe permute: probs and out_probs go together");
    PT_REQUIRE(E <= kPermThreads || probs == nullptr, "moe permute: at most %d experts with probabilities", kPermThreads);
    moe_permute_kernel<<<(unsigned) T, kPermThreads, 0, (cudaStream_t) stream>>>((const uint4 *) tokens, row_bytes / 16, (int) T, E, row_id_map,
                                                                                  (const uint8_t *) probs, probs_elem_bytes, num_out_tokens,
                                                                                  (uint4 *) out, (uint8_t *) out_probs);
    PT_LAUNCH_OK();
    return PT_OK;
}

#define PT_SWITCH_PROBS(dtype, PT_, ...)                                                                  \
    switch (dtype) {                                                                                      \
    case PT_BF16: { using PT_ = __nv_bfloat16; __VA_ARGS__; } break;                                      \
    case PT_F16: { using PT_ = __half; __VA_ARGS__; } break;                                              \
    case PT_F32: { using PT_ = float; __VA_ARGS__; } break;                                               \
    default: return set_error(PT_ERR_INVALID, "unsupported probability dtype %d", (int) dtype);          \
    }

int pt_moe_unpermute(const void *permuted, int dtype, int64_t T, int64_t H, int E, const int *row_id_map, const void *merging_probs,
                     const void *permuted_probs, int probs_dtype, void *out, void *unpermuted_probs, void *stream) {
    PT_REQUIRE(T >= 0 && H >= 0 && E >= 1, "moe unpermute: bad shape");
    if (T == 0) return PT_OK;
    PT_REQUIRE(row_id_map && (out || unpermuted_probs), "moe unpermute: null pointer");
    PT_REQUIRE(out == nullptr || (permuted && (H * (dtype == PT_F32 ? 4 : 2)) % 16 == 0 && aligned(permuted, 16) && aligned(out, 16)),
               "moe unpermute: rows must be multiples of 16 bytes, 16-byte aligned");
    PT_REQUIRE((permuted_probs == nullptr) == (unpermuted_probs == nullptr), "moe unpermute: permuted_probs and unpermuted_probs go together");
    PT_REQUIRE(E <= kPermThreads || unpermuted_probs == nullptr, "moe unpermute: at most %d experts with probabilities", kPermThreads);
    PT_SWITCH_SRC(dtype, T_, {
        PT_SWITCH_PROBS(probs_dtype, P_, {
            moe_unpermute_kernel<T_, P_><<<(unsigned) T, kPermThreads, 0, (cudaStream_t) stream>>>(
                (const T_ *) permuted, H, (int) T, E, row_id_map, (const P_ *) merging_probs, (const P_ *) permuted_probs, (T_ *) out,
                (P_ *) unpermuted_probs);
        });
    });
    PT_LAUNCH_OK();
    return PT_OK;
}

int pt_moe_unpermute_bwd_with_probs(const void *grad_out, const void *fwd_in, int dtype, int64_t T, int64_t H, int E, const int *row_id_map,
                                    const void *merging_probs, int probs_dtype, void *act_grad, void *probs_grad, void *stream) {
    PT_REQUIRE(T >= 0 && H >= 0 && E >= 1, "moe unpermute backward: bad shape");
    if (T == 0) return PT_OK;
    PT_REQUIRE(grad_out && fwd_in && row_id_map && merging_probs && act_grad && probs_grad, "moe unpermute backward: null pointer");
    PT_REQUIRE((H * (dtype == PT_F32 ? 4 : 2)) % 16 == 0 && aligned(grad_out, 16) && aligned(fwd_in, 16) && aligned(act_grad, 16),
               "moe unpermute backward: rows must be multiples of 16 bytes, 16-byte aligned");
    PT_SWITCH_SRC(dtype, T_, {
        PT_SWITCH_PROBS(probs_dtype, P_, {
            moe_unpermute_bwd_kernel<T_, P_><<<(unsigned) T, kPermThreads, 0, (cudaStream_t) stream>>>(
                (const T_ *) grad_out, (const T_ *) fwd_in, H, (int) T, E, row_id_map, (const P_ *) merging_probs, (T_ *) act_grad,
                (P_ *) probs_grad);
        });
    });
    PT_LAUNCH_OK();
    return PT_OK;
}

}  // extern "C"
