// Gated activations with routing probabilities (SwiGLU / GeGLU, forward and backward) and RMSNorm (forward with optional
// residual add, row statistics alone, backward): the element-wise steps on either side of the low-precision GEMMs.
//
// HBM-bound streaming kernels: persistent CTAs walk the rows (grid = min(rows, CTAs that fit)), 16-byte loads and stores,
// fp32 arithmetic (act_math.cuh), one block reduction per row where the operator needs one (the probability gradient,
// the mean square).  The reference's forms: primus_turbo/pytorch/ops/activation.py:23-80 with
// triton/activation/{swiglu,geglu}_kernel.py, and ops/normalization.py with triton/normalization/rmsnorm_kernel.py.
#include <algorithm>
#include <cstdlib>

#include "act_math.cuh"
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ptb {

constexpr int kAnThreads = 256;

template <typename T> __device__ __forceinline__ float an_to_f(T v);
template <> __device__ __forceinline__ float an_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float an_to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float an_to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T an_from_f(float v);
template <> __device__ __forceinline__ float an_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 an_from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half an_from_f<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float block_sum(float v, float *s_red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();   // s_red may still be read from the previous use
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kAnThreads / 32; ++w) t += s_red[w];
    return t;
}

// ---------------------------------------------------------------------------------------------- gated activation
// x [rows, 2H]: a = x[:, :H], b = x[:, H:]; out [rows, H] = act(a) * b * probs[row]; rows whose mask entry is 0 come out as zeros.
template <typename T, int ACT>
__global__ void __launch_bounds__(kAnThreads) glu_fwd_kernel(const T *__restrict__ x, const float *__restrict__ probs,
                                                             const int64_t *__restrict__ row_mask, int64_t rows, int64_t H,
                                                             T *__restrict__ out) {
    constexpr int V = 16 / sizeof(T);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        if (row_mask != nullptr && row_mask[r] == 0) {   // the reference leaves these rows unwritten; zeros keep the result deterministic
            for (int64_t h = (int64_t) threadIdx.x * V; h < H; h += (int64_t) kAnThreads * V) *reinterpret_cast<uint4 *>(out + r * H + h) = make_uint4(0, 0, 0, 0);
            continue;
        }
        const float p = probs[r];
        const T *a = x + r * 2 * H, *b = a + H;
        for (int64_t h = (int64_t) threadIdx.x * V; h < H; h += (int64_t) kAnThreads * V) {
            const uint4 ar = __ldg(reinterpret_cast<const uint4 *>(a + h)), br = __ldg(reinterpret_cast<const uint4 *>(b + h));
            const T *av = reinterpret_cast<const T *>(&ar), *bv = reinterpret_cast<const T *>(&br);
            uint4 o;
            T *ov = reinterpret_cast<T *>(&o);
#pragma unroll
            for (int i = 0; i < V; ++i) ov[i] = an_from_f<T>(glu_value<ACT>(an_to_f<T>(av[i]), an_to_f<T>(bv[i]), p));
            *reinterpret_cast<uint4 *>(out + r * H + h) = o;
        }
    }
}

// grad_x[:, :H] = g * p * b * act'(a); grad_x[:, H:] = g * p * act(a); grad_probs[row] = sum_h g * act(a) * b
template <typename T, int ACT>
__global__ void __launch_bounds__(kAnThreads) glu_bwd_kernel(const T *__restrict__ grad_out, const T *__restrict__ x,
                                                             const float *__restrict__ probs, const int64_t *__restrict__ row_mask,
                                                             int64_t rows, int64_t H, T *__restrict__ grad_x, float *__restrict__ grad_probs) {
    constexpr int V = 16 / sizeof(T);
    __shared__ float s_red[kAnThreads / 32];
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        if (row_mask != nullptr && row_mask[r] == 0) {
            for (int64_t h = (int64_t) threadIdx.x * V; h < 2 * H; h += (int64_t) kAnThreads * V)
                *reinterpret_cast<uint4 *>(grad_x + r * 2 * H + h) = make_uint4(0, 0, 0, 0);
            if (threadIdx.x == 0) grad_probs[r] = 0.f;
            continue;
        }
        const float p = probs[r];
        const T *a = x + r * 2 * H, *b = a + H, *g = grad_out + r * H;
        float dot = 0.f;
        for (int64_t h = (int64_t) threadIdx.x * V; h < H; h += (int64_t) kAnThreads * V) {
            const uint4 ar = __ldg(reinterpret_cast<const uint4 *>(a + h)), br = __ldg(reinterpret_cast<const uint4 *>(b + h));
            const uint4 gr = __ldg(reinterpret_cast<const uint4 *>(g + h));
            const T *av = reinterpret_cast<const T *>(&ar), *bv = reinterpret_cast<const T *>(&br), *gv = reinterpret_cast<const T *>(&gr);
            uint4 oa, ob;
            T *oav = reinterpret_cast<T *>(&oa), *obv = reinterpret_cast<T *>(&ob);
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const float af = an_to_f<T>(av[i]), bf = an_to_f<T>(bv[i]), gf = an_to_f<T>(gv[i]);
                const float act = act_value<ACT>(af);
                dot += gf * act * bf;
                const float gp = gf * p;
                oav[i] = an_from_f<T>(gp * (bf * act_grad<ACT>(af)));
                obv[i] = an_from_f<T>(gp * act);
            }
            *reinterpret_cast<uint4 *>(grad_x + r * 2 * H + h) = oa;
            *reinterpret_cast<uint4 *>(grad_x + r * 2 * H + H + h) = ob;
        }
        const float total = block_sum(dot, s_red);
        if (threadIdx.x == 0) grad_probs[r] = total;
    }
}

// V elements of T moved as one access (V * sizeof(T) = 16 bytes on the aligned path, V = 1 for ragged or unaligned rows)
template <typename T, int V> struct alignas(sizeof(T) * V) Vec { T e[V]; };
template <typename T, int V> __device__ __forceinline__ Vec<T, V> ldv(const T *p) {
    if constexpr (V * sizeof(T) == 16) {
        const uint4 r = __ldg(reinterpret_cast<const uint4 *>(p));
        return *reinterpret_cast<const Vec<T, V> *>(&r);
    } else {
        return *reinterpret_cast<const Vec<T, V> *>(p);
    }
}
template <typename T, int V> __device__ __forceinline__ Vec<T, V> ldv_plain(const T *p) { return *reinterpret_cast<const Vec<T, V> *>(p); }
template <typename T, int V> __device__ __forceinline__ void stv(T *p, const Vec<T, V> &v) { *reinterpret_cast<Vec<T, V> *>(p) = v; }

// ---------------------------------------------------------------------------------------------- RMSNorm
// y = (x [+ residual]) * rstd * g; rstd [rows] always written; x_plus_r written when a residual is given; y may be null
// (statistics only).  The row is read once when it fits the registers (H <= 4 vectors x 256 threads), twice else.
template <typename T, int V, bool RESIDUAL>
__global__ void __launch_bounds__(kAnThreads) rmsnorm_fwd_kernel(const T *__restrict__ x, const T *__restrict__ residual,
                                                                 const T *__restrict__ gamma, float eps, int zero_centered, int64_t rows,
                                                                 int64_t H, T *__restrict__ y, T *__restrict__ x_plus_r,
                                                                 float *__restrict__ rstd_out) {
    constexpr int kKeep = 4;   // 16-byte vectors a thread keeps between the two passes
    __shared__ float s_red[kAnThreads / 32];
    const bool fits = H <= (int64_t) kAnThreads * V * kKeep;
    auto load_sum = [&](int64_t r, int64_t h, float &ss) -> Vec<T, V> {   // x (+ residual) at [r, h .. h + V), its squares added to ss
        Vec<T, V> v = ldv<T, V>(x + r * H + h);
        T *e = v.e;
        if constexpr (RESIDUAL) {
            const Vec<T, V> rr = ldv<T, V>(residual + r * H + h);
            const T *re = rr.e;
#pragma unroll
            for (int i = 0; i < V; ++i) e[i] = an_from_f<T>(an_to_f<T>(e[i]) + an_to_f<T>(re[i]));
            stv<T, V>(x_plus_r + r * H + h, v);
        }
#pragma unroll
        for (int i = 0; i < V; ++i) { const float f = an_to_f<T>(e[i]); ss += f * f; }
        return v;
    };
    auto scale_store = [&](int64_t r, int64_t h, const Vec<T, V> &v, float rstd) {
        const Vec<T, V> gr = ldv<T, V>(gamma + h);
        const T *e = v.e, *ge = gr.e;
        Vec<T, V> o;
        T *oe = o.e;
#pragma unroll
        for (int i = 0; i < V; ++i)
            oe[i] = an_from_f<T>(rmsnorm_value(an_to_f<T>(e[i]), rstd, an_to_f<T>(ge[i]) + (zero_centered ? 1.0f : 0.0f)));
        stv<T, V>(y + r * H + h, o);
    };
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        float ss = 0.f;
        if (fits) {
            Vec<T, V> keep[kKeep];
#pragma unroll
            for (int k = 0; k < kKeep; ++k) {
                const int64_t h = ((int64_t) k * kAnThreads + threadIdx.x) * V;
                if (h < H) keep[k] = load_sum(r, h, ss);
            }
            const float rstd = rsqrtf(block_sum(ss, s_red) / (float) H + eps);
            if (threadIdx.x == 0) rstd_out[r] = rstd;
            if (y == nullptr) continue;
#pragma unroll
            for (int k = 0; k < kKeep; ++k) {
                const int64_t h = ((int64_t) k * kAnThreads + threadIdx.x) * V;
                if (h < H) scale_store(r, h, keep[k], rstd);
            }
        } else {
            for (int64_t h = (int64_t) threadIdx.x * V; h < H; h += (int64_t) kAnThreads * V) load_sum(r, h, ss);
            const float rstd = rsqrtf(block_sum(ss, s_red) / (float) H + eps);
            if (threadIdx.x == 0) rstd_out[r] = rstd;
            if (y == nullptr) continue;
            if (RESIDUAL) __syncthreads();   // x_plus_r written above is read back below (same thread, same addresses)
            for (int64_t h = (int64_t) threadIdx.x * V; h < H; h += (int64_t) kAnThreads * V) {
                const Vec<T, V> v = RESIDUAL ? ldv_plain<T, V>(x_plus_r + r * H + h) : ldv<T, V>(x + r * H + h);
                scale_store(r, h, v, rstd);
            }
        }
    }
}

// Row statistics alone (rstd), one warp per row, no block-wide barrier: the pass a normalising quantizer needs before it
// streams the tensor a second time.  The sum of squares is formed in the order rmsnorm_fwd_kernel forms it (the partial
// sums of its 256 threads, its eight warp reductions, then the eight warp sums in turn: lane l plays threads l, 32 + l,
// ...), so both kernels give the same rstd bit for bit.
template <typename T>
__global__ void __launch_bounds__(kAnThreads) rmsnorm_stats_kernel(const T *__restrict__ x, float eps, int64_t rows, int64_t H,
                                                                   float *__restrict__ rstd_out) {
    constexpr int V = 16 / sizeof(T);
    constexpr int kW = kAnThreads / 32;
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t) gridDim.x * kW;
    for (int64_t r = (int64_t) blockIdx.x * kW + (threadIdx.x >> 5); r < rows; r += warps) {
        const T *row = x + r * H;
        float ss[kW];
#pragma unroll
        for (int w = 0; w < kW; ++w) ss[w] = 0.f;
        for (int64_t h0 = 0; h0 < H; h0 += (int64_t) kAnThreads * V) {
#pragma unroll
            for (int w = 0; w < kW; ++w) {
                const int64_t h = h0 + (int64_t) (w * 32 + lane) * V;
                if (h < H) {
                    const Vec<T, V> v = ldv<T, V>(row + h);
#pragma unroll
                    for (int i = 0; i < V; ++i) { const float f = an_to_f<T>(v.e[i]); ss[w] += f * f; }
                }
            }
        }
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kW; ++w) {
            float v = ss[w];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            total += v;
        }
        if (lane == 0) rstd_out[r] = rsqrtf(total / (float) H + eps);
    }
}

// dx = (dy * g - x_hat * mean(dy * g * x_hat)) * rstd (+ grad of the x + residual sum when given);
// dgamma partial of this CTA: sum over its rows of dy * x_hat, written to dg_partial[blockIdx.x, :] (fp32).
template <typename T, int V>
__global__ void __launch_bounds__(kAnThreads, 2) rmsnorm_bwd_kernel(const T *__restrict__ dy, const T *__restrict__ dxpr, const T *__restrict__ x,
                                                                 const T *__restrict__ gamma, const float *__restrict__ rstd_in,
                                                                 int zero_centered, int64_t rows, int64_t H, T *__restrict__ dx,
                                                                 float *__restrict__ dg_partial) {
    constexpr int kKeep = 4;   // vectors of columns per thread whose dgamma sums stay in registers
    __shared__ float s_red[kAnThreads / 32];
    float *dg = dg_partial + (int64_t) blockIdx.x * H;
    const bool fits = H <= (int64_t) kAnThreads * V * kKeep;
    float dgr[kKeep][V];
#pragma unroll
    for (int k = 0; k < kKeep; ++k)
#pragma unroll
        for (int i = 0; i < V; ++i) dgr[k][i] = 0.f;
    if (!fits)
        for (int64_t h = threadIdx.x; h < H; h += kAnThreads) dg[h] = 0.f;
    __syncthreads();   // the zeros above are written by other threads than those that add to the same columns below
    const float zc = zero_centered ? 1.0f : 0.0f;
    // one row: its dot product sum_h dy * g * x_hat, then dx and the dgamma terms
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float rstd = rstd_in[r];
        float acc = 0.f;
        if (fits) {   // the row (x and dy) stays in registers between the two steps
            Vec<T, V> xk[kKeep], dk[kKeep];
#pragma unroll
            for (int k = 0; k < kKeep; ++k) {
                const int64_t h = ((int64_t) k * kAnThreads + threadIdx.x) * V;
                if (h < H) {
                    xk[k] = ldv<T, V>(x + r * H + h);
                    dk[k] = ldv<T, V>(dy + r * H + h);
                    const Vec<T, V> gr = ldv<T, V>(gamma + h);
#pragma unroll
                    for (int i = 0; i < V; ++i) acc += an_to_f<T>(dk[k].e[i]) * (an_to_f<T>(gr.e[i]) + zc) * (an_to_f<T>(xk[k].e[i]) * rstd);
                }
            }
            const float m = block_sum(acc, s_red) / (float) H;
#pragma unroll
            for (int k = 0; k < kKeep; ++k) {
                const int64_t h = ((int64_t) k * kAnThreads + threadIdx.x) * V;
                if (h < H) {
                    const Vec<T, V> gr = ldv<T, V>(gamma + h);
                    Vec<T, V> pr = {};
                    if (dxpr != nullptr) pr = ldv<T, V>(dxpr + r * H + h);
                    Vec<T, V> o;
#pragma unroll
                    for (int i = 0; i < V; ++i) {
                        const float x_hat = an_to_f<T>(xk[k].e[i]) * rstd, d = an_to_f<T>(dk[k].e[i]);
                        float v = (d * (an_to_f<T>(gr.e[i]) + zc) - x_hat * m) * rstd;
                        if (dxpr != nullptr) v += an_to_f<T>(pr.e[i]);
                        o.e[i] = an_from_f<T>(v);
                        dgr[k][i] += d * x_hat;
                    }
                    stv<T, V>(dx + r * H + h, o);
                }
            }
            continue;
        }
        for (int64_t h = (int64_t) threadIdx.x * V; h < H; h += (int64_t) kAnThreads * V) {
            const Vec<T, V> xr = ldv<T, V>(x + r * H + h), dr = ldv<T, V>(dy + r * H + h), gr = ldv<T, V>(gamma + h);
#pragma unroll
            for (int i = 0; i < V; ++i) acc += an_to_f<T>(dr.e[i]) * (an_to_f<T>(gr.e[i]) + zc) * (an_to_f<T>(xr.e[i]) * rstd);
        }
        const float m = block_sum(acc, s_red) / (float) H;
        for (int64_t h = (int64_t) threadIdx.x * V; h < H; h += (int64_t) kAnThreads * V) {
            const Vec<T, V> xr = ldv<T, V>(x + r * H + h), dr = ldv<T, V>(dy + r * H + h), gr = ldv<T, V>(gamma + h);
            Vec<T, V> pr = {};
            if (dxpr != nullptr) pr = ldv<T, V>(dxpr + r * H + h);
            Vec<T, V> o;
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const float x_hat = an_to_f<T>(xr.e[i]) * rstd, d = an_to_f<T>(dr.e[i]);
                float v = (d * (an_to_f<T>(gr.e[i]) + zc) - x_hat * m) * rstd;
                if (dxpr != nullptr) v += an_to_f<T>(pr.e[i]);
                o.e[i] = an_from_f<T>(v);
                dg[h + i] += d * x_hat;   // column h + i belongs to this thread alone in every row this CTA visits
            }
            stv<T, V>(dx + r * H + h, o);
        }
    }
    if (fits) {
#pragma unroll
        for (int k = 0; k < kKeep; ++k) {
            const int64_t h = ((int64_t) k * kAnThreads + threadIdx.x) * V;
            if (h < H) {
#pragma unroll
                for (int i = 0; i < V; ++i) dg[h + i] = dgr[k][i];
            }
        }
    }
}

// The same with the rows staged through shared memory: while a row is processed, the next one (x and dy) is already on
// its way into the other half of a double buffer (16-byte cp.async; a thread reads back only what it copied itself, so
// the buffers need no barrier).  For rows of up to 4 vectors per thread (8192 16-bit elements).  Element assignment and
// summation order are those of rmsnorm_bwd_kernel: both give the same bits.
template <typename T, int KEEP>
__global__ void __launch_bounds__(kAnThreads, 3) rmsnorm_bwd_staged_kernel(const T *__restrict__ dy, const T *__restrict__ dxpr, const T *__restrict__ x,
                                                                        const T *__restrict__ gamma, const float *__restrict__ rstd_in,
                                                                        int zero_centered, int64_t rows, int64_t H, T *__restrict__ dx,
                                                                        float *__restrict__ dg_partial, int stages) {
    constexpr int V = 16 / sizeof(T);
    constexpr int kKeep = KEEP;   // vectors per thread and row: 2 (rows of up to 512 vectors) or 4
    extern __shared__ __align__(16) uint8_t an_smem[];   // [stages][x row | dy row]
    __shared__ float s_red[kAnThreads / 32];
    const int64_t row_bytes = H * (int64_t) sizeof(T);
    auto sx = [&](int b) { return reinterpret_cast<T *>(an_smem + (int64_t) b * 2 * row_bytes); };
    auto sd = [&](int b) { return reinterpret_cast<T *>(an_smem + (int64_t) b * 2 * row_bytes + row_bytes); };
    auto issue = [&](int64_t r, int b) {
#pragma unroll
        for (int k = 0; k < kKeep; ++k) {
            const int64_t h = ((int64_t) k * kAnThreads + threadIdx.x) * V;
            if (h < H && r < rows) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sm100::smem_u32(sx(b) + h)), "l"(x + r * H + h) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sm100::smem_u32(sd(b) + h)), "l"(dy + r * H + h) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");   // one group per row slot, empty past the last row
    };
    // all but the newest stages - 2 groups have landed (the row about to be used is the oldest one in flight)
    auto wait_oldest = [&]() {
        switch (stages) {
            case 2: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
            case 3: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
            case 4: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
            case 5: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
            case 6: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
            case 7: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
            default: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
        }
    };
    float dgr[kKeep][V];
#pragma unroll
    for (int k = 0; k < kKeep; ++k)
#pragma unroll
        for (int i = 0; i < V; ++i) dgr[k][i] = 0.f;
    const float zc = zero_centered ? 1.0f : 0.0f;
    // Two vectors per thread: the thread's gains (the same for every row) are converted once, and a row's normalised values
    // stay in registers between its dot product and its write-out.  Four vectors per thread would spill: that form reads
    // them from shared memory twice.
    constexpr bool kInRegs = KEEP == 2;
    [[maybe_unused]] float gp[kInRegs ? kKeep : 1][V];
    if constexpr (kInRegs) {
#pragma unroll
        for (int k = 0; k < kKeep; ++k) {
            const int64_t h = ((int64_t) k * kAnThreads + threadIdx.x) * V;
            Vec<T, V> gr = {};
            if (h < H) gr = ldv<T, V>(gamma + h);
#pragma unroll
            for (int i = 0; i < V; ++i) gp[k][i] = an_to_f<T>(gr.e[i]) + zc;
        }
    }
    // Ring of `stages` row slots: stages - 1 rows are on their way while one is processed (a CTA keeps
    // (stages - 1) x 2 rows of bytes in flight; with one row ahead, three CTAs per SM of 4096-element rows asked for 48 KB
    // at a time and the kernel ran at the memory latency, not the bandwidth).
    int b = 0;
    for (int s0 = 0; s0 < stages - 1; ++s0) issue((int64_t) blockIdx.x + (int64_t) s0 * gridDim.x, s0);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x, b = b + 1 == stages ? 0 : b + 1) {
        wait_oldest();
        issue(r + (int64_t) (stages - 1) * gridDim.x, b == 0 ? stages - 1 : b - 1);   // the slot this thread read one row ago
        const float rstd = rstd_in[r];
        float acc = 0.f;
        if constexpr (!kInRegs) {
#pragma unroll
            for (int k = 0; k < kKeep; ++k) {
                const int64_t h = ((int64_t) k * kAnThreads + threadIdx.x) * V;
                if (h < H) {
                    const Vec<T, V> xv = ldv_plain<T, V>(sx(b) + h), dv = ldv_plain<T, V>(sd(b) + h), gr = ldv<T, V>(gamma + h);
#pragma unroll
                    for (int i = 0; i < V; ++i) acc += an_to_f<T>(dv.e[i]) * (an_to_f<T>(gr.e[i]) + zc) * (an_to_f<T>(xv.e[i]) * rstd);
                }
            }
            const float m = block_sum(acc, s_red) / (float) H;
#pragma unroll
            for (int k = 0; k < kKeep; ++k) {
                const int64_t h = ((int64_t) k * kAnThreads + threadIdx.x) * V;
                if (h < H) {
                    const Vec<T, V> xv = ldv_plain<T, V>(sx(b) + h), dv = ldv_plain<T, V>(sd(b) + h), gr = ldv<T, V>(gamma + h);
                    Vec<T, V> pr = {};
                    if (dxpr != nullptr) pr = ldv<T, V>(dxpr + r * H + h);
                    Vec<T, V> o;
#pragma unroll
                    for (int i = 0; i < V; ++i) {
                        const float x_hat = an_to_f<T>(xv.e[i]) * rstd, d = an_to_f<T>(dv.e[i]);
                        float v = (d * (an_to_f<T>(gr.e[i]) + zc) - x_hat * m) * rstd;
                        if (dxpr != nullptr) v += an_to_f<T>(pr.e[i]);
                        o.e[i] = an_from_f<T>(v);
                        dgr[k][i] += d * x_hat;
                    }
                    stv<T, V>(dx + r * H + h, o);
                }
            }
            continue;
        }
        float xh[kInRegs ? kKeep : 1][V];
        Vec<T, V> dvk[kInRegs ? kKeep : 1];
#pragma unroll
        for (int k = 0; k < kKeep; ++k) {
            const int64_t h = ((int64_t) k * kAnThreads + threadIdx.x) * V;
            if (h < H) {
                const Vec<T, V> xv = ldv_plain<T, V>(sx(b) + h);
                dvk[k] = ldv_plain<T, V>(sd(b) + h);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    xh[k][i] = an_to_f<T>(xv.e[i]) * rstd;
                    acc += an_to_f<T>(dvk[k].e[i]) * gp[k][i] * xh[k][i];
                }
            }
        }
        const float m = block_sum(acc, s_red) / (float) H;
#pragma unroll
        for (int k = 0; k < kKeep; ++k) {
            const int64_t h = ((int64_t) k * kAnThreads + threadIdx.x) * V;
            if (h < H) {
                Vec<T, V> pr = {};
                if (dxpr != nullptr) pr = ldv<T, V>(dxpr + r * H + h);
                Vec<T, V> o;
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    const float x_hat = xh[k][i], d = an_to_f<T>(dvk[k].e[i]);
                    float v = (d * gp[k][i] - x_hat * m) * rstd;
                    if (dxpr != nullptr) v += an_to_f<T>(pr.e[i]);
                    o.e[i] = an_from_f<T>(v);
                    dgr[k][i] += d * x_hat;
                }
                stv<T, V>(dx + r * H + h, o);
            }
        }
    }
    float *dg = dg_partial + (int64_t) blockIdx.x * H;
#pragma unroll
    for (int k = 0; k < kKeep; ++k) {
        const int64_t h = ((int64_t) k * kAnThreads + threadIdx.x) * V;
        if (h < H) {
#pragma unroll
            for (int i = 0; i < V; ++i) dg[h + i] = dgr[k][i];
        }
    }
}

// dgamma[h] = sum over parts of dg_partial[part, h]
// A CTA owns 32 columns; its 16 warps take every 16th part (128-byte coalesced reads, four in flight) and their sums meet
// in shared memory in a fixed order.  (One thread per column over all parts left 8-16 CTAs walking 444 dependent rows of
// the partial array: tens of microseconds behind every backward.)
constexpr int kDgLanes = 16;
template <typename T>
__global__ void __launch_bounds__(32 * kDgLanes) rmsnorm_dgamma_kernel(const float *__restrict__ dg_partial, int parts, int64_t H,
                                                                      T *__restrict__ dgamma) {
    __shared__ float s_part[kDgLanes][33];
    const int c = threadIdx.x & 31, pl = threadIdx.x >> 5;
    const int64_t h = (int64_t) blockIdx.x * 32 + c;
    float acc = 0.f;
    if (h < H) {
#pragma unroll 4
        for (int p = pl; p < parts; p += kDgLanes) acc += dg_partial[(int64_t) p * H + h];
    }
    s_part[pl][c] = acc;
    __syncthreads();
    if (pl == 0 && h < H) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < kDgLanes; ++i) t += s_part[i][c];
        dgamma[h] = an_from_f<T>(t);
    }
}

// Grid of a block-per-row kernel: no more CTAs than are resident at once, and the same number of rows for each, give or
// take one (a fixed "SMs x 8" grid left the last of its 1.6 waves 60 % full on kernels that fit five CTAs per SM).
template <typename Kernel> static int an_grid(Kernel kern, int64_t rows) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kAnThreads, 0) != cudaSuccess || per_sm <= 0) {
        cudaGetLastError();
        per_sm = 4;
    }
    const int64_t per_cta = std::max<int64_t>(1, ceil_div(rows, (int64_t) sm_count() * per_sm));
    return (int) std::max<int64_t>(1, ceil_div(rows, per_cta));
}

}  // namespace ptb

using namespace ptb;

extern "C" {

int pt_glu_fwd(const void *x, int dtype, const float *probs, const int64_t *row_mask, int64_t rows, int64_t H, int act, void *out, void *stream) {
    PT_REQUIRE(rows >= 0 && H >= 0 && (act == 0 || act == 1), "glu forward: bad arguments");
    if (rows * H == 0) return PT_OK;
    PT_REQUIRE(x && probs && out, "glu forward: null pointer");
    PT_REQUIRE((H * (dtype == PT_F32 ? 4 : 2)) % 16 == 0 && aligned(x, 16) && aligned(out, 16), "glu forward: H must give 16-byte rows, 16-byte aligned");
    PT_SWITCH_SRC(dtype, T, {
        if (act == 0) glu_fwd_kernel<T, PT_ACT_SILU><<<an_grid(glu_fwd_kernel<T, PT_ACT_SILU>, rows), kAnThreads, 0, (cudaStream_t) stream>>>((const T *) x, probs, row_mask, rows, H, (T *) out);
        else glu_fwd_kernel<T, PT_ACT_GELU><<<an_grid(glu_fwd_kernel<T, PT_ACT_GELU>, rows), kAnThreads, 0, (cudaStream_t) stream>>>((const T *) x, probs, row_mask, rows, H, (T *) out);
    });
    PT_LAUNCH_OK();
    return PT_OK;
}

int pt_glu_bwd(const void *grad_out, const void *x, int dtype, const float *probs, const int64_t *row_mask, int64_t rows, int64_t H, int act,
               void *grad_x, float *grad_probs, void *stream) {
    PT_REQUIRE(rows >= 0 && H >= 0 && (act == 0 || act == 1), "glu backward: bad arguments");
    if (rows * H == 0) return PT_OK;
    PT_REQUIRE(grad_out && x && probs && grad_x && grad_probs, "glu backward: null pointer");
    PT_REQUIRE((H * (dtype == PT_F32 ? 4 : 2)) % 16 == 0 && aligned(x, 16) && aligned(grad_out, 16) && aligned(grad_x, 16),
               "glu backward: H must give 16-byte rows, 16-byte aligned");
    PT_SWITCH_SRC(dtype, T, {
        if (act == 0)
            glu_bwd_kernel<T, PT_ACT_SILU><<<an_grid(glu_bwd_kernel<T, PT_ACT_SILU>, rows), kAnThreads, 0, (cudaStream_t) stream>>>((const T *) grad_out, (const T *) x, probs, row_mask, rows,
                                                                                                H, (T *) grad_x, grad_probs);
        else
            glu_bwd_kernel<T, PT_ACT_GELU><<<an_grid(glu_bwd_kernel<T, PT_ACT_GELU>, rows), kAnThreads, 0, (cudaStream_t) stream>>>((const T *) grad_out, (const T *) x, probs, row_mask, rows,
                                                                                                H, (T *) grad_x, grad_probs);
    });
    PT_LAUNCH_OK();
    return PT_OK;
}

int pt_rmsnorm_fwd(const void *x, const void *residual, const void *gamma, int dtype, float eps, int zero_centered, int64_t rows, int64_t H, void *y,
                   void *x_plus_r, float *rstd, void *stream) {
    PT_REQUIRE(rows >= 0 && H >= 1, "rmsnorm forward: bad shape");
    if (rows == 0) return PT_OK;
    PT_REQUIRE(x && rstd && (y == nullptr || gamma), "rmsnorm forward: null pointer");
    PT_REQUIRE((residual == nullptr) == (x_plus_r == nullptr), "rmsnorm forward: residual and x_plus_r go together");
    const bool vec = (H * (dtype == PT_F32 ? 4 : 2)) % 16 == 0 && aligned(x, 16) && aligned(y, 16) && aligned(gamma, 16) && aligned(residual, 16) &&
                     aligned(x_plus_r, 16);   // else element-wise accesses
    cudaStream_t st = (cudaStream_t) stream;
#define PT_RMS_FWD(V_, RES_) \
    rmsnorm_fwd_kernel<T, V_, RES_><<<an_grid(rmsnorm_fwd_kernel<T, V_, RES_>, rows), kAnThreads, 0, st>>>((const T *) x, (const T *) residual, (const T *) gamma, eps, zero_centered, rows, H, \
                                                                          (T *) y, (T *) x_plus_r, rstd)
    if (y == nullptr && residual == nullptr && vec) {   // statistics only
        PT_SWITCH_SRC(dtype, T, {
            const int grid = an_grid(rmsnorm_stats_kernel<T>, ceil_div(rows, kAnThreads / 32));   // a warp per row: groups of eight rows
            rmsnorm_stats_kernel<T><<<grid, kAnThreads, 0, st>>>((const T *) x, eps, rows, H, rstd);
        });
        PT_LAUNCH_OK();
        return PT_OK;
    }
    PT_SWITCH_SRC(dtype, T, {
        constexpr int VW = 16 / sizeof(T);
        if (vec) { if (residual) PT_RMS_FWD(VW, true); else PT_RMS_FWD(VW, false); }
        else { if (residual) PT_RMS_FWD(1, true); else PT_RMS_FWD(1, false); }
    });
#undef PT_RMS_FWD
    PT_LAUNCH_OK();
    return PT_OK;
}

int pt_rmsnorm_bwd_parts(int64_t rows) { return (int) std::min<int64_t>(std::max<int64_t>(rows, 1), (int64_t) sm_count() * 3); }

int pt_rmsnorm_bwd(const void *dy, const void *dxpr, const void *x, const void *gamma, const float *rstd, int dtype, int zero_centered, int64_t rows,
                   int64_t H, void *dx, void *dgamma, float *dg_partial, int parts, void *stream) {
    PT_REQUIRE(rows >= 0 && H >= 1, "rmsnorm backward: bad shape");
    PT_REQUIRE(dgamma && dg_partial && parts == pt_rmsnorm_bwd_parts(rows), "rmsnorm backward: dgamma buffers / part count");
    PT_REQUIRE(rows == 0 || (dy && x && gamma && rstd && dx), "rmsnorm backward: null pointer");
    const bool vec = (H * (dtype == PT_F32 ? 4 : 2)) % 16 == 0 && aligned(x, 16) && aligned(dy, 16) && aligned(dx, 16) && aligned(gamma, 16) && aligned(dxpr, 16);
    cudaStream_t st = (cudaStream_t) stream;
    PT_SWITCH_SRC(dtype, T, {
        constexpr int VW = 16 / sizeof(T);
        if (vec && H <= (int64_t) kAnThreads * VW * 4 && getenv("PT_RMSNORM_BWD_NO_STAGE") == nullptr) {
            // as many row slots as fit 72 KiB (three CTAs per SM), between 2 and 8
            const int64_t slot_bytes = 2 * H * (int64_t) sizeof(T);
            const int stages = (int) std::max<int64_t>(2, std::min<int64_t>(8, (72 * 1024) / slot_bytes));
            const int smem = (int) (stages * slot_bytes);
            auto kern = H <= (int64_t) kAnThreads * VW * 2 ? rmsnorm_bwd_staged_kernel<T, 2> : rmsnorm_bwd_staged_kernel<T, 4>;
            PT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            kern<<<parts, kAnThreads, smem, st>>>((const T *) dy, (const T *) dxpr, (const T *) x, (const T *) gamma, rstd, zero_centered, rows, H, (T *) dx,
                                                  dg_partial, stages);
        } else if (vec)
            rmsnorm_bwd_kernel<T, VW><<<parts, kAnThreads, 0, st>>>((const T *) dy, (const T *) dxpr, (const T *) x, (const T *) gamma, rstd, zero_centered, rows,
                                                                    H, (T *) dx, dg_partial);
        else
            rmsnorm_bwd_kernel<T, 1><<<parts, kAnThreads, 0, st>>>((const T *) dy, (const T *) dxpr, (const T *) x, (const T *) gamma, rstd, zero_centered, rows, H,
                                                                   (T *) dx, dg_partial);
        PT_LAUNCH_OK();
        rmsnorm_dgamma_kernel<T><<<(unsigned) ceil_div(H, 32), 32 * kDgLanes, 0, st>>>(dg_partial, parts, H, (T *) dgamma);
    });
    PT_LAUNCH_OK();
    return PT_OK;
}

}  // extern "C"
