// Fused composites that work on rows or elements: Softmax, RMSNorm
// (SimplifiedLayerNormalization, optionally with the preceding residual add),
// Gelu (optionally with the following multiply = GeGLU), RotaryEmbedding, and
// the greedy-sampling argmax.
//
// Each kernel follows the primitive sequence of its decomposition
// (crates/onyxia-ir/src/decomp.rs:174-355) and rounds to the tensor dtype at
// the same points, so for f16 tensors the result differs from the interpreter
// only where an f32 transcendental or an f32 sum differs from the f64 one.
#include "common.cuh"
#include "kernels.hpp"

namespace oxk {

// Round an f32 working value through the tensor dtype.
template <int DT> __device__ __forceinline__ float rnd(float v) {
    if constexpr (DT == DT_F16) return __half2float(__float2half_rn(v));
    else return v;
}
// Round an f64 value to the tensor dtype in one step.
template <int DT> __device__ __forceinline__ float rnd_d(double v) {
    if constexpr (DT == DT_F16) return __half2float(__double2half(v));
    else return (float)v;
}
// Block-wide f64 sum (the interpreter reduces in f64); `red` is 32 doubles of shared memory.
__device__ __forceinline__ double block_sum_d(double v, double* red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int k = 0; k < nw; k++) t += red[k];
        red[0] = t;
    }
    __syncthreads();
    return red[0];
}

// ───────────────────────────── Softmax ──────────────────────────────────
struct SoftmaxP {
    const void* x;
    void* y;
    long long rows, cols;
};

// One block per row: max, then exp and sum, then divide (decomp.rs:174-183).
template <int DT> __global__ void __launch_bounds__(256) fused_softmax(const SoftmaxP p) {
    __shared__ float red[32];
    __shared__ double redd[32];
    for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const long long base = row * p.cols;
        float mx = -INFINITY;
        for (long long c = threadIdx.x; c < p.cols; c += blockDim.x) mx = fmaxf(mx, ld<DT>(p.x, base + c));
        mx = block_max(mx, red);
        double dsum = 0.0;
        for (long long c = threadIdx.x; c < p.cols; c += blockDim.x)
            dsum += (double)rnd_d<DT>(exp((double)rnd<DT>(ld<DT>(p.x, base + c) - mx)));
        float sum = rnd_d<DT>(block_sum_d(dsum, redd));
        for (long long c = threadIdx.x; c < p.cols; c += blockDim.x) {
            float e = rnd_d<DT>(exp((double)rnd<DT>(ld<DT>(p.x, base + c) - mx)));
            st<DT>(p.y, base + c, e / sum);
        }
    }
}

void emit_softmax(Emitter& em, const TRef& x, const TRef& y) {
    SoftmaxP p{};
    p.cols = x.shape.empty() ? 1 : x.shape.back();
    p.rows = p.cols ? x.numel() / p.cols : 0;
    if (p.rows == 0 || p.cols == 0) return;
    dim3 g((unsigned)std::min<long long>(p.rows, sm_count() * 32LL)), b(256);
    if (x.dtype == DT_F32) em.launch(fused_softmax<DT_F32>, g, b, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}}, "fused_softmax");
    else em.launch(fused_softmax<DT_F16>, g, b, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}}, "fused_softmax");
}

// ───────────────────────────── RMSNorm ──────────────────────────────────
struct RmsNormP {
    const void* x;
    const void* res;  // optional residual added to x first
    const void* w;
    void* y;
    void* sum_out;    // optional: x + res
    long long rows, cols;
    float eps;        // already rounded to the tensor dtype
};

// x·rsqrt(mean(x²) + ε)·w with the decomposition's rounding points
// (decomp.rs:241-257). A row is one CTA; for rows of up to EPT·blockDim
// elements every operand is fetched in a single round of loads and the row
// stays in registers (one DRAM latency instead of three).
template <int DT, int EPT> __global__ void __launch_bounds__(1024) fused_rmsnorm(const RmsNormP p) {
    __shared__ double redd[32];
    pdl_enter();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const long long base = row * p.cols;
        float v[EPT > 0 ? EPT : 1], wv[EPT > 0 ? EPT : 1];
        double ss = 0.0;
        if constexpr (EPT > 0) {
#pragma unroll
            for (int e = 0; e < EPT; e++) {
                long long c = threadIdx.x + (long long)e * blockDim.x;
                bool in = c < p.cols;
                v[e] = in ? ld<DT>(p.x, base + c) : 0.f;
                wv[e] = in ? ld<DT>(p.w, c) : 0.f;
                if (p.res && in) v[e] = rnd<DT>(v[e] + ld<DT>(p.res, base + c));
            }
#pragma unroll
            for (int e = 0; e < EPT; e++) ss += (double)rnd<DT>(v[e] * v[e]);
        } else {
            for (long long c = threadIdx.x; c < p.cols; c += blockDim.x) {
                float x = ld<DT>(p.x, base + c);
                if (p.res) x = rnd<DT>(x + ld<DT>(p.res, base + c));
                ss += (double)rnd<DT>(x * x);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        __syncthreads();  // redd may still be read by the previous row
        if (lane == 0) redd[warp] = ss;
        __syncthreads();
        double tot = 0.0;
        for (int k = 0; k < nw; k++) tot += redd[k];
        float ms = rnd_d<DT>(tot / (double)p.cols);
        float denom = rnd<DT>(ms + p.eps);
        float inv = rnd_d<DT>(1.0 / sqrt((double)denom));
        if constexpr (EPT > 0) {
#pragma unroll
            for (int e = 0; e < EPT; e++) {
                long long c = threadIdx.x + (long long)e * blockDim.x;
                if (c < p.cols) {
                    if (p.res && p.sum_out) st<DT>(p.sum_out, base + c, v[e]);
                    st<DT>(p.y, base + c, rnd<DT>(v[e] * inv) * wv[e]);
                }
            }
        } else {
            for (long long c = threadIdx.x; c < p.cols; c += blockDim.x) {
                float x = ld<DT>(p.x, base + c);
                if (p.res) {
                    x = rnd<DT>(x + ld<DT>(p.res, base + c));
                    if (p.sum_out) st<DT>(p.sum_out, base + c, x);
                }
                st<DT>(p.y, base + c, rnd<DT>(x * inv) * ld<DT>(p.w, c));
            }
        }
    }
}

void emit_rmsnorm(Emitter& em, const TRef& x, const TRef& w, const TRef& y, double eps, const TRef* res,
                  const TRef* sum_out) {
    RmsNormP p{};
    p.cols = x.shape.back();
    p.rows = p.cols ? x.numel() / p.cols : 0;
    if (p.rows == 0 || p.cols == 0) return;
    p.eps = x.dtype == DT_F16 ? __half2float(__double2half(eps)) : (float)eps;
    // ≤ 4 elements per thread where the row allows it, warps of whole lanes
    long long threads = std::min<long long>(1024, std::max<long long>(64, ((p.cols + 3) / 4 + 31) / 32 * 32));
    long long ept = (p.cols + threads - 1) / threads;
    dim3 g((unsigned)std::min<long long>(p.rows, sm_count() * 32LL)), b((unsigned)threads);
    Buf rb = res ? res->buf : Buf{kSlotNull, 0}, sb = sum_out ? sum_out->buf : Buf{kSlotNull, 0};
#define GO(DT, E) \
    em.launch(fused_rmsnorm<DT, E>, g, b, 0, p, {{&p.x, x.buf}, {&p.res, rb}, {&p.w, w.buf}, {&p.y, y.buf}, {&p.sum_out, sb}}, "fused_rmsnorm", /*pdl=*/true)
#define GO_E(DT)                    \
    if (ept <= 1) GO(DT, 1);        \
    else if (ept <= 2) GO(DT, 2);   \
    else if (ept <= 4) GO(DT, 4);   \
    else if (ept <= 8) GO(DT, 8);   \
    else GO(DT, 0);
    if (x.dtype == DT_F32) { GO_E(DT_F32) } else { GO_E(DT_F16) }
#undef GO_E
#undef GO
}

// ───────────────────────────── Gelu / GeGLU ─────────────────────────────
struct GeluP {
    const void* x;
    const void* mul;  // optional second factor (GeGLU: gelu(gate)·up)
    void* y;
    long long n;
    int tanh_approx;
    float c_half, c_one, c_coef, c_k, c_inv_sqrt2;  // constants rounded to the tensor dtype
};

__device__ __forceinline__ double erf_as_f(float xf) {  // Abramowitz–Stegun 7.1.26 (interp.rs:860-872)
    double x = xf;
    double sign = x < 0.0 ? -1.0 : 1.0;
    x = fabs(x);
    double t = 1.0 / (1.0 + 0.3275911 * x);
    double y = 1.0 - (((((1.061405429 * t - 1.453152027) * t) + 1.421413741) * t - 0.284496736) * t + 0.254829592) * t *
                         exp(-x * x);
    return sign * y;
}

template <int DT> __global__ void fused_gelu(const GeluP p) {
    pdl_enter();
    for (long long i = global_tid(); i < p.n; i += global_threads()) {
        float x = ld<DT>(p.x, i);
        float inner;
        if (p.tanh_approx) {  // decomp.rs:192-202
            float x2 = rnd<DT>(x * x);
            float x3 = rnd<DT>(x2 * x);
            float cx3 = rnd<DT>(p.c_coef * x3);
            float s = rnd<DT>(x + cx3);
            float sc = rnd<DT>(p.c_k * s);
            inner = rnd_d<DT>(tanh((double)sc));
        } else {  // decomp.rs:203-208
            float sc = rnd<DT>(x * p.c_inv_sqrt2);
            inner = rnd_d<DT>(erf_as_f(sc));
        }
        float one_plus = rnd<DT>(p.c_one + inner);
        float hx = rnd<DT>(p.c_half * x);
        float out = hx * one_plus;
        if (p.mul) out = rnd<DT>(out) * ld<DT>(p.mul, i);
        st<DT>(p.y, i, out);
    }
}

void emit_gelu(Emitter& em, const TRef& x, const TRef& y, bool tanh_approx, const TRef* mul) {
    GeluP p{};
    p.n = x.numel();
    if (p.n == 0) return;
    p.tanh_approx = tanh_approx ? 1 : 0;
    auto r = [&](double v) { return x.dtype == DT_F16 ? __half2float(__double2half(v)) : (float)v; };
    p.c_half = r(0.5);
    p.c_one = r(1.0);
    p.c_coef = r(0.044715);
    p.c_k = r(std::sqrt(2.0 / 3.14159265358979323846));
    p.c_inv_sqrt2 = r(0.70710678118654752440);
    dim3 g(grid_for(p.n, 256)), b(256);
    Buf mb = mul ? mul->buf : Buf{kSlotNull, 0};
    const char* label = mul ? "fused_geglu" : "fused_gelu";
    if (x.dtype == DT_F32) em.launch(fused_gelu<DT_F32>, g, b, 0, p, {{&p.x, x.buf}, {&p.mul, mb}, {&p.y, y.buf}}, label, /*pdl=*/true);
    else em.launch(fused_gelu<DT_F16>, g, b, 0, p, {{&p.x, x.buf}, {&p.mul, mb}, {&p.y, y.buf}}, label, /*pdl=*/true);
}

// ───────────────────────────── RotaryEmbedding ──────────────────────────
struct RotaryP {
    const void* x;
    const long long* pos;  // [B·S]
    const void* cos;
    const void* sin;
    void* y;
    ErrWord* err;
    long long n;       // B·S·heads·D
    long long heads, d, half, cache_rows;
    int node;
};

// Half-split rotation with inline cos/sin gather by position (decomp.rs:259-355).
template <int DT> __global__ void fused_rotary(const RotaryP p) {
    for (long long i = global_tid(); i < p.n; i += global_threads()) {
        long long e = i % p.d, tok = i / (p.d * p.heads);
        float out;
        if (e >= 2 * p.half) {
            out = ld<DT>(p.x, i);
        } else {
            long long row = p.pos[tok];
            if (row < 0) row += p.cache_rows;
            if (row < 0 || row >= p.cache_rows) {
                report(p.err, ERR_GATHER_OOB, p.node, row, p.cache_rows);
                row = 0;
            }
            bool first = e < p.half;
            long long j = first ? e : e - p.half;
            float c = ld<DT>(p.cos, row * p.half + j), s = ld<DT>(p.sin, row * p.half + j);
            float x1 = ld<DT>(p.x, i - (first ? 0 : p.half)), x2 = ld<DT>(p.x, i + (first ? p.half : 0));
            out = first ? rnd<DT>(x1 * c) - rnd<DT>(x2 * s) : rnd<DT>(x2 * c) + rnd<DT>(x1 * s);
        }
        st<DT>(p.y, i, out);
    }
}

void emit_rotary(Emitter& em, const TRef& x, const TRef& pos, const TRef& cos, const TRef& sin, const TRef& y,
                 int64_t heads, int64_t half) {
    RotaryP p{};
    p.n = x.numel();
    if (p.n == 0) return;
    p.heads = heads;
    p.d = x.shape.back() / heads;
    p.half = half;
    p.cache_rows = cos.shape[0];
    p.node = em.node;
    dim3 g(grid_for(p.n, 256)), b(256);
    if (x.dtype == DT_F32)
        em.launch(fused_rotary<DT_F32>, g, b, 0, p,
                  {{&p.x, x.buf}, {&p.pos, pos.buf}, {&p.cos, cos.buf}, {&p.sin, sin.buf}, {&p.y, y.buf}, {&p.err, Buf{kSlotErr, 0}}}, "fused_rotary");
    else
        em.launch(fused_rotary<DT_F16>, g, b, 0, p,
                  {{&p.x, x.buf}, {&p.pos, pos.buf}, {&p.cos, cos.buf}, {&p.sin, sin.buf}, {&p.y, y.buf}, {&p.err, Buf{kSlotErr, 0}}}, "fused_rotary");
}

// ───────────────────────────── argmax over the last axis ────────────────
struct ArgmaxP {
    const void* x;
    long long* y;
    float* part_v;       // [rows][blocks] best value per block
    long long* part_i;   // [rows][blocks] its index
    unsigned* counters;  // one per row
    long long rows, cols;
    int blocks;          // blocks per row
};

// (v, i) beats (bv, b) if it is larger, or equal with a higher index: among
// equal maxima the last one wins, like `Iterator::max_by`
// (crates/onyxia-cli/src/sampling.rs:71-80).
__device__ __forceinline__ bool am_better(float v, long long i, float bv, long long b) {
    return b < 0 || (i >= 0 && (v > bv || (v == bv && i > b)));
}
__device__ __forceinline__ void am_block(float& best, long long& bi, float* sv, long long* si) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (am_better(ov, oi, best, bi)) {
            best = ov;
            bi = oi;
        }
    }
    __syncthreads();
    if (lane == 0) {
        sv[w] = best;
        si[w] = bi;
    }
    __syncthreads();
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : -1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (am_better(ov, oi, best, bi)) {
            best = ov;
            bi = oi;
        }
    }
}

// Each row is split over `blocks` CTAs; the last one to arrive merges.
template <int DT> __global__ void __launch_bounds__(256) sample_argmax(const ArgmaxP p) {
    __shared__ float sv[32];
    __shared__ long long si[32];
    __shared__ unsigned arrived;
    const long long row = blockIdx.y, base = row * p.cols;
    const long long per = (p.cols + p.blocks - 1) / p.blocks;
    const long long c0 = blockIdx.x * per, c1 = c0 + per < p.cols ? c0 + per : p.cols;
    float best = -INFINITY;
    long long bi = -1;
    for (long long c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        float v = ld<DT>(p.x, base + c);
        if (bi < 0 || v >= best) {  // columns ascend within a thread, so >= keeps the last maximum
            best = v;
            bi = c;
        }
    }
    am_block(best, bi, sv, si);
    if (p.blocks == 1) {
        if (threadIdx.x == 0) p.y[row] = bi < 0 ? 0 : bi;
        return;
    }
    if (threadIdx.x == 0) {
        p.part_v[row * p.blocks + blockIdx.x] = best;
        p.part_i[row * p.blocks + blockIdx.x] = bi;
        __threadfence();
        arrived = atomicAdd(p.counters + row, 1u);
        if (arrived == (unsigned)p.blocks - 1) p.counters[row] = 0;
    }
    __syncthreads();
    if (arrived != (unsigned)p.blocks - 1) return;
    __threadfence();
    best = -INFINITY;
    bi = -1;
    for (int k = threadIdx.x; k < p.blocks; k += blockDim.x) {
        float v = __ldcg(p.part_v + row * p.blocks + k);
        long long i = __ldcg(p.part_i + row * p.blocks + k);
        if (am_better(v, i, best, bi)) {
            best = v;
            bi = i;
        }
    }
    am_block(best, bi, sv, si);
    if (threadIdx.x == 0) p.y[row] = bi < 0 ? 0 : bi;
}

void emit_argmax_last(Emitter& em, const TRef& x, const TRef& y, Buf part, Buf counters) {
    ArgmaxP p{};
    p.cols = x.shape.back();
    p.rows = p.cols ? x.numel() / p.cols : 0;
    if (p.rows == 0) return;
    if (p.rows > 65535 || (size_t)p.rows > kCounterWords) throw std::runtime_error("argmax: too many rows");
    p.blocks = (int)std::max<long long>(1, std::min<long long>(kArgmaxMaxBlocks, p.cols / 2048));
    dim3 g((unsigned)p.blocks, (unsigned)p.rows), b(256);
    Buf pv = part, pi = part.at((int64_t)(p.rows * kArgmaxMaxBlocks * 4));
    if (x.dtype == DT_F32)
        em.launch(sample_argmax<DT_F32>, g, b, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}, {&p.part_v, pv}, {&p.part_i, pi}, {&p.counters, counters}}, "sample_argmax");
    else
        em.launch(sample_argmax<DT_F16>, g, b, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}, {&p.part_v, pv}, {&p.part_i, pi}, {&p.counters, counters}}, "sample_argmax");
}

}  // namespace oxk
