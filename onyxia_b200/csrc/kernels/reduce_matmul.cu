// Reduce, MatMul and Dequantize primitives
// (crates/onyxia-ir/src/interp.rs:960-1125, 764-797).
#include "common.cuh"
#include "kernels.hpp"

namespace oxk {

static std::vector<int64_t> row_major(const std::vector<int64_t>& dims) {
    std::vector<int64_t> st(dims.size(), 1);
    for (size_t i = dims.size(); i-- > 1;) st[i - 1] = st[i] * dims[i];
    return st;
}

// ───────────────────────────── Reduce ───────────────────────────────────
enum { R_SUM = 0, R_MEAN, R_MAX, R_MIN, R_PROD };

struct ReduceP {
    const void* x;
    void* y;
    long long out_n, count;
    int op;
    NdShape kept;   // kept dims, in order
    NdStride skept;
    NdShape red;    // reduced dims, in order
    NdStride sred;
};

template <typename W> __device__ __forceinline__ W red_init(int op);
template <> __device__ __forceinline__ float red_init<float>(int op) {
    return op == R_PROD ? 1.f : op == R_MAX ? -INFINITY : op == R_MIN ? INFINITY : 0.f;
}
template <> __device__ __forceinline__ long long red_init<long long>(int op) {
    return op == R_PROD ? 1 : op == R_MAX ? LLONG_MIN : op == R_MIN ? LLONG_MAX : 0;
}
__device__ __forceinline__ float red_step(int op, float a, float v) {
    switch (op) {
        case R_PROD: return a * v;
        case R_MAX: return fmaxf(a, v);
        case R_MIN: return fminf(a, v);
        default: return a + v;
    }
}
__device__ __forceinline__ long long red_step(int op, long long a, long long v) {
    switch (op) {
        case R_PROD: return (long long)((unsigned long long)a * (unsigned long long)v);
        case R_MAX: return a > v ? a : v;
        case R_MIN: return a < v ? a : v;
        default: return (long long)((unsigned long long)a + (unsigned long long)v);
    }
}

// One warp per output element; lanes stride over the reduced elements and are
// combined with shuffles. Integer results are exact (wrapping ops commute);
// float sums differ from the interpreter's f64 order only by rounding.
template <int DT> __global__ void prim_reduce(const ReduceP p) {
    using W = typename Ty<DT>::W;
    int lane = threadIdx.x & 31;
    long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long o = warp; o < p.out_n; o += nwarps) {
        long long base = nd_offset(o, p.kept, p.skept);
        W acc = red_init<W>(p.op);
        for (long long r = lane; r < p.count; r += 32) acc = red_step(p.op, acc, ld<DT>(p.x, base + nd_offset(r, p.red, p.sred)));
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            W other = __shfl_xor_sync(0xffffffffu, acc, s);
            acc = red_step(p.op, acc, other);
        }
        if (lane == 0) {
            if (p.op == R_MEAN) {
                if constexpr (Ty<DT>::is_float) acc = acc / (float)p.count;
                else if (p.count != 0) acc = acc / p.count;  // truncating integer mean
            }
            st<DT>(p.y, o, acc);
        }
    }
}

// Few outputs, each over many elements (the attention mask's row sums at batch 1): one CTA per output, four
// independent loads in flight per thread, warps combined through shared memory. Same operations and order
// classes as above (integers exact; float sums differ from the interpreter's only by rounding).
template <int DT> __global__ void __launch_bounds__(256) prim_reduce_block(const ReduceP p) {
    using W = typename Ty<DT>::W;
    __shared__ W part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (long long o = blockIdx.x; o < p.out_n; o += gridDim.x) {
        const long long base = nd_offset(o, p.kept, p.skept);
        W acc = red_init<W>(p.op);
        for (long long r0 = threadIdx.x; r0 < p.count; r0 += 4 * 256) {
            W v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const long long r = r0 + u * 256;
                v[u] = r < p.count ? (W)ld<DT>(p.x, base + nd_offset(r, p.red, p.sred)) : red_init<W>(p.op);
            }
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (r0 + u * 256 < p.count) acc = red_step(p.op, acc, v[u]);
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc = red_step(p.op, acc, __shfl_xor_sync(0xffffffffu, acc, s));
        if (lane == 0) part[warp] = acc;
        __syncthreads();
        if (warp == 0) {
            acc = lane < 8 ? part[lane] : red_init<W>(p.op);
#pragma unroll
            for (int s = 4; s > 0; s >>= 1) {
                W other = __shfl_xor_sync(0xffffffffu, acc, s);
                if (lane < 8) acc = red_step(p.op, acc, other);
            }
            if (lane == 0) {
                if (p.op == R_MEAN) {
                    if constexpr (Ty<DT>::is_float) acc = acc / (float)p.count;
                    else if (p.count != 0) acc = acc / p.count;  // truncating integer mean
                }
                st<DT>(p.y, o, acc);
            }
        }
        __syncthreads();  // `part` is reused by the next output
    }
}

void emit_reduce(Emitter& em, int op, const TRef& x, const TRef& y, const std::vector<size_t>& axes) {
    ReduceP p{};
    p.op = op;
    auto xs = row_major(x.shape);
    p.out_n = 1;
    p.count = 1;
    for (size_t d = 0; d < x.shape.size(); d++) {
        bool red = false;
        for (auto a : axes) red |= (a == d);
        if (red) {
            p.red.dim[p.red.rank] = x.shape[d];
            p.sred.s[p.red.rank++] = xs[d];
            p.count *= x.shape[d];
        } else {
            p.kept.dim[p.kept.rank] = x.shape[d];
            p.skept.s[p.kept.rank++] = xs[d];
            p.out_n *= x.shape[d];
        }
    }
    (void)y;
    const bool per_block = p.count >= 256 && p.out_n <= 2 * sm_count();
    dim3 g(per_block ? (unsigned)std::max<long long>(p.out_n, 1) : grid_for(p.out_n * 32, 256)), b(256);
#define CALL(DT)                                                                                              \
    if (per_block) em.launch(prim_reduce_block<DT>, g, b, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}}, "prim_reduce"); \
    else em.launch(prim_reduce<DT>, g, b, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}}, "prim_reduce")
    switch (x.dtype) {
        case DT_F32: CALL(DT_F32); break;
        case DT_F16: CALL(DT_F16); break;
        case DT_I64: CALL(DT_I64); break;
        case DT_I32: CALL(DT_I32); break;
        case DT_U32: CALL(DT_U32); break;
        case DT_U8: CALL(DT_U8); break;
        case DT_I8: CALL(DT_I8); break;
        default: throw std::runtime_error("reduce: unsupported dtype");
    }
#undef CALL
}

// ───────────────────────────── MatMul ───────────────────────────────────
// Generic batched matmul with transpose flags and batch broadcast. Operands
// are addressed as a(i,k) = a[batch_off_a + i·a_rs + k·a_cs] (likewise b), so
// the four layouts share one kernel. 32×32 output tiles, 32-deep K slabs in
// shared memory, f32 accumulation for floats, wrapping int64 for integers.
struct MatMulP {
    const void* a;
    const void* b;
    void* y;
    long long m, n, k;
    long long a_rs, a_cs, b_rs, b_cs;  // strides of (row, k) for a and (k, col) for b
    long long a_mat, b_mat;            // elements per matrix
    NdShape batch;
    NdStride sa, sb;                   // batch strides in units of matrices (0 = broadcast)
};

template <int DT> __global__ void __launch_bounds__(256) prim_matmul(const MatMulP p) {
    using W = typename Ty<DT>::W;
    constexpr int T = 32;
    __shared__ W As[T][T + 1];
    __shared__ W Bs[T][T + 1];
    long long bi = blockIdx.z;
    long long a_base = nd_offset(bi, p.batch, p.sa) * p.a_mat;
    long long b_base = nd_offset(bi, p.batch, p.sb) * p.b_mat;
    int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 × 8 threads, 4 rows each
    long long row0 = (long long)blockIdx.y * T, col0 = (long long)blockIdx.x * T;
    W acc[4];
#pragma unroll
    for (int r = 0; r < 4; r++) acc[r] = (W)0;
    for (long long k0 = 0; k0 < p.k; k0 += T) {
#pragma unroll
        for (int r = 0; r < 4; r++) {
            int i = ty * 4 + r;
            long long gi = row0 + i, gk = k0 + tx;
            As[i][tx] = (gi < p.m && gk < p.k) ? ld<DT>(p.a, a_base + gi * p.a_rs + gk * p.a_cs) : (W)0;
            long long gk2 = k0 + i, gj = col0 + tx;
            Bs[i][tx] = (gk2 < p.k && gj < p.n) ? ld<DT>(p.b, b_base + gk2 * p.b_rs + gj * p.b_cs) : (W)0;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < T; kk++) {
            W bv = Bs[kk][tx];
#pragma unroll
            for (int r = 0; r < 4; r++) {
                if constexpr (Ty<DT>::is_float) acc[r] = fmaf(As[ty * 4 + r][kk], bv, acc[r]);
                else acc[r] = (long long)((unsigned long long)acc[r] + (unsigned long long)As[ty * 4 + r][kk] * (unsigned long long)bv);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 4; r++) {
        long long gi = row0 + ty * 4 + r, gj = col0 + tx;
        if (gi < p.m && gj < p.n) st<DT>(p.y, (bi * p.m + gi) * p.n + gj, acc[r]);
    }
}

void emit_matmul(Emitter& em, const TRef& a, const TRef& b, const TRef& y, bool ta, bool tb) {
    MatMulP p{};
    size_t ar = a.shape.size(), br = b.shape.size();
    int64_t a_r = a.shape[ar - 2], a_c = a.shape[ar - 1], b_r = b.shape[br - 2], b_c = b.shape[br - 1];
    p.m = ta ? a_c : a_r;
    p.k = ta ? a_r : a_c;
    p.n = tb ? b_r : b_c;
    p.a_rs = ta ? 1 : a_c;
    p.a_cs = ta ? a_c : 1;
    p.b_rs = tb ? 1 : b_c;  // stride of k
    p.b_cs = tb ? b_c : 1;  // stride of column
    p.a_mat = a_r * a_c;
    p.b_mat = b_r * b_c;
    std::vector<int64_t> batch(y.shape.begin(), y.shape.end() - 2);
    std::vector<int64_t> ab(a.shape.begin(), a.shape.end() - 2), bb(b.shape.begin(), b.shape.end() - 2);
    if (batch.size() > (size_t)kMaxRank) throw std::runtime_error("matmul: batch rank exceeds 8");
    p.batch.rank = (int)batch.size();
    int64_t nb = 1;
    for (size_t i = 0; i < batch.size(); i++) {
        p.batch.dim[i] = batch[i];
        nb *= batch[i];
    }
    auto fill = [&](const std::vector<int64_t>& in, NdStride& s) {
        size_t off = batch.size() - in.size();
        long long run = 1;
        for (size_t i = in.size(); i-- > 0;) {
            s.s[i + off] = in[i] == 1 ? 0 : run;
            run *= in[i];
        }
    };
    fill(ab, p.sa);
    fill(bb, p.sb);
    if (nb == 0 || p.m == 0 || p.n == 0) return;
    if (nb > 65535) throw std::runtime_error("matmul: more than 65535 batch matrices");
    dim3 g((unsigned)((p.n + 31) / 32), (unsigned)((p.m + 31) / 32), (unsigned)nb), blk(256);
#define CALL(DT) em.launch(prim_matmul<DT>, g, blk, 0, p, {{&p.a, a.buf}, {&p.b, b.buf}, {&p.y, y.buf}}, "prim_matmul")
    switch (a.dtype) {
        case DT_F32: CALL(DT_F32); break;
        case DT_F16: CALL(DT_F16); break;
        case DT_I64: CALL(DT_I64); break;
        case DT_I32: CALL(DT_I32); break;
        case DT_U32: CALL(DT_U32); break;
        case DT_U8: CALL(DT_U8); break;
        case DT_I8: CALL(DT_I8); break;
        default: throw std::runtime_error("matmul: unsupported dtype");
    }
#undef CALL
}

// ───────────────────────────── Dequantize ───────────────────────────────
// out[i] = (q[i] − zp[i / bs]) · scale[i / bs], rounded to the scales' dtype.
// The product of a small integer and one scale is exact in f32, so a single
// rounding on store matches the interpreter's f64 evaluation bit for bit.
struct DequantP {
    const void* q;
    const void* scales;
    const void* zp;  // may be null
    void* y;
    long long n, block_size;
    int default_zp;
};

template <int QDT, int SDT> __global__ void prim_dequantize(const DequantP p) {
    // each thread handles 8 consecutive elements (one 32-bit word of nibbles for u4/i4)
    long long groups = (p.n + 7) / 8;
    for (long long g = global_tid(); g < groups; g += global_threads()) {
        long long i0 = g * 8;
#pragma unroll
        for (int e = 0; e < 8; e++) {
            long long i = i0 + e;
            if (i >= p.n) break;
            long long blockk = i / p.block_size;
            long long q, z = p.default_zp;
            if constexpr (QDT == DT_U4) {
                q = ld_u4(p.q, i);
                if (p.zp) z = ld_u4(p.zp, blockk);
            } else if constexpr (QDT == DT_I4) {
                q = ld_i4(p.q, i);
                if (p.zp) z = ld_i4(p.zp, blockk);
            } else {
                q = ((const unsigned char*)p.q)[i];
                if (p.zp) z = ((const unsigned char*)p.zp)[blockk];
            }
            float s = ld<SDT>(p.scales, blockk);
            st<SDT>(p.y, i, (float)(q - z) * s);
        }
    }
}

void emit_dequantize(Emitter& em, const TRef& q, const TRef& scales, const TRef* zp, const TRef& y, int64_t block_size) {
    DequantP p{};
    p.n = y.numel();
    p.block_size = block_size;
    p.default_zp = q.dtype == DT_I4 ? 0 : (q.dtype == DT_U4 ? 8 : 128);
    dim3 g(grid_for((p.n + 7) / 8, 256)), b(256);
    Buf zb = zp ? zp->buf : Buf{kSlotNull, 0};
#define CALL(Q, S) \
    em.launch(prim_dequantize<Q, S>, g, b, 0, p, {{&p.q, q.buf}, {&p.scales, scales.buf}, {&p.zp, zb}, {&p.y, y.buf}}, "prim_dequantize")
    if (scales.dtype == DT_F32) {
        if (q.dtype == DT_U4) CALL(DT_U4, DT_F32);
        else if (q.dtype == DT_I4) CALL(DT_I4, DT_F32);
        else CALL(DT_U8, DT_F32);
    } else {
        if (q.dtype == DT_U4) CALL(DT_U4, DT_F16);
        else if (q.dtype == DT_I4) CALL(DT_I4, DT_F16);
        else CALL(DT_U8, DT_F16);
    }
#undef CALL
}

}  // namespace oxk
