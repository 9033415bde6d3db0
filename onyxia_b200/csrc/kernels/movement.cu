// Data-movement primitives: Reshape (copy form), Transpose, Broadcast, Concat,
// Slice, Gather, Scatter. They move whole elements by size and never look
// inside them (crates/onyxia-ir/src/interp.rs:579-748).
#include "common.cuh"
#include "kernels.hpp"

namespace oxk {

static int elem_bytes(int dt) {
    switch (dt) {
        case DT_I64: return 8;
        case DT_F32: case DT_I32: case DT_U32: return 4;
        case DT_F16: return 2;
        case DT_U8: case DT_I8: case DT_BOOL: return 1;
    }
    throw std::runtime_error("data-movement kernel: packed dtype must be cast or dequantized first");
}

static NdShape nd_shape(const std::vector<int64_t>& dims) {
    if (dims.size() > (size_t)kMaxRank) throw std::runtime_error("tensor rank exceeds 8");
    NdShape s{};
    s.rank = (int)dims.size();
    for (size_t i = 0; i < dims.size(); i++) s.dim[i] = dims[i];
    return s;
}

static std::vector<int64_t> row_major(const std::vector<int64_t>& dims) {
    std::vector<int64_t> st(dims.size(), 1);
    for (size_t i = dims.size(); i-- > 1;) st[i - 1] = st[i] * dims[i];
    return st;
}

// y[i] = x[base + Σ coord_d · stride_d]; covers transpose, broadcast and slice.
struct StridedP {
    const void* x;
    void* y;
    long long n;
    long long base;
    NdShape shp;
    NdStride sx;
};

template <typename E> __device__ __forceinline__ void strided_body(const StridedP& p) {
    for (long long i = global_tid(); i < p.n; i += global_threads())
        ((E*)p.y)[i] = ((const E*)p.x)[p.base + nd_offset(i, p.shp, p.sx)];
}
template <typename E> __global__ void prim_transpose(const StridedP p) { strided_body<E>(p); }
template <typename E> __global__ void prim_broadcast(const StridedP p) { strided_body<E>(p); }
template <typename E> __global__ void prim_slice(const StridedP p) { strided_body<E>(p); }

struct CopyP {
    const void* x;
    void* y;
    long long nbytes;
};
__global__ void prim_reshape_copy(const CopyP p) {
    // byte copy, 16 bytes per thread where alignment allows
    long long n16 = (((uintptr_t)p.x | (uintptr_t)p.y) & 15) == 0 ? p.nbytes / 16 : 0;
    for (long long i = global_tid(); i < n16; i += global_threads()) ((uint4*)p.y)[i] = ((const uint4*)p.x)[i];
    for (long long i = n16 * 16 + global_tid(); i < p.nbytes; i += global_threads())
        ((unsigned char*)p.y)[i] = ((const unsigned char*)p.x)[i];
}

void emit_reshape_copy(Emitter& em, const TRef& x, const TRef& y) {
    CopyP p{};
    int bits = (x.dtype == DT_U4 || x.dtype == DT_I4) ? 4 : elem_bytes(x.dtype) * 8;
    p.nbytes = (x.numel() * bits + 7) / 8;
    em.launch(prim_reshape_copy, dim3(grid_for(p.nbytes / 16 + 1, 256)), dim3(256), 0, p, {{&p.x, x.buf}, {&p.y, y.buf}},
              "prim_reshape");
}

#define OX_BY_SIZE(dt, K, ...)                                            \
    switch (elem_bytes(dt)) {                                             \
        case 8: em.launch(K<unsigned long long>, __VA_ARGS__); break;     \
        case 4: em.launch(K<unsigned>, __VA_ARGS__); break;               \
        case 2: em.launch(K<unsigned short>, __VA_ARGS__); break;         \
        default: em.launch(K<unsigned char>, __VA_ARGS__); break;         \
    }

void emit_transpose(Emitter& em, const TRef& x, const TRef& y, const std::vector<size_t>& perm) {
    StridedP p{};
    p.n = y.numel();
    p.shp = nd_shape(y.shape);
    auto xs = row_major(x.shape);
    for (size_t d = 0; d < perm.size(); d++) p.sx.s[d] = xs[perm[d]];
    dim3 g(grid_for(p.n, 256)), b(256);
    OX_BY_SIZE(x.dtype, prim_transpose, g, b, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}}, "prim_transpose")
}

void emit_broadcast(Emitter& em, const TRef& x, const TRef& y) {
    StridedP p{};
    p.n = y.numel();
    p.shp = nd_shape(y.shape);
    size_t off = y.shape.size() - x.shape.size();
    auto xs = row_major(x.shape);
    for (size_t d = 0; d < x.shape.size(); d++) p.sx.s[d + off] = x.shape[d] == 1 ? 0 : xs[d];
    dim3 g(grid_for(p.n, 256)), b(256);
    OX_BY_SIZE(x.dtype, prim_broadcast, g, b, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}}, "prim_broadcast")
}

void emit_slice(Emitter& em, const TRef& x, const TRef& y, const std::vector<int64_t>& starts,
                const std::vector<int64_t>& steps) {
    StridedP p{};
    p.n = y.numel();
    p.shp = nd_shape(y.shape);
    auto xs = row_major(x.shape);
    for (size_t d = 0; d < x.shape.size(); d++) {
        p.base += starts[d] * xs[d];
        p.sx.s[d] = steps[d] * xs[d];
    }
    dim3 g(grid_for(p.n, 256)), b(256);
    OX_BY_SIZE(x.dtype, prim_slice, g, b, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}}, "prim_slice")
}

// ───────────────────────────── Concat ───────────────────────────────────
// One launch per input: its [outer, len·inner] block lands at column offset
// `off·inner` of the output's [outer, total·inner] view.
struct ConcatP {
    const void* x;
    void* y;
    long long n;          // elements of this input
    long long in_row;     // len·inner
    long long out_row;    // total·inner
    long long out_off;    // off·inner
};
template <typename E> __global__ void prim_concat(const ConcatP p) {
    for (long long i = global_tid(); i < p.n; i += global_threads()) {
        long long o = i / p.in_row, r = i % p.in_row;
        ((E*)p.y)[o * p.out_row + p.out_off + r] = ((const E*)p.x)[i];
    }
}

void emit_concat(Emitter& em, const std::vector<TRef>& xs, const TRef& y, size_t axis) {
    long long inner = 1;
    for (size_t d = axis + 1; d < y.shape.size(); d++) inner *= y.shape[d];
    long long total = y.shape[axis], off = 0;
    for (auto& x : xs) {
        ConcatP p{};
        p.n = x.numel();
        p.in_row = x.shape[axis] * inner;
        p.out_row = total * inner;
        p.out_off = off * inner;
        off += x.shape[axis];
        if (p.n == 0) continue;
        dim3 g(grid_for(p.n, 256)), b(256);
        OX_BY_SIZE(y.dtype, prim_concat, g, b, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}}, "prim_concat")
    }
}

// ───────────────────────────── Gather ───────────────────────────────────
struct GatherP {
    const void* data;
    const long long* idx;
    void* y;
    ErrWord* err;
    long long n, inner, ni, dim;
    int node;
};
template <typename E> __global__ void prim_gather(const GatherP p) {
    for (long long i = global_tid(); i < p.n; i += global_threads()) {
        long long r = i % p.inner, ii = (i / p.inner) % p.ni, o = i / (p.inner * p.ni);
        long long raw = p.idx[ii];
        if (raw < 0) raw += p.dim;
        if (raw < 0 || raw >= p.dim) {  // the interpreter reports this (interp.rs:702-706)
            report(p.err, ERR_GATHER_OOB, p.node, raw, p.dim);
            ((E*)p.y)[i] = 0;
            continue;
        }
        ((E*)p.y)[i] = ((const E*)p.data)[(o * p.dim + raw) * p.inner + r];
    }
}

void emit_gather(Emitter& em, const TRef& data, const TRef& idx, const TRef& y, size_t axis) {
    GatherP p{};
    p.n = y.numel();
    p.inner = 1;
    for (size_t d = axis + 1; d < data.shape.size(); d++) p.inner *= data.shape[d];
    p.ni = idx.numel();
    p.dim = data.shape[axis];
    p.node = em.node;
    dim3 g(grid_for(p.n, 256)), b(256);
    OX_BY_SIZE(data.dtype, prim_gather, g, b, 0, p,
               {{&p.data, data.buf}, {&p.idx, idx.buf}, {&p.y, y.buf}, {&p.err, Buf{kSlotErr, 0}}}, "prim_gather")
}

// ───────────────────────────── Scatter ──────────────────────────────────
// Copy, then apply updates. Duplicate targets: the last update wins
// (interp.rs:726-747). Each thread owns one position j of the update slice and
// walks the updates in order, so the result does not depend on scheduling.
struct ScatterP {
    const long long* idx;
    const void* upd;
    void* y;
    ErrWord* err;
    long long num_updates, slice_len;
    int k;
    int node;
    long long dims[kMaxRank];
};
template <typename E> __global__ void prim_scatter(const ScatterP p) {
    for (long long j = global_tid(); j < p.slice_len; j += global_threads()) {
        for (long long u = 0; u < p.num_updates; u++) {
            long long base = 0;
            bool ok = true;
            for (int d = 0; d < p.k; d++) {
                long long raw = p.idx[u * p.k + d];
                if (raw < 0) raw += p.dims[d];
                if (raw < 0 || raw >= p.dims[d]) {
                    report(p.err, ERR_SCATTER_OOB, p.node, raw, p.dims[d]);
                    ok = false;
                    break;
                }
                base = base * p.dims[d] + raw;
            }
            if (ok) ((E*)p.y)[base * p.slice_len + j] = ((const E*)p.upd)[u * p.slice_len + j];
        }
    }
}

void emit_scatter(Emitter& em, const TRef& data, const TRef& idx, const TRef& upd, const TRef& y) {
    emit_reshape_copy(em, data, y);
    em.recs.back().label = "prim_scatter_copy";
    ScatterP p{};
    p.k = (int)idx.shape.back();
    p.num_updates = idx.numel() / (p.k > 0 ? p.k : 1);
    p.slice_len = 1;
    for (size_t d = p.k; d < data.shape.size(); d++) p.slice_len *= data.shape[d];
    for (int d = 0; d < p.k; d++) p.dims[d] = data.shape[d];
    p.node = em.node;
    if (p.num_updates == 0 || p.slice_len == 0) return;
    dim3 g(grid_for(p.slice_len, 128)), b(128);
    OX_BY_SIZE(data.dtype, prim_scatter, g, b, 0, p,
               {{&p.idx, idx.buf}, {&p.upd, upd.buf}, {&p.y, y.buf}, {&p.err, Buf{kSlotErr, 0}}}, "prim_scatter")
}

}  // namespace oxk
