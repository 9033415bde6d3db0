// Element-wise primitives: Unary, Binary, Compare, Select, Cast, Iota, DimValues.
// Semantics follow the interpreter's scalar rules
// (crates/onyxia-ir/src/interp.rs:513-573, 842-958, 142-259).
#include "common.cuh"
#include "kernels.hpp"

namespace oxk {

// ───────────────────────────── Unary ────────────────────────────────────
enum { U_NEG = 0, U_ABS, U_SQRT, U_RSQRT, U_EXP, U_LOG, U_SIN, U_COS, U_TANH, U_ERF, U_FLOOR, U_CEIL, U_NOT };

// Abramowitz–Stegun 7.1.26, the interpreter's erf (interp.rs:860-872).
__device__ __forceinline__ double erf_as(double x) {
    double sign = x < 0.0 ? -1.0 : 1.0;
    x = fabs(x);
    double t = 1.0 / (1.0 + 0.3275911 * x);
    double y = 1.0 - (((((1.061405429 * t - 1.453152027) * t) + 1.421413741) * t - 0.284496736) * t + 0.254829592) * t *
                         exp(-x * x);
    return sign * y;
}

// Correctly rounded basic ops stay in f32 (identical to f64-then-round);
// everything else is evaluated in f64 like the interpreter.
__device__ __forceinline__ float unary_f(int op, float a) {
    switch (op) {
        case U_NEG: return -a;
        case U_ABS: return fabsf(a);
        case U_SQRT: return sqrtf(a);
        case U_RSQRT: return (float)(1.0 / sqrt((double)a));
        case U_EXP: return (float)exp((double)a);
        case U_LOG: return (float)log((double)a);
        case U_SIN: return (float)sin((double)a);
        case U_COS: return (float)cos((double)a);
        case U_TANH: return (float)tanh((double)a);
        case U_ERF: return (float)erf_as((double)a);
        case U_FLOOR: return floorf(a);
        case U_CEIL: return ceilf(a);
    }
    return a;
}
// For f16 results the f64 value must be rounded to f16 in one step.
__device__ __forceinline__ __half unary_h(int op, float a) {
    switch (op) {
        case U_RSQRT: return __double2half(1.0 / sqrt((double)a));
        case U_EXP: return __double2half(exp((double)a));
        case U_LOG: return __double2half(log((double)a));
        case U_SIN: return __double2half(sin((double)a));
        case U_COS: return __double2half(cos((double)a));
        case U_TANH: return __double2half(tanh((double)a));
        case U_ERF: return __double2half(erf_as((double)a));
        default: return __float2half_rn(unary_f(op, a));
    }
}

struct UnaryP {
    const void* x;
    void* y;
    long long n;
    int op;
};

template <int DT> __global__ void prim_unary(const UnaryP p) {
    for (long long i = global_tid(); i < p.n; i += global_threads()) {
        if constexpr (DT == DT_F32) {
            st<DT>(p.y, i, unary_f(p.op, ld<DT>(p.x, i)));
        } else if constexpr (DT == DT_F16) {
            ((__half*)p.y)[i] = unary_h(p.op, ld<DT>(p.x, i));
        } else if constexpr (DT == DT_BOOL) {
            st<DT>(p.y, i, !ld<DT>(p.x, i));
        } else {
            long long a = ld<DT>(p.x, i);
            unsigned long long neg = 0ull - (unsigned long long)a;
            long long r = p.op == U_NEG ? (long long)neg : (a < 0 ? (long long)neg : a);
            st<DT>(p.y, i, r);
        }
    }
}

#define OX_DISPATCH_DT(dt, CALL)                      \
    switch (dt) {                                     \
        case DT_F32: { CALL(DT_F32); break; }         \
        case DT_F16: { CALL(DT_F16); break; }         \
        case DT_I64: { CALL(DT_I64); break; }         \
        case DT_I32: { CALL(DT_I32); break; }         \
        case DT_U32: { CALL(DT_U32); break; }         \
        case DT_U8: { CALL(DT_U8); break; }           \
        case DT_I8: { CALL(DT_I8); break; }           \
        case DT_BOOL: { CALL(DT_BOOL); break; }       \
        default: throw std::runtime_error("element-wise kernel: packed dtype"); \
    }

void emit_unary(Emitter& em, int op, const TRef& x, const TRef& y) {
    UnaryP p{};
    p.n = y.numel();
    p.op = op;
    dim3 g(grid_for(p.n, 256)), b(256);
#define CALL(DT) em.launch(prim_unary<DT>, g, b, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}}, "prim_unary")
    OX_DISPATCH_DT(x.dtype, CALL)
#undef CALL
}

// ───────────────────────────── Binary / Compare ─────────────────────────
enum { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_POW, B_MAX, B_MIN, B_AND, B_OR, B_XOR };
enum { C_EQ = 0, C_NE, C_LT, C_LE, C_GT, C_GE };

struct BinaryP {
    const void* a;
    const void* b;
    void* y;
    ErrWord* err;
    long long n;
    int op;
    int node;
    int contiguous;  // both operands have the output's shape
    NdShape shp;
    NdStride sa, sb;
};

__device__ __forceinline__ float binary_f(int op, float x, float y) {
    switch (op) {
        case B_ADD: return x + y;
        case B_SUB: return x - y;
        case B_MUL: return x * y;
        case B_DIV: return x / y;
        case B_POW: return (float)pow((double)x, (double)y);
        case B_MAX: return fmaxf(x, y);  // the non-NaN operand wins, like f64::max
        case B_MIN: return fminf(x, y);
    }
    return x;
}

__device__ __forceinline__ long long binary_i(int op, long long x, long long y, ErrWord* err, int node) {
    unsigned long long ux = (unsigned long long)x, uy = (unsigned long long)y;
    switch (op) {
        case B_ADD: return (long long)(ux + uy);
        case B_SUB: return (long long)(ux - uy);
        case B_MUL: return (long long)(ux * uy);
        case B_DIV:
            if (y == 0) {
                report(err, ERR_INT_DIV_ZERO, node, x, 0);
                return 0;
            }
            if (x == LLONG_MIN && y == -1) return LLONG_MIN;  // wrapping_div
            return x / y;
        case B_POW: {
            if (y < 0) {
                report(err, ERR_INT_POW_NEG, node, y, 0);
                return 0;
            }
            unsigned long long acc = 1, base = ux, e = uy;
            while (e) {
                if (e & 1) acc *= base;
                base *= base;
                e >>= 1;
            }
            return (long long)acc;
        }
        case B_MAX: return x > y ? x : y;
        case B_MIN: return x < y ? x : y;
    }
    return x;
}

template <int DT> __global__ void prim_binary(const BinaryP p) {
    for (long long i = global_tid(); i < p.n; i += global_threads()) {
        long long ia = i, ib = i;
        if (!p.contiguous) {
            ia = nd_offset(i, p.shp, p.sa);
            ib = nd_offset(i, p.shp, p.sb);
        }
        auto x = ld<DT>(p.a, ia);
        auto y = ld<DT>(p.b, ib);
        if constexpr (DT == DT_F32) {
            st<DT>(p.y, i, binary_f(p.op, x, y));
        } else if constexpr (DT == DT_F16) {
            if (p.op == B_POW) ((__half*)p.y)[i] = __double2half(pow((double)x, (double)y));
            else st<DT>(p.y, i, binary_f(p.op, x, y));
        } else if constexpr (DT == DT_BOOL) {
            bool r = p.op == B_AND ? (x && y) : p.op == B_OR ? (x || y) : (x != y);
            st<DT>(p.y, i, r);
        } else {
            st<DT>(p.y, i, binary_i(p.op, x, y, p.err, p.node));
        }
    }
}

template <int DT> __global__ void prim_compare(const BinaryP p) {
    for (long long i = global_tid(); i < p.n; i += global_threads()) {
        long long ia = i, ib = i;
        if (!p.contiguous) {
            ia = nd_offset(i, p.shp, p.sa);
            ib = nd_offset(i, p.shp, p.sb);
        }
        auto x = ld<DT>(p.a, ia);
        auto y = ld<DT>(p.b, ib);
        bool r;
        switch (p.op) {  // IEEE comparisons: with a NaN only != is true
            case C_EQ: r = x == y; break;
            case C_NE: r = x != y; break;
            case C_LT: r = x < y; break;
            case C_LE: r = x <= y; break;
            case C_GT: r = x > y; break;
            default: r = x >= y; break;
        }
        ((unsigned char*)p.y)[i] = r ? 1 : 0;
    }
}

// Strides of `in` over the coordinates of `out` (right-aligned, 0 where in's dim is 1).
static NdStride bcast_strides(const std::vector<int64_t>& in, const std::vector<int64_t>& out) {
    NdStride s{};
    size_t off = out.size() - in.size();
    long long run = 1;
    for (size_t i = in.size(); i-- > 0;) {
        s.s[i + off] = in[i] == 1 ? 0 : run;
        run *= in[i];
    }
    return s;
}

static NdShape nd_shape(const std::vector<int64_t>& dims) {
    if (dims.size() > (size_t)kMaxRank) throw std::runtime_error("tensor rank exceeds 8");
    NdShape s{};
    s.rank = (int)dims.size();
    for (size_t i = 0; i < dims.size(); i++) s.dim[i] = dims[i];
    return s;
}

static BinaryP binary_params(Emitter& em, int op, const TRef& a, const TRef& b, const TRef& y) {
    BinaryP p{};
    p.n = y.numel();
    p.op = op;
    p.node = em.node;
    p.contiguous = (a.shape == y.shape && b.shape == y.shape) ? 1 : 0;
    p.shp = nd_shape(y.shape);
    p.sa = bcast_strides(a.shape, y.shape);
    p.sb = bcast_strides(b.shape, y.shape);
    return p;
}

void emit_binary(Emitter& em, int op, const TRef& a, const TRef& b, const TRef& y) {
    BinaryP p = binary_params(em, op, a, b, y);
    dim3 g(grid_for(p.n, 256)), blk(256);
#define CALL(DT) \
    em.launch(prim_binary<DT>, g, blk, 0, p, {{&p.a, a.buf}, {&p.b, b.buf}, {&p.y, y.buf}, {&p.err, Buf{kSlotErr, 0}}}, "prim_binary")
    OX_DISPATCH_DT(a.dtype, CALL)
#undef CALL
}

void emit_compare(Emitter& em, int op, const TRef& a, const TRef& b, const TRef& y) {
    BinaryP p = binary_params(em, op, a, b, y);
    dim3 g(grid_for(p.n, 256)), blk(256);
#define CALL(DT) \
    em.launch(prim_compare<DT>, g, blk, 0, p, {{&p.a, a.buf}, {&p.b, b.buf}, {&p.y, y.buf}, {&p.err, Buf{kSlotErr, 0}}}, "prim_compare")
    OX_DISPATCH_DT(a.dtype, CALL)
#undef CALL
}

// ───────────────────────────── Select ───────────────────────────────────
struct SelectP {
    const unsigned char* c;
    const void* a;
    const void* b;
    void* y;
    long long n;
    NdShape shp;
    NdStride sc, sa, sb;
};

template <typename E> __global__ void prim_select(const SelectP p) {
    for (long long i = global_tid(); i < p.n; i += global_threads()) {
        bool pick = p.c[nd_offset(i, p.shp, p.sc)] != 0;
        ((E*)p.y)[i] = pick ? ((const E*)p.a)[nd_offset(i, p.shp, p.sa)] : ((const E*)p.b)[nd_offset(i, p.shp, p.sb)];
    }
}

static int elem_bytes(int dt) {
    switch (dt) {
        case DT_I64: return 8;
        case DT_F32: case DT_I32: case DT_U32: return 4;
        case DT_F16: return 2;
        case DT_U8: case DT_I8: case DT_BOOL: return 1;
    }
    throw std::runtime_error("packed dtype has no whole-byte element size");
}

void emit_select(Emitter& em, const TRef& c, const TRef& a, const TRef& b, const TRef& y) {
    SelectP p{};
    p.n = y.numel();
    p.shp = nd_shape(y.shape);
    p.sc = bcast_strides(c.shape, y.shape);
    p.sa = bcast_strides(a.shape, y.shape);
    p.sb = bcast_strides(b.shape, y.shape);
    dim3 g(grid_for(p.n, 256)), blk(256);
#define SEL(E) em.launch(prim_select<E>, g, blk, 0, p, {{&p.c, c.buf}, {&p.a, a.buf}, {&p.b, b.buf}, {&p.y, y.buf}}, "prim_select")
    switch (elem_bytes(a.dtype)) {
        case 8: SEL(unsigned long long); break;
        case 4: SEL(unsigned); break;
        case 2: SEL(unsigned short); break;
        default: SEL(unsigned char); break;
    }
#undef SEL
}

// ───────────────────────────── Cast ─────────────────────────────────────
struct CastP {
    const void* x;
    void* y;
    long long n;
};

// Rust `as i64` on a float: saturating, NaN → 0 (the hardware conversion
// saturates too but maps NaN to INT64_MIN).
__device__ __forceinline__ long long f2ll(float v) { return isnan(v) ? 0ll : (long long)v; }

// Working-domain conversion (interp.rs:210-279): float→int saturates (NaN→0)
// then wraps to the target width; int→float goes through f64; →bool is != 0.
template <int SRC, int DST> __device__ __forceinline__ void cast_one(const void* x, void* y, long long i, long long o) {
    if constexpr (SRC == DT_U4 || SRC == DT_I4) {
        long long v = SRC == DT_U4 ? ld_u4(x, i) : ld_i4(x, i);
        if constexpr (DST == DT_F32) ((float*)y)[o] = (float)v;
        else if constexpr (DST == DT_F16) ((__half*)y)[o] = __float2half_rn((float)v);
        else if constexpr (DST == DT_BOOL) ((unsigned char*)y)[o] = v != 0;
        else st<DST>(y, o, v);
    } else if constexpr (Ty<SRC>::is_float) {
        float v = ld<SRC>(x, i);
        if constexpr (DST == DT_F32) ((float*)y)[o] = v;
        else if constexpr (DST == DT_F16) ((__half*)y)[o] = __float2half_rn(v);
        else if constexpr (DST == DT_BOOL) ((unsigned char*)y)[o] = (v != 0.0f) ? 1 : 0;
        else st<DST>(y, o, f2ll(v));
    } else if constexpr (SRC == DT_BOOL) {
        bool v = ld<SRC>(x, i);
        if constexpr (DST == DT_F32) ((float*)y)[o] = v ? 1.f : 0.f;
        else if constexpr (DST == DT_F16) ((__half*)y)[o] = __float2half_rn(v ? 1.f : 0.f);
        else if constexpr (DST == DT_BOOL) ((unsigned char*)y)[o] = v;
        else st<DST>(y, o, (long long)v);
    } else {
        long long v = ld<SRC>(x, i);
        if constexpr (DST == DT_F32) ((float*)y)[o] = (float)(double)v;
        else if constexpr (DST == DT_F16) ((__half*)y)[o] = __double2half((double)v);
        else if constexpr (DST == DT_BOOL) ((unsigned char*)y)[o] = v != 0;
        else st<DST>(y, o, v);
    }
}

template <int SRC, int DST> __global__ void prim_cast(const CastP p) {
    for (long long i = global_tid(); i < p.n; i += global_threads()) cast_one<SRC, DST>(p.x, p.y, i, i);
}

// Packing casts write one byte (two nibbles) per thread.
template <int SRC> __global__ void prim_cast_pack4(const CastP p) {
    long long nbytes = (p.n + 1) / 2;
    for (long long j = global_tid(); j < nbytes; j += global_threads()) {
        unsigned char out = 0;
        for (int h = 0; h < 2; h++) {
            long long i = 2 * j + h;
            if (i >= p.n) break;
            long long v;
            if constexpr (SRC == DT_U4) v = ld_u4(p.x, i);
            else if constexpr (SRC == DT_I4) v = ld_i4(p.x, i);
            else if constexpr (Ty<SRC>::is_float) v = f2ll(ld<SRC>(p.x, i));
            else v = (long long)ld<SRC>(p.x, i);
            out |= (unsigned char)(((unsigned)v & 0xF) << (4 * h));
        }
        ((unsigned char*)p.y)[j] = out;
    }
}

template <int SRC> static void emit_cast_from(Emitter& em, const TRef& x, const TRef& y, const CastP& p) {
    dim3 g(grid_for(p.n, 256)), blk(256);
#define TO(DST) em.launch(prim_cast<SRC, DST>, g, blk, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}}, "prim_cast")
    switch (y.dtype) {
        case DT_F32: TO(DT_F32); break;
        case DT_F16: TO(DT_F16); break;
        case DT_I64: TO(DT_I64); break;
        case DT_I32: TO(DT_I32); break;
        case DT_U32: TO(DT_U32); break;
        case DT_U8: TO(DT_U8); break;
        case DT_I8: TO(DT_I8); break;
        case DT_BOOL: TO(DT_BOOL); break;
        default:
            em.launch(prim_cast_pack4<SRC>, g, blk, 0, p, {{&p.x, x.buf}, {&p.y, y.buf}}, "prim_cast_pack4");
    }
#undef TO
}

void emit_cast(Emitter& em, const TRef& x, const TRef& y) {
    CastP p{};
    p.n = y.numel();
    switch (x.dtype) {
        case DT_F32: emit_cast_from<DT_F32>(em, x, y, p); break;
        case DT_F16: emit_cast_from<DT_F16>(em, x, y, p); break;
        case DT_I64: emit_cast_from<DT_I64>(em, x, y, p); break;
        case DT_I32: emit_cast_from<DT_I32>(em, x, y, p); break;
        case DT_U32: emit_cast_from<DT_U32>(em, x, y, p); break;
        case DT_U8: emit_cast_from<DT_U8>(em, x, y, p); break;
        case DT_I8: emit_cast_from<DT_I8>(em, x, y, p); break;
        case DT_BOOL: emit_cast_from<DT_BOOL>(em, x, y, p); break;
        case DT_U4: emit_cast_from<DT_U4>(em, x, y, p); break;
        case DT_I4: emit_cast_from<DT_I4>(em, x, y, p); break;
        default: throw std::runtime_error("cast: unknown dtype");
    }
}

// ───────────────────────────── Iota / DimValues ─────────────────────────
struct IotaP {
    void* y;
    long long n;
};
template <int DT> __global__ void prim_iota(const IotaP p) {
    for (long long i = global_tid(); i < p.n; i += global_threads()) {
        if constexpr (DT == DT_F32) ((float*)p.y)[i] = (float)(double)i;
        else if constexpr (DT == DT_F16) ((__half*)p.y)[i] = __double2half((double)i);
        else st<DT>(p.y, i, i);
    }
}

void emit_iota(Emitter& em, const TRef& y) {
    IotaP p{};
    p.n = y.numel();
    dim3 g(grid_for(p.n, 256)), blk(256);
#define CALL(DT) em.launch(prim_iota<DT>, g, blk, 0, p, {{&p.y, y.buf}}, "prim_iota")
    switch (y.dtype) {
        case DT_F32: CALL(DT_F32); break;
        case DT_F16: CALL(DT_F16); break;
        case DT_I64: CALL(DT_I64); break;
        case DT_I32: CALL(DT_I32); break;
        case DT_U32: CALL(DT_U32); break;
        case DT_U8: CALL(DT_U8); break;
        case DT_I8: CALL(DT_I8); break;
        default: throw std::runtime_error("iota: unsupported dtype");
    }
#undef CALL
}

constexpr int kMaxDimValues = 32;
struct DimValuesP {
    long long* y;
    int n;
    long long v[kMaxDimValues];
};
__global__ void prim_dim_values(const DimValuesP p) {
    int i = threadIdx.x;
    if (i < p.n) p.y[i] = p.v[i];
}

void emit_dim_values(Emitter& em, const std::vector<int64_t>& vals, const TRef& y) {
    if (vals.size() > (size_t)kMaxDimValues) throw std::runtime_error("dim_values: more than 32 expressions");
    DimValuesP p{};
    p.n = (int)vals.size();
    for (size_t i = 0; i < vals.size(); i++) p.v[i] = vals[i];
    em.launch(prim_dim_values, dim3(1), dim3(32), 0, p, {{&p.y, y.buf}}, "prim_dim_values");
}

}  // namespace oxk
