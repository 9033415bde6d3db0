// TEST INFRASTRUCTURE — CPU oracle (see interp.hpp). Each function names the
// part of crates/onyxia-ir/src/interp.rs it restates.
#include "interp.hpp"

#include <omp.h>

#include <cmath>
#include <cstring>
#include <limits>

#if defined(__F16C__)
#include <immintrin.h>
#endif

namespace oxref {

using namespace ox;

static int g_threads = 1;
void set_threads(int n) { g_threads = n < 1 ? 1 : n; }
int get_threads() { return g_threads; }
// Parallelise a loop only when it is worth a fork.
#define OXREF_PAR(n) if ((n) > 4096 && g_threads > 1) num_threads(g_threads)

// ───────────────────────────── Tensor ──────────────────────────────────
Tensor Tensor::alloc(DType dt, std::vector<size_t> shape) {
    Tensor t;
    t.dtype = dt;
    t.shape = std::move(shape);
    t.own = std::make_shared<std::vector<uint8_t>>(t.nbytes(), 0);
    t.data = t.own->data();
    return t;
}

Tensor Tensor::from_bytes(DType dt, std::vector<size_t> shape, const void* bytes, size_t nbytes) {
    Tensor t;
    t.dtype = dt;
    t.shape = std::move(shape);
    size_t expect = t.nbytes();
    if (nbytes != expect)
        fail(ErrKind::Interp, "tensor data size mismatch: " + std::to_string(nbytes) + " bytes for " + dtype_name(dt) +
                                  " (expected " + std::to_string(expect) + ")");
    t.own = std::make_shared<std::vector<uint8_t>>((const uint8_t*)bytes, (const uint8_t*)bytes + nbytes);
    t.data = t.own->data();
    return t;
}

Tensor Tensor::view(DType dt, std::vector<size_t> shape, const uint8_t* bytes) {
    Tensor t;
    t.dtype = dt;
    t.shape = std::move(shape);
    t.data = bytes;
    return t;
}

// ─────────────── working-domain loads / stores (interp.rs:142-279) ─────
enum class Dom { F, I, B };
static Dom dom_of(DType d) { return dtype_is_float(d) ? Dom::F : (d == DType::Bool ? Dom::B : Dom::I); }

static inline double f16_to_f64_fast(uint16_t h) {
#if defined(__F16C__)
    return (double)_cvtsh_ss(h);
#else
    return f16_bits_to_f64(h);
#endif
}

static inline double ld_f(const Tensor& t, size_t i) {
    if (t.dtype == DType::F32) {
        float v;
        std::memcpy(&v, t.data + 4 * i, 4);
        return (double)v;
    }
    uint16_t h;
    std::memcpy(&h, t.data + 2 * i, 2);
    return f16_to_f64_fast(h);
}

static inline int64_t ld_i(const Tensor& t, size_t i) {
    switch (t.dtype) {
        case DType::I64: { int64_t v; std::memcpy(&v, t.data + 8 * i, 8); return v; }
        case DType::I32: { int32_t v; std::memcpy(&v, t.data + 4 * i, 4); return v; }
        case DType::U32: { uint32_t v; std::memcpy(&v, t.data + 4 * i, 4); return (int64_t)v; }
        case DType::U8: return (int64_t)t.data[i];
        case DType::I8: return (int64_t)(int8_t)t.data[i];
        case DType::U4: return (int64_t)((t.data[i / 2] >> ((i % 2) * 4)) & 0xF);
        case DType::I4: {
            uint8_t nib = (t.data[i / 2] >> ((i % 2) * 4)) & 0xF;
            return (int64_t)((int8_t)(nib << 4) >> 4);  // sign-extend from 4 bits
        }
        default: fail(ErrKind::Interp, std::string(dtype_name(t.dtype)) + " is not an int tensor");
    }
}

static inline bool ld_b(const Tensor& t, size_t i) { return t.data[i] != 0; }

// Rust `f64 as i64`: saturating, NaN → 0.
static inline int64_t f64_as_i64(double x) {
    if (std::isnan(x)) return 0;
    if (x >= 9223372036854775808.0) return INT64_MAX;
    if (x <= -9223372036854775808.0) return INT64_MIN;
    return (int64_t)x;
}

// One scalar of the working domain.
struct Scalar {
    Dom dom;
    double f;
    int64_t i;
    bool b;
};
static inline Scalar SF(double v) { return Scalar{Dom::F, v, 0, false}; }
static inline Scalar SI(int64_t v) { return Scalar{Dom::I, 0, v, false}; }
static inline Scalar SB(bool v) { return Scalar{Dom::B, 0, 0, v}; }

static inline Scalar ld(const Tensor& t, size_t i) {
    switch (dom_of(t.dtype)) {
        case Dom::F: return SF(ld_f(t, i));
        case Dom::I: return SI(ld_i(t, i));
        default: return SB(ld_b(t, i));
    }
}

static inline double as_f(const Scalar& s) { return s.dom == Dom::F ? s.f : s.dom == Dom::I ? (double)s.i : (s.b ? 1.0 : 0.0); }
static inline int64_t as_i(const Scalar& s) { return s.dom == Dom::F ? f64_as_i64(s.f) : s.dom == Dom::I ? s.i : (int64_t)s.b; }

// Values::encode for one element (interp.rs:214-259). Packed nibbles are OR-ed
// into zero-initialised storage, so concurrent writers must not share a byte.
static inline void st(uint8_t* data, DType dt, size_t i, const Scalar& s) {
    switch (dt) {
        case DType::F32: { float v = (float)as_f(s); std::memcpy(data + 4 * i, &v, 4); break; }
        case DType::F16: { uint16_t h = f64_to_f16_bits(as_f(s)); std::memcpy(data + 2 * i, &h, 2); break; }
        case DType::I64: { int64_t v = as_i(s); std::memcpy(data + 8 * i, &v, 8); break; }
        case DType::I32: { int32_t v = (int32_t)(uint32_t)(uint64_t)as_i(s); std::memcpy(data + 4 * i, &v, 4); break; }
        case DType::U32: { uint32_t v = (uint32_t)(uint64_t)as_i(s); std::memcpy(data + 4 * i, &v, 4); break; }
        case DType::U8: data[i] = (uint8_t)(uint64_t)as_i(s); break;
        case DType::I8: data[i] = (uint8_t)(uint64_t)as_i(s); break;
        case DType::Bool:
            data[i] = s.dom == Dom::B ? (uint8_t)s.b : s.dom == Dom::F ? (uint8_t)(s.f != 0.0) : (uint8_t)(s.i != 0);
            break;
        case DType::U4: case DType::I4: {
            uint8_t nib = (uint8_t)(uint64_t)as_i(s) & 0xF;
            data[i / 2] |= (uint8_t)(nib << ((i % 2) * 4));
            break;
        }
    }
}

// Raw element moves for the data-movement primitives. The reference moves
// values through its working domain and re-encodes them in the same dtype,
// which preserves every bit pattern except NaN payloads.
static inline uint64_t ld_raw(const Tensor& t, size_t i) {
    switch (dtype_bits(t.dtype)) {
        case 64: { uint64_t v; std::memcpy(&v, t.data + 8 * i, 8); return v; }
        case 32: { uint32_t v; std::memcpy(&v, t.data + 4 * i, 4); return v; }
        case 16: { uint16_t v; std::memcpy(&v, t.data + 2 * i, 2); return v; }
        case 8: return t.data[i];
        default: return (t.data[i / 2] >> ((i % 2) * 4)) & 0xF;
    }
}
static inline void st_raw(uint8_t* data, DType dt, size_t i, uint64_t v) {
    switch (dtype_bits(dt)) {
        case 64: std::memcpy(data + 8 * i, &v, 8); break;
        case 32: { uint32_t x = (uint32_t)v; std::memcpy(data + 4 * i, &x, 4); break; }
        case 16: { uint16_t x = (uint16_t)v; std::memcpy(data + 2 * i, &x, 2); break; }
        case 8: data[i] = (uint8_t)v; break;
        default: data[i / 2] |= (uint8_t)((v & 0xF) << ((i % 2) * 4)); break;
    }
}

// ─────────────── shape / index helpers (interp.rs:283-331) ─────────────
static std::vector<size_t> broadcast_shape(const std::vector<size_t>& a, const std::vector<size_t>& b) {
    size_t rank = std::max(a.size(), b.size());
    std::vector<size_t> out;
    for (size_t i = 0; i < rank; i++) {
        size_t da = (i + a.size() >= rank) ? a[i + a.size() - rank] : 1;
        size_t db = (i + b.size() >= rank) ? b[i + b.size() - rank] : 1;
        // a size-1 dim stretches to the other side, including to 0
        if (da == db || db == 1) out.push_back(da);
        else if (da == 1) out.push_back(db);
        else fail(ErrKind::Interp, "cannot broadcast shapes");
    }
    return out;
}

static size_t prod(const std::vector<size_t>& s, size_t from = 0, size_t to = SIZE_MAX) {
    if (to > s.size()) to = s.size();
    size_t n = 1;
    for (size_t i = from; i < to; i++) n *= s[i];
    return n;
}

static std::vector<size_t> row_major_strides(const std::vector<size_t>& shape) {
    std::vector<size_t> st(shape.size(), 1);
    for (size_t i = shape.size(); i-- > 1;) st[i - 1] = st[i] * shape[i];
    return st;
}

// Strides of `in_shape` expressed over `out_shape` coordinates, right-aligned,
// 0 where the input dim is 1 (broadcast_index, interp.rs:301-309).
static std::vector<size_t> bcast_strides(const std::vector<size_t>& in_shape, const std::vector<size_t>& out_shape) {
    std::vector<size_t> st(out_shape.size(), 0);
    auto rs = row_major_strides(in_shape);
    size_t off = out_shape.size() - in_shape.size();
    for (size_t i = 0; i < in_shape.size(); i++) st[i + off] = in_shape[i] == 1 ? 0 : rs[i];
    return st;
}

static inline size_t map_index(size_t linear, const std::vector<size_t>& out_shape, const std::vector<size_t>& strides) {
    size_t idx = 0;
    for (size_t d = out_shape.size(); d-- > 0;) {
        size_t c = linear % out_shape[d];
        linear /= out_shape[d];
        idx += c * strides[d];
    }
    return idx;
}

// ─────────────── scalar semantics (interp.rs:842-939) ──────────────────
static double erf_as(double x) {  // Abramowitz–Stegun 7.1.26 (interp.rs:860-872)
    double sign = x < 0.0 ? -1.0 : 1.0;
    x = std::fabs(x);
    double t = 1.0 / (1.0 + 0.3275911 * x);
    double y = 1.0 - (((((1.061405429 * t - 1.453152027) * t) + 1.421413741) * t - 0.284496736) * t + 0.254829592) * t *
                         std::exp(-x * x);
    return sign * y;
}

static double unary_f(UnaryOp op, double a) {
    switch (op) {
        case UnaryOp::Neg: return -a;
        case UnaryOp::Abs: return std::fabs(a);
        case UnaryOp::Sqrt: return std::sqrt(a);
        case UnaryOp::Rsqrt: return 1.0 / std::sqrt(a);
        case UnaryOp::Exp: return std::exp(a);
        case UnaryOp::Log: return std::log(a);
        case UnaryOp::Sin: return std::sin(a);
        case UnaryOp::Cos: return std::cos(a);
        case UnaryOp::Tanh: return std::tanh(a);
        case UnaryOp::Erf: return erf_as(a);
        case UnaryOp::Floor: return std::floor(a);
        case UnaryOp::Ceil: return std::ceil(a);
        default: fail(ErrKind::Interp, "unary op on the wrong domain");
    }
}

static inline int64_t wadd(int64_t a, int64_t b) { return (int64_t)((uint64_t)a + (uint64_t)b); }
static inline int64_t wsub(int64_t a, int64_t b) { return (int64_t)((uint64_t)a - (uint64_t)b); }
static inline int64_t wmul(int64_t a, int64_t b) { return (int64_t)((uint64_t)a * (uint64_t)b); }

static Scalar binary_val(BinaryOp op, const Scalar& a, const Scalar& b) {
    if (a.dom == Dom::F) {
        double x = a.f, y = b.f;
        switch (op) {
            case BinaryOp::Add: return SF(x + y);
            case BinaryOp::Sub: return SF(x - y);
            case BinaryOp::Mul: return SF(x * y);
            case BinaryOp::Div: return SF(x / y);
            case BinaryOp::Pow: return SF(std::pow(x, y));
            case BinaryOp::Max: return SF(std::fmax(x, y));  // non-NaN operand wins, like f64::max
            case BinaryOp::Min: return SF(std::fmin(x, y));
            default: fail(ErrKind::Interp, "bool op on floats");
        }
    }
    if (a.dom == Dom::I) {
        int64_t x = a.i, y = b.i;
        switch (op) {
            case BinaryOp::Add: return SI(wadd(x, y));
            case BinaryOp::Sub: return SI(wsub(x, y));
            case BinaryOp::Mul: return SI(wmul(x, y));
            case BinaryOp::Div:
                if (y == 0) fail(ErrKind::Interp, "integer division by zero");
                if (x == INT64_MIN && y == -1) return SI(INT64_MIN);  // wrapping_div
                return SI(x / y);
            case BinaryOp::Pow: {
                if (y < 0) fail(ErrKind::Interp, "integer pow with negative exponent");
                // repeated wrapping multiplication == square-and-multiply mod 2^64
                int64_t acc = 1, base = x;
                uint64_t e = (uint64_t)y;
                while (e) {
                    if (e & 1) acc = wmul(acc, base);
                    base = wmul(base, base);
                    e >>= 1;
                }
                return SI(acc);
            }
            case BinaryOp::Max: return SI(std::max(x, y));
            case BinaryOp::Min: return SI(std::min(x, y));
            default: fail(ErrKind::Interp, "bool op on ints");
        }
    }
    switch (op) {
        case BinaryOp::And: return SB(a.b && b.b);
        case BinaryOp::Or: return SB(a.b || b.b);
        case BinaryOp::Xor: return SB(a.b != b.b);
        default: fail(ErrKind::Interp, "numeric op on bools");
    }
}

static bool compare_val(CmpOp op, const Scalar& a, const Scalar& b) {
    int ord;  // -1, 0, 1, or 2 = unordered
    if (a.dom == Dom::F) {
        if (std::isnan(a.f) || std::isnan(b.f)) ord = 2;
        else ord = a.f < b.f ? -1 : (a.f > b.f ? 1 : 0);
    } else if (a.dom == Dom::I) {
        ord = a.i < b.i ? -1 : (a.i > b.i ? 1 : 0);
    } else {
        ord = (int)a.b - (int)b.b;
    }
    if (ord == 2) return op == CmpOp::Ne;  // NaN: only Ne is true
    switch (op) {
        case CmpOp::Eq: return ord == 0;
        case CmpOp::Ne: return ord != 0;
        case CmpOp::Lt: return ord < 0;
        case CmpOp::Le: return ord <= 0;
        case CmpOp::Gt: return ord > 0;
        case CmpOp::Ge: return ord >= 0;
    }
    return false;
}

// Errors raised inside OpenMP regions are carried out through this.
struct ParError {
    bool set = false;
    ErrKind kind = ErrKind::Interp;
    std::string msg;
    void capture(const Error& e) {
#pragma omp critical(oxref_err)
        if (!set) {
            set = true;
            kind = e.kind;
            msg = e.detail;
        }
    }
    void rethrow() const {
        if (set) fail(kind, msg);
    }
};

// ─────────────── dequantisation (interp.rs:764-797) ────────────────────
static inline int64_t default_zp(DType d) { return d == DType::I4 ? 0 : (int64_t)1 << (dtype_bits(d) - 1); }

// Round an f64 to the scales' dtype and return it widened back to f64.
static inline double round_to(DType dt, double v) {
    if (dt == DType::F32) return (double)(float)v;
    return f16_bits_to_f64(f64_to_f16_bits(v));
}

// One dequantised row segment [start, start+count) of the flattened tensor,
// already rounded to the scales' dtype, widened to f64.
static void dequant_range(const LazyDequant& lz, size_t start, size_t count, double* out) {
    const Tensor &q = lz.q, &s = lz.scales;
    int64_t dz = default_zp(q.dtype);
    bool f16 = s.dtype == DType::F16;
    for (size_t j = 0; j < count; j++) {
        size_t i = start + j;
        size_t block = i / lz.block_size;
        int64_t z = lz.has_zp ? ld_i(lz.zp, block) : dz;
        int64_t d = ld_i(q, i) - z;
#if defined(__F16C__)
        if (f16 && d > -2048 && d < 2048) {
            // (q − zp)·s has ≤ 11+11 significant bits: exact in f32, so one
            // hardware f32→f16 rounding equals the direct f64→f16 rounding.
            uint16_t hs;
            std::memcpy(&hs, s.data + 2 * block, 2);
            float p = (float)d * _cvtsh_ss(hs);
            out[j] = (double)_cvtsh_ss(_cvtss_sh(p, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
            continue;
        }
#endif
        (void)f16;
        out[j] = round_to(s.dtype, (double)d * ld_f(s, block));
    }
}

void materialize(Tensor& t) {
    if (!t.lazy) return;
    std::shared_ptr<LazyDequant> lz = t.lazy;
    size_t n = t.numel();
    Tensor out = Tensor::alloc(t.dtype, t.shape);
    uint8_t* dst = out.mut();
    const size_t chunk = 4096;
    size_t chunks = (n + chunk - 1) / chunk;
#pragma omp parallel for schedule(static) OXREF_PAR(n)
    for (size_t c = 0; c < chunks; c++) {
        double buf[chunk];
        size_t start = c * chunk, cnt = std::min(chunk, n - start);
        dequant_range(*lz, start, cnt, buf);
        for (size_t j = 0; j < cnt; j++) st(dst, out.dtype, start + j, SF(buf[j]));
    }
    t = out;
}

// ─────────────── matmul (interp.rs:960-1029) ───────────────────────────
static Tensor matmul(const Tensor& a_in, const Tensor& b_in, bool ta, bool tb) {
    Tensor a = a_in, b = b_in;
    materialize(a);
    size_t ar = a.shape.size(), br = b.shape.size();
    size_t m = ta ? a.shape[ar - 1] : a.shape[ar - 2];
    size_t ka = ta ? a.shape[ar - 2] : a.shape[ar - 1];
    size_t kb = tb ? b.shape[br - 1] : b.shape[br - 2];
    size_t n = tb ? b.shape[br - 2] : b.shape[br - 1];
    if (ka != kb) fail(ErrKind::Interp, "matmul contraction mismatch: " + std::to_string(ka) + " vs " + std::to_string(kb));
    std::vector<size_t> a_batch(a.shape.begin(), a.shape.end() - 2), b_batch(b.shape.begin(), b.shape.end() - 2);
    std::vector<size_t> batch = broadcast_shape(a_batch, b_batch);
    std::vector<size_t> out_shape = batch;
    out_shape.push_back(m);
    out_shape.push_back(n);
    size_t nb = prod(batch);
    auto a_bs = bcast_strides(a_batch, batch), b_bs = bcast_strides(b_batch, batch);
    size_t a_mat = m * ka, b_mat = kb * n;
    Tensor out = Tensor::alloc(a.dtype, out_shape);
    uint8_t* dst = out.mut();
    bool is_float = dtype_is_float(a.dtype);

    if (!is_float) {
        materialize(b);
        for (size_t bi = 0; bi < nb; bi++) {
            size_t a_base = map_index(bi, batch, a_bs) * a_mat, b_base = map_index(bi, batch, b_bs) * b_mat;
            for (size_t i = 0; i < m; i++)
                for (size_t j = 0; j < n; j++) {
                    int64_t acc = 0;
                    for (size_t kk = 0; kk < ka; kk++) {
                        int64_t x = ld_i(a, a_base + (ta ? kk * m + i : i * ka + kk));
                        int64_t y = ld_i(b, b_base + (tb ? j * kb + kk : kk * n + j));
                        acc = wadd(acc, wmul(x, y));
                    }
                    st(dst, out.dtype, (bi * m + i) * n + j, SI(acc));
                }
        }
        return out;
    }

    // Float path: A widened to f64 once (activations are small); B read row by
    // row. Accumulation is f64 in k order for every output, as in the
    // reference, whatever the loop nest around it.
    size_t a_elems = a.numel();
    std::vector<double> fa(a_elems);
#pragma omp parallel for schedule(static) OXREF_PAR(a_elems)
    for (size_t i = 0; i < a_elems; i++) fa[i] = ld_f(a, i);

    if (b.lazy && !(tb && br == 2)) materialize(b);
    if (tb) {
        // B is [.., N, K]: one contiguous K-row per output column.
        for (size_t bi = 0; bi < nb; bi++) {
            size_t a_base = map_index(bi, batch, a_bs) * a_mat, b_base = map_index(bi, batch, b_bs) * b_mat;
#pragma omp parallel OXREF_PAR(n * ka * m)
            {
                std::vector<double> row(kb);
#pragma omp for schedule(static)
                for (size_t j = 0; j < n; j++) {
                    if (b.lazy) dequant_range(*b.lazy, b_base + j * kb, kb, row.data());
                    else
                        for (size_t kk = 0; kk < kb; kk++) row[kk] = ld_f(b, b_base + j * kb + kk);
                    for (size_t i = 0; i < m; i++) {
                        double acc = 0.0;
                        if (ta)
                            for (size_t kk = 0; kk < ka; kk++) acc += fa[a_base + kk * m + i] * row[kk];
                        else {
                            const double* ap = &fa[a_base + i * ka];
                            for (size_t kk = 0; kk < ka; kk++) acc += ap[kk] * row[kk];
                        }
                        st(dst, out.dtype, (bi * m + i) * n + j, SF(acc));
                    }
                }
            }
        }
    } else {
        size_t b_elems = b.numel();
        std::vector<double> fb(b_elems);
#pragma omp parallel for schedule(static) OXREF_PAR(b_elems)
        for (size_t i = 0; i < b_elems; i++) fb[i] = ld_f(b, i);
        for (size_t bi = 0; bi < nb; bi++) {
            size_t a_base = map_index(bi, batch, a_bs) * a_mat, b_base = map_index(bi, batch, b_bs) * b_mat;
#pragma omp parallel for schedule(static) OXREF_PAR(m * n * ka)
            for (size_t ij = 0; ij < m * n; ij++) {
                size_t i = ij / n, j = ij % n;
                double acc = 0.0;
                for (size_t kk = 0; kk < ka; kk++)
                    acc += fa[a_base + (ta ? kk * m + i : i * ka + kk)] * fb[b_base + kk * n + j];
                st(dst, out.dtype, (bi * m + i) * n + j, SF(acc));
            }
        }
    }
    return out;
}

// ─────────────── reduce (interp.rs:1031-1125) ──────────────────────────
static Tensor reduce(const Tensor& x, ReduceOp op, const std::vector<size_t>& axes, bool keepdims) {
    const auto& in_shape = x.shape;
    size_t rank = in_shape.size();
    std::vector<char> is_red(rank, 0);
    for (auto a : axes) is_red[a] = 1;
    std::vector<size_t> out_shape, kept_dims, red_dims, kept_str, red_str;
    auto in_str = row_major_strides(in_shape);
    size_t count = 1;
    for (size_t i = 0; i < rank; i++) {
        if (is_red[i]) {
            if (keepdims) out_shape.push_back(1);
            red_dims.push_back(in_shape[i]);
            red_str.push_back(in_str[i]);
            count *= in_shape[i];
        } else {
            out_shape.push_back(in_shape[i]);
            kept_dims.push_back(in_shape[i]);
            kept_str.push_back(in_str[i]);
        }
    }
    size_t out_n = prod(kept_dims);
    Tensor out = Tensor::alloc(x.dtype, out_shape);
    uint8_t* dst = out.mut();
    bool is_float = dtype_is_float(x.dtype);
    // For each output, the reduced elements are visited in increasing input
    // linear index — the order the reference's single pass produces.
#pragma omp parallel for schedule(static) OXREF_PAR(out_n * count)
    for (size_t o = 0; o < out_n; o++) {
        size_t base = map_index(o, kept_dims, kept_str);
        if (is_float) {
            double acc = (op == ReduceOp::Sum || op == ReduceOp::Mean) ? 0.0
                         : op == ReduceOp::Prod                        ? 1.0
                         : op == ReduceOp::Max                         ? -INFINITY
                                                                       : INFINITY;
            for (size_t r = 0; r < count; r++) {
                double v = ld_f(x, base + map_index(r, red_dims, red_str));
                switch (op) {
                    case ReduceOp::Sum: case ReduceOp::Mean: acc += v; break;
                    case ReduceOp::Prod: acc *= v; break;
                    case ReduceOp::Max: acc = std::fmax(acc, v); break;
                    case ReduceOp::Min: acc = std::fmin(acc, v); break;
                }
            }
            if (op == ReduceOp::Mean) acc /= (double)count;
            st(dst, out.dtype, o, SF(acc));
        } else {
            int64_t acc = (op == ReduceOp::Sum || op == ReduceOp::Mean) ? 0
                          : op == ReduceOp::Prod                        ? 1
                          : op == ReduceOp::Max                         ? INT64_MIN
                                                                        : INT64_MAX;
            for (size_t r = 0; r < count; r++) {
                int64_t v = ld_i(x, base + map_index(r, red_dims, red_str));
                switch (op) {
                    case ReduceOp::Sum: case ReduceOp::Mean: acc = wadd(acc, v); break;
                    case ReduceOp::Prod: acc = wmul(acc, v); break;
                    case ReduceOp::Max: acc = std::max(acc, v); break;
                    case ReduceOp::Min: acc = std::min(acc, v); break;
                }
            }
            if (op == ReduceOp::Mean && count != 0) acc /= (int64_t)count;  // truncating
            st(dst, out.dtype, o, SI(acc));
        }
    }
    return out;
}

// ─────────────── parameter evaluation (interp.rs:1129-1182) ────────────
static std::vector<size_t> eval_dims(const SymShape& dims, const Bindings& b) {
    std::vector<size_t> out;
    for (auto& d : dims) out.push_back((size_t)d.eval(b));
    return out;
}

static std::vector<size_t> resolve_reshape(const SymShape& shape, size_t numel, Bindings& b) {
    std::vector<size_t> dims;
    bool have_unknown = false;
    size_t unk_i = 0;
    SymId unk_sym = 0;
    for (size_t i = 0; i < shape.size(); i++) {
        uint64_t v;
        std::string why;
        if (shape[i].try_eval(b, &v, &why)) {
            dims.push_back((size_t)v);
        } else {
            auto s = shape[i].as_sym();
            if (s && !have_unknown) {
                have_unknown = true;
                unk_i = i;
                unk_sym = *s;
                dims.push_back(0);
            } else {
                shape[i].eval(b);  // rethrows the binding error
            }
        }
    }
    if (have_unknown) {
        size_t rest = 1;
        for (size_t j = 0; j < dims.size(); j++)
            if (j != unk_i) rest *= dims[j];
        if (rest == 0 || numel % rest != 0)
            fail(ErrKind::Interp, "cannot infer reshape dim: " + std::to_string(numel) + " elements over " + std::to_string(rest));
        dims[unk_i] = numel / rest;
        b.bind(unk_sym, dims[unk_i]);
    }
    return dims;
}

static int64_t ceil_div_euclid(int64_t num, int64_t d) {
    int64_t x = num + d - 1, q = x / d;
    if (x % d < 0) q -= 1;
    return q;
}

// Copy `n` elements chosen by `src_of(i)`; packed outputs are written serially.
template <class F>
static void move_elems(const Tensor& src, Tensor& out, size_t n, F src_of, ParError& perr) {
    uint8_t* dst = out.mut();
    if (dtype_is_packed(out.dtype)) {
        for (size_t i = 0; i < n; i++) st_raw(dst, out.dtype, i, ld_raw(src, src_of(i)));
        return;
    }
#pragma omp parallel for schedule(static) OXREF_PAR(n)
    for (size_t i = 0; i < n; i++) {
        try {
            st_raw(dst, out.dtype, i, ld_raw(src, src_of(i)));
        } catch (const Error& e) {
            perr.capture(e);
        }
    }
}

// ─────────────── eval_prim (interp.rs:511-799) ─────────────────────────
Tensor eval_prim(const Prim& p, const std::vector<const Tensor*>& ins_in, Bindings& bindings) {
    // Only MatMul understands a lazily dequantised operand.
    std::vector<Tensor> held;
    std::vector<const Tensor*> ins = ins_in;
    if (p.kind != PrimKind::MatMul) {
        held.reserve(ins.size());
        for (size_t i = 0; i < ins.size(); i++)
            if (ins[i]->lazy) {
                held.push_back(*ins[i]);
                materialize(held.back());
                ins[i] = &held.back();
            }
    }
    ParError perr;
    switch (p.kind) {
        case PrimKind::Unary: {
            const Tensor& x = *ins[0];
            size_t n = x.numel();
            Tensor out = Tensor::alloc(x.dtype, x.shape);
            uint8_t* dst = out.mut();
            UnaryOp op = (UnaryOp)p.op;
            Dom dom = dom_of(x.dtype);
#pragma omp parallel for schedule(static) OXREF_PAR(n)
            for (size_t i = 0; i < n; i++) {
                if (dom == Dom::F) st(dst, out.dtype, i, SF(unary_f(op, ld_f(x, i))));
                else if (dom == Dom::I) {
                    int64_t a = ld_i(x, i);
                    int64_t r = op == UnaryOp::Neg ? wsub(0, a) : (a < 0 ? wsub(0, a) : a);
                    st(dst, out.dtype, i, SI(r));
                } else
                    st(dst, out.dtype, i, SB(!ld_b(x, i)));
            }
            return out;
        }
        case PrimKind::Binary: case PrimKind::Compare: {
            const Tensor &a = *ins[0], &b = *ins[1];
            auto shape = broadcast_shape(a.shape, b.shape);
            size_t n = prod(shape);
            auto sa = bcast_strides(a.shape, shape), sb = bcast_strides(b.shape, shape);
            bool is_cmp = p.kind == PrimKind::Compare;
            Tensor out = Tensor::alloc(is_cmp ? DType::Bool : a.dtype, shape);
            uint8_t* dst = out.mut();
#pragma omp parallel for schedule(static) OXREF_PAR(n)
            for (size_t i = 0; i < n; i++) {
                try {
                    Scalar x = ld(a, map_index(i, shape, sa)), y = ld(b, map_index(i, shape, sb));
                    if (is_cmp) st(dst, out.dtype, i, SB(compare_val((CmpOp)p.op, x, y)));
                    else st(dst, out.dtype, i, binary_val((BinaryOp)p.op, x, y));
                } catch (const Error& e) {
                    perr.capture(e);
                }
            }
            perr.rethrow();
            return out;
        }
        case PrimKind::Select: {
            const Tensor &c = *ins[0], &a = *ins[1], &b = *ins[2];
            auto shape = broadcast_shape(broadcast_shape(c.shape, a.shape), b.shape);
            size_t n = prod(shape);
            auto sc = bcast_strides(c.shape, shape), sa = bcast_strides(a.shape, shape), sb = bcast_strides(b.shape, shape);
            Tensor out = Tensor::alloc(a.dtype, shape);
            uint8_t* dst = out.mut();
#pragma omp parallel for schedule(static) OXREF_PAR(n)
            for (size_t i = 0; i < n; i++) {
                bool pick_a = ld_b(c, map_index(i, shape, sc));
                uint64_t v = pick_a ? ld_raw(a, map_index(i, shape, sa)) : ld_raw(b, map_index(i, shape, sb));
                st_raw(dst, out.dtype, i, v);
            }
            return out;
        }
        case PrimKind::Cast: {
            const Tensor& x = *ins[0];
            size_t n = x.numel();
            Tensor out = Tensor::alloc(p.dtype, x.shape);
            uint8_t* dst = out.mut();
            if (dtype_is_packed(p.dtype)) {
                for (size_t i = 0; i < n; i++) st(dst, out.dtype, i, ld(x, i));
            } else {
#pragma omp parallel for schedule(static) OXREF_PAR(n)
                for (size_t i = 0; i < n; i++) st(dst, out.dtype, i, ld(x, i));
            }
            return out;
        }
        case PrimKind::MatMul:
            return matmul(*ins[0], *ins[1], p.trans_a, p.trans_b);
        case PrimKind::Reduce:
            return reduce(*ins[0], (ReduceOp)p.op, p.axes, p.keepdims);
        case PrimKind::Reshape: {
            const Tensor& x = *ins[0];
            auto dims = resolve_reshape(p.shape, x.numel(), bindings);
            if (prod(dims) != x.numel())
                fail(ErrKind::Interp, "reshape element count mismatch: input has " + std::to_string(x.numel()) + " elements");
            Tensor out = x;  // shares storage: value semantics, tensors are immutable
            out.shape = dims;
            return out;
        }
        case PrimKind::Transpose: {
            const Tensor& x = *ins[0];
            size_t rank = x.shape.size();
            if (p.axes.size() != rank) fail(ErrKind::Interp, "transpose perm does not match rank " + std::to_string(rank));
            std::vector<char> seen(rank, 0);
            for (auto a : p.axes) {
                if (a >= rank || seen[a]) fail(ErrKind::Interp, "transpose perm is not a permutation");
                seen[a] = 1;
            }
            std::vector<size_t> out_shape, strides;
            auto in_str = row_major_strides(x.shape);
            for (auto a : p.axes) {
                out_shape.push_back(x.shape[a]);
                strides.push_back(in_str[a]);
            }
            size_t n = x.numel();
            Tensor out = Tensor::alloc(x.dtype, out_shape);
            move_elems(x, out, n, [&](size_t i) { return map_index(i, out_shape, strides); }, perr);
            return out;
        }
        case PrimKind::Broadcast: {
            const Tensor& x = *ins[0];
            auto target = eval_dims(p.shape, bindings);
            auto out_shape = broadcast_shape(x.shape, target);
            auto strides = bcast_strides(x.shape, out_shape);
            size_t n = prod(out_shape);
            Tensor out = Tensor::alloc(x.dtype, out_shape);
            move_elems(x, out, n, [&](size_t i) { return map_index(i, out_shape, strides); }, perr);
            return out;
        }
        case PrimKind::Concat: {
            const Tensor& first = *ins[0];
            size_t axis = p.axis;
            std::vector<size_t> out_shape = first.shape;
            size_t total = 0;
            for (auto* t : ins) total += t->shape[axis];
            out_shape[axis] = total;
            Tensor out = Tensor::alloc(first.dtype, out_shape);
            uint8_t* dst = out.mut();
            size_t outer = prod(out_shape, 0, axis), inner = prod(out_shape, axis + 1);
            size_t off = 0;
            for (auto* t : ins) {
                size_t len = t->shape[axis];
                bool packed = dtype_is_packed(out.dtype);
                size_t cnt = outer * len * inner;
                if (packed) {
                    for (size_t e = 0; e < cnt; e++) {
                        size_t o = e / (len * inner), r = e % (len * inner);
                        st_raw(dst, out.dtype, (o * total + off) * inner + r, ld_raw(*t, e));
                    }
                } else {
                    size_t esz = dtype_bits(out.dtype) / 8;
                    for (size_t o = 0; o < outer; o++)
                        std::memcpy(dst + ((o * total + off) * inner) * esz, t->data + (o * len * inner) * esz, len * inner * esz);
                }
                off += len;
            }
            return out;
        }
        case PrimKind::Slice: {
            const Tensor& x = *ins[0];
            size_t rank = x.shape.size();
            std::vector<size_t> out_shape = x.shape;
            std::vector<int64_t> starts(rank, 0), steps(rank, 1);
            for (auto& s : p.specs) {
                int64_t start = (int64_t)s.start.eval(bindings), end = (int64_t)s.end.eval(bindings);
                int64_t len = s.step > 0 ? ceil_div_euclid(end - start, s.step) : ceil_div_euclid(start - end, -s.step);
                out_shape[s.axis] = (size_t)std::max<int64_t>(len, 0);
                starts[s.axis] = start;
                steps[s.axis] = s.step;
            }
            auto in_str = row_major_strides(x.shape);
            size_t n = prod(out_shape);
            size_t xn = x.numel();
            Tensor out = Tensor::alloc(x.dtype, out_shape);
            move_elems(x, out, n,
                       [&](size_t i) {
                           size_t idx = 0, lin = i;
                           for (size_t d = rank; d-- > 0;) {
                               size_t c = lin % out_shape[d];
                               lin /= out_shape[d];
                               idx += (size_t)(starts[d] + (int64_t)c * steps[d]) * in_str[d];
                           }
                           if (idx >= xn) fail(ErrKind::Interp, "slice reads outside its input");
                           return idx;
                       },
                       perr);
            perr.rethrow();
            return out;
        }
        case PrimKind::Gather: {
            const Tensor &data = *ins[0], &indices = *ins[1];
            size_t axis = p.axis;
            int64_t dim = (int64_t)data.shape[axis];
            std::vector<size_t> out_shape(data.shape.begin(), data.shape.begin() + axis);
            out_shape.insert(out_shape.end(), indices.shape.begin(), indices.shape.end());
            out_shape.insert(out_shape.end(), data.shape.begin() + axis + 1, data.shape.end());
            size_t outer = prod(data.shape, 0, axis), inner = prod(data.shape, axis + 1), ni = indices.numel();
            size_t n = outer * ni * inner;
            Tensor out = Tensor::alloc(data.dtype, out_shape);
            move_elems(data, out, n,
                       [&](size_t i) {
                           size_t r = i % inner, ii = (i / inner) % ni, o = i / (inner * ni);
                           int64_t raw = ld_i(indices, ii);
                           if (raw < 0) raw += dim;
                           if (raw < 0 || raw >= dim)
                               fail(ErrKind::Interp, "gather index " + std::to_string(raw) + " out of range for dim " + std::to_string(dim));
                           return (o * (size_t)dim + (size_t)raw) * inner + r;
                       },
                       perr);
            perr.rethrow();
            return out;
        }
        case PrimKind::Scatter: {
            const Tensor &data = *ins[0], &indices = *ins[1], &updates = *ins[2];
            size_t ir = indices.shape.size();
            size_t k = indices.shape[ir - 1];
            size_t num_updates = prod(indices.shape, 0, ir - 1);
            size_t slice_len = prod(data.shape, k);
            Tensor out = Tensor::alloc(data.dtype, data.shape);
            uint8_t* dst = out.mut();
            bool packed = dtype_is_packed(data.dtype);
            if (!packed) std::memcpy(dst, data.data, data.nbytes());
            std::vector<uint64_t> nib;  // packed types go through an unpacked copy
            if (packed) {
                nib.resize(data.numel());
                for (size_t i = 0; i < nib.size(); i++) nib[i] = ld_raw(data, i);
            }
            // duplicates: last write wins (interp.rs:726-747)
            for (size_t u = 0; u < num_updates; u++) {
                size_t base = 0;
                for (size_t d = 0; d < k; d++) {
                    int64_t raw = ld_i(indices, u * k + d);
                    int64_t dim = (int64_t)data.shape[d];
                    if (raw < 0) raw += dim;
                    if (raw < 0 || raw >= dim)
                        fail(ErrKind::Interp, "scatter index " + std::to_string(raw) + " out of range for dim " + std::to_string(dim));
                    base = base * data.shape[d] + (size_t)raw;
                }
                for (size_t j = 0; j < slice_len; j++) {
                    uint64_t v = ld_raw(updates, u * slice_len + j);
                    if (packed) nib[base * slice_len + j] = v;
                    else st_raw(dst, out.dtype, base * slice_len + j, v);
                }
            }
            if (packed)
                for (size_t i = 0; i < nib.size(); i++) st_raw(dst, out.dtype, i, nib[i]);
            return out;
        }
        case PrimKind::Iota: {
            size_t n = (size_t)p.len.eval(bindings);
            Tensor out = Tensor::alloc(p.dtype, {n});
            for (size_t i = 0; i < n; i++) st(out.mut(), out.dtype, i, SI((int64_t)i));
            return out;
        }
        case PrimKind::DimValues: {
            size_t n = p.shape.size();
            Tensor out = Tensor::alloc(DType::I64, {n});
            for (size_t i = 0; i < n; i++) st(out.mut(), out.dtype, i, SI(p.shape[i].eval_signed(bindings)));
            return out;
        }
        case PrimKind::Dequantize: {
            const Tensor &data = *ins[0], &scales = *ins[1];
            if (dom_of(data.dtype) != Dom::I || !dtype_is_float(scales.dtype))
                fail(ErrKind::Interp, "dequantize operand domains");
            auto lz = std::make_shared<LazyDequant>();
            lz->q = data;
            lz->scales = scales;
            lz->block_size = p.block_size;
            if (ins.size() > 2) {
                if (dom_of(ins[2]->dtype) != Dom::I)
                    fail(ErrKind::Interp, std::string(dtype_name(ins[2]->dtype)) + " is not an int tensor");
                lz->has_zp = true;
                lz->zp = *ins[2];
            }
            Tensor out;
            out.dtype = scales.dtype;
            out.shape = eval_dims(p.shape, bindings);
            if (out.numel() != data.numel())
                fail(ErrKind::Interp, "encode length mismatch: " + std::to_string(data.numel()) + " values into the output shape");
            size_t n_blocks = (data.numel() + p.block_size - 1) / p.block_size;
            if (scales.numel() < n_blocks || (lz->has_zp && lz->zp.numel() < n_blocks))
                fail(ErrKind::Interp, "dequantize: too few scales or zero points for the data");
            out.lazy = lz;
            // Small results are written out at once; big weight matrices stay
            // lazy so a following MatMul can stream them.
            if (out.numel() <= (1u << 16)) materialize(out);
            return out;
        }
    }
    fail(ErrKind::Interp, "unknown primitive");
}

// ─────────────── eval (interp.rs:419-495) ──────────────────────────────
static std::vector<std::pair<std::string, Tensor>> eval_with(const Module& m, const std::vector<NodeId>& order,
                                                             const std::vector<std::vector<ValueId>>* deaths,
                                                             const std::vector<std::pair<std::string, Tensor>>& inputs) {
    std::vector<InputDesc> descs;
    for (auto& in : inputs) descs.push_back(InputDesc{in.first.c_str(), in.second.dtype, in.second.shape.data(), in.second.shape.size()});
    Bindings bindings = bind_shapes(m, descs);
    std::vector<Tensor> slots(m.values.size());
    std::vector<char> have(m.values.size(), 0);
    for (ValueId id = 0; id < m.values.size(); id++) {
        const ValueDef& def = m.values[id];
        if (def.origin.kind == Origin::Input) {
            std::string name = def.name ? *def.name : std::string();
            const Tensor* found = nullptr;
            for (auto& in : inputs)
                if (in.first == name) found = &in.second;
            if (!found) fail(ErrKind::Binding, "missing input '" + name + "'");
            slots[id] = *found;
            have[id] = 1;
        } else if (def.origin.kind == Origin::Const) {
            const TensorType& ty = m.consts.ty(def.origin.id);
            auto dims = *shape_as_static(ty.shape);
            std::vector<size_t> shape(dims.begin(), dims.end());
            if (!m.consts.bytes(def.origin.id)) fail(ErrKind::Interp, "constant bytes were released");
            slots[id] = Tensor::view(ty.dtype, shape, m.consts.bytes(def.origin.id));
            have[id] = 1;
        }
    }
    for (size_t step = 0; step < order.size(); step++) {
        const Node& node = m.nodes[order[step]];
        if (!node.is_prim && node.composite.name == "onyxia.AllReduce") {
            // The sum over tensor-parallel ranks: the test harness supplies it (another thread or process
            // holds the other ranks' interpreters). Element type and count travel with the call.
            if (!allreduce_hook()) fail(ErrKind::Interp, "onyxia.AllReduce needs an all-reduce hook");
            if (!have[node.inputs[0]]) fail(ErrKind::Interp, "input value not yet materialized");
            Tensor t = slots[node.inputs[0]];
            materialize(t);
            Tensor out = Tensor::from_bytes(t.dtype, t.shape, t.data, t.nbytes());
            allreduce_hook()(out.mut(), (uint64_t)out.numel(), (int32_t)out.dtype);
            slots[node.outputs[0]] = std::move(out);
            have[node.outputs[0]] = 1;
            if (deaths)
                for (auto v : (*deaths)[step]) slots[v] = Tensor();
            continue;
        }
        if (!node.is_prim)
            fail(ErrKind::Interp, "composite '" + node.composite.name + "' must be inlined before interpretation");
        std::vector<const Tensor*> ins;
        for (auto v : node.inputs) {
            if (!have[v]) fail(ErrKind::Interp, "input value not yet materialized");
            ins.push_back(&slots[v]);
        }
        Tensor out;
        try {
            out = eval_prim(node.prim, ins, bindings);
        } catch (const Error& e) {
            std::string loc = node.loc_name ? *node.loc_name : "<unnamed>";
            fail(ErrKind::Interp, std::string(node.prim.name()) + " (node '" + loc + "'): " + e.what());
        }
        ValueId out_id = node.outputs[0];
        const SymShape& declared = m.values[out_id].ty.shape;
        if (declared.size() == out.shape.size())
            for (size_t d = 0; d < declared.size(); d++)
                if (auto s = declared[d].as_sym())
                    if (!bindings.get(*s)) bindings.bind(*s, out.shape[d]);
        slots[out_id] = std::move(out);
        have[out_id] = 1;
        if (deaths)
            for (auto v : (*deaths)[step]) slots[v] = Tensor();
    }
    std::vector<std::pair<std::string, Tensor>> outs;
    for (auto& o : m.outputs) {
        if (!have[o.second]) fail(ErrKind::Interp, "output '" + o.first + "' was never produced");
        Tensor t = slots[o.second];
        materialize(t);
        outs.emplace_back(o.first, std::move(t));
    }
    return outs;
}

AllReduceHook& allreduce_hook() {
    static AllReduceHook hook = nullptr;
    return hook;
}

std::vector<std::pair<std::string, Tensor>> eval(const Module& m, const std::vector<std::pair<std::string, Tensor>>& inputs) {
    return eval_with(m, m.topo_order(), nullptr, inputs);
}

RefSession prepare(Module m) {
    RefSession s;
    s.module = inline_composites(std::move(m), standard_decompositions(),
                                 [](const Module&, const Node& n) { return !n.is_prim && n.composite.name == "onyxia.AllReduce"; });
    validate(s.module);
    s.order = s.module.topo_order();
    // Values are dropped after their last reader so big models fit in host
    // memory; results do not depend on it.
    std::vector<int64_t> last(s.module.values.size(), -1);
    for (size_t step = 0; step < s.order.size(); step++)
        for (auto v : s.module.nodes[s.order[step]].inputs) last[v] = (int64_t)step;
    for (auto& o : s.module.outputs) last[o.second] = -1;
    s.deaths.assign(s.order.size(), {});
    for (ValueId v = 0; v < last.size(); v++)
        if (last[v] >= 0 && s.module.values[v].origin.kind == Origin::Node) s.deaths[last[v]].push_back(v);
    return s;
}

std::vector<std::pair<std::string, Tensor>> RefSession::run(const std::vector<std::pair<std::string, Tensor>>& inputs) const {
    return eval_with(module, order, &deaths, inputs);
}

}  // namespace oxref
