// Shape/dtype inference over the closed primitive set, and structural
// validation. Reference behaviour: crates/onyxia-ir/src/infer.rs:26-491 and
// crates/onyxia-ir/src/validate.rs:15-140.
#include "ir.hpp"

#include <unordered_set>

namespace ox {

static void require_same_dtype(DType a, DType b, const std::string& what) {
    if (a != b)
        fail(ErrKind::DType, what + ": dtype mismatch " + dtype_name(a) + " vs " + dtype_name(b) +
                                 " (no implicit promotion; lowering must insert casts)");
}
static void require_numeric(DType d, const std::string& what) {
    if (d == DType::Bool || dtype_is_packed(d))
        fail(ErrKind::DType, what + ": dtype " + dtype_name(d) + " not supported");
}
static void require_unpacked(DType d, const std::string& what) {
    if (dtype_is_packed(d))
        fail(ErrKind::DType, what + ": packed dtype " + dtype_name(d) + " must be cast/dequantized first");
}
static void require_bool(DType d, const std::string& what) {
    if (d != DType::Bool) fail(ErrKind::DType, what + ": expected bool, got " + dtype_name(d));
}

static SymShape broadcast_dims(const DimExpr* a, size_t na, const DimExpr* b, size_t nb) {
    size_t rank = na > nb ? na : nb;
    DimExpr one = DimExpr::constant(1);
    SymShape out;
    for (size_t i = 0; i < rank; i++) {
        const DimExpr* x = (i + na >= rank) ? &a[i + na - rank] : nullptr;
        const DimExpr* y = (i + nb >= rank) ? &b[i + nb - rank] : nullptr;
        if (x && y) {
            if (*x == *y) out.push_back(*x);
            else if (*x == one) out.push_back(*y);
            else if (*y == one) out.push_back(*x);
            else
                fail(ErrKind::Shape, "cannot broadcast dim " + x->to_string() + " with " + y->to_string() +
                                         " (dims that must match should share a symbol)");
        } else {
            out.push_back(x ? *x : *y);
        }
    }
    return out;
}

SymShape broadcast_shapes(const SymShape& a, const SymShape& b) {
    return broadcast_dims(a.data(), a.size(), b.data(), b.size());
}

static void check_axes(const std::vector<size_t>& axes, size_t rank, const std::string& what) {
    if (axes.empty()) fail(ErrKind::Shape, what + ": axes must be non-empty (reduce-over-all lists every axis)");
    bool have_prev = false;
    size_t prev = 0;
    for (size_t a : axes) {
        if (a >= rank)
            fail(ErrKind::Shape, what + ": axis " + std::to_string(a) + " out of range for rank " + std::to_string(rank));
        if (have_prev && prev >= a) fail(ErrKind::Shape, what + ": axes must be sorted and unique");
        prev = a;
        have_prev = true;
    }
}

static int64_t ceil_div_euclid(int64_t num, int64_t d) {
    // (num + d - 1).div_euclid(d) for d > 0
    int64_t x = num + d - 1;
    int64_t q = x / d;
    if (x % d < 0) q -= 1;
    return q;
}

static DimExpr slice_out_dim(const SliceSpec& s) {
    if (s.step == 0) fail(ErrKind::Shape, "slice step must be nonzero");
    if (s.step == 1) return s.end - s.start;
    if (s.step == -1) return s.start - s.end;
    auto st = s.start.as_const(), en = s.end.as_const();
    if (!st || !en)
        fail(ErrKind::Shape, "slice with step " + std::to_string(s.step) + " requires constant bounds, got [" +
                                 s.start.to_string() + ", " + s.end.to_string() + ")");
    int64_t start = (int64_t)*st, end = (int64_t)*en;
    int64_t len = s.step > 0 ? ceil_div_euclid(end - start, s.step) : ceil_div_euclid(start - end, -s.step);
    if (len < 0)
        fail(ErrKind::Shape, "slice [" + std::to_string(start) + ", " + std::to_string(end) + ") step " +
                                 std::to_string(s.step) + " has negative length");
    return DimExpr::constant((uint64_t)len);
}

static void check_unary_dtype(UnaryOp op, DType dt) {
    bool ok = false;
    switch (op) {
        case UnaryOp::Neg: ok = dtype_is_float(dt) || dt == DType::I64 || dt == DType::I32 || dt == DType::I8; break;
        case UnaryOp::Abs: ok = dtype_is_float(dt) || (dtype_is_int(dt) && !dtype_is_packed(dt)); break;
        case UnaryOp::Not: ok = dt == DType::Bool; break;
        default: ok = dtype_is_float(dt);
    }
    if (!ok) fail(ErrKind::DType, std::string("unary op does not support dtype ") + dtype_name(dt));
}

std::vector<TensorType> infer_prim(const Prim& p, const std::vector<const TensorType*>& in) {
    auto ar = p.arity();
    if (in.size() < ar.first || in.size() > ar.second) {
        std::string want = ar.first == ar.second ? std::to_string(ar.first)
                           : ar.second == SIZE_MAX ? ">= " + std::to_string(ar.first)
                                                   : std::to_string(ar.first) + "..=" + std::to_string(ar.second);
        fail(ErrKind::InvalidGraph, std::string(p.name()) + " expects " + want + " inputs, got " + std::to_string(in.size()));
    }
    TensorType out;
    switch (p.kind) {
        case PrimKind::Unary:
            check_unary_dtype((UnaryOp)p.op, in[0]->dtype);
            out = *in[0];
            break;
        case PrimKind::Binary: {
            require_same_dtype(in[0]->dtype, in[1]->dtype, p.name());
            BinaryOp op = (BinaryOp)p.op;
            if (op == BinaryOp::And || op == BinaryOp::Or || op == BinaryOp::Xor)
                require_bool(in[0]->dtype, p.name());
            else
                require_numeric(in[0]->dtype, p.name());
            out = TensorType{in[0]->dtype, broadcast_shapes(in[0]->shape, in[1]->shape)};
            break;
        }
        case PrimKind::Compare:
            require_same_dtype(in[0]->dtype, in[1]->dtype, p.name());
            require_unpacked(in[0]->dtype, p.name());
            out = TensorType{DType::Bool, broadcast_shapes(in[0]->shape, in[1]->shape)};
            break;
        case PrimKind::Select: {
            require_bool(in[0]->dtype, "select condition");
            require_same_dtype(in[1]->dtype, in[2]->dtype, "select branches");
            require_unpacked(in[1]->dtype, "select");
            SymShape s = broadcast_shapes(in[0]->shape, in[1]->shape);
            out = TensorType{in[1]->dtype, broadcast_shapes(s, in[2]->shape)};
            break;
        }
        case PrimKind::Cast:
            out = TensorType{p.dtype, in[0]->shape};
            break;
        case PrimKind::MatMul: {
            const TensorType &a = *in[0], &b = *in[1];
            require_same_dtype(a.dtype, b.dtype, "matmul");
            require_numeric(a.dtype, "matmul");
            if (a.shape.size() < 2 || b.shape.size() < 2)
                fail(ErrKind::Shape, "matmul requires rank >= 2 operands, got " + shape_to_string(a.shape) + " and " +
                                         shape_to_string(b.shape) + " (lowering handles rank-1 promotion)");
            size_t ra = a.shape.size(), rb = b.shape.size();
            const DimExpr& m = p.trans_a ? a.shape[ra - 1] : a.shape[ra - 2];
            const DimExpr& ka = p.trans_a ? a.shape[ra - 2] : a.shape[ra - 1];
            const DimExpr& kb = p.trans_b ? b.shape[rb - 1] : b.shape[rb - 2];
            const DimExpr& n = p.trans_b ? b.shape[rb - 2] : b.shape[rb - 1];
            if (ka != kb)
                fail(ErrKind::Shape, "matmul contraction mismatch: " + ka.to_string() + " vs " + kb.to_string() +
                                         " (shapes " + shape_to_string(a.shape) + " x " + shape_to_string(b.shape) + ")");
            SymShape dims = broadcast_dims(a.shape.data(), ra - 2, b.shape.data(), rb - 2);
            dims.push_back(m);
            dims.push_back(n);
            out = TensorType{a.dtype, dims};
            break;
        }
        case PrimKind::Reduce: {
            const TensorType& x = *in[0];
            require_numeric(x.dtype, "reduce");
            check_axes(p.axes, x.shape.size(), "reduce");
            SymShape dims;
            for (size_t i = 0; i < x.shape.size(); i++) {
                bool red = false;
                for (size_t a : p.axes) red |= (a == i);
                if (red) {
                    if (p.keepdims) dims.push_back(DimExpr::constant(1));
                } else {
                    dims.push_back(x.shape[i]);
                }
            }
            out = TensorType{x.dtype, dims};
            break;
        }
        case PrimKind::Reshape: {
            const TensorType& x = *in[0];
            DimExpr in_n = shape_numel(x.shape), out_n = shape_numel(p.shape);
            if (in_n != out_n) {
                auto a = in_n.as_const(), b = out_n.as_const();
                if (a && b)
                    fail(ErrKind::Shape, "reshape element count mismatch: " + shape_to_string(x.shape) + " (" +
                                             std::to_string(*a) + " elements) -> " + shape_to_string(p.shape) + " (" +
                                             std::to_string(*b) + " elements)");
            }
            out = TensorType{x.dtype, p.shape};
            break;
        }
        case PrimKind::Transpose: {
            const TensorType& x = *in[0];
            size_t rank = x.shape.size();
            std::vector<char> seen(rank, 0);
            bool ok = p.axes.size() == rank;
            if (ok)
                for (size_t a : p.axes) {
                    if (a >= rank || seen[a]) {
                        ok = false;
                        break;
                    }
                    seen[a] = 1;
                }
            if (!ok) fail(ErrKind::Shape, "transpose perm is not a permutation of rank " + std::to_string(rank));
            SymShape dims;
            for (size_t a : p.axes) dims.push_back(x.shape[a]);
            out = TensorType{x.dtype, dims};
            break;
        }
        case PrimKind::Broadcast:
            out = TensorType{in[0]->dtype, broadcast_shapes(in[0]->shape, p.shape)};
            break;
        case PrimKind::Concat: {
            const TensorType& first = *in[0];
            size_t rank = first.shape.size();
            if (p.axis >= rank)
                fail(ErrKind::Shape, "concat axis " + std::to_string(p.axis) + " out of range for rank " + std::to_string(rank));
            DimExpr axis_dim = DimExpr::constant(0);
            for (auto* x : in) {
                require_same_dtype(first.dtype, x->dtype, "concat");
                if (x->shape.size() != rank)
                    fail(ErrKind::Shape, "concat rank mismatch: " + shape_to_string(first.shape) + " vs " + shape_to_string(x->shape));
                for (size_t i = 0; i < rank; i++)
                    if (i != p.axis && first.shape[i] != x->shape[i])
                        fail(ErrKind::Shape, "concat dim " + std::to_string(i) + " mismatch: " +
                                                 shape_to_string(first.shape) + " vs " + shape_to_string(x->shape));
                axis_dim = axis_dim + x->shape[p.axis];
            }
            SymShape dims = first.shape;
            dims[p.axis] = axis_dim;
            out = TensorType{first.dtype, dims};
            break;
        }
        case PrimKind::Slice: {
            const TensorType& x = *in[0];
            size_t rank = x.shape.size();
            SymShape dims = x.shape;
            std::unordered_set<size_t> seen;
            for (auto& s : p.specs) {
                if (s.axis >= rank)
                    fail(ErrKind::Shape, "slice axis " + std::to_string(s.axis) + " out of range for rank " + std::to_string(rank));
                if (!seen.insert(s.axis).second)
                    fail(ErrKind::Shape, "slice axis " + std::to_string(s.axis) + " specified twice");
                dims[s.axis] = slice_out_dim(s);
            }
            out = TensorType{x.dtype, dims};
            break;
        }
        case PrimKind::Gather: {
            const TensorType &data = *in[0], &idx = *in[1];
            if (idx.dtype != DType::I64)
                fail(ErrKind::DType, std::string("gather indices must be i64, got ") + dtype_name(idx.dtype));
            size_t rank = data.shape.size();
            if (rank == 0 || p.axis >= rank)
                fail(ErrKind::Shape, "gather axis " + std::to_string(p.axis) + " out of range for rank " + std::to_string(rank));
            SymShape dims(data.shape.begin(), data.shape.begin() + p.axis);
            dims.insert(dims.end(), idx.shape.begin(), idx.shape.end());
            dims.insert(dims.end(), data.shape.begin() + p.axis + 1, data.shape.end());
            out = TensorType{data.dtype, dims};
            break;
        }
        case PrimKind::Scatter: {
            const TensorType &data = *in[0], &idx = *in[1], &upd = *in[2];
            require_same_dtype(data.dtype, upd.dtype, "scatter");
            if (idx.dtype != DType::I64)
                fail(ErrKind::DType, std::string("scatter indices must be i64, got ") + dtype_name(idx.dtype));
            size_t ir = idx.shape.size();
            if (ir == 0) fail(ErrKind::Shape, "scatter indices must have rank >= 1");
            auto kc = idx.shape[ir - 1].as_const();
            if (!kc) fail(ErrKind::Shape, "scatter requires a constant last indices dim, got " + shape_to_string(idx.shape));
            size_t k = (size_t)*kc, dr = data.shape.size();
            if (k > dr)
                fail(ErrKind::Shape, "scatter index depth " + std::to_string(k) + " exceeds data rank " + std::to_string(dr));
            SymShape expect(idx.shape.begin(), idx.shape.end() - 1);
            expect.insert(expect.end(), data.shape.begin() + k, data.shape.end());
            if (upd.shape != expect)
                fail(ErrKind::Shape, "scatter updates shape " + shape_to_string(upd.shape) + " does not match expected " +
                                         shape_to_string(expect));
            out = data;
            break;
        }
        case PrimKind::Iota:
            require_numeric(p.dtype, "iota");
            out = TensorType{p.dtype, SymShape{p.len}};
            break;
        case PrimKind::DimValues:
            out = TensorType{DType::I64, fixed_shape({(uint64_t)p.shape.size()})};
            break;
        case PrimKind::Dequantize: {
            const TensorType &data = *in[0], &scales = *in[1];
            if (p.block_size == 0) fail(ErrKind::Shape, "dequantize block_size must be > 0");
            if (data.dtype != DType::U4 && data.dtype != DType::I4 && data.dtype != DType::U8)
                fail(ErrKind::DType, std::string("dequantize data must be u4/i4/u8, got ") + dtype_name(data.dtype));
            if (!dtype_is_float(scales.dtype))
                fail(ErrKind::DType, std::string("dequantize scales must be float, got ") + dtype_name(scales.dtype));
            if (in.size() > 2) require_same_dtype(data.dtype, in[2]->dtype, "dequantize zero_points");
            if (data.shape.empty()) fail(ErrKind::Shape, "dequantize data must have rank >= 1");
            if (auto l = data.shape.back().as_const())
                if (*l != p.block_size)
                    fail(ErrKind::Shape, "dequantize data last dim " + std::to_string(*l) + " != block_size " +
                                             std::to_string(p.block_size));
            auto a = shape_numel(data.shape).as_const(), b = shape_numel(p.shape).as_const();
            if (a && b && *a != *b)
                fail(ErrKind::Shape, "dequantize element count mismatch: data " + shape_to_string(data.shape) +
                                         " vs out " + shape_to_string(p.shape));
            out = TensorType{scales.dtype, p.shape};
            break;
        }
    }
    return {out};
}

// ───────────────────────────── validate ────────────────────────────────
static std::string node_label(const Module& m, size_t i) {
    const Node& n = m.nodes[i];
    std::string kind = n.is_prim ? n.prim.name() : n.composite.name;
    return "node " + std::to_string(i) + " (" + kind + (n.loc_name ? ", '" + *n.loc_name + "'" : std::string()) + ")";
}

void validate(const Module& m) {
    size_t nv = m.values.size(), nn = m.nodes.size();
    for (size_t i = 0; i < nv; i++) {
        const ValueDef& d = m.values[i];
        auto bad = [&](const std::string& msg) {
            fail(ErrKind::InvalidGraph, "value " + std::to_string(i) + (d.name ? " ('" + *d.name + "')" : std::string()) + ": " + msg);
        };
        if (d.origin.kind == Origin::Const) {
            if (d.origin.id >= m.consts.size()) bad("const id out of range");
            if (m.consts.ty(d.origin.id) != d.ty)
                bad("type " + d.ty.to_string() + " disagrees with pool entry type " + m.consts.ty(d.origin.id).to_string());
        } else if (d.origin.kind == Origin::Node) {
            if (d.origin.id >= nn) bad("producer node id out of range");
            const Node& p = m.nodes[d.origin.id];
            if (d.origin.output >= p.outputs.size() || p.outputs[d.origin.output] != i)
                bad("producer node's outputs do not point back to this value");
        }
    }
    for (size_t i = 0; i < nn; i++) {
        const Node& n = m.nodes[i];
        auto bad = [&](const std::string& msg) { fail(ErrKind::InvalidGraph, node_label(m, i) + ": " + msg); };
        for (auto v : n.inputs)
            if (v >= nv) bad("input value id out of range");
        for (size_t oi = 0; oi < n.outputs.size(); oi++) {
            if (n.outputs[oi] >= nv) bad("output value id out of range");
            const Origin& o = m.values[n.outputs[oi]].origin;
            if (!(o.kind == Origin::Node && o.id == i && o.output == oi))
                bad("output " + std::to_string(oi) + " does not record this node as its origin");
        }
        if (n.is_prim) {
            std::vector<const TensorType*> tys;
            for (auto v : n.inputs) tys.push_back(&m.values[v].ty);
            std::vector<TensorType> inferred;
            try {
                inferred = infer_prim(n.prim, tys);
            } catch (const Error& e) {
                bad(e.what());
            }
            if (inferred.size() != n.outputs.size())
                bad("produces " + std::to_string(n.outputs.size()) + " outputs but inference expects " +
                    std::to_string(inferred.size()));
            for (size_t oi = 0; oi < inferred.size(); oi++)
                if (inferred[oi] != m.values[n.outputs[oi]].ty)
                    bad("output " + std::to_string(oi) + " declared as " + m.values[n.outputs[oi]].ty.to_string(&m.symbols) +
                        " but inference says " + inferred[oi].to_string(&m.symbols));
        }
    }
    for (auto& io : m.inputs) {
        if (io.second >= nv) fail(ErrKind::InvalidGraph, "input '" + io.first + "' has out-of-range value id");
        if (m.values[io.second].origin.kind != Origin::Input)
            fail(ErrKind::InvalidGraph, "input '" + io.first + "' refers to a value whose origin is not Input");
    }
    for (auto& io : m.outputs)
        if (io.second >= nv) fail(ErrKind::InvalidGraph, "output '" + io.first + "' has out-of-range value id");
    m.topo_order();
}

}  // namespace ox
