// Tensor-parallel partition of a module: the part of it that one of `tp` ranks
// executes.
//
// The pass finds MatMulNBits nodes whose results flow — through
// GroupQueryAttention, unary element-wise nodes and binary element-wise nodes of
// two equally split operands — only into the activation input of another
// MatMulNBits. Those producers are split along N (each rank keeps a contiguous
// band of rows of the packed weight: N/tp output features), everything in
// between works on the rank's band (attention on the rank's heads and its share
// of the KV cache), and the consuming MatMulNBits is split along K (each rank
// multiplies its band of input features by the matching blocks of the weight).
// The K-split result is a partial sum; an `onyxia.AllReduce` composite after it
// stands for the sum over ranks. Everything else (norms, residual adds, the
// embedding, lm_head) is replicated.
//
// The reference has no multi-device execution; the contract this pass keeps is
// its single-device semantics: summing the partial results of all ranks gives
// the unpartitioned MatMulNBits up to the rounding of the partial sums.
#include <algorithm>
#include <cstring>
#include <map>
#include <set>

#include "ir.hpp"

namespace ox {

namespace {

bool is_composite(const Node& n, const char* name) { return !n.is_prim && n.composite.name == name; }

struct Analysis {
    std::set<NodeId> col, row, gqa, elementwise;
    std::vector<char> split;  // per value: holds only this rank's band of the last axis (KV caches: of axis 1)
};

// Nodes a split value may pass through.
bool passes_split(const Node& n) {
    if (!n.is_prim) return n.composite.name == "Gelu";
    return n.prim.kind == PrimKind::Unary || n.prim.kind == PrimKind::Binary;
}

Analysis analyse(const Module& m, int tp) {
    const size_t nv = m.values.size();
    std::vector<std::vector<NodeId>> readers(nv);
    for (NodeId i = 0; i < m.nodes.size(); i++)
        for (auto v : m.nodes[i].inputs) readers[v].push_back(i);
    std::vector<char> is_output(nv, 0);
    for (auto& o : m.outputs) is_output[o.second] = 1;
    std::vector<int> input_index(nv, -1);
    for (size_t i = 0; i < m.inputs.size(); i++) input_index[m.inputs[i].second] = (int)i;

    auto last_dim_ok = [&](ValueId v) {
        const auto& shp = m.values[v].ty.shape;
        if (shp.empty()) return false;
        auto c = shp.back().as_const();
        return c && *c % (uint64_t)tp == 0;
    };
    // candidates for the N split: constant 4-bit weights, N and the scale/zero-point rows divisible
    std::set<NodeId> cand;
    for (NodeId i = 0; i < m.nodes.size(); i++) {
        const Node& n = m.nodes[i];
        if (!is_composite(n, "com.microsoft.MatMulNBits")) continue;
        const int64_t N = n.composite.attrs.int_or("N", 0), K = n.composite.attrs.int_or("K", 0);
        const int64_t nb = (K + 31) / 32;
        bool ok = N > 0 && N % tp == 0 && last_dim_ok(n.outputs[0]) && n.composite.attrs.int_or("block_size", 0) == 32;
        for (size_t j = 1; j < n.inputs.size() && ok; j++) ok = m.values[n.inputs[j]].origin.kind == Origin::Const;
        if (n.inputs.size() > 3 && ((N / tp) * nb) % 2 != 0) ok = false;  // zero points are packed two per byte
        if (ok) cand.insert(i);
    }

    Analysis a;
    for (;;) {
        a = Analysis{};
        a.split.assign(nv, 0);
        std::vector<std::set<NodeId>> source(nv);  // which candidates a split value descends from
        std::set<NodeId> bad;                       // candidates that have to stay whole
        for (NodeId i : m.topo_order()) {
            const Node& n = m.nodes[i];
            std::set<NodeId> src;
            bool any_split = false, all_split = !n.inputs.empty();
            for (auto v : n.inputs) {
                if (a.split[v]) {
                    any_split = true;
                    src.insert(source[v].begin(), source[v].end());
                } else {
                    all_split = false;
                }
            }
            auto mark = [&](ValueId v) {
                a.split[v] = 1;
                source[v] = src;
            };
            if (is_composite(n, "com.microsoft.MatMulNBits")) {
                if (a.split[n.inputs[0]]) {
                    // consumes a band of features: K split, partial result
                    const int64_t K = n.composite.attrs.int_or("K", 0), nb = (K + 31) / 32;
                    bool ok = K % 32 == 0 && nb % tp == 0 && n.composite.attrs.int_or("block_size", 0) == 32;
                    for (size_t j = 1; j < n.inputs.size() && ok; j++) ok = m.values[n.inputs[j]].origin.kind == Origin::Const;
                    if (ok) a.row.insert(i);
                    else bad.insert(src.begin(), src.end());
                } else if (cand.count(i)) {
                    src = {i};
                    a.col.insert(i);
                    mark(n.outputs[0]);
                }
                continue;
            }
            if (!any_split) continue;
            if (is_composite(n, "com.microsoft.GroupQueryAttention")) {
                const int64_t H = n.composite.attrs.int_or("num_heads", 0), KV = n.composite.attrs.int_or("kv_num_heads", 0);
                bool ok = a.split[n.inputs[0]] && a.split[n.inputs[1]] && a.split[n.inputs[2]] && H % tp == 0 && KV % tp == 0 &&
                          n.outputs.size() == 3;
                // the caches must be plain module inputs nothing else reads, so that their declared shape can shrink
                for (int s = 3; s <= 4 && ok; s++)
                    ok = input_index[n.inputs[s]] >= 0 && readers[n.inputs[s]].size() == 1 && m.values[n.inputs[s]].ty.shape.size() == 4;
                for (size_t j = 5; j < n.inputs.size() && ok; j++) ok = !a.split[n.inputs[j]];
                // a bias tensor is indexed by head: not handled
                if (n.composite.attrs.int_or("has_attention_bias", 0) != 0) ok = false;
                if (ok) {
                    a.gqa.insert(i);
                    for (auto v : n.outputs) mark(v);
                } else {
                    bad.insert(src.begin(), src.end());
                }
                continue;
            }
            bool ok = passes_split(n) && all_split && n.outputs.size() == 1;
            if (ok)
                for (auto v : n.inputs) ok = ok && m.values[v].ty.shape == m.values[n.outputs[0]].ty.shape;
            if (ok) {
                a.elementwise.insert(i);
                mark(n.outputs[0]);
            } else {
                bad.insert(src.begin(), src.end());
            }
        }
        // a split value may only leave the module as a KV cache
        for (ValueId v = 0; v < nv; v++) {
            if (!a.split[v]) continue;
            const bool is_cache = m.values[v].origin.kind == Origin::Node && a.gqa.count(m.values[v].origin.id) &&
                                  m.values[v].origin.output >= 1;
            if ((is_output[v] && !is_cache) || (readers[v].empty() && !is_output[v])) bad.insert(source[v].begin(), source[v].end());
            if (is_cache && !readers[v].empty()) bad.insert(source[v].begin(), source[v].end());
        }
        if (bad.empty()) break;
        for (auto b : bad) cand.erase(b);
    }
    return a;
}

// Rows [r0, r0 + rows) of a constant laid out as `total_rows` equal rows.
std::vector<uint8_t> slice_rows(const uint8_t* data, size_t nbytes, uint64_t total_rows, uint64_t r0, uint64_t rows) {
    const size_t row_bytes = nbytes / total_rows;
    return std::vector<uint8_t>(data + r0 * row_bytes, data + (r0 + rows) * row_bytes);
}

// Columns [c0, c0 + cols) of every row of a [rows, total_cols] constant whose elements take `bits` bits
// (4-bit elements are packed low nibble first over the flattened tensor).
std::vector<uint8_t> slice_cols(const uint8_t* data, uint64_t rows, uint64_t total_cols, uint64_t c0, uint64_t cols, int bits) {
    if (bits % 8 == 0) {
        const size_t eb = bits / 8;
        std::vector<uint8_t> out(rows * cols * eb);
        for (uint64_t r = 0; r < rows; r++) std::memcpy(out.data() + r * cols * eb, data + (r * total_cols + c0) * eb, cols * eb);
        return out;
    }
    std::vector<uint8_t> out((rows * cols + 1) / 2, 0);
    for (uint64_t r = 0; r < rows; r++)
        for (uint64_t c = 0; c < cols; c++) {
            const uint64_t si = r * total_cols + c0 + c, di = r * cols + c;
            const uint8_t nib = (data[si >> 1] >> ((si & 1) * 4)) & 0xF;
            out[di >> 1] |= (uint8_t)(nib << ((di & 1) * 4));
        }
    return out;
}

uint64_t static_numel(const TensorType& t) {
    uint64_t n = 1;
    for (auto& d : t.shape) n *= d.as_const().value();
    return n;
}

}  // namespace

Module tp_partition(const Module& src, int tp, int rank) {
    if (tp < 1 || rank < 0 || rank >= tp) fail(ErrKind::Attribute, "tensor-parallel partition: rank out of range");
    Module m = src;
    if (tp == 1) return m;
    const Analysis a = analyse(src, tp);
    const uint64_t utp = (uint64_t)tp, ur = (uint64_t)rank;

    auto shrink_dim = [&](ValueId v, size_t axis) {
        auto& shp = m.values[v].ty.shape;
        shp[axis] = DimExpr::constant(shp[axis].as_const().value() / utp);
    };
    auto set_const = [&](ValueId v, TensorType ty, std::vector<uint8_t> bytes) {
        ConstId id = m.consts.add(ty, std::move(bytes));
        m.values[v].ty = ty;
        m.values[v].origin.kind = Origin::Const;
        m.values[v].origin.id = id;
    };
    auto const_bytes = [&](ValueId v) {
        const ConstId id = src.values[v].origin.id;
        if (!src.consts.bytes(id)) fail(ErrKind::InvalidGraph, "tensor-parallel partition: constant bytes are gone");
        return std::make_pair(src.consts.bytes(id), src.consts.nbytes(id));
    };

    for (NodeId i : a.col) {
        Node& n = m.nodes[i];
        const uint64_t N = (uint64_t)n.composite.attrs.int_("N"), K = (uint64_t)n.composite.attrs.int_("K"), nb = (K + 31) / 32;
        const uint64_t rows = N / utp, r0 = ur * rows;
        for (size_t j = 1; j < n.inputs.size(); j++) {
            const ValueId v = n.inputs[j];
            auto [data, nbytes] = const_bytes(v);
            TensorType ty = src.values[v].ty;
            // weight [N, nb, 32]; scales and zero points: N·nb elements in row-major order, any rank
            if (j == 1) {
                ty.shape[0] = DimExpr::constant(rows);
                set_const(v, ty, slice_rows(data, nbytes, N, r0, rows));
            } else {
                const uint64_t total = static_numel(ty);
                if (total != N * nb) fail(ErrKind::Shape, "tensor-parallel partition: unexpected scale / zero-point shape");
                const int bits = dtype_is_packed(ty.dtype) ? 4 : (int)(dtype_storage_bytes(ty.dtype, 1) * 8);
                ty.shape = {DimExpr::constant(rows * nb)};
                set_const(v, ty, slice_cols(data, 1, N * nb, r0 * nb, rows * nb, bits));
            }
        }
        n.composite.attrs.set("N", AttrValue::of_int((int64_t)rows));
        shrink_dim(n.outputs[0], m.values[n.outputs[0]].ty.shape.size() - 1);
    }
    for (NodeId i : a.elementwise) shrink_dim(m.nodes[i].outputs[0], m.values[m.nodes[i].outputs[0]].ty.shape.size() - 1);
    for (NodeId i : a.gqa) {
        Node& n = m.nodes[i];
        n.composite.attrs.set("num_heads", AttrValue::of_int(n.composite.attrs.int_("num_heads") / tp));
        n.composite.attrs.set("kv_num_heads", AttrValue::of_int(n.composite.attrs.int_("kv_num_heads") / tp));
        shrink_dim(n.outputs[0], m.values[n.outputs[0]].ty.shape.size() - 1);
        shrink_dim(n.outputs[1], 1);
        shrink_dim(n.outputs[2], 1);
        shrink_dim(n.inputs[3], 1);
        shrink_dim(n.inputs[4], 1);
    }
    for (NodeId i : a.row) {
        const uint64_t N = (uint64_t)m.nodes[i].composite.attrs.int_("N"), K = (uint64_t)m.nodes[i].composite.attrs.int_("K");
        const uint64_t nb = K / 32, cols = nb / utp, c0 = ur * cols;
        for (size_t j = 1; j < m.nodes[i].inputs.size(); j++) {
            const ValueId v = m.nodes[i].inputs[j];
            auto [data, nbytes] = const_bytes(v);
            (void)nbytes;
            TensorType ty = src.values[v].ty;
            if (j == 1) {  // [N, nb, 32] 4-bit: keep blocks c0 … c0 + cols of every row (a block is 16 bytes)
                ty.shape[1] = DimExpr::constant(cols);
                set_const(v, ty, slice_cols(data, N, nb * 16, c0 * 16, cols * 16, 8));
            } else {
                if (static_numel(ty) != N * nb) fail(ErrKind::Shape, "tensor-parallel partition: unexpected scale / zero-point shape");
                const int bits = dtype_is_packed(ty.dtype) ? 4 : (int)(dtype_storage_bytes(ty.dtype, 1) * 8);
                ty.shape = {DimExpr::constant(N * cols)};
                set_const(v, ty, slice_cols(data, N, nb, c0, cols, bits));
            }
        }
        m.nodes[i].composite.attrs.set("K", AttrValue::of_int((int64_t)(K / utp)));
        // the node now yields a partial sum; the sum over ranks takes its place downstream
        const ValueId full = m.nodes[i].outputs[0];
        ValueDef pd;
        pd.ty = m.values[full].ty;
        pd.origin.kind = Origin::Node;
        pd.origin.id = i;
        pd.origin.output = 0;
        const ValueId partial = m.add_value(pd);
        m.nodes[i].outputs[0] = partial;
        Node ar;
        ar.is_prim = false;
        ar.composite.name = "onyxia.AllReduce";
        ar.composite.attrs.set("world", AttrValue::of_int((int64_t)tp));
        ar.inputs = {partial};
        ar.outputs = {full};
        ar.loc_name = m.nodes[i].loc_name ? std::optional<std::string>(*m.nodes[i].loc_name + "/AllReduce") : std::nullopt;
        ar.loc_op = std::string("AllReduce");
        const NodeId arn = m.add_node(std::move(ar));
        m.values[full].origin.kind = Origin::Node;
        m.values[full].origin.id = arn;
        m.values[full].origin.output = 0;
    }
    validate(m);
    return m;
}

// How many MatMulNBits nodes were split along N and along K for `tp` ranks (diagnostics, tests).
void tp_partition_stats(const Module& m, int tp, size_t* col, size_t* row, size_t* attn) {
    const Analysis a = analyse(m, tp);
    if (col) *col = a.col.size();
    if (row) *row = a.row.size();
    if (attn) *attn = a.gqa.size();
}

}  // namespace ox
