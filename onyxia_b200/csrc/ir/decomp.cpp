// Standard decompositions of the composite set into primitives, and the
// legaliser that inlines them.
//
// These are the *specification* of every fused kernel: the primitive sequence
// (and therefore every store-rounding point) follows the reference
// crates/onyxia-ir/src/decomp.rs:
//   Softmax :174-183, Gelu :185-213, Trilu :215-239,
//   SimplifiedLayerNormalization :241-257, RotaryEmbedding :259-355,
//   GroupQueryAttention :357-613, MatMulNBits :615-663,
//   inline_composites :73-133.
#include <cmath>
#include <cstring>

#include "ir.hpp"

namespace ox {

const DecompFn* DecompositionRegistry::get(const std::string& name) const {
    auto it = map_.find(name);
    return it == map_.end() ? nullptr : &it->second;
}

namespace {

using Ins = std::vector<ValueId>;
DimExpr C(uint64_t v) { return DimExpr::constant(v); }

// Rank-0 constant of `dt` holding v (rounded like the reference: f32 via C
// cast, f16 straight from f64, ints by saturating truncation).
ValueId scalar(GraphBuilder& b, DType dt, double v) {
    std::vector<uint8_t> bytes;
    auto put = [&](const void* p, size_t n) { bytes.assign((const uint8_t*)p, (const uint8_t*)p + n); };
    switch (dt) {
        case DType::F32: { float f = (float)v; put(&f, 4); break; }
        case DType::F16: { uint16_t h = f64_to_f16_bits(v); put(&h, 2); break; }
        case DType::I64: { int64_t i = (int64_t)v; put(&i, 8); break; }
        case DType::I32: { int32_t i = (int32_t)v; put(&i, 4); break; }
        default: fail(ErrKind::Unsupported, std::string("scalar constant of dtype ") + dtype_name(dt));
    }
    return b.constant(TensorType{dt, {}}, std::move(bytes));
}

ValueId slice1(GraphBuilder& b, ValueId x, size_t axis, DimExpr start, DimExpr end) {
    SliceSpec s;
    s.axis = axis;
    s.start = std::move(start);
    s.end = std::move(end);
    s.step = 1;
    return b.slice(x, {s});
}

Ins softmax(const Composite& c, const Ins& in, GraphBuilder& b) {
    size_t axis = (size_t)c.attrs.int_("axis");
    ValueId x = in[0];
    ValueId mx = b.reduce(ReduceOp::Max, x, {axis}, true);
    ValueId e = b.unary(UnaryOp::Exp, b.sub(x, mx));
    ValueId sum = b.reduce(ReduceOp::Sum, e, {axis}, true);
    return {b.div(e, sum)};
}

Ins gelu(const Composite& c, const Ins& in, GraphBuilder& b) {
    ValueId x = in[0];
    DType dt = b.ty(x).dtype;
    ValueId half_c = scalar(b, dt, 0.5);
    ValueId one = scalar(b, dt, 1.0);
    ValueId inner;
    if (c.attrs.str_or("approximate", "none") == "tanh") {
        // 0.5·x·(1 + tanh(√(2/π)·(x + 0.044715·x³)))
        ValueId coef = scalar(b, dt, 0.044715);
        ValueId k = scalar(b, dt, std::sqrt(2.0 / M_PI));
        ValueId x2 = b.mul(x, x);
        ValueId x3 = b.mul(x2, x);
        ValueId cx3 = b.mul(coef, x3);
        ValueId sum = b.add(x, cx3);
        inner = b.unary(UnaryOp::Tanh, b.mul(k, sum));
    } else {
        // 0.5·x·(1 + erf(x/√2))
        ValueId inv_sqrt2 = scalar(b, dt, M_SQRT1_2);
        inner = b.unary(UnaryOp::Erf, b.mul(x, inv_sqrt2));
    }
    ValueId one_plus = b.add(one, inner);
    ValueId hx = b.mul(half_c, x);
    return {b.mul(hx, one_plus)};
}

Ins trilu(const Composite& c, const Ins& in, GraphBuilder& b) {
    ValueId x = in[0];
    bool upper = c.attrs.int_or("upper", 1) != 0;
    int64_t k = c.attrs.int_or("k", 0);
    SymShape dims = b.ty(x).shape;
    if (dims.size() < 2) fail(ErrKind::Shape, "Trilu requires rank >= 2");
    DimExpr r = dims[dims.size() - 2], cd = dims[dims.size() - 1];
    ValueId rows = b.reshape(b.iota(r, DType::I64), {r, C(1)});
    ValueId cols = b.reshape(b.iota(cd, DType::I64), {C(1), cd});
    ValueId shifted = b.add(rows, scalar(b, DType::I64, (double)k));
    // upper keeps col >= row + k, lower keeps col <= row + k
    ValueId keep = b.cmp(upper ? CmpOp::Ge : CmpOp::Le, cols, shifted);
    ValueId zero = scalar(b, b.ty(x).dtype, 0.0);
    return {b.select(keep, x, zero)};
}

Ins simplified_layer_norm(const Composite& c, const Ins& in, GraphBuilder& b) {
    ValueId x = in[0], w = in[1];
    double eps = c.attrs.float_or("epsilon", 1e-5);
    size_t last = b.ty(x).shape.size() - 1;
    ValueId ms = b.reduce(ReduceOp::Mean, b.mul(x, x), {last}, true);
    ValueId denom = b.add(ms, scalar(b, b.ty(x).dtype, eps));
    ValueId inv = b.unary(UnaryOp::Rsqrt, denom);
    return {b.mul(b.mul(x, inv), w)};
}

Ins rotary_embedding(const Composite& c, const Ins& in, GraphBuilder& b) {
    if (c.attrs.int_or("interleaved", 0) != 0)
        fail(ErrKind::Unsupported, "RotaryEmbedding interleaved=1 decomposition");
    ValueId x = in[0], pos = in[1], cos_cache = in[2], sin_cache = in[3];
    SymShape xd = b.ty(x).shape;
    if (xd.size() != 3)
        fail(ErrKind::Unsupported, "RotaryEmbedding expects 3-D input, got " + shape_to_string(xd));
    DimExpr bsz = xd[0], seq = xd[1], hidden = xd[2];
    // num_heads = 0 means "infer from the cache width".
    uint64_t heads;
    int64_t nh = c.attrs.int_or("num_heads", 0);
    if (nh > 0) {
        heads = (uint64_t)nh;
    } else {
        heads = 1;
        auto half = b.ty(cos_cache).shape[1].as_const();
        auto h = hidden.as_const();
        if (h && half) {
            uint64_t r = *half * 2;
            if (r > 0 && *h % r == 0) heads = *h / r;
        }
    }
    auto d_opt = hidden.div_exact(C(heads));
    if (!d_opt)
        fail(ErrKind::Shape, "hidden dim " + hidden.to_string() + " not divisible by num_heads " + std::to_string(heads));
    DimExpr d = *d_opt;
    int64_t rdim = c.attrs.int_or("rotary_embedding_dim", 0);
    DimExpr half_r = rdim == 0 ? b.ty(cos_cache).shape[1] : C((uint64_t)rdim / 2);
    DimExpr r_full = half_r * C(2);

    SymShape bc = {bsz, seq, C(1), half_r};
    ValueId cosv = b.reshape(b.gather(cos_cache, pos, 0), bc);
    ValueId sinv = b.reshape(b.gather(sin_cache, pos, 0), bc);

    ValueId x4 = b.reshape(x, {bsz, seq, C(heads), d});
    ValueId x1 = slice1(b, x4, 3, C(0), half_r);
    ValueId x2 = slice1(b, x4, 3, half_r, r_full);

    ValueId x1c = b.mul(x1, cosv);
    ValueId x2s = b.mul(x2, sinv);
    ValueId o1 = b.sub(x1c, x2s);
    ValueId x2c = b.mul(x2, cosv);
    ValueId x1s = b.mul(x1, sinv);
    ValueId o2 = b.add(x2c, x1s);

    DimExpr rest_len = d - r_full;
    Ins parts = {o1, o2};
    if (rest_len.as_const() != std::optional<uint64_t>(0)) parts.push_back(slice1(b, x4, 3, r_full, d));
    ValueId joined = b.concat(parts, 3);
    return {b.reshape(joined, {bsz, seq, hidden})};
}

Ins group_query_attention(const Composite& c, const Ins& in, GraphBuilder& b) {
    if (in.size() < 6) fail(ErrKind::InvalidGraph, "GQA expects at least 6 inputs");
    ValueId q = in[0], k = in[1], v = in[2], past_k = in[3], past_v = in[4], seqlens = in[5];
    uint64_t heads = (uint64_t)c.attrs.int_("num_heads");
    uint64_t kv_heads = (uint64_t)c.attrs.int_("kv_num_heads");
    if (heads == 0 || kv_heads == 0 || heads % kv_heads != 0)
        fail(ErrKind::Attribute, "GQA num_heads=" + std::to_string(heads) +
                                     " must be a positive multiple of kv_num_heads=" + std::to_string(kv_heads));
    uint64_t group = heads / kv_heads;
    int64_t window = c.attrs.int_or("local_window_size", -1);

    SymShape qd = b.ty(q).shape;
    DimExpr bsz = qd[0], seq = qd[1], hidden = qd[2];
    auto d_opt = hidden.div_exact(C(heads));
    if (!d_opt) fail(ErrKind::Shape, "GQA hidden " + hidden.to_string() + " not divisible by num_heads " + std::to_string(heads));
    DimExpr d = *d_opt;
    DimExpr past = b.ty(past_k).shape[2];
    DimExpr total = past + seq;
    DType dt = b.ty(q).dtype;
    DimExpr one = C(1);

    // tot_b = seqlens_k[b] + 1 as i64 [B,1,1,1]; past_b = max(tot_b - S, 0).
    ValueId sl = b.cast(b.reshape(seqlens, {bsz, one, one, one}), DType::I64);
    ValueId tot_b = b.add(sl, scalar(b, DType::I64, 1.0));
    ValueId s_dim = b.prim(Prim::dim_values({seq}), {});
    ValueId past_b_raw = b.sub(tot_b, s_dim);
    ValueId past_b = b.binary(BinaryOp::Max, past_b_raw, scalar(b, DType::I64, 0.0));
    ValueId jrel = b.reshape(b.iota(seq, DType::I64), {one, one, seq, one});

    // Rotary positions come from the per-row past length, like the mask.
    if (c.attrs.int_or("do_rotary", 0) != 0) {
        if (in.size() < 8) fail(ErrKind::InvalidGraph, "GQA with do_rotary=1 needs cos/sin caches");
        ValueId cosc = in[6], sinc = in[7];
        int64_t interleaved = c.attrs.int_or("rotary_interleaved", 0);
        ValueId qpos = b.add(past_b, jrel);
        ValueId pos2 = b.reshape(qpos, {bsz, seq});
        auto rope = [&](ValueId x, uint64_t n) {
            Attrs a;
            a.set("num_heads", AttrValue::of_int((int64_t)n));
            a.set("interleaved", AttrValue::of_int(interleaved));
            TensorType ty = b.ty(x);
            return b.composite("com.microsoft.RotaryEmbedding", a, {x, pos2, cosc, sinc}, {ty})[0];
        };
        q = rope(q, heads);
        k = rope(k, kv_heads);
    }

    // [B,S,N·D] → [B,S,N,D] → [B,N,S,D]
    auto to_heads = [&](ValueId x, uint64_t n) {
        return b.transpose(b.reshape(x, {bsz, seq, C(n), d}), {0, 2, 1, 3});
    };
    ValueId q4 = to_heads(q, heads);
    ValueId k4 = to_heads(k, kv_heads);
    ValueId v4 = to_heads(v, kv_heads);

    // present[b] = valid past rows ++ new rows ++ zeros, placed per row with a
    // one-hot matmul (onehot[b,t,j] = (t == past_b + j)).
    ValueId zero_f = scalar(b, dt, 0.0);
    ValueId one_f = scalar(b, dt, 1.0);
    ValueId pcols = b.reshape(b.iota(past, DType::I64), {one, one, past, one});
    ValueId past_valid = b.cmp(CmpOp::Lt, pcols, past_b);
    DimExpr kvc = C(kv_heads);
    ValueId new_zeros = b.broadcast(zero_f, {bsz, kvc, seq, d});
    ValueId tcols = b.reshape(b.iota(total, DType::I64), {one, one, total, one});
    ValueId jrow = b.reshape(jrel, {one, one, one, seq});
    ValueId tpos = b.add(past_b, jrow);
    ValueId hot = b.cmp(CmpOp::Eq, tcols, tpos);
    ValueId onehot = b.broadcast(b.select(hot, one_f, zero_f), {bsz, kvc, total, seq});

    auto place_present = [&](ValueId past_kv, ValueId new4) {
        ValueId kept = b.select(past_valid, past_kv, zero_f);
        ValueId padded = b.concat({kept, new_zeros}, 2);
        ValueId placed = b.matmul(onehot, new4);
        return b.add(padded, placed);
    };
    ValueId present_k = place_present(past_k, k4);
    ValueId present_v = place_present(past_v, v4);

    auto repeat = [&](ValueId x) {
        if (group == 1) return x;
        ValueId with_g = b.reshape(x, {bsz, kvc, C(1), total, d});
        ValueId grown = b.broadcast(with_g, {bsz, kvc, C(group), total, d});
        return b.reshape(grown, {bsz, C(heads), total, d});
    };
    ValueId k_rep = repeat(present_k);
    ValueId v_rep = repeat(present_v);

    ValueId scores = b.matmul(q4, k_rep, false, true);
    double scale_attr = c.attrs.float_or("scale", 0.0);
    double scale = scale_attr;
    if (scale_attr == 0.0) {
        auto dc = d.as_const();
        if (!dc) fail(ErrKind::Shape, "GQA head dim must be constant for the default scale");
        scale = 1.0 / std::sqrt((double)*dc);
    }
    scores = b.mul(scores, scalar(b, dt, scale));
    if (c.attrs.int_or("has_attention_bias", 0) != 0) scores = b.add(scores, in.back());

    // allow col ≤ qpos and, with a window, col ≥ qpos − window
    ValueId qpos = b.add(past_b, jrel);
    ValueId cols = b.reshape(b.iota(total, DType::I64), {one, one, one, total});
    ValueId allowed = b.cmp(CmpOp::Le, cols, qpos);
    if (window >= 0) {
        ValueId min_col = b.sub(qpos, scalar(b, DType::I64, (double)window));
        ValueId in_window = b.cmp(CmpOp::Ge, cols, min_col);
        allowed = b.binary(BinaryOp::And, allowed, in_window);
    }
    ValueId masked = b.select(allowed, scores, scalar(b, dt, -INFINITY));

    Attrs sa;
    sa.set("axis", AttrValue::of_int(3));
    TensorType mty = b.ty(masked);
    ValueId probs = b.composite("Softmax", sa, {masked}, {mty})[0];

    ValueId ctx = b.transpose(b.matmul(probs, v_rep), {0, 2, 1, 3});
    ValueId out = b.reshape(ctx, {bsz, seq, hidden});
    return {out, present_k, present_v};
}

Ins matmul_nbits(const Composite& c, const Ins& in, GraphBuilder& b) {
    if (in.size() < 3) fail(ErrKind::InvalidGraph, "MatMulNBits expects at least 3 inputs");
    ValueId a = in[0], bq = in[1], scales = in[2];
    int64_t bits = c.attrs.int_or("bits", 4);
    if (bits != 4) fail(ErrKind::Unsupported, "MatMulNBits with bits=" + std::to_string(bits));
    uint64_t k = (uint64_t)c.attrs.int_("K");
    uint64_t n = (uint64_t)c.attrs.int_("N");
    size_t block = (size_t)c.attrs.int_("block_size");

    DimExpr n_blocks = b.ty(bq).shape[1];
    ValueId scales2 = b.reshape(scales, {C(n), n_blocks});
    DimExpr padded_k = n_blocks * C(block);
    Ins deq_in = {bq, scales2};
    if (in.size() > 3) deq_in.push_back(in[3]);
    ValueId w = b.prim(Prim::dequantize(block, {C(n), padded_k}), deq_in);
    if (padded_k.as_const() != std::optional<uint64_t>(k)) w = slice1(b, w, 1, C(0), C(k));
    if (b.ty(w).dtype != b.ty(a).dtype) w = b.cast(w, b.ty(a).dtype);
    return {b.matmul(a, w, false, true)};
}

}  // namespace

const DecompositionRegistry& standard_decompositions() {
    static const DecompositionRegistry reg = [] {
        DecompositionRegistry r;
        r.register_("Softmax", softmax);
        r.register_("Gelu", gelu);
        r.register_("Trilu", trilu);
        r.register_("SimplifiedLayerNormalization", simplified_layer_norm);
        r.register_("com.microsoft.RotaryEmbedding", rotary_embedding);
        r.register_("com.microsoft.GemmaRotaryEmbedding", rotary_embedding);
        r.register_("com.microsoft.GroupQueryAttention", group_query_attention);
        r.register_("com.microsoft.MatMulNBits", matmul_nbits);
        return r;
    }();
    return reg;
}

Module inline_composites(Module m, const DecompositionRegistry& reg,
                         const std::function<bool(const Module&, const Node&)>& supports) {
    for (;;) {
        NodeId target = UINT32_MAX;
        for (NodeId i = 0; i < m.nodes.size(); i++)
            if (!m.nodes[i].is_prim && !supports(m, m.nodes[i])) {
                target = i;
                break;
            }
        if (target == UINT32_MAX) {
            eliminate_dead(m);
            return m;
        }
        Composite comp = m.nodes[target].composite;
        Ins inputs = m.nodes[target].inputs;
        Ins old_out = m.nodes[target].outputs;
        auto loc_name = m.nodes[target].loc_name;
        auto loc_op = m.nodes[target].loc_op;

        const DecompFn* fn = reg.get(comp.name);
        if (!fn)
            fail(ErrKind::Unsupported, "no kernel and no decomposition for composite '" + comp.name + "'" +
                                           (loc_name ? " (node " + *loc_name + ")" : std::string()));
        GraphBuilder b(std::move(m));
        b.set_loc(loc_name, loc_op);
        Ins new_out = (*fn)(comp, inputs, b);
        m = b.into_module();

        if (new_out.size() != old_out.size())
            fail(ErrKind::InvalidGraph, "decomposition of '" + comp.name + "' produced " + std::to_string(new_out.size()) +
                                            " outputs, composite declares " + std::to_string(old_out.size()));
        for (size_t i = 0; i < old_out.size(); i++) {
            const TensorType &ot = m.values[old_out[i]].ty, &nt = m.values[new_out[i]].ty;
            if (ot != nt)
                fail(ErrKind::InvalidGraph, "decomposition of '" + comp.name + "': declared output type " +
                                                ot.to_string(&m.symbols) + " but decomposition produces " +
                                                nt.to_string(&m.symbols));
            m.replace_uses(old_out[i], new_out[i]);
        }
        m.remove_nodes({target});
    }
}

}  // namespace ox
