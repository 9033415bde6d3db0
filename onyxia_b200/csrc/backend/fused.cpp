// Fused-composite registry (≙ standard_kernels,
// crates/onyxia-backend-wgpu/src/fused.rs:71-86). Registry membership is what
// `Backend::supports` reports; `accepts` narrows a kernel to the operand types
// it implements, every other instance of the composite is legalised through
// its decomposition.
#include <cmath>

#include "../kernels/common.cuh"
#include "runtime.hpp"

namespace oxrt {

using namespace ox;
using oxk::TRef;

namespace {

const TensorType& ty(const Module& m, ValueId v) { return m.values[v].ty; }
bool is_float(DType d) { return d == DType::F32 || d == DType::F16; }

// ── Softmax ──
bool softmax_accepts(const Module& m, const Node& n) {
    if (n.inputs.size() != 1) return false;
    const TensorType& x = ty(m, n.inputs[0]);
    if (!is_float(x.dtype) || x.shape.empty()) return false;
    auto* a = n.composite.attrs.get("axis");
    return a && a->kind == AttrValue::Int && (size_t)a->i == x.shape.size() - 1;
}
void softmax_lower(FusedCtx& c) { oxk::emit_softmax(c.em, c.ins[0], c.outs[0]); }

// ── SimplifiedLayerNormalization ──
bool rmsnorm_accepts(const Module& m, const Node& n) {
    if (n.inputs.size() != 2) return false;
    const TensorType &x = ty(m, n.inputs[0]), &w = ty(m, n.inputs[1]);
    if (!is_float(x.dtype) || w.dtype != x.dtype || x.shape.empty()) return false;
    return w.shape.size() == 1 && w.shape[0] == x.shape.back();
}
void rmsnorm_lower(FusedCtx& c) {
    double eps = c.node.composite.attrs.float_or("epsilon", 1e-5);
    oxk::emit_rmsnorm(c.em, c.ins[0], c.ins[1], c.outs[0], eps, nullptr, nullptr);
}

// ── Gelu ──
bool gelu_accepts(const Module& m, const Node& n) { return n.inputs.size() == 1 && is_float(ty(m, n.inputs[0]).dtype); }
void gelu_lower(FusedCtx& c) {
    bool tanh = c.node.composite.attrs.str_or("approximate", "none") == "tanh";
    oxk::emit_gelu(c.em, c.ins[0], c.outs[0], tanh, nullptr);
}

// ── RotaryEmbedding ──
// Head count and rotary width are resolved exactly like the decomposition
// (crates/onyxia-ir/src/decomp.rs:283-311).
bool rotary_geometry(const Module& m, const Node& n, int64_t* heads, int64_t* half) {
    const TensorType &x = ty(m, n.inputs[0]), &cosc = ty(m, n.inputs[2]);
    auto hidden = x.shape[2].as_const();
    auto cache_half = cosc.shape[1].as_const();
    if (!hidden || !cache_half) return false;
    int64_t nh = n.composite.attrs.int_or("num_heads", 0);
    int64_t h;
    if (nh > 0) h = nh;
    else {
        int64_t r = (int64_t)*cache_half * 2;
        h = (r > 0 && (int64_t)*hidden % r == 0) ? (int64_t)*hidden / r : 1;
    }
    if ((int64_t)*hidden % h != 0) return false;
    int64_t rdim = n.composite.attrs.int_or("rotary_embedding_dim", 0);
    int64_t hf = rdim == 0 ? (int64_t)*cache_half : rdim / 2;
    int64_t d = (int64_t)*hidden / h;
    if (hf <= 0 || 2 * hf > d || hf > (int64_t)*cache_half) return false;
    // the decomposition reshapes the gathered cache row to `half` columns
    if (hf != (int64_t)*cache_half) return false;
    *heads = h;
    *half = hf;
    return true;
}
bool rotary_accepts(const Module& m, const Node& n) {
    if (n.inputs.size() != 4) return false;
    if (n.composite.attrs.int_or("interleaved", 0) != 0) return false;
    const TensorType &x = ty(m, n.inputs[0]), &pos = ty(m, n.inputs[1]), &cosc = ty(m, n.inputs[2]), &sinc = ty(m, n.inputs[3]);
    if (!is_float(x.dtype) || x.shape.size() != 3 || pos.dtype != DType::I64 || pos.shape.size() != 2) return false;
    if (cosc.dtype != x.dtype || sinc.dtype != x.dtype || cosc.shape.size() != 2 || sinc.shape != cosc.shape) return false;
    int64_t h, hf;
    return rotary_geometry(m, n, &h, &hf);
}
// geometry is recomputed from concrete shapes at lowering time
void rotary_lower(FusedCtx& c) {
    int64_t hidden = c.ins[0].shape[2], cache_half = c.ins[2].shape[1];
    int64_t nh = c.node.composite.attrs.int_or("num_heads", 0);
    int64_t heads = nh > 0 ? nh : ((cache_half > 0 && hidden % (2 * cache_half) == 0) ? hidden / (2 * cache_half) : 1);
    oxk::emit_rotary(c.em, c.ins[0], c.ins[1], c.ins[2], c.ins[3], c.outs[0], heads, cache_half);
}

// ── GroupQueryAttention ──
bool gqa_accepts(const Module& m, const Node& n) {
    const Attrs& a = n.composite.attrs;
    if (n.inputs.size() < 6) return false;
    int64_t heads = a.int_or("num_heads", 0), kv = a.int_or("kv_num_heads", 0);
    if (heads <= 0 || kv <= 0 || heads % kv != 0) return false;
    bool rot = a.int_or("do_rotary", 0) != 0, bias = a.int_or("has_attention_bias", 0) != 0;
    if (n.inputs.size() != (size_t)(6 + (rot ? 2 : 0) + (bias ? 1 : 0))) return false;
    if (rot && a.int_or("rotary_interleaved", 0) != 0) return false;
    const TensorType &q = ty(m, n.inputs[0]), &k = ty(m, n.inputs[1]), &v = ty(m, n.inputs[2]);
    const TensorType &pk = ty(m, n.inputs[3]), &pv = ty(m, n.inputs[4]), &sl = ty(m, n.inputs[5]);
    if (!is_float(q.dtype) || k.dtype != q.dtype || v.dtype != q.dtype || pk.dtype != q.dtype || pv.dtype != q.dtype) return false;
    if (sl.dtype != DType::I32) return false;
    if (q.shape.size() != 3 || k.shape.size() != 3 || v.shape.size() != 3 || pk.shape.size() != 4 || pv.shape.size() != 4) return false;
    auto hidden = q.shape[2].as_const();
    if (!hidden || *hidden % (uint64_t)heads != 0) return false;
    uint64_t d = *hidden / (uint64_t)heads;
    if (d != 32 && d != 64 && d != 128 && d != 256) return false;
    if (pk.shape[3].as_const() != std::optional<uint64_t>(d) || pk.shape[1].as_const() != std::optional<uint64_t>((uint64_t)kv)) return false;
    if (pv.shape != pk.shape) return false;
    if (rot) {
        const TensorType &cosc = ty(m, n.inputs[6]), &sinc = ty(m, n.inputs[7]);
        if (cosc.dtype != q.dtype || sinc.dtype != q.dtype || cosc.shape.size() != 2 || sinc.shape != cosc.shape) return false;
        auto half = cosc.shape[1].as_const();
        if (!half || *half == 0 || 2 * *half > d) return false;
    }
    if (bias) {
        const TensorType& bt = ty(m, n.inputs.back());
        if (bt.dtype != q.dtype || bt.shape.size() != 4) return false;
    }
    if (a.float_or("scale", 0.0) == 0.0 && !q.shape[2].as_const()) return false;
    return true;
}
void gqa_lower(FusedCtx& c) {
    const Attrs& a = c.node.composite.attrs;
    oxk::GqaDesc d{};
    d.batch = c.ins[0].shape[0];
    d.seq = c.ins[0].shape[1];
    d.heads = a.int_("num_heads");
    d.kv_heads = a.int_("kv_num_heads");
    d.head_dim = c.ins[0].shape[2] / d.heads;
    d.past = c.ins[3].shape[2];
    double sc = a.float_or("scale", 0.0);
    d.scale = sc == 0.0 ? 1.0 / std::sqrt((double)d.head_dim) : sc;
    d.window = a.int_or("local_window_size", -1);
    bool rot = a.int_or("do_rotary", 0) != 0;
    d.has_bias = a.int_or("has_attention_bias", 0) != 0;
    const TRef *cosr = nullptr, *sinr = nullptr, *biasr = nullptr;
    if (rot) {
        cosr = &c.ins[6];
        sinr = &c.ins[7];
        d.rot_half = cosr->shape[1];
        d.cache_rows = cosr->shape[0];
        // ≙ the rope-cache bound of the reference kernel (fused.rs:417-422)
        if (d.past + d.seq > d.cache_rows)
            fail(ErrKind::Shape, "GQA rope cache has " + std::to_string(d.cache_rows) + " positions but the sequence reaches " +
                                     std::to_string(d.past + d.seq));
    }
    if (c.ins[5].numel() != d.batch)
        fail(ErrKind::Shape, "GQA seqlens_k has " + std::to_string(c.ins[5].numel()) + " elements for batch size " + std::to_string(d.batch));
    if (d.has_bias) {
        biasr = &c.ins.back();
        const auto& bs = biasr->shape;
        int64_t T = d.past + d.seq;
        bool ok = (bs[0] == d.batch || bs[0] == 1) && (bs[1] == d.heads || bs[1] == 1) && bs[2] == d.seq && bs[3] == T;
        if (!ok) fail(ErrKind::Shape, "GQA attention_bias does not broadcast over the scores");
        d.bias_b = bs[0];
        d.bias_h = bs[1];
    }
    d.in_place = c.kv_in_place;
    // A decode step on a cache that is appended to in place: size the launch for
    // the next multiple of 256 rows and pass the true length as a per-run scalar.
    if (d.in_place && d.seq == 1 && !d.has_bias) {
        d.t_bucket = (d.past + d.seq + 255) / 256 * 256;
        c.bucket = d.t_bucket;
        c.bucket_step = 256;
    }
    oxk::emit_gqa(c.em, d, c.ins[0], c.ins[1], c.ins[2], c.ins[3], c.ins[4], c.ins[5], cosr, sinr, biasr, c.outs[0], c.outs[1], c.outs[2]);
}

// ── MatMulNBits ──
bool nbits_accepts(const Module& m, const Node& n) {
    const Attrs& a = n.composite.attrs;
    if (n.inputs.size() < 3 || n.inputs.size() > 4) return false;
    if (a.int_or("bits", 4) != 4 || a.int_or("block_size", 0) != 32) return false;
    const TensorType &x = ty(m, n.inputs[0]), &w = ty(m, n.inputs[1]), &s = ty(m, n.inputs[2]);
    if (!is_float(x.dtype) || !is_float(s.dtype) || w.dtype != DType::U4 || x.shape.empty()) return false;
    int64_t K = a.int_or("K", 0), N = a.int_or("N", 0);
    if (K <= 0 || N <= 0) return false;
    auto wd = shape_as_static(w.shape);
    if (!wd || wd->size() != 3 || (*wd)[0] != (uint64_t)N || (*wd)[2] != 32 || (*wd)[1] != (uint64_t)((K + 31) / 32)) return false;
    if (x.shape.back().as_const() != std::optional<uint64_t>((uint64_t)K)) return false;
    auto sd = shape_as_static(s.shape);
    if (!sd) return false;
    uint64_t sn = 1;
    for (auto d : *sd) sn *= d;
    if (sn != (uint64_t)N * (*wd)[1]) return false;
    if (n.inputs.size() == 4) {
        const TensorType& z = ty(m, n.inputs[3]);
        auto zd = shape_as_static(z.shape);
        if (z.dtype != DType::U4 || !zd) return false;
        uint64_t zn = 1;
        for (auto d : *zd) zn *= d;
        if (zn != sn) return false;
    }
    // weights must be constants: their device copy is 16-byte aligned and immutable
    return m.values[n.inputs[1]].origin.kind == Origin::Const;
}
void nbits_lower(FusedCtx& c) {
    const Attrs& a = c.node.composite.attrs;
    oxk::NBitsDesc d{};
    d.k = a.int_("K");
    d.n = a.int_("N");
    d.block_size = 32;
    d.n_blocks = (d.k + 31) / 32;
    d.m = c.ins[0].numel() / d.k;
    d.act_dtype = c.ins[0].dtype;
    d.scale_dtype = c.ins[2].dtype;
    d.has_zp = c.ins.size() > 3;
    d.interleaved = c.weights_layout == 1;
    d.tiled = c.weights_layout == 2;
    oxk::emit_matmul_nbits(c.em, d, c.ins[0], c.ins[1], c.ins[2], d.has_zp ? &c.ins[3] : nullptr, c.outs[0]);
}

// ── onyxia.AllReduce (tensor parallelism) ──
bool allreduce_accepts(const Module& m, const Node& n) {
    if (n.inputs.size() != 1 || n.outputs.size() != 1) return false;
    const TensorType& t = ty(m, n.inputs[0]);
    return (t.dtype == DType::F16 || t.dtype == DType::F32) && t == ty(m, n.outputs[0]);
}
void allreduce_lower(FusedCtx& c) { oxk::emit_allreduce(c.em, c.ins[0], c.outs[0]); }

}  // namespace

}  // namespace oxrt

namespace oxk {
void emit_allreduce(Emitter& em, const TRef& x, const TRef& y) {
    if (x.numel() == 0) return;
    CollP p{};
    p.count = (unsigned long long)x.numel();
    p.dtype = x.dtype;
    LaunchRec r;
    r.coll = 1;
    r.params.resize(sizeof(CollP));
    std::memcpy(r.params.data(), &p, sizeof(CollP));
    r.relocs.push_back(Reloc{(uint32_t)offsetof(CollP, send), x.buf});
    r.relocs.push_back(Reloc{(uint32_t)offsetof(CollP, recv), y.buf});
    r.label = "allreduce";
    r.node = em.node;
    em.recs.push_back(std::move(r));
}
}  // namespace oxk

namespace oxrt {

const KernelRegistry& standard_kernels() {
    static const KernelRegistry reg = [] {
        KernelRegistry r;
        r.add({"Softmax", softmax_accepts, softmax_lower});
        r.add({"SimplifiedLayerNormalization", rmsnorm_accepts, rmsnorm_lower});
        r.add({"Gelu", gelu_accepts, gelu_lower});
        r.add({"com.microsoft.RotaryEmbedding", rotary_accepts, rotary_lower});
        r.add({"com.microsoft.GemmaRotaryEmbedding", rotary_accepts, rotary_lower});
        r.add({"com.microsoft.GroupQueryAttention", gqa_accepts, gqa_lower});
        r.add({"com.microsoft.MatMulNBits", nbits_accepts, nbits_lower});
        r.add({"onyxia.AllReduce", allreduce_accepts, allreduce_lower});
        return r;
    }();
    return reg;
}

}  // namespace oxrt
