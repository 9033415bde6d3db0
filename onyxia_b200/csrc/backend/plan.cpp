// Planning and execution: from a binding of the dimension symbols to a list of
// kernel launches with an arena layout, kept across runs, updated in place when
// only a few symbols move, and replayed as a CUDA graph.
//
// Behavioural model: WgpuSession::run
// (crates/onyxia-backend-wgpu/src/session.rs:532-611) — bind, evaluate shapes,
// register file, per-node dispatch, frees — restated so that the steady state
// of a decode loop costs one graph launch and a handful of parameter patches.
#include <algorithm>
#include <chrono>
#include <climits>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <cuda.h>

#include "../kernels/common.cuh"
#include "session.hpp"

namespace oxrt {

using namespace ox;
using oxk::Buf;
using oxk::TRef;

namespace {

// Best-fit allocator over byte offsets of the plan's arena.
struct OffsetAlloc {
    std::map<size_t, size_t> free_;  // offset → size
    size_t end = 0;
    static size_t round(size_t b) { return b == 0 ? 256 : (b + 255) / 256 * 256; }
    size_t alloc(size_t bytes) {
        bytes = round(bytes);
        auto best = free_.end();
        for (auto it = free_.begin(); it != free_.end(); ++it)
            if (it->second >= bytes && (best == free_.end() || it->second < best->second)) best = it;
        if (best != free_.end()) {
            size_t off = best->first, sz = best->second;
            free_.erase(best);
            if (sz > bytes) free_[off + bytes] = sz - bytes;
            return off;
        }
        if (!free_.empty()) {  // grow a trailing free block
            auto last = std::prev(free_.end());
            if (last->first + last->second == end) {
                size_t off = last->first;
                free_.erase(last);
                end = off + bytes;
                return off;
            }
        }
        size_t off = end;
        end += bytes;
        return off;
    }
    void release(size_t off, size_t bytes) {
        bytes = round(bytes);
        auto it = free_.emplace(off, bytes).first;
        auto next = std::next(it);
        if (next != free_.end() && it->first + it->second == next->first) {
            it->second += next->second;
            free_.erase(next);
        }
        if (it != free_.begin()) {
            auto prev = std::prev(it);
            if (prev->first + prev->second == it->first) {
                prev->second += it->second;
                free_.erase(it);
            }
        }
    }
};

// Rows a new KV buffer gets room for. Outgrowing it costs a step that copies every cache of the model into new
// buffers, through plans and graphs of their own (measured: 20–460 ms on the 1B model), so small caches get room for
// at least 4 096 more tokens and double; large ones (a batch of long sequences) grow by half.
int64_t grow_capacity(int64_t rows, int64_t row_bytes) {
    int64_t extra = std::max<int64_t>(256, rows / 2);
    if ((rows + std::max<int64_t>(4096, rows)) * row_bytes <= (int64_t)64 << 20) extra = std::max<int64_t>(4096, rows);
    else if ((rows + std::max<int64_t>(1024, rows)) * row_bytes <= (int64_t)64 << 20) extra = std::max<int64_t>(1024, rows);
    if (const char* e = std::getenv("ONYXIA_KV_ROOM")) {  // tests: a fixed number of spare rows, so that growth happens soon
        const long long v = std::atoll(e);
        if (v > 0) extra = v;
    }
    return (rows + extra + 63) / 64 * 64;
}

void add_syms(std::vector<SymId>& out, const DimExpr& e) {
    for (auto s : e.syms()) out.push_back(s);
}
void add_syms(std::vector<SymId>& out, const SymShape& s) {
    for (auto& d : s) add_syms(out, d);
}

bool same_bindings(const Bindings& a, const Bindings& b) {
    if (a.items().size() != b.items().size()) return false;
    for (auto& kv : a.items()) {
        auto v = b.get(kv.first);
        if (!v || *v != kv.second) return false;
    }
    return true;
}

inline bool moves_elements(PrimKind k) {
    return k == PrimKind::Transpose || k == PrimKind::Broadcast || k == PrimKind::Concat || k == PrimKind::Slice ||
           k == PrimKind::Gather || k == PrimKind::Scatter;
}

}  // namespace

// Which symbols can change a node's launch records: those in the types of its
// operands and results and in its own parameters (plus its fusion partner's).
void Session::collect_node_syms() {
    const Module& m = module_;
    auto of_node = [&](size_t i, std::vector<SymId>& out) {
        const Node& n = m.nodes[i];
        for (auto v : n.inputs) add_syms(out, m.values[v].ty.shape);
        for (auto v : n.outputs) add_syms(out, m.values[v].ty.shape);
        if (n.is_prim) {
            add_syms(out, n.prim.shape);
            add_syms(out, n.prim.len);
            for (auto& s : n.prim.specs) {
                add_syms(out, s.start);
                add_syms(out, s.end);
            }
        }
    };
    for (size_t i = 0; i < m.nodes.size(); i++) {
        std::vector<SymId> s;
        of_node(i, s);
        if (info_[i].fuse_with >= 0) of_node((size_t)info_[i].fuse_with, s);
        if (info_[i].absorbed_by >= 0) of_node((size_t)info_[i].absorbed_by, s);
        if (group_of_leader_[i] >= 0) {
            const GemvGroup& g = groups_[group_of_leader_[i]];
            for (auto mem : g.members) of_node(mem, s);
            for (int extra : {g.gelu_node, g.mul_node, g.norm2, g.slice, g.add, g.norm1})
                if (extra >= 0) of_node((size_t)extra, s);
        }
        std::sort(s.begin(), s.end());
        s.erase(std::unique(s.begin(), s.end()), s.end());
        info_[i].syms = std::move(s);
    }
}

std::vector<uint64_t> Session::structure_key(const std::vector<DTensor>& inputs, const std::vector<char>& kv_in_place) const {
    std::vector<uint64_t> key;
    key.reserve(inputs.size() + kv_in_place.size() / 64 + 2);
    for (auto& t : inputs) key.push_back((uint64_t)t.cap);
    uint64_t bits = 0;
    int nbits = 0;
    for (char c : kv_in_place) {
        bits = (bits << 1) | (uint64_t)(c != 0);
        if (++nbits == 64) {
            key.push_back(bits);
            bits = 0;
            nbits = 0;
        }
    }
    key.push_back(bits);
    return key;
}

bool Session::lower_step(Plan& plan, oxk::Emitter& em, size_t step, Bindings& bindings, const std::vector<DTensor>& inputs,
                         const std::vector<char>& kv_in_place, void* arena_ptr) {
    const Module& m = module_;
    OffsetAlloc* arena = static_cast<OffsetAlloc*>(arena_ptr);
    NodeId nid = order_[step];
    const Node& node = m.nodes[nid];
    em.begin_node((int)nid);
    try {
        bool fused_gqa = !node.is_prim && node.composite.name == "com.microsoft.GroupQueryAttention";
        for (size_t oi = 0; oi < node.outputs.size(); oi++) {
            ValueId o = node.outputs[oi];
            // ── shape ──
            std::vector<int64_t> shp;
            if (node.is_prim && node.prim.kind == PrimKind::Reshape) {
                // at most one unbound bare symbol is inferred from the element count
                // (crates/onyxia-ir/src/interp.rs:1138-1169)
                int64_t numel = plan.trefs[node.inputs[0]].numel();
                int unknown = -1;
                SymId unk_sym = 0;
                for (size_t i = 0; i < node.prim.shape.size(); i++) {
                    uint64_t val;
                    std::string why;
                    if (node.prim.shape[i].try_eval(bindings, &val, &why)) {
                        shp.push_back((int64_t)val);
                    } else {
                        auto s = node.prim.shape[i].as_sym();
                        if (s && unknown < 0) {
                            unknown = (int)i;
                            unk_sym = *s;
                            shp.push_back(0);
                        } else {
                            node.prim.shape[i].eval(bindings);
                        }
                    }
                }
                if (unknown >= 0) {
                    int64_t rest = 1;
                    for (size_t j = 0; j < shp.size(); j++)
                        if ((int)j != unknown) rest *= shp[j];
                    if (rest == 0 || numel % rest != 0)
                        fail(ErrKind::Runtime, "cannot infer reshape dim: " + std::to_string(numel) + " elements over " + std::to_string(rest));
                    shp[unknown] = numel / rest;
                    bindings.bind(unk_sym, (uint64_t)shp[unknown]);
                }
                int64_t out_n = 1;
                for (auto d : shp) out_n *= d;
                if (out_n != numel)
                    fail(ErrKind::Runtime, "reshape element count mismatch: input has " + std::to_string(numel) + " elements");
            } else {
                for (auto& d : m.values[o].ty.shape) shp.push_back((int64_t)d.eval(bindings));
            }

            // ── storage ──
            DType dt = m.values[o].ty.dtype;
            ValueId root = alias_root_[o];
            TRef tr;
            tr.dtype = (int)dt;
            tr.shape = std::move(shp);
            if (root != o) {
                plan.loc[o].kind = ValueLoc::Alias;
                plan.loc[o].index = root;
                tr.buf = plan.trefs[root].buf;
                if (plan.trefs[root].cap) fail(ErrKind::Unsupported, "reshape of a KV-cache view");
                plan.trefs[o] = std::move(tr);
                continue;
            }
            size_t bytes = dtype_storage_bytes(dt, (uint64_t)tr.numel());
            if (is_output_root_[o]) {
                OutBuf ob;
                ob.bytes = bytes;
                if (fused_gqa && oi >= 1 && tr.shape.size() == 4) {
                    int s = (int)oi - 1;
                    if (kv_in_place[nid]) {
                        int in_idx = gqa_past_input_[s][nid];
                        ob.alias_input = in_idx;
                        tr.cap = inputs[in_idx].cap;
                    } else {
                        tr.cap = grow_capacity(tr.shape[2], (int64_t)dtype_storage_bytes(dt, (uint64_t)(tr.shape[0] * tr.shape[1] * tr.shape[3])));
                        ob.kv_cap = tr.cap;
                        ob.bytes = dtype_storage_bytes(dt, (uint64_t)(tr.shape[0] * tr.shape[1] * tr.cap * tr.shape[3]));
                    }
                    ob.kv_rows = tr.shape[2];
                }
                if (arena) {
                    plan.loc[o].kind = ValueLoc::Output;
                    plan.loc[o].index = (uint32_t)plan.out_bufs.size();
                    plan.out_bufs.push_back(ob);
                } else {
                    plan.out_bufs[plan.loc[o].index] = ob;
                }
            } else if (arena) {
                plan.loc[o].kind = ValueLoc::Arena;
                plan.loc[o].offset = arena->alloc(bytes);
                plan.arena_size[o] = OffsetAlloc::round(bytes);
            } else if (OffsetAlloc::round(bytes) > plan.arena_size[o]) {
                return false;  // the value outgrew its slot: the arena has to be laid out again
            }
            tr.buf = Buf{o, 0};
            plan.trefs[o] = std::move(tr);
        }

        // ── kernels ──
        if (info_[nid].absorbed_by < 0) {
            std::vector<TRef> ins, outs;
            for (auto v : node.inputs) ins.push_back(plan.trefs[v]);
            for (auto v : node.outputs) outs.push_back(plan.trefs[v]);
            if (group_of_leader_[nid] >= 0) {
                lower_group(em, groups_[group_of_leader_[nid]], plan, bindings);
            } else if (node.is_prim && node.prim.kind == PrimKind::Reshape) {
                // a view: nothing to launch
            } else if (info_[nid].fuse_kind == FUSE_GEGLU) {
                const Node& g = m.nodes[info_[nid].fuse_with];
                bool tanh = g.composite.attrs.str_or("approximate", "none") == "tanh";
                oxk::emit_gelu(em, plan.trefs[g.inputs[0]], outs[0], tanh, &ins[1]);
            } else if (info_[nid].fuse_kind == FUSE_ADD_NORM) {
                const Node& a = m.nodes[info_[nid].fuse_with];
                double eps = node.composite.attrs.float_or("epsilon", 1e-5);
                TRef sum = plan.trefs[a.outputs[0]];
                oxk::emit_rmsnorm(em, plan.trefs[a.inputs[0]], ins[1], outs[0], eps, &plan.trefs[a.inputs[1]], &sum);
            } else if (node.is_prim && moves_elements(node.prim.kind) && !outs.empty() && dtype_is_packed((DType)outs[0].dtype)) {
                // Packed nibbles have no address of their own: the interpreter moves them through its integer domain
                // (crates/onyxia-ir/src/interp.rs:579-748, types.rs:7-11). Here: widen every packed operand to bytes,
                // move the bytes, pack the result. Bit-exact; two extra launches per operand.
                const DType byte_dt = (DType)outs[0].dtype == DType::U4 ? DType::U8 : DType::I8;
                auto bytes_like = [&](const TRef& t) {
                    TRef b;
                    b.dtype = (int)byte_dt;
                    b.shape = t.shape;
                    b.buf = em.scratch((size_t)std::max<int64_t>(t.numel(), 1));
                    return b;
                };
                std::vector<TRef> wide = ins;
                for (size_t i = 0; i < ins.size(); i++)
                    if (dtype_is_packed((DType)ins[i].dtype)) {
                        wide[i] = bytes_like(ins[i]);
                        if (ins[i].numel()) oxk::emit_cast(em, ins[i], wide[i]);
                    }
                TRef moved = bytes_like(outs[0]);
                lower_prim(em, node, bindings, wide, {moved});
                if (outs[0].numel()) oxk::emit_cast(em, moved, outs[0]);
            } else if (node.is_prim) {
                lower_prim(em, node, bindings, ins, outs);
            } else {
                FusedCtx fc{em, node, ins, outs, (bool)kv_in_place[nid], false};
                if (node.inputs.size() > 1) fc.weights_layout = interleaved_[node.inputs[1]];
                info_[nid].fused->lower(fc);
                plan.node_bucket[nid] = fc.bucket;
                plan.node_bucket_step[nid] = fc.bucket_step;
            }
            for (size_t j = 0; j < em.dyn_vals.size(); j++) plan.dyn_host[(size_t)nid * oxk::kDynPerNode + j] = em.dyn_vals[j];
            if (!em.dyn_vals.empty()) plan.dyn_used = true;
        }
    } catch (const Error& e) {
        if (e.kind == ErrKind::Binding) throw;
        std::string kind = node.is_prim ? node.prim.name() : node.composite.name;
        std::string loc = node.loc_name ? *node.loc_name : "<unnamed>";
        fail(ErrKind::Runtime, kind + " (node '" + loc + "'): " + e.what());
    } catch (const std::exception& e) {
        std::string kind = node.is_prim ? node.prim.name() : node.composite.name;
        std::string loc = node.loc_name ? *node.loc_name : "<unnamed>";
        fail(ErrKind::Runtime, kind + " (node '" + loc + "'): " + e.what());
    }
    if (arena)
        for (auto v : deaths_[step])
            if (plan.loc[v].kind == ValueLoc::Arena) arena->release(plan.loc[v].offset, plan.arena_size[v]);
    return true;
}

// One launch for a group of MatMulNBits nodes with its prologue and epilogue.
void Session::lower_group(oxk::Emitter& em, const GemvGroup& g, Plan& plan, const Bindings& bindings) {
    const Module& m = module_;
    oxk::NBitsGroup gr{};
    gr.k = g.k;
    gr.has_zp = g.has_zp;
    gr.n_seg = (int)g.members.size();
    for (size_t i = 0; i < g.members.size(); i++) {
        const Node& n = m.nodes[g.members[i]];
        gr.seg_n[i] = n.composite.attrs.int_("N");
        gr.y[i] = plan.trefs[n.outputs[0]];
    }
    gr.geglu = g.geglu;
    if (g.geglu) gr.y[0] = plan.trefs[m.nodes[g.mul_node].outputs[0]];
    const TRef tiles = plan.trefs[m.nodes[g.members[0]].inputs[1]];  // the group's tile stream lives in the slot of the first member's weight constant
    TRef src = plan.trefs[g.src];
    TRef w1, w2, res, sum;
    if (g.norm1 >= 0) {
        w1 = plan.trefs[m.nodes[g.norm1].inputs[1]];
        gr.eps1 = m.nodes[g.norm1].composite.attrs.float_or("epsilon", 1e-5);
    }
    if (g.add >= 0) {
        res = plan.trefs[g.res];
        sum = plan.trefs[m.nodes[g.add].outputs[0]];
    }
    if (g.norm2 >= 0) {
        w2 = plan.trefs[m.nodes[g.norm2].inputs[1]];
        gr.eps2 = m.nodes[g.norm2].composite.attrs.float_or("epsilon", 1e-5);
    }
    if (g.slice >= 0) {
        // Which rows of the chain's [rows, K] operands the slice keeps. When they are one contiguous range the prologue
        // simply starts there; otherwise the chain runs as separate launches in front of the slice.
        const Node& sl = m.nodes[g.slice];
        const std::vector<int64_t>& shp = plan.trefs[sl.inputs[0]].shape;
        const size_t rank = shp.size();
        std::vector<int64_t> lo(rank, 0), hi(shp);
        for (auto& sp : sl.prim.specs) {
            lo[sp.axis] = (int64_t)sp.start.eval(bindings);
            hi[sp.axis] = (int64_t)sp.end.eval(bindings);
            if (lo[sp.axis] < 0 || hi[sp.axis] > shp[sp.axis] || lo[sp.axis] > hi[sp.axis]) fail(ErrKind::Runtime, "slice bounds outside the tensor");
        }
        size_t j = 0;
        while (j + 1 < rank && lo[j] == 0 && hi[j] == shp[j]) j++;  // first axis that is cut (rank − 1: none)
        bool contiguous = true;
        for (size_t a = 0; a < j && j + 1 < rank; a++) contiguous = contiguous && shp[a] == 1;
        for (size_t a = j + 1; a + 1 < rank; a++) contiguous = contiguous && lo[a] == 0 && hi[a] == shp[a];
        if (contiguous) {
            int64_t inner = 1;
            for (size_t a = j + 1; a + 1 < rank; a++) inner *= shp[a];
            const int64_t row0 = j + 1 < rank ? lo[j] * inner : 0;
            int64_t rows = 1;
            for (size_t a = 0; a + 1 < rank; a++) rows *= hi[a] - lo[a];
            const int64_t off = row0 * g.k * 2;  // f16 rows
            auto rows_of = [&](TRef& t) {
                t.buf.off += off;
                t.shape = {rows, g.k};
            };
            rows_of(src);
            if (g.add >= 0) {
                rows_of(res);
                rows_of(sum);
            }
        } else {
            TRef cur = src;
            if (g.norm1 >= 0) {
                const TRef out = plan.trefs[m.nodes[g.norm1].outputs[0]];
                oxk::emit_rmsnorm(em, cur, w1, out, gr.eps1, nullptr, nullptr);
                cur = out;
            }
            if (g.add >= 0) {
                const Node& ad = m.nodes[g.add];
                // the operands in graph order: one of them is what the step above wrote (or the plain source)
                lower_prim(em, ad, bindings, {plan.trefs[ad.inputs[0]], plan.trefs[ad.inputs[1]]}, {sum});
                cur = sum;
            }
            const TRef cut = plan.trefs[sl.outputs[0]];
            if (g.slice_last) {  // … → norm2 → Slice → the matrices
                const TRef normed = plan.trefs[m.nodes[g.norm2].outputs[0]];
                oxk::emit_rmsnorm(em, cur, w2, normed, gr.eps2, nullptr, nullptr);
                lower_prim(em, sl, bindings, {normed}, {cut});
            } else {             // … → Slice → norm2 (as the launch's prologue) → the matrices
                lower_prim(em, sl, bindings, {cur}, {cut});
                if (g.norm2 >= 0) gr.w2 = &w2;
            }
            src = cut;
            gr.m = src.numel() / g.k;
            oxk::emit_nbits_group(em, gr, src, tiles);
            return;
        }
    }
    gr.m = src.numel() / g.k;
    if (g.norm1 >= 0) gr.w1 = &w1;
    if (g.add >= 0) {
        gr.res = &res;
        gr.sum_out = &sum;
    }
    if (g.norm2 >= 0) gr.w2 = &w2;
    oxk::emit_nbits_group(em, gr, src, tiles);
}

void Session::finish_outputs(Plan& plan) {
    const Module& m = module_;
    plan.outputs.clear();
    for (auto& o : m.outputs) {
        OutSpec s;
        s.name = o.first;
        s.value = o.second;
        s.dtype = m.values[o.second].ty.dtype;
        s.shape = plan.trefs[o.second].shape;
        s.cap = plan.trefs[o.second].cap;
        plan.outputs.push_back(std::move(s));
    }
}

std::unique_ptr<Plan> Session::build_plan(const Bindings& bindings_in, const std::vector<DTensor>& inputs,
                                          const std::vector<char>& kv_in_place) {
    const Module& m = module_;
    auto plan = std::make_unique<Plan>();
    size_t nv = m.values.size();
    plan->loc.assign(nv, ValueLoc{});
    plan->trefs.assign(nv, TRef{});
    plan->arena_size.assign(nv, 0);
    plan->node_recs.assign(m.nodes.size(), {0, 0});
    plan->dyn_host.assign(m.nodes.size() * oxk::kDynPerNode + 1, 0);  // the last slot holds the run's epoch
    plan->node_bucket.assign(m.nodes.size(), 0);
    plan->node_bucket_step.assign(m.nodes.size(), 0);
    plan->structure = structure_key(inputs, kv_in_place);
    Bindings bindings = bindings_in;

    for (ValueId v = 0; v < nv; v++) {
        const ValueDef& def = m.values[v];
        if (def.origin.kind == Origin::Const) {
            plan->loc[v].kind = ValueLoc::Const;
            plan->trefs[v] = TRef{Buf{v, 0}, (int)def.ty.dtype, consts_[v].shape, 0};
        } else if (def.origin.kind == Origin::Input && input_index_[v] >= 0) {
            const DTensor& t = inputs[input_index_[v]];
            plan->loc[v].kind = ValueLoc::Input;
            plan->loc[v].index = (uint32_t)input_index_[v];
            plan->trefs[v] = TRef{Buf{v, 0}, (int)def.ty.dtype, t.shape, t.cap};
        }
    }

    OffsetAlloc arena;
    oxk::Emitter em;
    for (size_t step = 0; step < order_.size(); step++) {
        uint32_t begin = (uint32_t)em.recs.size();
        lower_step(*plan, em, step, bindings, inputs, kv_in_place, &arena);
        plan->node_recs[order_[step]] = {begin, (uint32_t)em.recs.size() - begin};
    }
    plan->arena_bytes = arena.end;
    plan->scratch_bytes = em.scratch_bytes;
    plan->recs = std::move(em.recs);
    plan->bindings = bindings;
    finish_outputs(*plan);
    fuse_persistent(*plan);
    plans_built++;
    return plan;
}

// Re-lower only the nodes that depend on a symbol whose value changed. Returns
// false when the plan cannot be patched (a different launch count, a value
// that outgrew its arena slot, symbols bound while running): the caller then
// builds a new plan.
bool Session::update_plan(Plan& plan, const Bindings& bindings_in, const std::vector<DTensor>& inputs,
                          const std::vector<char>& kv_in_place) {
    const Module& m = module_;
    if (plan.bindings.items().size() != bindings_in.items().size()) return false;  // late-bound symbols involved
    std::vector<SymId> changed;
    for (auto& kv : bindings_in.items()) {
        auto old = plan.bindings.get(kv.first);
        if (!old) return false;
        if (*old != kv.second) changed.push_back(kv.first);
    }
    std::sort(changed.begin(), changed.end());
    Bindings bindings = bindings_in;
    // inputs first: their shapes follow the new binding
    for (size_t i = 0; i < m.inputs.size(); i++) plan.trefs[m.inputs[i].second].shape = inputs[i].shape;
    size_t scratch = plan.scratch_bytes;
    for (size_t step = 0; step < order_.size(); step++) {
        NodeId nid = order_[step];
        const auto& syms = info_[nid].syms;
        bool hit = false;
        for (auto s : syms)
            if (std::binary_search(changed.begin(), changed.end(), s)) {
                hit = true;
                break;
            }
        if (!hit) continue;
        oxk::Emitter em;
        if (!lower_step(plan, em, step, bindings, inputs, kv_in_place, nullptr)) return false;
        auto range = plan.node_recs[nid];
        if (em.recs.size() != range.second) return false;
        for (uint32_t i = 0; i < range.second; i++) plan.recs[range.first + i] = std::move(em.recs[i]);
        scratch = std::max(scratch, em.scratch_bytes);
    }
    plan.scratch_bytes = scratch;
    plan.bindings = bindings;
    finish_outputs(plan);
    fuse_persistent(plan);
    plans_updated++;
    return true;
}

// Builds the list of launches a run executes. Every maximal run of consecutive records that carry a
// persistent-operation descriptor becomes one launch of the persistent step kernel; the launch is
// rebuilt only when the operations it was built from changed.
void Session::fuse_persistent(Plan& plan) {
    static const bool disabled = [] {
        const char* e = std::getenv("ONYXIA_DISABLE_PERSIST");  // diagnostics: keep one launch per operation
        return e && std::atoi(e) != 0;
    }();
    const bool enabled = !disabled && !opt_.without_fused && !opt_.disable_pattern_fusion && !opt_.disable_persist;
    const auto& recs = plan.recs;
    const size_t max_ops = (size_t)oxk::persist_max_ops();
    const Buf epoch{oxk::kSlotDyn, (int64_t)((plan.dyn_host.size() - 1) * sizeof(int64_t))};
    plan.launches.clear();
    std::vector<Plan::PersistRun> runs;
    size_t xoff = 0, i = 0;
    while (i < recs.size()) {
        size_t j = i;
        while (enabled && j < recs.size() && recs[j].pop && j - i < max_ops) j++;
        if (j - i >= 2) {
            Plan::PersistRun run;
            const size_t idx = runs.size();
            bool cached = idx < plan.persist_runs.size() && plan.persist_runs[idx].ops.size() == j - i && plan.persist_runs[idx].xoff == xoff;
            for (size_t k = i; cached && k < j; k++) cached = oxk::same_op(plan.persist_runs[idx].ops[k - i], *recs[k].pop);
            if (cached) {
                run = std::move(plan.persist_runs[idx]);
            } else {
                std::vector<const oxk::PersistOp*> ops;
                for (size_t k = i; k < j; k++) {
                    run.ops.push_back(*recs[k].pop);
                    ops.push_back(recs[k].pop.get());
                }
                run.xoff = xoff;
                std::string why;
                run.ok = oxk::build_persist_launch(ops, epoch, &run.launch, &why);
                static const bool debug = std::getenv("ONYXIA_PERSIST_DEBUG") != nullptr;  // diagnostics
                if (debug) std::fprintf(stderr, "persistent step: %zu operations: %s\n", ops.size(), run.ok ? "fused" : why.c_str());
                if (run.ok)  // this run's words live after those of the runs before it
                    for (auto& rl : run.launch.rec.relocs)
                        if (rl.buf.slot == oxk::kSlotXbuf) rl.buf.off += (int64_t)xoff;
            }
            const bool ok = run.ok;
            if (ok) xoff += (run.launch.xbuf_bytes + 255) / 256 * 256;
            runs.push_back(std::move(run));
            if (ok) {
                plan.launches.push_back(nullptr);  // patched below, once `runs` no longer moves
                i = j;
                continue;
            }
        }
        if (j == i) j = i + 1;
        for (size_t k = i; k < j; k++) plan.launches.push_back(&recs[k]);
        i = j;
    }
    plan.persist_runs = std::move(runs);
    size_t r = 0;
    for (auto& l : plan.launches)
        if (!l) {
            while (!plan.persist_runs[r].ok) r++;
            l = &plan.persist_runs[r++].launch.rec;
        }
    plan.xbuf_bytes = xoff;
    if (xoff) plan.dyn_used = true;
}

void Session::lower_prim(oxk::Emitter& em, const Node& node, const Bindings& b, const std::vector<TRef>& ins,
                         const std::vector<TRef>& outs) {
    const Prim& p = node.prim;
    const TRef& y = outs[0];
    for (auto& t : ins)
        if (t.cap) fail(ErrKind::Unsupported, "a KV-cache view reached a primitive; it should have been packed first");
    if (y.numel() == 0) return;
    switch (p.kind) {
        case PrimKind::Unary: oxk::emit_unary(em, p.op, ins[0], y); break;
        case PrimKind::Binary: oxk::emit_binary(em, p.op, ins[0], ins[1], y); break;
        case PrimKind::Compare: oxk::emit_compare(em, p.op, ins[0], ins[1], y); break;
        case PrimKind::Select: oxk::emit_select(em, ins[0], ins[1], ins[2], y); break;
        case PrimKind::Cast: oxk::emit_cast(em, ins[0], y); break;
        case PrimKind::MatMul:
            if (ins[0].numel() == 0 || ins[1].numel() == 0) fail(ErrKind::Unsupported, "matmul with an empty contraction dimension");
            oxk::emit_matmul(em, ins[0], ins[1], y, p.trans_a, p.trans_b);
            break;
        case PrimKind::Reduce: oxk::emit_reduce(em, p.op, ins[0], y, p.axes); break;
        case PrimKind::Reshape: break;
        case PrimKind::Transpose: oxk::emit_transpose(em, ins[0], y, p.axes); break;
        case PrimKind::Broadcast: oxk::emit_broadcast(em, ins[0], y); break;
        case PrimKind::Concat: oxk::emit_concat(em, ins, y, p.axis); break;
        case PrimKind::Slice: {
            size_t rank = ins[0].shape.size();
            std::vector<int64_t> starts(rank, 0), steps(rank, 1);
            for (auto& s : p.specs) {
                int64_t start = (int64_t)s.start.eval(b), end = (int64_t)s.end.eval(b);
                int64_t dim = ins[0].shape[s.axis];
                int64_t len = y.shape[s.axis];
                int64_t last = start + (len - 1) * s.step;
                if (len > 0 && (start < 0 || start >= dim || last < 0 || last >= dim))
                    fail(ErrKind::Runtime, "slice [" + std::to_string(start) + ", " + std::to_string(end) + ") step " +
                                               std::to_string(s.step) + " reads outside dim " + std::to_string(dim));
                starts[s.axis] = start;
                steps[s.axis] = s.step;
            }
            oxk::emit_slice(em, ins[0], y, starts, steps);
            break;
        }
        case PrimKind::Gather: oxk::emit_gather(em, ins[0], ins[1], y, p.axis); break;
        case PrimKind::Scatter: oxk::emit_scatter(em, ins[0], ins[1], ins[2], y); break;
        case PrimKind::Iota: oxk::emit_iota(em, y); break;
        case PrimKind::DimValues: {
            std::vector<int64_t> vals;
            for (auto& e : p.shape) vals.push_back(e.eval_signed(b));
            oxk::emit_dim_values(em, vals, y);
            break;
        }
        case PrimKind::Dequantize:
            oxk::emit_dequantize(em, ins[0], ins[1], ins.size() > 2 ? &ins[2] : nullptr, y, (int64_t)p.block_size);
            break;
    }
}

// ───────────────────────────── execution ────────────────────────────────
cudaEvent_t Session::prof_event() {
    if (!prof_free_.empty()) {
        cudaEvent_t e = prof_free_.back();
        prof_free_.pop_back();
        return e;
    }
    cudaEvent_t e;
    OX_CUDA(cudaEventCreate(&e));
    return e;
}

std::vector<Timing> Session::take_timings() {
    OX_CUDA(cudaSetDevice(device_));
    OX_CUDA(cudaStreamSynchronize(stream_));
    std::vector<Timing> out;
    for (auto& r : prof_) {
        float ms = 0.f;
        OX_CUDA(cudaEventElapsedTime(&ms, r.a, r.b));
        Timing t;
        t.kernel = r.kernel;
        t.node = (r.node >= 0 && (size_t)r.node < info_.size()) ? info_[r.node].label : "";
        t.time_ns = (uint64_t)(ms * 1e6f);
        out.push_back(std::move(t));
        prof_free_.push_back(r.a);
        prof_free_.push_back(r.b);
    }
    prof_.clear();
    return out;
}

// Encodes a tiled 2-D f16 tensor map (128-byte swizzle, zero fill outside the tensor) for the address a
// record's tensor has in this run. The driver entry point is looked up through the runtime, so the
// library still has no link-time dependency on the driver.
static void encode_tensor_map(const oxk::TmapReloc& tm, void* base, uint8_t* params) {
    uint8_t* dst = params + tm.field_off;
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0) {
        // only known now: the tensor is a view at an odd offset of its buffer
        if (tm.enable_off == 0xFFFFFFFFu) fail(ErrKind::Runtime, "a tensor read through a tensor map is not 16-byte aligned");
        const int32_t off = 0;
        std::memcpy(params + tm.enable_off, &off, sizeof(off));
        return;
    }
    using Encode = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static Encode encode = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn)
            fail(ErrKind::Runtime, "cuTensorMapEncodeTiled is not available from this driver");
        return reinterpret_cast<Encode>(fn);
    }();
    alignas(64) CUtensorMap map;
    const cuuint64_t dims[2] = {tm.dim0, tm.dim1};
    const cuuint64_t strides[1] = {tm.stride1_bytes};
    const cuuint32_t box[2] = {tm.box0, tm.box1};
    const cuuint32_t elem[2] = {1, 1};
    CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) fail(ErrKind::Runtime, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)rc));
    std::memcpy(dst, &map, sizeof(map));
}

// One launch of a record with its parameter bytes. Kernels written for
// programmatic dependent launch get the stream-serialisation attribute, so they
// may begin while the launch before them is still running.
void Session::launch_rec(const oxk::LaunchRec& r, void* param_bytes, bool allow_pdl) {
    if (r.coll) {
        oxk::CollP c;
        std::memcpy(&c, param_bytes, sizeof(c));
        Communicator* comm = backend_.communicator();
        if (!comm) fail(ErrKind::Runtime, "all-reduce without a tensor-parallel group");
        comm->allreduce_sum(c.send, c.recv, (size_t)c.count, (DType)c.dtype, stream_, d_err_, r.node);
        return;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = r.grid;
    cfg.blockDim = r.block;
    cfg.dynamicSmemBytes = r.smem;
    cfg.stream = stream_;
    cudaLaunchAttribute attr[3];
    unsigned n_attr = 0;
    static const bool coop_off = [] {
        const char* e = std::getenv("ONYXIA_PERSIST_COOP");  // diagnostics: "0" launches the persistent kernel the ordinary way
        return e && std::atoi(e) == 0;
    }();
    if (r.cooperative && !coop_off) {
        attr[n_attr].id = cudaLaunchAttributeCooperative;
        attr[n_attr].val.cooperative = 1;
        n_attr++;
    }
    if (allow_pdl && r.pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        n_attr++;
    }
    if (r.cluster.x) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = r.cluster.x;
        attr[n_attr].val.clusterDim.y = r.cluster.y;
        attr[n_attr].val.clusterDim.z = r.cluster.z;
        n_attr++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    void* args[1] = {param_bytes};
    OX_CUDA(cudaLaunchKernelExC(&cfg, r.func, args));
}

// The plan's launch list as a CUDA graph, recorded by capturing the launches so
// that programmatic-dependent-launch edges are kept. The node created by each
// launch is remembered for later parameter updates.
void Session::build_graph(Plan& plan, const std::vector<std::vector<uint8_t>>& params) {
    if (plan.exec) cudaGraphExecDestroy(plan.exec);
    if (plan.graph) cudaGraphDestroy(plan.graph);
    plan.exec = nullptr;
    plan.graph = nullptr;
    plan.graph_nodes.clear();
    OX_CUDA(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeRelaxed));
    try {
        for (size_t i = 0; i < plan.launches.size(); i++) {
            launch_rec(*plan.launches[i], const_cast<uint8_t*>(params[i].data()), !opt_.disable_pdl);
            cudaStreamCaptureStatus status;
            const cudaGraphNode_t* deps = nullptr;
            size_t n_deps = 0;
            OX_CUDA(cudaStreamGetCaptureInfo_v3(stream_, &status, nullptr, nullptr, &deps, nullptr, &n_deps));
            if (plan.launches[i]->coll) {  // a collective may record several nodes; it is never patched in place
                plan.graph_nodes.push_back(nullptr);
                continue;
            }
            if (status != cudaStreamCaptureStatusActive || n_deps != 1)
                fail(ErrKind::Runtime, "internal: stream capture lost track of a launch");
            plan.graph_nodes.push_back(deps[0]);
        }
    } catch (...) {
        cudaGraph_t dead = nullptr;
        cudaStreamEndCapture(stream_, &dead);
        if (dead) cudaGraphDestroy(dead);
        cudaGetLastError();
        plan.graph_nodes.clear();
        throw;
    }
    OX_CUDA(cudaStreamEndCapture(stream_, &plan.graph));
    OX_CUDA(cudaGraphInstantiate(&plan.exec, plan.graph, 0));
    plan.graph_params = params;
    plan.graph_grids.clear();
    plan.graph_clusters.clear();
    plan.graph_funcs.clear();
    for (auto* r : plan.launches) {
        plan.graph_grids.push_back(r->grid);
        plan.graph_clusters.push_back(r->cluster);
        plan.graph_funcs.push_back(r->func);
    }
}

void Session::execute(Plan& plan, const std::vector<DTensor>& inputs, std::vector<BufferRef>& out_bufs) {
    size_t need = plan.arena_bytes + plan.scratch_bytes + 512;
    if (!plan.arena || plan.arena->bytes < need) {
        // leave head-room so a growing scratch area does not move the arena at every step
        plan.arena = pool_->alloc(plan.arena_bytes + plan.scratch_bytes * 2 + 512);
    }
    if (plan.dyn_used && !plan.dyn_dev) plan.dyn_dev = pool_->alloc(plan.dyn_host.size() * sizeof(int64_t));
    if (plan.xbuf_bytes && (!plan.xbuf || plan.xbuf->bytes < plan.xbuf_bytes)) {
        // tags of earlier epochs never match again, so only a fresh area has to be cleared
        plan.xbuf = pool_->alloc(plan.xbuf_bytes);
        OX_CUDA(cudaMemsetAsync(plan.xbuf->ptr, 0, plan.xbuf->bytes, stream_));
    }
    if (plan.xbuf_bytes) {  // a fresh non-zero 32-bit tag for this run's words
        if ((++plan.epoch & 0xFFFFFFFFull) == 0) ++plan.epoch;
        plan.dyn_host.back() = (int64_t)(plan.epoch & 0xFFFFFFFFull);
    }
    char* arena_base = (char*)plan.arena->ptr;
    size_t scratch_off = (plan.arena_bytes + 255) / 256 * 256;

    out_bufs.clear();
    for (auto& ob : plan.out_bufs) {
        if (ob.alias_input >= 0) out_bufs.push_back(inputs[ob.alias_input].buf);
        else out_bufs.push_back(pool_->alloc(std::max<size_t>(ob.bytes, 1)));
    }

    auto resolve = [&](const Buf& buf) -> void* {
        switch (buf.slot) {
            case oxk::kSlotErr: return (void*)d_err_;
            case oxk::kSlotNull: return nullptr;
            case oxk::kSlotCounters: return (void*)d_counters_;
            case oxk::kSlotDyn: return (char*)plan.dyn_dev->ptr + buf.off;
            case oxk::kSlotScratch: return arena_base + scratch_off + buf.off;
            case oxk::kSlotXbuf: return (char*)plan.xbuf->ptr + buf.off;
            default: break;
        }
        const ValueLoc& l = plan.loc[buf.slot];
        char* base = nullptr;
        switch (l.kind) {
            case ValueLoc::Arena: base = arena_base + l.offset; break;
            case ValueLoc::Const: base = (char*)consts_[buf.slot].ptr(); break;
            case ValueLoc::Input: base = (char*)inputs[l.index].ptr(); break;
            case ValueLoc::Output: base = (char*)out_bufs[l.index]->ptr; break;
            default: fail(ErrKind::Runtime, "internal: unresolved value slot");
        }
        return base + buf.off;
    };

    // per-run scalars: staged through a small ring of pinned copies so the host
    // may run ahead of the device
    if (plan.dyn_used) {
        size_t bytes = plan.dyn_host.size() * sizeof(int64_t);
        if (!plan.dyn_pinned) {
            OX_CUDA(cudaMallocHost((void**)&plan.dyn_pinned, bytes * Plan::kDynRing));
            for (auto& e : plan.dyn_events) OX_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        }
        unsigned slot = plan.dyn_cursor++ % Plan::kDynRing;
        if (plan.dyn_cursor > Plan::kDynRing) OX_CUDA(cudaEventSynchronize(plan.dyn_events[slot]));
        int64_t* stage = plan.dyn_pinned + (size_t)slot * plan.dyn_host.size();
        std::memcpy(stage, plan.dyn_host.data(), bytes);
        OX_CUDA(cudaMemcpyAsync(plan.dyn_dev->ptr, stage, bytes, cudaMemcpyHostToDevice, stream_));
        OX_CUDA(cudaEventRecord(plan.dyn_events[slot], stream_));
    }

    plan.uses++;
    const size_t n = plan.launches.size();
    bool use_graph = !profiling && !opt_.disable_graphs && n >= 2 && plan.uses >= 2;

    if (use_graph) {
        bool rebuild = !plan.exec || plan.graph_nodes.size() != n;
        // patched parameter bytes for every launch
        static thread_local std::vector<std::vector<uint8_t>> params;
        params.resize(n);
        for (size_t i = 0; i < n; i++) {
            const oxk::LaunchRec& r = *plan.launches[i];
            params[i].assign(r.params.begin(), r.params.end());
            for (auto& rl : r.relocs) {
                void* p = resolve(rl.buf);
                std::memcpy(params[i].data() + rl.field_off, &p, sizeof(void*));
            }
            for (auto& tm : r.tmaps) encode_tensor_map(tm, resolve(tm.buf), params[i].data());
        }
        if (!rebuild) {
            for (size_t i = 0; i < n && !rebuild; i++) {
                const oxk::LaunchRec& r = *plan.launches[i];
                bool same_grid = plan.graph_grids[i].x == r.grid.x && plan.graph_grids[i].y == r.grid.y && plan.graph_grids[i].z == r.grid.z;
                // The cluster shape and the cooperative attribute belong to the captured node and cannot be
                // patched: a launch that changed either (or its kernel) has the graph recorded again.
                const dim3& gc = plan.graph_clusters[i];
                if (gc.x != r.cluster.x || gc.y != r.cluster.y || gc.z != r.cluster.z || plan.graph_funcs[i] != r.func) {
                    rebuild = true;
                    break;
                }
                if (same_grid && params[i] == plan.graph_params[i]) continue;
                if (r.coll) {  // the buffers of a captured collective moved: record the graph again
                    rebuild = true;
                    break;
                }
                cudaKernelNodeParams kp{};
                void* args[1] = {params[i].data()};
                kp.func = const_cast<void*>(r.func);
                kp.gridDim = r.grid;
                kp.blockDim = r.block;
                kp.sharedMemBytes = r.smem;
                kp.kernelParams = args;
                cudaError_t e = cudaGraphExecKernelNodeSetParams(plan.exec, plan.graph_nodes[i], &kp);
                if (e != cudaSuccess) {
                    cudaGetLastError();
                    rebuild = true;  // e.g. a different kernel function: instantiate afresh
                    break;
                }
                plan.graph_params[i] = params[i];
                plan.graph_grids[i] = r.grid;
                graph_node_updates++;
            }
        }
        if (rebuild) build_graph(plan, params);
        OX_CUDA(cudaGraphLaunch(plan.exec, stream_));
        graph_launches++;
        launch_count += n;
    } else {
        std::vector<uint8_t> params;
        for (size_t i = 0; i < n; i++) {
            const oxk::LaunchRec& r = *plan.launches[i];
            params = r.params;
            for (auto& rl : r.relocs) {
                void* p = resolve(rl.buf);
                std::memcpy(params.data() + rl.field_off, &p, sizeof(void*));
            }
            for (auto& tm : r.tmaps) encode_tensor_map(tm, resolve(tm.buf), params.data());
            void* args[1] = {params.data()};
            ProfRec pr{};
            if (profiling) {
                pr.a = prof_event();
                pr.b = prof_event();
                pr.kernel = r.label;
                pr.node = r.node;
                OX_CUDA(cudaEventRecord(pr.a, stream_));
            }
            launch_rec(r, args[0], !profiling && !opt_.disable_pdl);
            launch_count++;
            if (profiling) {
                OX_CUDA(cudaEventRecord(pr.b, stream_));
                prof_.push_back(pr);
            }
        }
    }
    for (size_t i = 0; i < plan.out_bufs.size(); i++)
        if (plan.out_bufs[i].kv_rows >= 0) out_bufs[i]->kv_rows = plan.out_bufs[i].kv_rows;

    OX_CUDA(cudaMemcpyAsync(h_err_, d_err_, sizeof(oxk::ErrWord), cudaMemcpyDeviceToHost, stream_));
    err_pending_ = true;
}

namespace {
inline double now_us() {
    return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
}  // namespace

// Selects (patches, builds) the plan for a set of inputs. With `shapes_only` the inputs need no buffers
// except the KV caches: the call only gets the plan for an announced next step ready.
Plan* Session::plan_for(const std::vector<std::pair<std::string, DTensor>>& named, std::vector<DTensor>& inputs, bool shapes_only,
                        double* t_bound_out) {
    const Module& m = module_;
    // match by name against the signature (crates/onyxia-ir/src/backend.rs:47-50);
    // callers usually pass inputs in signature order, which is checked first
    inputs.assign(m.inputs.size(), DTensor{});
    std::vector<std::vector<size_t>> shape_store(m.inputs.size());
    std::vector<InputDesc> descs;
    descs.reserve(m.inputs.size());
    for (size_t i = 0; i < m.inputs.size(); i++) {
        const DTensor* found = nullptr;
        if (i < named.size() && named[i].first == m.inputs[i].first) found = &named[i].second;
        else
            for (auto& kv : named)
                if (kv.first == m.inputs[i].first) found = &kv.second;
        if (!found) fail(ErrKind::Binding, "missing input '" + m.inputs[i].first + "'");
        if (!found->buf && !shapes_only)
            fail(ErrKind::Runtime, "input '" + m.inputs[i].first + "' is not a device tensor of this backend");
        inputs[i] = *found;
        shape_store[i].assign(found->shape.begin(), found->shape.end());
        descs.push_back(InputDesc{m.inputs[i].first.c_str(), inputs[i].dtype, shape_store[i].data(), shape_store[i].size()});
    }
    Bindings bindings = bind_shapes(m, descs);

    for (size_t i = 0; i < inputs.size(); i++)
        if (inputs[i].cap && input_needs_dense_[i]) {
            if (shapes_only) return nullptr;  // would have to copy: leave it to the real run
            inputs[i] = dense_copy(inputs[i]);
        }

    // Which KV caches can be appended to in place this time?
    std::vector<char> kv_in_place(m.nodes.size(), 0);
    for (size_t n = 0; n < m.nodes.size(); n++) {
        int ik = gqa_past_input_[0][n], iv = gqa_past_input_[1][n];
        if (ik < 0 || iv < 0) continue;
        const DTensor &tk = inputs[ik], &tv = inputs[iv];
        ValueId pres = m.nodes[n].outputs[1];
        int64_t total = (int64_t)m.values[pres].ty.shape[2].eval(bindings);
        auto ok = [&](const DTensor& t) {
            return t.buf && t.cap >= total && t.offset == 0 && t.shape.size() == 4 && t.buf->kv_rows == t.shape[2];
        };
        bool outs = is_output_root_[m.nodes[n].outputs[1]] && is_output_root_[m.nodes[n].outputs[2]];
        kv_in_place[n] = ok(tk) && ok(tv) && tk.buf != tv.buf && outs;
    }

    if (t_bound_out) *t_bound_out = now_us();
    // ── find, patch or build the plan ──
    std::vector<uint64_t> key = structure_key(inputs, kv_in_place);
    Plan* plan = nullptr;
    for (auto it = plans_.begin(); it != plans_.end(); ++it)
        if ((*it)->structure == key && same_bindings((*it)->bindings, bindings)) {
            plans_.splice(plans_.begin(), plans_, it);
            plan = plans_.front().get();
            plans_reused++;
            break;
        }
    if (!plan)
        for (auto it = plans_.begin(); it != plans_.end(); ++it)
            if ((*it)->structure == key) {
                // patching may leave the plan half-updated when it gives up: such a plan is dropped
                if (update_plan(**it, bindings, inputs, kv_in_place)) {
                    plans_.splice(plans_.begin(), plans_, it);
                    plan = plans_.front().get();
                } else {
                    plans_.erase(it);
                }
                break;
            }
    if (!plan) {
        if (shapes_only) return nullptr;  // a full build needs the real inputs
        plans_.push_front(build_plan(bindings, inputs, kv_in_place));
        plan = plans_.front().get();
        while (plans_.size() > 6) plans_.pop_back();
    }
    return plan;
}

// Announces the shapes of the next run (buffers are only needed for the KV caches) so that its plan is
// patched now, while the device is still busy with the current step.
void Session::preplan(const std::vector<std::pair<std::string, DTensor>>& named) {
    std::vector<DTensor> inputs;
    try {
        plan_for(named, inputs, true, nullptr);
    } catch (const Error&) {
        // the real run reports whatever is wrong with its inputs
    }
}

std::vector<std::pair<std::string, DTensor>> Session::run(const std::vector<std::pair<std::string, DTensor>>& named) {
    const double t_start = now_us();
    OX_CUDA(cudaSetDevice(device_));
    std::vector<DTensor> inputs;
    double t_bound = t_start;
    Plan* plan = plan_for(named, inputs, false, &t_bound);

    const double t_planned = now_us();
    std::vector<BufferRef> out_bufs;
    execute(*plan, inputs, out_bufs);
    const double t_executed = now_us();
    host_us[0] += t_bound - t_start;
    host_us[1] += t_planned - t_bound;
    host_us[2] += t_executed - t_planned;
    host_runs++;

    std::vector<std::pair<std::string, DTensor>> outs;
    outs.reserve(plan->outputs.size());
    for (auto& spec : plan->outputs) {
        ValueId root = alias_root_[spec.value];
        const ValueLoc& l = plan->loc[root];
        DTensor t;
        t.dtype = spec.dtype;
        t.shape = spec.shape;
        t.cap = spec.cap;
        switch (l.kind) {
            case ValueLoc::Output: t.buf = out_bufs[l.index]; break;
            case ValueLoc::Input:
                t.buf = inputs[l.index].buf;
                t.offset = inputs[l.index].offset;
                t.cap = inputs[l.index].cap;
                break;
            case ValueLoc::Const: t.buf = consts_[root].buf; break;
            default: fail(ErrKind::Runtime, "internal: module output without storage");
        }
        outs.emplace_back(spec.name, std::move(t));
    }
    return outs;
}

}  // namespace oxrt
