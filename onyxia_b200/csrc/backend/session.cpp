// Session: prepare-time analysis, per-binding plans, execution.
#include "session.hpp"

#include <algorithm>
#include <climits>
#include <cstdlib>
#include <cstring>

#include "../kernels/common.cuh"

namespace oxrt {

using namespace ox;
using oxk::Buf;
using oxk::TRef;

void cuda_fail(cudaError_t e, const char* what) {
    fail(ErrKind::Runtime, std::string("CUDA error ") + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ") in " + what);
}

// ───────────────────────────── Pool ─────────────────────────────────────
DeviceBuffer::~DeviceBuffer() {
    if (pool && ptr) pool->release(ptr, bytes);
}

Pool::~Pool() {
    for (auto& kv : free_) cudaFree(kv.second);
}

static size_t round_size(size_t bytes) {
    if (bytes < 512) return 512;
    if (bytes < (1u << 20)) return (bytes + 511) / 512 * 512;
    return (bytes + (1u << 16) - 1) / (1u << 16) * (1u << 16);
}

BufferRef Pool::alloc(size_t bytes) {
    size_t want = round_size(bytes);
    auto b = std::make_shared<DeviceBuffer>();
    b->pool = shared_from_this();
    auto it = free_.lower_bound(want);
    if (it != free_.end() && it->first <= want + want / 4 + 4096) {
        b->ptr = it->second;
        b->bytes = it->first;
        cached_ -= it->first;
        free_.erase(it);
        reuses++;
    } else {
        OX_CUDA(cudaSetDevice(device_));
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, want);
        if (e != cudaSuccess) {
            trim();  // give cached blocks back and retry once
            cudaGetLastError();
            e = cudaMalloc(&p, want);
        }
        if (e != cudaSuccess) {
            b->pool.reset();
            cuda_fail(e, "cudaMalloc");
        }
        b->ptr = p;
        b->bytes = want;
        fresh_allocations++;
    }
    live_ += b->bytes;
    if (live_ > peak_) peak_ = live_;
    return b;
}

void Pool::release(void* ptr, size_t bytes) {
    live_ -= bytes;
    cached_ += bytes;
    free_.emplace(bytes, ptr);
}

void Pool::trim() {
    for (auto& kv : free_) cudaFree(kv.second);
    free_.clear();
    cached_ = 0;
}

Plan::~Plan() {
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    if (dyn_pinned) {
        for (auto e : dyn_events)
            if (e) cudaEventDestroy(e);
        cudaFreeHost(dyn_pinned);
    }
}

// ───────────────────────────── Backend ──────────────────────────────────
Backend::Backend(std::vector<int> devices, Options opt) : devices_(std::move(devices)), opt_(opt) {
    if (devices_.empty()) devices_.push_back(0);
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        fail(ErrKind::Runtime, "no CUDA device available: this backend has no CPU fallback");
    for (int d : devices_)
        if (d < 0 || d >= count) fail(ErrKind::Runtime, "CUDA device ordinal " + std::to_string(d) + " out of range");
}

std::unique_ptr<Session> Backend::prepare(Module m) {
    const KernelRegistry& reg = standard_kernels();
    bool fused = !opt_.without_fused;
    // Diagnostics: ONYXIA_DISABLE_FUSED="Name1,Name2" legalises those composites
    // through their decompositions even though a kernel exists.
    std::string disabled = std::string(",") + (std::getenv("ONYXIA_DISABLE_FUSED") ? std::getenv("ONYXIA_DISABLE_FUSED") : "") + ",";
    Module legal = inline_composites(std::move(m), standard_decompositions(), [&](const Module& mod, const Node& n) {
        if (n.composite.name == "onyxia.AllReduce") {
            if (!comm_) fail(ErrKind::Unsupported, "the module was partitioned for tensor parallelism but this backend has not joined a group");
            return true;
        }
        if (!fused) return false;
        if (disabled.find("," + n.composite.name + ",") != std::string::npos) return false;
        const FusedKernel* k = reg.get(n.composite.name);
        return k && k->accepts(mod, n);
    });
    validate(legal);
    return std::make_unique<Session>(*this, std::move(legal));
}

// ───────────────────────────── Session ──────────────────────────────────
Session::Session(Backend& backend, Module legalized)
    : backend_(backend), opt_(backend.options()), device_(backend.device()), pool_(std::make_shared<Pool>(backend.device())),
      module_(std::move(legalized)) {
    OX_CUDA(cudaSetDevice(device_));
    if (const char* e = std::getenv("ONYXIA_DISABLE_PDL")) opt_.disable_pdl = opt_.disable_pdl || std::atoi(e) != 0;  // diagnostics
    OX_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    OX_CUDA(cudaMalloc((void**)&d_err_, kErrAreaBytes));  // the error word, then room for a developer trace log
    OX_CUDA(cudaMemset(d_err_, 0, kErrAreaBytes));
    OX_CUDA(cudaMallocHost((void**)&h_err_, sizeof(oxk::ErrWord)));
    std::memset(h_err_, 0, sizeof(oxk::ErrWord));
    OX_CUDA(cudaEventCreate(&ev_t0_));
    OX_CUDA(cudaEventCreate(&ev_t1_));
    OX_CUDA(cudaMalloc((void**)&d_counters_, oxk::kCounterWords * sizeof(unsigned)));
    OX_CUDA(cudaMemset(d_counters_, 0, oxk::kCounterWords * sizeof(unsigned)));
    analyse();
    upload_constants();
    interleave_weights();
}

Session::~Session() {
    cudaSetDevice(device_);
    if (stream_) cudaStreamSynchronize(stream_);
    plans_.clear();
    consts_.clear();
    if (d_err_) cudaFree(d_err_);
    if (d_counters_) cudaFree(d_counters_);
    if (h_err_) cudaFreeHost(h_err_);
    for (auto& r : prof_) {
        cudaEventDestroy(r.a);
        cudaEventDestroy(r.b);
    }
    for (auto e : prof_free_) cudaEventDestroy(e);
    if (stage_pinned_) {
        cudaFreeHost(stage_pinned_);
        for (auto e : stage_events_) cudaEventDestroy(e);
    }
    if (ev_t0_) cudaEventDestroy(ev_t0_);
    if (ev_t1_) cudaEventDestroy(ev_t1_);
    if (stream_) cudaStreamDestroy(stream_);
}

void Session::analyse() {
    const Module& m = module_;
    order_ = m.topo_order();
    size_t nv = m.values.size(), nn = m.nodes.size();
    step_of_node_.assign(nn, -1);
    for (size_t s = 0; s < order_.size(); s++) step_of_node_[order_[s]] = (int)s;

    info_.assign(nn, NodeInfo{});
    const KernelRegistry& reg = standard_kernels();
    for (size_t i = 0; i < nn; i++) {
        const Node& n = m.nodes[i];
        if (n.is_prim) {
            info_[i].label = n.prim.name();
        } else {
            info_[i].fused = reg.get(n.composite.name);
            if (!info_[i].fused) fail(ErrKind::Unsupported, "composite '" + n.composite.name + "' survived legalisation without a kernel");
            info_[i].label = n.composite.name;
        }
        if (n.loc_name) info_[i].label = *n.loc_name;
        if (n.is_prim) {
            PrimKind k = n.prim.kind;
            if (k == PrimKind::DimValues && n.prim.shape.size() > 32) fail(ErrKind::Unsupported, "dim_values with more than 32 expressions");
        }
        for (auto v : n.outputs)
            if (m.values[v].ty.shape.size() > (size_t)oxk::kMaxRank) fail(ErrKind::Unsupported, "tensor rank above 8");
    }

    // Reshape outputs alias their input (value semantics allow a view).
    alias_root_.resize(nv);
    for (ValueId v = 0; v < nv; v++) alias_root_[v] = v;
    for (auto nid : order_) {
        const Node& n = m.nodes[nid];
        if (n.is_prim && n.prim.kind == PrimKind::Reshape) alias_root_[n.outputs[0]] = alias_root_[n.inputs[0]];
    }

    input_index_.assign(nv, -1);
    for (size_t i = 0; i < m.inputs.size(); i++) input_index_[m.inputs[i].second] = (int)i;
    is_output_root_.assign(nv, 0);
    output_names_.clear();
    for (auto& o : m.outputs) {
        is_output_root_[alias_root_[o.second]] = 1;
        output_names_.push_back(o.first);
    }

    find_gemv_groups();
    if (!opt_.disable_pattern_fusion && !opt_.without_fused) find_pattern_fusions();
    collect_node_syms();

    last_use_.assign(nv, -1);
    for (size_t s = 0; s < order_.size(); s++) {
        NodeId nid = order_[s];
        // a node whose work is issued by another node's kernel reads its inputs at that node's step
        int at = info_[nid].absorbed_by >= 0 ? std::max((int)s, step_of_node_[info_[nid].absorbed_by]) : (int)s;
        for (auto v : m.nodes[nid].inputs) {
            ValueId r = alias_root_[v];
            if (last_use_[r] < at) last_use_[r] = at;
        }
    }
    // a value nobody reads still has to exist until its producer ran
    for (size_t s = 0; s < order_.size(); s++)
        for (auto v : m.nodes[order_[s]].outputs) {
            ValueId r = alias_root_[v];
            if (last_use_[r] < (int)s) last_use_[r] = (int)s;
        }
    deaths_.assign(order_.size(), {});
    for (ValueId v = 0; v < nv; v++) {
        if (alias_root_[v] != v || is_output_root_[v]) continue;
        if (m.values[v].origin.kind != Origin::Node) continue;
        if (last_use_[v] >= 0) deaths_[last_use_[v]].push_back(v);
    }

    // KV caches that may be appended to in place: a fused GQA whose past K/V
    // are module inputs read by nothing else.
    std::vector<int> consumers(nv, 0);
    for (auto& n : m.nodes)
        for (auto v : n.inputs) consumers[v]++;
    for (auto& o : m.outputs) consumers[o.second]++;
    gqa_past_input_[0].assign(nn, -1);
    gqa_past_input_[1].assign(nn, -1);
    input_needs_dense_.assign(m.inputs.size(), 0);
    std::vector<char> is_kv_slot(nv, 0);
    for (size_t i = 0; i < nn; i++) {
        const Node& n = m.nodes[i];
        if (n.is_prim || n.composite.name != "com.microsoft.GroupQueryAttention") continue;
        for (int s = 0; s < 2; s++) {
            ValueId pv = n.inputs[3 + s];
            if (input_index_[pv] >= 0 && consumers[pv] == 1) {
                gqa_past_input_[s][i] = input_index_[pv];
                is_kv_slot[pv] = 1;
            }
        }
        if (gqa_past_input_[0][i] < 0 || gqa_past_input_[1][i] < 0 || n.inputs[3] == n.inputs[4])
            gqa_past_input_[0][i] = gqa_past_input_[1][i] = -1;
    }
    for (size_t i = 0; i < m.inputs.size(); i++) {
        ValueId v = m.inputs[i].second;
        bool kv_only = false;
        for (size_t n = 0; n < nn; n++)
            if (gqa_past_input_[0][n] == (int)i || gqa_past_input_[1][n] == (int)i) kv_only = true;
        input_needs_dense_[i] = kv_only && is_kv_slot[v] ? 0 : 1;
    }
}

// Groups MatMulNBits nodes that read the same f16 activations (and whose
// constant weights nobody else reads) into single launches, and attaches to a
// group the norm/add/norm chain that feeds it and the Gelu·Mul pair it feeds
// when these touch nothing else. The arithmetic and its rounding points are the
// ones of the separate kernels.
void Session::find_gemv_groups() {
    const Module& m = module_;
    const size_t nn = m.nodes.size(), nv = m.values.size();
    groups_.clear();
    group_of_leader_.assign(nn, -1);
    if (opt_.without_fused || opt_.disable_pattern_fusion) return;
    if (const char* e = std::getenv("ONYXIA_DISABLE_GEMV_GROUPS"))  // diagnostics
        if (std::atoi(e) != 0) return;
    const char* layout_env = std::getenv("ONYXIA_GEMV_LAYOUT");
    if (layout_env && std::string(layout_env) == "interleaved") return;

    std::vector<int> uses(nv, 0);
    std::vector<std::vector<int>> readers(nv);
    for (size_t i = 0; i < nn; i++)
        for (auto v : m.nodes[i].inputs) {
            uses[v]++;
            readers[v].push_back((int)i);
        }
    std::vector<int> out_uses(nv, 0);
    for (auto& o : m.outputs) out_uses[o.second]++;

    auto is_norm = [&](int i) {
        const Node& n = m.nodes[i];
        return !n.is_prim && n.composite.name == "SimplifiedLayerNormalization" && info_[i].fused && info_[i].absorbed_by < 0 &&
               info_[i].fuse_with < 0 && m.values[n.inputs[0]].ty.dtype == DType::F16 && m.values[n.inputs[1]].ty.dtype == DType::F16 &&
               m.values[n.outputs[0]].ty == m.values[n.inputs[0]].ty && m.values[n.inputs[1]].origin.kind == Origin::Const;
    };
    auto producer = [&](ValueId v) { return m.values[v].origin.kind == Origin::Node ? (int)m.values[v].origin.id : -1; };

    // eligible members, keyed by the activations they read
    auto eligible = [&](size_t i) {
        const Node& n = m.nodes[i];
        if (n.is_prim || n.composite.name != "com.microsoft.MatMulNBits" || !info_[i].fused || info_[i].absorbed_by >= 0) return false;
        if (m.values[n.inputs[0]].ty.dtype != DType::F16 || m.values[n.inputs[2]].ty.dtype != DType::F16) return false;
        if (m.values[n.outputs[0]].ty.dtype != DType::F16) return false;
        for (size_t j = 1; j < n.inputs.size(); j++) {
            ValueId c = n.inputs[j];
            if (m.values[c].origin.kind != Origin::Const || uses[c] != 1 || out_uses[c]) return false;
            // constants sharing one pool entry would share one device buffer
            for (ValueId u = 0; u < nv; u++)
                if (u != c && m.values[u].origin.kind == Origin::Const && m.values[u].origin.id == m.values[c].origin.id) return false;
        }
        auto wd = shape_as_static(m.values[n.inputs[1]].ty.shape);
        return wd && wd->size() == 3;
    };
    std::vector<char> taken(nn, 0);
    for (size_t s = 0; s < order_.size(); s++) {
        const size_t i = order_[s];
        if (taken[i] || !eligible(i)) continue;
        const Node& n0 = m.nodes[i];
        GemvGroup g;
        g.k = n0.composite.attrs.int_("K");
        g.has_zp = n0.inputs.size() > 3;
        g.members.push_back((ox::NodeId)i);
        const ValueId a = n0.inputs[0];
        for (size_t s2 = s + 1; s2 < order_.size() && g.members.size() < 3; s2++) {
            const size_t j = order_[s2];
            if (taken[j] || !eligible(j)) continue;
            const Node& nj = m.nodes[j];
            if (nj.inputs[0] != a || nj.composite.attrs.int_("K") != g.k || (nj.inputs.size() > 3) != g.has_zp) continue;
            g.members.push_back((ox::NodeId)j);
        }
        // every reader of a member's output must run after the launch
        auto readers_after = [&](int leader) {
            for (auto mem : g.members)
                for (int r : readers[m.nodes[mem].outputs[0]])
                    if (r != leader && step_of_node_[r] <= step_of_node_[leader]) return false;
            return true;
        };
        g.leader = (int)g.members.back();
        // Gelu(member 0) · member 1 with nothing else reading either
        if (g.members.size() == 2) {
            const ValueId o0 = m.nodes[g.members[0]].outputs[0], o1 = m.nodes[g.members[1]].outputs[0];
            if (uses[o0] == 1 && uses[o1] == 1 && !out_uses[o0] && !out_uses[o1] && m.values[o0].ty == m.values[o1].ty) {
                const int gi = readers[o0][0], mi = readers[o1][0];
                const Node &gn = m.nodes[gi], &mn = m.nodes[mi];
                if (!gn.is_prim && gn.composite.name == "Gelu" && info_[gi].fused && info_[gi].absorbed_by < 0 && mn.is_prim &&
                    mn.prim.kind == PrimKind::Binary && (BinaryOp)mn.prim.op == BinaryOp::Mul && info_[mi].absorbed_by < 0 &&
                    info_[mi].fuse_with < 0 && mn.inputs[0] == gn.outputs[0] && mn.inputs[1] == o1 &&
                    uses[gn.outputs[0]] == 1 && !out_uses[gn.outputs[0]] && m.values[mn.outputs[0]].ty == m.values[o0].ty &&
                    alias_root_[mn.outputs[0]] == mn.outputs[0]) {
                    g.geglu = gn.composite.attrs.str_or("approximate", "none") == "tanh" ? 1 : 2;
                    g.gelu_node = gi;
                    g.mul_node = mi;
                    g.leader = mi;
                }
            }
        }
        while (!g.geglu && !readers_after(g.leader) && g.members.size() > 1) {
            g.members.pop_back();  // fall back to a smaller group
            g.leader = (int)g.members.back();
        }
        // the chain that produces the activations
        g.src = a;
        // A Slice that only selects rows (the last-token slice in front of the lm_head) commutes with the row-wise
        // chain: the prologue then works on the selected rows of the chain's operands.
        auto row_slice = [&](ValueId v) {  // the node when `v` is such a Slice's result that nothing else reads
            const int sn = producer(v);
            if (sn < 0 || !m.nodes[sn].is_prim || m.nodes[sn].prim.kind != PrimKind::Slice || info_[sn].absorbed_by >= 0 ||
                info_[sn].fuse_with >= 0 || out_uses[v] || alias_root_[v] != v)
                return -1;
            const Node& sl = m.nodes[sn];
            const size_t rank = m.values[sl.inputs[0]].ty.shape.size();
            if (rank < 2 || m.values[sl.inputs[0]].ty.dtype != DType::F16) return -1;
            for (auto& sp : sl.prim.specs)
                if (sp.axis + 1 >= rank || sp.step != 1) return -1;
            return sn;
        };
        int pn = producer(a), slice_first = -1;
        ValueId na = a;  // the value norm2 produces
        if (uses[a] == (int)g.members.size() && !out_uses[a] && alias_root_[a] == a) {
            const int sn = row_slice(a);
            if (sn >= 0) {
                const ValueId v = m.nodes[sn].inputs[0];
                const int p2 = producer(v);
                if (p2 >= 0 && is_norm(p2) && uses[v] == 1 && !out_uses[v] && alias_root_[v] == v) {
                    slice_first = sn;
                    pn = p2;
                    na = v;
                }
            }
        }
        if (pn >= 0 && is_norm(pn) && (slice_first >= 0 || (uses[a] == (int)g.members.size() && !out_uses[a] && alias_root_[a] == a))) {
            const Node& n2 = m.nodes[pn];
            bool ok = true;
            GemvGroup c = g;
            c.norm2 = pn;
            ValueId z = n2.inputs[0];
            if (slice_first >= 0) {
                c.slice = slice_first;
                c.slice_last = true;
            } else if (uses[z] == 1) {
                const int sn = row_slice(z);
                if (sn >= 0) {
                    c.slice = sn;
                    z = m.nodes[sn].inputs[0];
                }
            }
            c.src = z;
            const int an = producer(z);
            if (an >= 0 && m.nodes[an].is_prim && m.nodes[an].prim.kind == PrimKind::Binary &&
                (BinaryOp)m.nodes[an].prim.op == BinaryOp::Add && info_[an].absorbed_by < 0 && info_[an].fuse_with < 0 &&
                alias_root_[z] == z) {
                const Node& ad = m.nodes[an];
                const TensorType& ts = m.values[ad.outputs[0]].ty;
                if (m.values[ad.inputs[0]].ty == ts && m.values[ad.inputs[1]].ty == ts && ts.dtype == DType::F16) {
                    // every other reader of the sum must run after the launch; behind a slice only some rows of the
                    // sum are formed, so there must be no other reader at all
                    for (int r : readers[ad.outputs[0]])
                        if (r != pn && r != c.slice && (c.slice >= 0 || step_of_node_[r] <= step_of_node_[g.leader])) ok = false;
                    if (c.slice >= 0 && out_uses[ad.outputs[0]]) ok = false;
                    if (ok) {
                        c.add = an;
                        int which = -1;  // the operand that is itself a norm nothing else reads
                        for (int side = 1; side >= 0 && which < 0; side--) {
                            const ValueId ov = ad.inputs[side];
                            const int p1 = producer(ov);
                            if (p1 >= 0 && is_norm(p1) && uses[ov] == 1 && !out_uses[ov] && alias_root_[ov] == ov) which = side;
                        }
                        if (which >= 0) {
                            c.norm1 = producer(ad.inputs[which]);
                            c.src = m.nodes[c.norm1].inputs[0];
                            c.res = ad.inputs[1 - which];
                        } else {
                            c.src = ad.inputs[1];
                            c.res = ad.inputs[0];
                        }
                    }
                }
            }
            if (ok) g = c;
        }
        // record
        const int gid = (int)groups_.size();
        auto absorb = [&](int node) {
            if (node >= 0 && node != g.leader) info_[node].absorbed_by = g.leader;
        };
        for (auto mem : g.members) {
            taken[mem] = 1;
            absorb((int)mem);
        }
        absorb(g.gelu_node);
        absorb(g.norm2);
        absorb(g.slice);
        absorb(g.add);
        absorb(g.norm1);
        group_of_leader_[g.leader] = gid;
        groups_.push_back(std::move(g));
    }
}

// Cross-node fusions the registry cannot express by name: Gelu followed by a
// multiply (GeGLU) and a residual add followed by an RMS norm. Either pair
// becomes one launch of the corresponding fused kernel; the arithmetic and its
// rounding points are unchanged.
void Session::find_pattern_fusions() {
    const Module& m = module_;
    std::vector<int> uses(m.values.size(), 0);
    for (auto& n : m.nodes)
        for (auto v : n.inputs) uses[v]++;
    for (auto& o : m.outputs) uses[o.second] += 2;  // outputs must stay materialised
    for (size_t i = 0; i < m.nodes.size(); i++) {
        const Node& n = m.nodes[i];
        if (n.is_prim || info_[i].absorbed_by >= 0) continue;
        if (n.composite.name == "Gelu") {
            ValueId g = n.outputs[0];
            if (uses[g] != 1) continue;
            for (size_t j = 0; j < m.nodes.size(); j++) {
                const Node& c = m.nodes[j];
                if (!c.is_prim || c.prim.kind != PrimKind::Binary || (BinaryOp)c.prim.op != BinaryOp::Mul) continue;
                if (c.inputs[0] != g || c.inputs[1] == g) continue;  // gelu(gate)·up, gelu on the left
                const TensorType &tg = m.values[g].ty, &tu = m.values[c.inputs[1]].ty;
                if (tg != tu || info_[j].absorbed_by >= 0 || info_[j].fuse_with >= 0) continue;
                // `up` must already exist when the Gelu node runs: the fused
                // launch is issued at the Mul's step instead.
                info_[i].absorbed_by = (int)j;
                info_[j].fuse_with = (int)i;
                info_[j].fuse_kind = FUSE_GEGLU;
                break;
            }
        } else if (n.composite.name == "SimplifiedLayerNormalization") {
            ValueId x = n.inputs[0];
            const Origin& o = m.values[x].origin;
            if (o.kind != Origin::Node) continue;
            const Node& a = m.nodes[o.id];
            if (!a.is_prim || a.prim.kind != PrimKind::Binary || (BinaryOp)a.prim.op != BinaryOp::Add) continue;
            if (info_[o.id].absorbed_by >= 0 || info_[o.id].fuse_with >= 0) continue;
            const TensorType &t0 = m.values[a.inputs[0]].ty, &t1 = m.values[a.inputs[1]].ty;
            if (t0 != t1 || t0 != m.values[x].ty) continue;  // no broadcasting in the add
            if (alias_root_[x] != x) continue;
            // the add must directly precede the norm in execution order
            if (step_of_node_[o.id] + 1 != step_of_node_[i]) continue;
            info_[o.id].absorbed_by = (int)i;
            info_[i].fuse_with = (int)o.id;
            info_[i].fuse_kind = FUSE_ADD_NORM;
        }
    }
}

void Session::upload_constants() {
    Module& m = module_;
    consts_.assign(m.values.size(), DTensor{});
    std::unordered_map<ConstId, ValueId> seen;
    for (ValueId v = 0; v < m.values.size(); v++) {
        const ValueDef& def = m.values[v];
        if (def.origin.kind != Origin::Const) continue;
        ConstId cid = def.origin.id;
        auto it = seen.find(cid);
        if (it != seen.end()) {
            consts_[v] = consts_[it->second];
            continue;
        }
        auto dims = shape_as_static(m.consts.ty(cid).shape);
        DTensor t;
        t.dtype = def.ty.dtype;
        for (auto d : *dims) t.shape.push_back((int64_t)d);
        size_t nbytes = m.consts.nbytes(cid);
        t.buf = pool_->alloc(nbytes ? nbytes : 1);
        if (nbytes) {
            if (!m.consts.bytes(cid)) fail(ErrKind::InvalidGraph, "constant bytes are gone");
            OX_CUDA(cudaMemcpyAsync(t.buf->ptr, m.consts.bytes(cid), nbytes, cudaMemcpyHostToDevice, stream_));
        }
        consts_[v] = t;
        seen[cid] = v;
    }
    OX_CUDA(cudaStreamSynchronize(stream_));
    // prepare() consumed the module: the host copies of the weights are dropped
    for (auto& kv : seen) m.consts.release(kv.first);
}

// Launch an emitter's records right away; slot i resolves to slots[i].
void Session::launch_now(const oxk::Emitter& em, const std::vector<void*>& slots) {
    for (auto& r : em.recs) {
        std::vector<uint8_t> params = r.params;
        for (auto& rl : r.relocs) {
            void* p = rl.buf.slot < slots.size() ? (char*)slots[rl.buf.slot] + rl.buf.off : nullptr;
            std::memcpy(params.data() + rl.field_off, &p, sizeof(void*));
        }
        void* args[1] = {params.data()};
        OX_CUDA(cudaLaunchKernel(r.func, r.grid, r.block, args, r.smem, stream_));
        launch_count++;
    }
}

// Weight constants read only by f16 MatMulNBits nodes are re-laid out for the
// decode kernels (backend-private layouts; the caller's bytes were consumed by
// prepare). Preferred: tile records that hold a tile's nibbles, scales and zero
// points together, which needs every reader of the weight to use the same
// constant scales and zero points. Otherwise: nibbles interleaved in place.
void Session::interleave_weights() {
    const Module& m = module_;
    interleaved_.assign(m.values.size(), 0);
    if (opt_.without_fused) return;
    const char* layout_env = std::getenv("ONYXIA_GEMV_LAYOUT");  // "interleaved" forces the older layout
    const bool allow_tiled = !(layout_env && std::string(layout_env) == "interleaved");
    std::vector<int> total(m.values.size(), 0), eligible(m.values.size(), 0);
    // per weight: the scales / zero-point values its readers use (−1 none yet, −2 readers disagree)
    std::vector<long long> w_scales(m.values.size(), -1), w_zp(m.values.size(), -1);
    for (auto& n : m.nodes)
        for (auto v : n.inputs) total[v]++;
    for (auto& o : m.outputs) total[o.second]++;
    for (size_t i = 0; i < m.nodes.size(); i++) {
        const Node& n = m.nodes[i];
        if (n.is_prim || n.composite.name != "com.microsoft.MatMulNBits" || !info_[i].fused) continue;
        if (m.values[n.inputs[0]].ty.dtype != DType::F16 || m.values[n.inputs[2]].ty.dtype != DType::F16) continue;
        ValueId w = n.inputs[1];
        eligible[w]++;
        long long sc = m.values[n.inputs[2]].origin.kind == Origin::Const ? (long long)n.inputs[2] : -2;
        long long zp = n.inputs.size() > 3 ? (m.values[n.inputs[3]].origin.kind == Origin::Const ? (long long)n.inputs[3] : -2) : -3;
        w_scales[w] = w_scales[w] == -1 || w_scales[w] == sc ? sc : -2;
        w_zp[w] = w_zp[w] == -1 || w_zp[w] == zp ? zp : -2;
    }
    // groups first: one tile stream per group, kept in the slot of the first member's weight
    for (auto& g : groups_) {
        const long long nb = (g.k + 31) / 32;
        std::vector<long long> rts;
        long long total_rt = 0;
        for (auto mem : g.members) {
            rts.push_back((m.nodes[mem].composite.attrs.int_("N") + 15) / 16);
            total_rt += rts.back();
        }
        const size_t tile_bytes = oxk::nbits_tiled_bytes(16, nb, g.has_zp);  // bytes of one row tile (all its k tiles)
        BufferRef dst = pool_->alloc(std::max<size_t>((size_t)total_rt * tile_bytes, 16));
        long long rt_add = 0;
        for (size_t i = 0; i < g.members.size(); i++) {
            const Node& n = m.nodes[g.members[i]];
            oxk::Emitter em;
            // GeGLU: row tiles of gate and up alternate; otherwise one matrix after the other
            oxk::emit_nbits_pack_tiles(em, oxk::Buf{0, 0}, oxk::Buf{1, 0}, oxk::Buf{2, 0}, oxk::Buf{3, 0},
                                       n.composite.attrs.int_("N"), nb, g.has_zp, g.geglu ? 2 : 1, g.geglu ? (long long)i : rt_add);
            launch_now(em, {consts_[n.inputs[1]].ptr(), consts_[n.inputs[2]].ptr(), g.has_zp ? consts_[n.inputs[3]].ptr() : nullptr,
                            dst->ptr});
            rt_add += rts[i];
        }
        OX_CUDA(cudaStreamSynchronize(stream_));
        for (size_t i = 0; i < g.members.size(); i++) {
            const Node& n = m.nodes[g.members[i]];
            interleaved_[n.inputs[1]] = 3;  // part of a group's stream; not usable on its own
            consts_[n.inputs[1]].buf = i == 0 ? dst : BufferRef();
            consts_[n.inputs[2]].buf = BufferRef();  // the scales (and zero points) live inside the tile records
            if (g.has_zp) consts_[n.inputs[3]].buf = BufferRef();
        }
    }
    std::unordered_map<void*, char> done;
    for (ValueId v = 0; v < m.values.size(); v++) {
        if (interleaved_[v] == 3) continue;
        if (!eligible[v] || eligible[v] != total[v] || !consts_[v].buf) continue;
        // constants sharing one pool entry share one device buffer
        bool shared = false;
        for (ValueId u = 0; u < m.values.size(); u++)
            if (u != v && consts_[u].buf == consts_[v].buf) shared = true;
        auto wd = shape_as_static(m.values[v].ty.shape);
        const bool tiled = allow_tiled && !shared && w_scales[v] >= 0 && w_zp[v] != -2 && wd && wd->size() == 3 &&
                           consts_[(ValueId)w_scales[v]].buf && (w_zp[v] < 0 || consts_[(ValueId)w_zp[v]].buf);
        if (tiled) {
            const long long n_rows = (long long)(*wd)[0], nb = (long long)(*wd)[1];
            const bool has_zp = w_zp[v] >= 0;
            BufferRef dst = pool_->alloc(std::max<size_t>(oxk::nbits_tiled_bytes(n_rows, nb, has_zp), 16));
            oxk::Emitter em;
            oxk::emit_nbits_pack_tiles(em, oxk::Buf{0, 0}, oxk::Buf{1, 0}, oxk::Buf{2, 0}, oxk::Buf{3, 0}, n_rows, nb, has_zp);
            launch_now(em, {consts_[v].buf->ptr, consts_[(ValueId)w_scales[v]].ptr(),
                            has_zp ? consts_[(ValueId)w_zp[v]].ptr() : nullptr, dst->ptr});
            OX_CUDA(cudaStreamSynchronize(stream_));  // the source buffer may be released below
            consts_[v].buf = dst;
            interleaved_[v] = 2;
            continue;
        }
        bool shared_ok = true;
        for (ValueId u = 0; u < m.values.size(); u++)
            if (u != v && consts_[u].buf == consts_[v].buf && (eligible[u] != total[u] || !eligible[u])) shared_ok = false;
        if (!shared_ok) continue;
        interleaved_[v] = 1;
        if (done.count(consts_[v].buf->ptr)) continue;
        done[consts_[v].buf->ptr] = 1;
        size_t bytes = consts_[v].nbytes();
        BufferRef dst = pool_->alloc(std::max<size_t>(bytes, 4));
        oxk::Emitter em;
        oxk::emit_nbits_interleave(em, oxk::Buf{0, 0}, oxk::Buf{1, 0}, (long long)bytes);
        launch_now(em, {consts_[v].buf->ptr, dst->ptr});
        for (ValueId u = 0; u < m.values.size(); u++)
            if (u != v && consts_[u].buf == consts_[v].buf) consts_[u].buf = dst;
        consts_[v].buf = dst;
    }
    OX_CUDA(cudaStreamSynchronize(stream_));
}

DTensor Session::upload(DType dtype, const std::vector<int64_t>& shape, const void* bytes, size_t nbytes) {
    OX_CUDA(cudaSetDevice(device_));
    DTensor t;
    t.dtype = dtype;
    t.shape = shape;
    if (t.nbytes() != nbytes)
        fail(ErrKind::Interp, "tensor data size mismatch: " + std::to_string(nbytes) + " bytes for " + dtype_name(dtype) +
                                  " (expected " + std::to_string(t.nbytes()) + ")");
    t.buf = pool_->alloc(nbytes ? nbytes : 1);
    if (nbytes && nbytes <= kStageBytes) {
        // Small uploads (token ids, masks) go through a ring of pinned staging slots: the copy is truly
        // asynchronous and the caller's memory is free for reuse when this returns.
        if (!stage_pinned_) {
            OX_CUDA(cudaMallocHost((void**)&stage_pinned_, kStageBytes * kStageSlots));
            for (auto& e : stage_events_) OX_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        }
        const unsigned slot = stage_cursor_++ % kStageSlots;
        if (stage_cursor_ > kStageSlots) OX_CUDA(cudaEventSynchronize(stage_events_[slot]));
        std::memcpy(stage_pinned_ + (size_t)slot * kStageBytes, bytes, nbytes);
        OX_CUDA(cudaMemcpyAsync(t.buf->ptr, stage_pinned_ + (size_t)slot * kStageBytes, nbytes, cudaMemcpyHostToDevice, stream_));
        OX_CUDA(cudaEventRecord(stage_events_[slot], stream_));
    } else if (nbytes) {
        OX_CUDA(cudaMemcpyAsync(t.buf->ptr, bytes, nbytes, cudaMemcpyHostToDevice, stream_));
    }
    return t;
}

void Session::check_device_error() {
    if (!err_pending_) return;
    err_pending_ = false;
    if (h_err_->code == 0) return;
    oxk::ErrWord e = *h_err_;
    std::memset(h_err_, 0, sizeof(*h_err_));
    OX_CUDA(cudaMemsetAsync(d_err_, 0, sizeof(oxk::ErrWord), stream_));
    std::string node = "<unnamed>", kind = "kernel";
    if (e.node >= 0 && (size_t)e.node < module_.nodes.size()) {
        const Node& n = module_.nodes[e.node];
        kind = n.is_prim ? n.prim.name() : n.composite.name;
        if (n.loc_name) node = *n.loc_name;
    }
    std::string what;
    switch (e.code) {
        case oxk::ERR_GATHER_OOB: what = "gather index " + std::to_string(e.a) + " out of range for dim " + std::to_string(e.b); break;
        case oxk::ERR_SCATTER_OOB: what = "scatter index " + std::to_string(e.a) + " out of range for dim " + std::to_string(e.b); break;
        case oxk::ERR_INT_DIV_ZERO: what = "integer division by zero"; break;
        case oxk::ERR_INT_POW_NEG: what = "integer pow with negative exponent"; break;
        case oxk::ERR_WAIT_TIMEOUT: what = "a bounded device-side wait gave up"; break;
        case oxk::ERR_SAMPLE_NO_FINITE: what = "All logits are NaN or Inf, cannot sample (row " + std::to_string(e.a) + ")"; break;
        default: what = "device error code " + std::to_string(e.code);
    }
    fail(ErrKind::Runtime, kind + " (node '" + node + "'): " + what);
}

void Session::wait_idle() {
    OX_CUDA(cudaSetDevice(device_));
    OX_CUDA(cudaStreamSynchronize(stream_));
    check_device_error();
}

void Session::timer_start() {
    OX_CUDA(cudaSetDevice(device_));
    OX_CUDA(cudaEventRecord(ev_t0_, stream_));
}

float Session::timer_stop() {
    OX_CUDA(cudaSetDevice(device_));
    OX_CUDA(cudaEventRecord(ev_t1_, stream_));
    OX_CUDA(cudaEventSynchronize(ev_t1_));
    float ms = 0.f;
    OX_CUDA(cudaEventElapsedTime(&ms, ev_t0_, ev_t1_));
    check_device_error();
    return ms;
}

DTensor Session::dense_copy(const DTensor& t) {
    if (t.cap == 0 || t.shape.size() != 4 || t.cap == t.shape[2]) {
        DTensor d = t;
        d.cap = 0;
        return d;
    }
    DTensor d;
    d.dtype = t.dtype;
    d.shape = t.shape;
    d.buf = pool_->alloc(std::max<size_t>(d.nbytes(), 1));
    size_t row = (size_t)t.shape[3] * dtype_bits(t.dtype) / 8;
    size_t heads = (size_t)(t.shape[0] * t.shape[1]);
    if (heads && t.shape[2] && row)
        OX_CUDA(cudaMemcpy2DAsync(d.buf->ptr, (size_t)t.shape[2] * row, t.ptr(), (size_t)t.cap * row, (size_t)t.shape[2] * row,
                                  heads, cudaMemcpyDeviceToDevice, stream_));
    return d;
}

void Session::download(const DTensor& t, void* dst, size_t cap, size_t* written) {
    OX_CUDA(cudaSetDevice(device_));
    size_t nbytes = t.nbytes();
    if (cap < nbytes) fail(ErrKind::Runtime, "download buffer too small: " + std::to_string(cap) + " < " + std::to_string(nbytes));
    if (nbytes) {
        if (t.cap && t.shape.size() == 4 && t.cap != t.shape[2]) {
            size_t row = (size_t)t.shape[3] * dtype_bits(t.dtype) / 8;
            size_t heads = (size_t)(t.shape[0] * t.shape[1]);
            OX_CUDA(cudaMemcpy2DAsync(dst, (size_t)t.shape[2] * row, t.ptr(), (size_t)t.cap * row, (size_t)t.shape[2] * row, heads,
                                      cudaMemcpyDeviceToHost, stream_));
        } else {
            OX_CUDA(cudaMemcpyAsync(dst, t.ptr(), nbytes, cudaMemcpyDeviceToHost, stream_));
        }
    }
    OX_CUDA(cudaStreamSynchronize(stream_));
    if (written) *written = nbytes;
    check_device_error();
}

void Session::download_async(const DTensor& t, void* pinned_dst) {
    OX_CUDA(cudaSetDevice(device_));
    if (t.cap) fail(ErrKind::Shape, "download_async: the tensor must be densely packed");
    if (t.nbytes()) OX_CUDA(cudaMemcpyAsync(pinned_dst, t.ptr(), t.nbytes(), cudaMemcpyDeviceToHost, stream_));
}

DTensor Session::argmax_last(const DTensor& logits) {
    OX_CUDA(cudaSetDevice(device_));
    if (!dtype_is_float(logits.dtype) || logits.shape.empty() || logits.shape.back() == 0)
        fail(ErrKind::DType, "argmax needs a float tensor with a non-empty last axis");
    DTensor out;
    out.dtype = DType::I64;
    out.shape.assign(logits.shape.begin(), logits.shape.end() - 1);
    out.buf = pool_->alloc(std::max<size_t>(out.nbytes(), 8));
    oxk::Emitter em;
    TRef x{Buf{0, 0}, (int)logits.dtype, logits.shape, 0}, y{Buf{1, 0}, (int)DType::I64, out.shape, 0};
    int64_t rows = out.numel();
    BufferRef part = pool_->alloc(oxk::argmax_scratch_bytes(rows));
    oxk::emit_argmax_last(em, x, y, Buf{2, 0}, Buf{3, 0});
    launch_now(em, {logits.ptr(), out.ptr(), part->ptr, (void*)d_counters_});
    return out;
}

// Temperature / top-k / top-p sampling of one token per row (crates/onyxia-cli/src/sampling.rs:36-65); `u` holds one
// uniform number in [0, 1] per row. A temperature at or below 1e-6 selects greedily, like the reference.
DTensor Session::sample_last(const DTensor& logits, float temperature, long long top_k, float top_p, const float* u, size_t n_u) {
    if (temperature <= 0.f || temperature < 1e-6f) return argmax_last(logits);
    OX_CUDA(cudaSetDevice(device_));
    if (!dtype_is_float(logits.dtype) || logits.shape.empty() || logits.shape.back() == 0)
        fail(ErrKind::DType, "sampling needs a float tensor with a non-empty last axis");
    if (logits.cap != 0) fail(ErrKind::Shape, "sampling: logits must be densely packed");
    if (top_k < 0) fail(ErrKind::Attribute, "top_k must not be negative");
    DTensor out;
    out.dtype = DType::I64;
    out.shape.assign(logits.shape.begin(), logits.shape.end() - 1);
    const int64_t rows = out.numel();
    if ((int64_t)n_u != rows) fail(ErrKind::Shape, "sampling needs one uniform number per row of the logits: " + std::to_string(rows));
    out.buf = pool_->alloc(std::max<size_t>(out.nbytes(), 8));
    DTensor ud = upload(DType::F32, {rows}, u, sizeof(float) * (size_t)rows);
    oxk::Emitter em;
    TRef x{Buf{0, 0}, (int)logits.dtype, logits.shape, 0}, y{Buf{1, 0}, (int)DType::I64, out.shape, 0};
    oxk::emit_sample_rows(em, x, y, Buf{2, 0}, temperature, top_k, top_p);
    // slot kSlotErr resolves through launch_now's slot table only for small indices: patch the error word by hand
    for (auto& r : em.recs)
        for (auto& rl : r.relocs)
            if (rl.buf.slot == oxk::kSlotErr) rl.buf = Buf{3, rl.buf.off};
    launch_now(em, {logits.ptr(), out.ptr(), ud.ptr(), (void*)d_err_});
    OX_CUDA(cudaMemcpyAsync(h_err_, d_err_, sizeof(oxk::ErrWord), cudaMemcpyDeviceToHost, stream_));
    err_pending_ = true;
    return out;
}

void Session::argmax_last_into(const DTensor& logits, const DTensor& out) {
    OX_CUDA(cudaSetDevice(device_));
    if (logits.shape.empty() || logits.shape.back() == 0 || !logits.buf)
        fail(ErrKind::Shape, "argmax needs a tensor with a non-empty last axis");
    if (logits.cap != 0) fail(ErrKind::Shape, "argmax: logits must be densely packed");
    const int64_t cols = logits.shape.back(), rows = logits.numel() / cols;
    if (out.dtype != DType::I64 || !out.buf || out.numel() != rows || out.cap != 0)
        fail(ErrKind::Shape, "argmax: the result tensor must be a densely packed I64 tensor with one element per row of the logits");
    const char* err = oxk::argmax_last_static(device_, stream_, logits.ptr(), (int)logits.dtype, rows, cols,
                                              (long long*)out.ptr());
    if (err) fail(ErrKind::Runtime, err);
}

}  // namespace oxrt
