// Session: prepare-time analysis, per-binding plans, execution.
#include "session.hpp"

#include <algorithm>
#include <climits>
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
    b->pool = this;
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
            b->pool = nullptr;
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
    Module legal = inline_composites(std::move(m), standard_decompositions(), [&](const Module& mod, const Node& n) {
        if (!fused) return false;
        const FusedKernel* k = reg.get(n.composite.name);
        return k && k->accepts(mod, n);
    });
    validate(legal);
    return std::make_unique<Session>(*this, std::move(legal));
}

// ───────────────────────────── Session ──────────────────────────────────
Session::Session(Backend& backend, Module legalized)
    : backend_(backend), opt_(backend.options()), device_(backend.device()), pool_(backend.device()),
      module_(std::move(legalized)) {
    OX_CUDA(cudaSetDevice(device_));
    OX_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    OX_CUDA(cudaMalloc((void**)&d_err_, sizeof(oxk::ErrWord)));
    OX_CUDA(cudaMemset(d_err_, 0, sizeof(oxk::ErrWord)));
    OX_CUDA(cudaMallocHost((void**)&h_err_, sizeof(oxk::ErrWord)));
    std::memset(h_err_, 0, sizeof(oxk::ErrWord));
    OX_CUDA(cudaEventCreate(&ev_a_));
    OX_CUDA(cudaEventCreate(&ev_b_));
    OX_CUDA(cudaEventCreate(&ev_t0_));
    OX_CUDA(cudaEventCreate(&ev_t1_));
    analyse();
    upload_constants();
}

Session::~Session() {
    cudaSetDevice(device_);
    if (stream_) cudaStreamSynchronize(stream_);
    plans_.clear();
    consts_.clear();
    if (d_err_) cudaFree(d_err_);
    if (h_err_) cudaFreeHost(h_err_);
    if (ev_a_) cudaEventDestroy(ev_a_);
    if (ev_b_) cudaEventDestroy(ev_b_);
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
        // movement primitives cannot interpret packed nibbles
        if (n.is_prim) {
            PrimKind k = n.prim.kind;
            bool moves = k == PrimKind::Transpose || k == PrimKind::Broadcast || k == PrimKind::Concat || k == PrimKind::Slice ||
                         k == PrimKind::Gather || k == PrimKind::Scatter || k == PrimKind::Select;
            if (moves && !n.inputs.empty()) {
                DType dt = m.values[n.inputs[k == PrimKind::Select ? 1 : 0]].ty.dtype;
                if (dtype_is_packed(dt))
                    fail(ErrKind::Unsupported, std::string(n.prim.name()) + " on packed dtype " + dtype_name(dt) +
                                                   ": cast or dequantize first");
            }
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

    if (!opt_.disable_pattern_fusion && !opt_.without_fused) find_pattern_fusions();

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
        t.buf = pool_.alloc(nbytes ? nbytes : 1);
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

DTensor Session::upload(DType dtype, const std::vector<int64_t>& shape, const void* bytes, size_t nbytes) {
    OX_CUDA(cudaSetDevice(device_));
    DTensor t;
    t.dtype = dtype;
    t.shape = shape;
    if (t.nbytes() != nbytes)
        fail(ErrKind::Interp, "tensor data size mismatch: " + std::to_string(nbytes) + " bytes for " + dtype_name(dtype) +
                                  " (expected " + std::to_string(t.nbytes()) + ")");
    t.buf = pool_.alloc(nbytes ? nbytes : 1);
    if (nbytes) OX_CUDA(cudaMemcpyAsync(t.buf->ptr, bytes, nbytes, cudaMemcpyHostToDevice, stream_));
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
    d.buf = pool_.alloc(std::max<size_t>(d.nbytes(), 1));
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

DTensor Session::argmax_last(const DTensor& logits) {
    OX_CUDA(cudaSetDevice(device_));
    if (!dtype_is_float(logits.dtype) || logits.shape.empty() || logits.shape.back() == 0)
        fail(ErrKind::DType, "argmax needs a float tensor with a non-empty last axis");
    DTensor out;
    out.dtype = DType::I64;
    out.shape.assign(logits.shape.begin(), logits.shape.end() - 1);
    out.buf = pool_.alloc(std::max<size_t>(out.nbytes(), 8));
    oxk::Emitter em;
    TRef x{Buf{0, 0}, (int)logits.dtype, logits.shape, 0}, y{Buf{1, 0}, (int)DType::I64, out.shape, 0};
    oxk::emit_argmax_last(em, x, y);
    for (auto& r : em.recs) {
        std::vector<uint8_t> params = r.params;
        for (auto& rl : r.relocs) {
            void* p = rl.buf.slot == 0 ? logits.ptr() : out.ptr();
            std::memcpy(params.data() + rl.field_off, &p, sizeof(void*));
        }
        void* args[1] = {params.data()};
        OX_CUDA(cudaLaunchKernel(r.func, r.grid, r.block, args, r.smem, stream_));
        launch_count++;
    }
    return out;
}

// ───────────────────────────── planning ─────────────────────────────────
namespace {

// Best-fit allocator over byte offsets of the plan's arena.
struct OffsetAlloc {
    std::map<size_t, size_t> free_;  // offset → size
    size_t end = 0;
    size_t alloc(size_t bytes) {
        bytes = (bytes + 255) / 256 * 256;
        if (bytes == 0) bytes = 256;
        auto best = free_.end();
        for (auto it = free_.begin(); it != free_.end(); ++it)
            if (it->second >= bytes && (best == free_.end() || it->second < best->second)) best = it;
        if (best != free_.end()) {
            size_t off = best->first, sz = best->second;
            free_.erase(best);
            if (sz > bytes) free_[off + bytes] = sz - bytes;
            return off;
        }
        // grow: extend a trailing free block if there is one
        if (!free_.empty()) {
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
        bytes = (bytes + 255) / 256 * 256;
        if (bytes == 0) bytes = 256;
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

int64_t grow_capacity(int64_t rows) {
    // room for the next appends: +50 %, at least 256 rows, multiple of 64
    int64_t extra = std::max<int64_t>(256, rows / 2);
    return (rows + extra + 63) / 64 * 64;
}

}  // namespace

std::unique_ptr<Plan> Session::build_plan(const Bindings& bindings_in, const std::vector<DTensor>& inputs,
                                          const std::vector<char>& kv_in_place) {
    const Module& m = module_;
    Bindings bindings = bindings_in;
    auto plan = std::make_unique<Plan>();
    size_t nv = m.values.size();
    plan->loc.assign(nv, ValueLoc{});
    plan->shapes.assign(nv, {});
    std::vector<TRef> trefs(nv);
    std::vector<size_t> arena_size(nv, 0);
    OffsetAlloc arena;
    oxk::Emitter em;

    for (ValueId v = 0; v < nv; v++) {
        const ValueDef& def = m.values[v];
        if (def.origin.kind == Origin::Const) {
            plan->loc[v].kind = ValueLoc::Const;
            plan->shapes[v] = consts_[v].shape;
            trefs[v] = TRef{Buf{v, 0}, (int)def.ty.dtype, consts_[v].shape, 0};
        } else if (def.origin.kind == Origin::Input && input_index_[v] >= 0) {
            const DTensor& t = inputs[input_index_[v]];
            plan->loc[v].kind = ValueLoc::Input;
            plan->loc[v].index = (uint32_t)input_index_[v];
            plan->shapes[v] = t.shape;
            trefs[v] = TRef{Buf{v, 0}, (int)def.ty.dtype, t.shape, t.cap};
        }
    }

    struct Ctx {
        OffsetAlloc& arena;
        std::vector<size_t>& arena_size;
    } ctx{arena, arena_size};
    (void)ctx;

    for (size_t step = 0; step < order_.size(); step++) {
        NodeId nid = order_[step];
        const Node& node = m.nodes[nid];
        em.begin_node((int)nid);
        try {
            // ── output shapes ──
            for (auto o : node.outputs) {
                const SymShape& sym = m.values[o].ty.shape;
                std::vector<int64_t> shp;
                if (node.is_prim && node.prim.kind == PrimKind::Reshape) {
                    // at most one unbound bare symbol is inferred from the element count
                    // (crates/onyxia-ir/src/interp.rs:1138-1169)
                    int64_t numel = 1;
                    for (auto d : plan->shapes[node.inputs[0]]) numel *= d;
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
                    for (auto& d : sym) shp.push_back((int64_t)d.eval(bindings));
                }
                plan->shapes[o] = shp;
            }

            // ── output storage ──
            bool fused_gqa = !node.is_prim && node.composite.name == "com.microsoft.GroupQueryAttention";
            for (size_t oi = 0; oi < node.outputs.size(); oi++) {
                ValueId o = node.outputs[oi];
                DType dt = m.values[o].ty.dtype;
                ValueId root = alias_root_[o];
                TRef tr;
                tr.dtype = (int)dt;
                tr.shape = plan->shapes[o];
                if (root != o) {
                    plan->loc[o].kind = ValueLoc::Alias;
                    plan->loc[o].index = root;
                    tr.buf = trefs[root].buf;
                    tr.cap = trefs[root].cap;
                    if (tr.cap) {
                        // a reshaped KV view would need strides: work on a packed copy instead
                        fail(ErrKind::Unsupported, "reshape of a KV-cache view");
                    }
                    trefs[o] = tr;
                    continue;
                }
                int64_t numel = 1;
                for (auto d : tr.shape) numel *= d;
                size_t bytes = dtype_storage_bytes(dt, (uint64_t)numel);
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
                            tr.cap = grow_capacity(tr.shape[2]);
                            ob.kv_cap = tr.cap;
                            ob.bytes = dtype_storage_bytes(dt, (uint64_t)(tr.shape[0] * tr.shape[1] * tr.cap * tr.shape[3]));
                        }
                        ob.kv_rows = tr.shape[2];
                    }
                    plan->loc[o].kind = ValueLoc::Output;
                    plan->loc[o].index = (uint32_t)plan->out_bufs.size();
                    plan->out_bufs.push_back(ob);
                } else {
                    plan->loc[o].kind = ValueLoc::Arena;
                    plan->loc[o].offset = arena.alloc(bytes);
                    arena_size[o] = bytes;
                }
                tr.buf = Buf{o, 0};
                trefs[o] = tr;
            }

            // ── kernels ──
            if (info_[nid].absorbed_by < 0) {
                std::vector<TRef> ins, outs;
                for (auto v : node.inputs) ins.push_back(trefs[v]);
                for (auto v : node.outputs) outs.push_back(trefs[v]);
                if (node.is_prim && node.prim.kind == PrimKind::Reshape) {
                    // a view: nothing to launch
                } else if (info_[nid].fuse_kind == FUSE_GEGLU) {
                    const Node& g = m.nodes[info_[nid].fuse_with];
                    bool tanh = g.composite.attrs.str_or("approximate", "none") == "tanh";
                    oxk::emit_gelu(em, trefs[g.inputs[0]], outs[0], tanh, &ins[1]);
                } else if (info_[nid].fuse_kind == FUSE_ADD_NORM) {
                    const Node& a = m.nodes[info_[nid].fuse_with];
                    double eps = node.composite.attrs.float_or("epsilon", 1e-5);
                    TRef sum = trefs[a.outputs[0]];
                    oxk::emit_rmsnorm(em, trefs[a.inputs[0]], ins[1], outs[0], eps, &trefs[a.inputs[1]], &sum);
                } else if (node.is_prim) {
                    lower_prim(em, node, bindings, ins, outs);
                } else {
                    FusedCtx fc{em, node, ins, outs, (bool)kv_in_place[nid]};
                    info_[nid].fused->lower(fc);
                }
            }
        } catch (const Error& e) {
            std::string kind = node.is_prim ? node.prim.name() : node.composite.name;
            std::string loc = node.loc_name ? *node.loc_name : "<unnamed>";
            if (e.kind == ErrKind::Binding) throw;
            fail(ErrKind::Runtime, kind + " (node '" + loc + "'): " + e.what());
        } catch (const std::exception& e) {
            std::string kind = node.is_prim ? node.prim.name() : node.composite.name;
            std::string loc = node.loc_name ? *node.loc_name : "<unnamed>";
            fail(ErrKind::Runtime, kind + " (node '" + loc + "'): " + e.what());
        }

        for (auto v : deaths_[step])
            if (plan->loc[v].kind == ValueLoc::Arena) arena.release(plan->loc[v].offset, arena_size[v]);
    }

    plan->arena_bytes = arena.end;
    plan->scratch_bytes = em.scratch_bytes;
    plan->recs = std::move(em.recs);
    for (auto& o : m.outputs) {
        OutSpec s;
        s.name = o.first;
        s.value = o.second;
        s.dtype = m.values[o.second].ty.dtype;
        s.shape = plan->shapes[o.second];
        s.cap = trefs[o.second].cap;
        plan->outputs.push_back(std::move(s));
    }
    return plan;
}

void Session::lower_prim(oxk::Emitter& em, const Node& node, const Bindings& b, const std::vector<TRef>& ins,
                         const std::vector<TRef>& outs) {
    const Prim& p = node.prim;
    const TRef& y = outs[0];
    for (auto& t : ins)
        if (t.cap) fail(ErrKind::Unsupported, "a KV-cache view reached a primitive; it should have been packed first");
    if (y.numel() == 0 && p.kind != PrimKind::Scatter) return;
    switch (p.kind) {
        case PrimKind::Unary: oxk::emit_unary(em, p.op, ins[0], y); break;
        case PrimKind::Binary: oxk::emit_binary(em, p.op, ins[0], ins[1], y); break;
        case PrimKind::Compare: oxk::emit_compare(em, p.op, ins[0], ins[1], y); break;
        case PrimKind::Select: oxk::emit_select(em, ins[0], ins[1], ins[2], y); break;
        case PrimKind::Cast: oxk::emit_cast(em, ins[0], y); break;
        case PrimKind::MatMul:
            if (ins[0].numel() == 0 || ins[1].numel() == 0)
                fail(ErrKind::Unsupported, "matmul with an empty contraction dimension");
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
        case PrimKind::Dequantize: oxk::emit_dequantize(em, ins[0], ins[1], ins.size() > 2 ? &ins[2] : nullptr, y, (int64_t)p.block_size); break;
    }
}

// ───────────────────────────── execution ────────────────────────────────
void Session::execute(Plan& plan, const std::vector<DTensor>& inputs, std::vector<BufferRef>& out_bufs) {
    if (!plan.arena && plan.arena_bytes + plan.scratch_bytes > 0) plan.arena = pool_.alloc(plan.arena_bytes + plan.scratch_bytes + 256);
    char* arena_base = plan.arena ? (char*)plan.arena->ptr : nullptr;
    size_t scratch_off = (plan.arena_bytes + 255) / 256 * 256;

    out_bufs.clear();
    for (auto& ob : plan.out_bufs) {
        if (ob.alias_input >= 0) {
            out_bufs.push_back(inputs[ob.alias_input].buf);
        } else {
            BufferRef b = pool_.alloc(std::max<size_t>(ob.bytes, 1));
            out_bufs.push_back(b);
        }
    }

    auto resolve = [&](const Buf& buf) -> void* {
        if (buf.slot == oxk::kSlotErr) return (void*)d_err_;
        if (buf.slot == oxk::kSlotNull) return nullptr;
        if (buf.slot == oxk::kSlotScratch) return arena_base + scratch_off + buf.off;
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

    std::vector<uint8_t> params;
    for (size_t i = 0; i < plan.recs.size(); i++) {
        const oxk::LaunchRec& r = plan.recs[i];
        params = r.params;
        for (auto& rl : r.relocs) {
            void* p = resolve(rl.buf);
            std::memcpy(params.data() + rl.field_off, &p, sizeof(void*));
        }
        void* args[1] = {params.data()};
        if (profiling) OX_CUDA(cudaEventRecord(ev_a_, stream_));
        OX_CUDA(cudaLaunchKernel(r.func, r.grid, r.block, args, r.smem, stream_));
        launch_count++;
        if (profiling) {
            OX_CUDA(cudaEventRecord(ev_b_, stream_));
            OX_CUDA(cudaEventSynchronize(ev_b_));
            float ms = 0;
            OX_CUDA(cudaEventElapsedTime(&ms, ev_a_, ev_b_));
            Timing t;
            t.kernel = r.label;
            t.node = (r.node >= 0 && (size_t)r.node < info_.size()) ? info_[r.node].label : "";
            t.time_ns = (uint64_t)(ms * 1e6);
            timings.push_back(std::move(t));
        }
    }
    for (size_t i = 0; i < plan.out_bufs.size(); i++)
        if (plan.out_bufs[i].kv_rows >= 0) out_bufs[i]->kv_rows = plan.out_bufs[i].kv_rows;

    OX_CUDA(cudaMemcpyAsync(h_err_, d_err_, sizeof(oxk::ErrWord), cudaMemcpyDeviceToHost, stream_));
    err_pending_ = true;
}

std::vector<std::pair<std::string, DTensor>> Session::run(const std::vector<std::pair<std::string, DTensor>>& named) {
    OX_CUDA(cudaSetDevice(device_));
    const Module& m = module_;
    // match by name against the signature (crates/onyxia-ir/src/backend.rs:47-50)
    std::vector<DTensor> inputs(m.inputs.size());
    std::vector<InputDesc> descs;
    std::vector<std::vector<size_t>> shape_store(m.inputs.size());
    for (size_t i = 0; i < m.inputs.size(); i++) {
        const DTensor* found = nullptr;
        for (auto& kv : named)
            if (kv.first == m.inputs[i].first) found = &kv.second;
        if (!found) fail(ErrKind::Binding, "missing input '" + m.inputs[i].first + "'");
        if (!found->buf) fail(ErrKind::Runtime, "input '" + m.inputs[i].first + "' is not a device tensor of this backend");
        inputs[i] = *found;
        for (auto d : found->shape) shape_store[i].push_back((size_t)d);
    }
    for (size_t i = 0; i < m.inputs.size(); i++)
        descs.push_back(InputDesc{m.inputs[i].first.c_str(), inputs[i].dtype, shape_store[i].data(), shape_store[i].size()});
    Bindings bindings = bind_shapes(m, descs);

    for (size_t i = 0; i < inputs.size(); i++)
        if (inputs[i].cap && input_needs_dense_[i]) inputs[i] = dense_copy(inputs[i]);

    // Which KV caches can be appended to in place this time?
    std::vector<char> kv_in_place(m.nodes.size(), 0);
    for (size_t n = 0; n < m.nodes.size(); n++) {
        int ik = gqa_past_input_[0][n], iv = gqa_past_input_[1][n];
        if (ik < 0 || iv < 0) continue;
        const DTensor &tk = inputs[ik], &tv = inputs[iv];
        ValueId pres = m.nodes[n].outputs[1];
        int64_t total = (int64_t)m.values[pres].ty.shape[2].eval(bindings);
        auto ok = [&](const DTensor& t) {
            return t.cap >= total && t.offset == 0 && t.shape.size() == 4 && t.buf->kv_rows == t.shape[2];
        };
        // only when both present tensors are module outputs with their own buffers
        bool outs = is_output_root_[m.nodes[n].outputs[1]] && is_output_root_[m.nodes[n].outputs[2]];
        kv_in_place[n] = ok(tk) && ok(tv) && tk.buf != tv.buf && outs;
        if (!kv_in_place[n]) {
            // a capacity view that cannot be extended is read as it is
        }
    }

    std::unique_ptr<Plan> plan = build_plan(bindings, inputs, kv_in_place);
    std::vector<BufferRef> out_bufs;
    execute(*plan, inputs, out_bufs);

    std::vector<std::pair<std::string, DTensor>> outs;
    for (auto& spec : plan->outputs) {
        ValueId root = alias_root_[spec.value];
        const ValueLoc& l = plan->loc[root];
        DTensor t;
        t.dtype = spec.dtype;
        t.shape = spec.shape;
        t.cap = spec.cap;
        switch (l.kind) {
            case ValueLoc::Output: t.buf = out_bufs[l.index]; break;
            case ValueLoc::Input: t.buf = inputs[l.index].buf; t.offset = inputs[l.index].offset; t.cap = inputs[l.index].cap; break;
            case ValueLoc::Const: t.buf = consts_[root].buf; break;
            default: fail(ErrKind::Runtime, "internal: module output without storage");
        }
        outs.emplace_back(spec.name, std::move(t));
    }
    // the plan (and its arena) may be recycled once the stream has passed it:
    // keep it until the next run replaces it
    plans_.push_front(std::move(plan));
    while (plans_.size() > 2) plans_.pop_back();
    return outs;
}

}  // namespace oxrt
