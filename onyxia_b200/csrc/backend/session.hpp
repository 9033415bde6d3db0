// The prepared session: plans (one per binding of the dimension symbols),
// their execution, and the host<->device boundary.
#pragma once
#include <list>

#include "runtime.hpp"
#include "../kernels/persist.hpp"

namespace oxrt {

// Where a value's bytes live while a plan runs.
struct ValueLoc {
    enum Kind : uint8_t { None, Arena, Const, Input, Output, Alias } kind = None;
    uint32_t index = 0;   // Input: position in module.inputs; Output: position in Plan::out_bufs; Alias: root value
    size_t offset = 0;    // Arena: byte offset
};

// One output buffer a run has to provide (several module outputs may share it).
struct OutBuf {
    size_t bytes = 0;
    int alias_input = -1;  // ≥ 0: the buffer of that module input is reused (in-place KV append)
    int64_t kv_cap = 0;    // rows per head for a freshly allocated KV cache
    int64_t kv_rows = -1;  // rows valid after this run (KV caches)
};

struct OutSpec {
    std::string name;
    ValueId value;
    DType dtype;
    std::vector<int64_t> shape;
    int64_t cap = 0;
};

// Everything needed to execute the module for one binding of the symbols.
//
// A plan is a flat list of launch records. Pointers inside the records are
// symbolic (value slot + offset) and are resolved against the current buffers
// at every run, so the same plan serves any set of input/output buffers. When
// only some dimension symbols change between runs (a decode loop: the KV
// length grows by one), the plan is updated in place: only the nodes whose
// types mention a changed symbol are lowered again.
struct Plan {
    std::vector<uint64_t> structure;             // what must match exactly (caps, in-place flags)
    ox::Bindings bindings;
    std::vector<oxk::LaunchRec> recs;
    std::vector<std::pair<uint32_t, uint32_t>> node_recs;  // per node: [begin, count) in recs
    std::vector<ValueLoc> loc;                   // per value
    std::vector<oxk::TRef> trefs;                // per value
    std::vector<size_t> arena_size;              // per value (Arena values)
    std::vector<OutBuf> out_bufs;
    std::vector<OutSpec> outputs;                // module outputs, signature order
    size_t arena_bytes = 0, scratch_bytes = 0, scratch_capacity = 0;
    BufferRef arena;                             // arena + scratch, owned by the plan
    // Per-run scalars (kDynPerNode int64 slots per node) and the bucket each
    // node's launch was sized for (0 = the node has none).
    std::vector<int64_t> dyn_host;
    std::vector<int64_t> node_bucket, node_bucket_step;
    bool dyn_used = false;
    BufferRef dyn_dev;
    static constexpr int kDynRing = 8;
    int64_t* dyn_pinned = nullptr;               // kDynRing staging copies of dyn_host
    cudaEvent_t dyn_events[kDynRing] = {};
    unsigned dyn_cursor = 0;
    // What a run executes: the records of `recs`, with every run of consecutive records that the
    // persistent step kernel can execute replaced by one launch of it.
    struct PersistRun {
        std::vector<oxk::PersistOp> ops;  // what the launch was built from (compared on every re-lowering)
        bool ok = false;                  // false: the run was found unsuitable, its records launch one by one
        size_t xoff = 0;                  // where the run's words start in the exchange area
        oxk::PersistLaunch launch;
    };
    std::vector<PersistRun> persist_runs;
    std::vector<const oxk::LaunchRec*> launches;
    BufferRef xbuf;                              // exchange area of the persistent launches (tagged words)
    size_t xbuf_bytes = 0;
    uint64_t epoch = 0;                          // tags the words of one run; never repeats within a plan
    // CUDA graph of the launch list, with the launch state each node currently holds.
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    std::vector<cudaGraphNode_t> graph_nodes;
    std::vector<std::vector<uint8_t>> graph_params;
    std::vector<dim3> graph_grids, graph_clusters;
    std::vector<const void*> graph_funcs;
    uint64_t uses = 0;
    ~Plan();
};

class Session {
public:
    Session(Backend& backend, Module legalized);
    ~Session();

    DTensor upload(DType dtype, const std::vector<int64_t>& shape, const void* bytes, size_t nbytes);
    std::vector<std::pair<std::string, DTensor>> run(const std::vector<std::pair<std::string, DTensor>>& inputs);
    void preplan(const std::vector<std::pair<std::string, DTensor>>& next_inputs);
    void download(const DTensor& t, void* dst, size_t cap, size_t* written);
    // Enqueues the copy of a densely packed tensor into pinned host memory and returns at once; the bytes are there
    // after the next wait_idle().
    void download_async(const DTensor& t, void* pinned_dst);
    DTensor argmax_last(const DTensor& logits);
    DTensor sample_last(const DTensor& logits, float temperature, long long top_k, float top_p, const float* u, size_t n_u);
    void argmax_last_into(const DTensor& logits, const DTensor& out);
    void wait_idle();
    void timer_start();
    float timer_stop();
    std::vector<Timing> take_timings();

    uint64_t resident_bytes() const { return pool_->live_bytes(); }
    uint64_t peak_resident_bytes() const { return pool_->peak_bytes(); }
    const Pool& pool() const { return *pool_; }
    bool profiling = false;
    uint64_t launch_count = 0;
    // planner statistics: plans built from scratch, updated in place, reused as they were
    uint64_t plans_built = 0, plans_updated = 0, plans_reused = 0, graph_node_updates = 0, graph_launches = 0;
    // host time spent inside run(): binding, planning, patching + launching (µs, summed)
    double host_us[3] = {0, 0, 0};
    uint64_t host_runs = 0;
    const Module& module() const { return module_; }
    void* error_area() const { return d_err_; }
    const std::vector<std::string>& output_names() const { return output_names_; }

private:
    struct NodeInfo {
        const FusedKernel* fused = nullptr;
        // Pattern fusion: this node's work is done by `absorbed_by`'s kernel.
        int absorbed_by = -1;
        int fuse_with = -1;  // the partner node this node's kernel also covers
        int fuse_kind = 0;
        std::string label;
        std::vector<ox::SymId> syms;  // symbols the node's lowering depends on
    };
    enum { FUSE_NONE = 0, FUSE_GEGLU = 1, FUSE_ADD_NORM = 2 };

    // MatMulNBits nodes that read the same activations run as one launch of the
    // streaming kernel over one tile stream. The launch may also cover the RMS
    // norm / residual add / RMS norm chain that produces the activations (as the
    // kernel's prologue) and a Gelu·Mul pair that consumes two members (as its
    // epilogue). All covered nodes are absorbed by the leader, the node at whose
    // step the launch is issued.
    struct GemvGroup {
        std::vector<ox::NodeId> members;  // in stream order
        int leader = -1;
        int geglu = 0;                    // 0 none, 1 tanh form, 2 erf form
        int gelu_node = -1, mul_node = -1;
        int norm2 = -1, add = -1, norm1 = -1;  // prologue chain, −1 = absent
        int slice = -1;                   // a row-selecting Slice in the chain (the last-token slice), −1 = absent
        bool slice_last = false;          // the Slice reads norm2's result (else norm2 reads the Slice's)
        ValueId src = 0, res = 0;         // what the prologue reads (src = the members' input without a prologue)
        bool has_zp = false;
        int64_t k = 0;
    };
    std::vector<GemvGroup> groups_;
    std::vector<int> group_of_leader_;    // per node: index into groups_ or −1
    void find_gemv_groups();
    void lower_group(oxk::Emitter& em, const GemvGroup& g, Plan& plan, const ox::Bindings& bindings);

    void upload_constants();
    void interleave_weights();
    void launch_now(const oxk::Emitter& em, const std::vector<void*>& slots);
    void analyse();
    void find_pattern_fusions();
    void collect_node_syms();

    std::vector<uint64_t> structure_key(const std::vector<DTensor>& inputs, const std::vector<char>& kv_in_place) const;
    std::unique_ptr<Plan> build_plan(const ox::Bindings& bindings, const std::vector<DTensor>& inputs,
                                     const std::vector<char>& kv_in_place);
    bool update_plan(Plan& plan, const ox::Bindings& bindings, const std::vector<DTensor>& inputs,
                     const std::vector<char>& kv_in_place);
    // Shapes, storage and launch records of one node. With `arena` set the
    // node's outputs are placed (full build); without, their placement is kept
    // and the call reports false if a size no longer fits (in-place update).
    bool lower_step(Plan& plan, oxk::Emitter& em, size_t step, ox::Bindings& bindings, const std::vector<DTensor>& inputs,
                    const std::vector<char>& kv_in_place, void* arena);
    void lower_prim(oxk::Emitter& em, const Node& node, const ox::Bindings& b, const std::vector<oxk::TRef>& ins,
                    const std::vector<oxk::TRef>& outs);
    void finish_outputs(Plan& plan);
    void fuse_persistent(Plan& plan);
    void execute(Plan& plan, const std::vector<DTensor>& inputs, std::vector<BufferRef>& out_bufs);
    Plan* plan_for(const std::vector<std::pair<std::string, DTensor>>& named, std::vector<DTensor>& inputs, bool shapes_only,
                   double* t_bound_out);
    void build_graph(Plan& plan, const std::vector<std::vector<uint8_t>>& params);
    void launch_rec(const oxk::LaunchRec& r, void* param_bytes, bool allow_pdl);
    void check_device_error();
    DTensor dense_copy(const DTensor& t);

    Backend& backend_;
    Options opt_;
    int device_;
    cudaStream_t stream_ = nullptr;
    std::shared_ptr<Pool> pool_;
    Module module_;
    std::vector<ox::NodeId> order_;
    std::vector<int> step_of_node_;
    std::vector<NodeInfo> info_;            // per node
    std::vector<ValueId> alias_root_;       // per value (itself when not an alias)
    std::vector<int> last_use_;             // per root value: last step reading it
    std::vector<std::vector<ValueId>> deaths_;  // per step: roots that die after it
    std::vector<DTensor> consts_;           // per value (empty unless Origin::Const)
    std::vector<char> interleaved_;         // per value: layout of a u4 weight constant (0 as uploaded, 1 interleaved, 2 tiled)
    unsigned* d_counters_ = nullptr;        // kCounterWords zeroed arrival counters
    std::vector<int> input_index_;          // per value: position in module.inputs or −1
    std::vector<char> is_output_root_;      // per value
    std::vector<char> input_needs_dense_;   // per module input
    std::vector<int> gqa_past_input_[2];    // per node: module-input index feeding past_k / past_v in place, or −1
    std::vector<std::string> output_names_;
    static constexpr size_t kErrAreaBytes = 256 + 8 * 8192;
    oxk::ErrWord* d_err_ = nullptr;
    oxk::ErrWord* h_err_ = nullptr;
    bool err_pending_ = false;
    std::list<std::unique_ptr<Plan>> plans_;  // most recently used first
    cudaEvent_t ev_t0_ = nullptr, ev_t1_ = nullptr;
    // pinned staging for small uploads
    static constexpr size_t kStageBytes = 64 * 1024;
    static constexpr unsigned kStageSlots = 16;
    uint8_t* stage_pinned_ = nullptr;
    cudaEvent_t stage_events_[kStageSlots] = {};
    unsigned stage_cursor_ = 0;
    // profiling: one event pair per launch, read back in take_timings
    struct ProfRec {
        cudaEvent_t a, b;
        const char* kernel;
        int node;
    };
    std::vector<ProfRec> prof_;
    std::vector<cudaEvent_t> prof_free_;
    cudaEvent_t prof_event();
};

}  // namespace oxrt
