/* onyxia_cuda.h — C ABI of the B200 execution backend for the Onyxia IR.
 *
 * This is the surface a Rust `onyxia-backend-cuda` crate binds to implement
 * the two traits of the reference unchanged:
 *
 *   trait Backend { fn supports(&self,&str)->bool; fn prepare(&self, Module)->Result<Session>; }
 *   trait Session { fn upload(..); async fn run(..); async fn download(..); }
 *       — crates/onyxia-ir/src/backend.rs:24-54
 *
 * A `Module` (crates/onyxia-ir/src/graph.rs:253-275) crosses the boundary
 * through the builder calls below, which mirror `GraphBuilder`
 * (crates/onyxia-ir/src/builder.rs:39-248): primitives are type-inferred as
 * they are added, composites declare their output types.
 *
 * Rules: plain pointers and sizes only; no exceptions cross the boundary;
 * every fallible call returns an `ox_status` and leaves a message readable
 * with `ox_last_error()` (per thread). One session is used by one host thread
 * at a time (`&mut self` in the reference).
 */
#ifndef ONYXIA_CUDA_H
#define ONYXIA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Error kinds = the variants of onyxia_ir::Error (crates/onyxia-ir/src/lib.rs:55-89). */
typedef enum ox_status {
    OX_OK = 0,
    OX_ERR_SHAPE = 1,
    OX_ERR_INVALID_GRAPH = 2,
    OX_ERR_DTYPE = 3,
    OX_ERR_ATTRIBUTE = 4,
    OX_ERR_BINDING = 5,
    OX_ERR_INTERP = 6,
    OX_ERR_UNSUPPORTED = 7,
    OX_ERR_RUNTIME = 8
} ox_status;

/* Element types (crates/onyxia-ir/src/types.rs:13-26). U4/I4 are bit-packed,
 * two elements per byte, low nibble first, total rounded up to a byte. */
typedef enum ox_dtype {
    OX_F32 = 0, OX_F16, OX_I64, OX_I32, OX_U32, OX_U8, OX_I8, OX_BOOL, OX_U4, OX_I4
} ox_dtype;

/* Primitive kinds (crates/onyxia-ir/src/prim.rs:130-214), in declaration order. */
typedef enum ox_prim_kind {
    OX_PRIM_UNARY = 0, OX_PRIM_BINARY, OX_PRIM_COMPARE, OX_PRIM_SELECT, OX_PRIM_CAST,
    OX_PRIM_MATMUL, OX_PRIM_REDUCE, OX_PRIM_RESHAPE, OX_PRIM_TRANSPOSE, OX_PRIM_BROADCAST,
    OX_PRIM_CONCAT, OX_PRIM_SLICE, OX_PRIM_GATHER, OX_PRIM_SCATTER, OX_PRIM_IOTA,
    OX_PRIM_DIM_VALUES, OX_PRIM_DEQUANTIZE
} ox_prim_kind;

/* Operator codes for ox_prim_desc.op (crates/onyxia-ir/src/prim.rs:27-107). */
enum { OX_NEG = 0, OX_ABS, OX_SQRT, OX_RSQRT, OX_EXP, OX_LOG, OX_SIN, OX_COS, OX_TANH, OX_ERF,
       OX_FLOOR, OX_CEIL, OX_NOT };
enum { OX_ADD = 0, OX_SUB, OX_MUL, OX_DIV, OX_POW, OX_MAX, OX_MIN, OX_AND, OX_OR, OX_XOR };
enum { OX_EQ = 0, OX_NE, OX_LT, OX_LE, OX_GT, OX_GE };
enum { OX_SUM = 0, OX_MEAN, OX_RMAX, OX_RMIN, OX_PROD };

/* A symbolic dimension: sum of terms, each coeff × product of symbols
 * (crates/onyxia-ir/src/dim.rs:131-162). A constant c is one term with
 * n_syms = 0; zero is n_terms = 0. Symbols are ids from
 * ox_module_intern_symbol. */
#define OX_MAX_TERM_SYMS 6
typedef struct ox_dimterm {
    int64_t coeff;
    int32_t n_syms;
    int32_t syms[OX_MAX_TERM_SYMS];
} ox_dimterm;

typedef struct ox_dimexpr {
    const ox_dimterm* terms;
    int32_t n_terms;
} ox_dimexpr;

typedef struct ox_slice_spec {
    uint64_t axis;
    ox_dimexpr start; /* inclusive, in the direction of travel */
    ox_dimexpr end;   /* exclusive */
    int64_t step;     /* never 0 */
} ox_slice_spec;

/* Parameters of one primitive; only the fields of `kind` are read. */
typedef struct ox_prim_desc {
    int32_t kind;             /* ox_prim_kind */
    int32_t op;               /* unary / binary / compare / reduce operator */
    int32_t dtype;            /* Cast target, Iota element type */
    int32_t trans_a, trans_b; /* MatMul */
    int32_t keepdims;         /* Reduce */
    const uint64_t* axes;     /* Reduce axes (sorted) or Transpose perm */
    int32_t n_axes;
    const ox_dimexpr* shape;  /* Reshape/Broadcast target, Dequantize out_shape, DimValues exprs */
    int32_t n_shape;
    uint64_t axis;            /* Concat / Gather */
    const ox_slice_spec* specs;
    int32_t n_specs;
    ox_dimexpr len;           /* Iota */
    uint64_t block_size;      /* Dequantize */
} ox_prim_desc;

/* Composite attribute (crates/onyxia-ir/src/attrs.rs:12-23). */
typedef enum ox_attr_kind { OX_ATTR_INT = 0, OX_ATTR_INTS, OX_ATTR_FLOAT, OX_ATTR_FLOATS, OX_ATTR_STR, OX_ATTR_BOOL } ox_attr_kind;
typedef struct ox_attr {
    const char* name;
    int32_t kind; /* ox_attr_kind */
    int64_t i;    /* INT, BOOL */
    double f;     /* FLOAT */
    const char* s;
    const int64_t* ints;
    const double* floats;
    int32_t n; /* element count for INTS / FLOATS */
} ox_attr;

typedef struct ox_tensor_type {
    int32_t dtype;
    const ox_dimexpr* dims;
    int32_t rank;
} ox_tensor_type;

typedef struct ox_module ox_module;
typedef struct ox_backend ox_backend;
typedef struct ox_session ox_session;
typedef struct ox_tensor ox_tensor;

/* Message of the last failed call on this thread (includes the node name for
 * execution errors, like crates/onyxia-backend-wgpu/src/session.rs:583-587). */
const char* ox_last_error(void);

/* ── Module construction ≙ GraphBuilder (crates/onyxia-ir/src/builder.rs) ── */
ox_module* ox_module_new(void);
void ox_module_free(ox_module*);
/* Deep copy of the graph; constant bytes are shared, not copied. */
ox_module* ox_module_clone(const ox_module*);
/* Tensor-parallel partition (no counterpart in the reference, which executes on one
 * device): a new module holding what rank `rank` of `tp` ranks executes. Pairs of
 * MatMulNBits nodes are split along N then K (column-split Q/K/V/gate/up, row-split
 * O/down), attention runs on the rank's heads and its share of the KV cache (the
 * declared shapes of the cache inputs and outputs shrink by `tp` along the head axis),
 * and an `onyxia.AllReduce` composite follows every K-split node; a backend created
 * with ox_backend_create_tp executes it as a sum over the ranks. The source module is
 * left untouched. `ox_module_tp_stats` reports how many nodes would be split along N
 * (out[0]), along K (out[1]) and how many attention nodes (out[2]). */
ox_status ox_module_tp_partition(const ox_module*, int32_t tp, int32_t rank, ox_module** out);
void ox_module_tp_stats(const ox_module*, int32_t tp, uint64_t out[3]);
/* ≙ GraphBuilder::sym (builder.rs:69-71). */
int32_t ox_module_intern_symbol(ox_module*, const char* name);
/* ≙ GraphBuilder::constant (builder.rs:127-135). With borrow != 0 the bytes
 * are not copied and must stay valid until the module (and its clones) have
 * been prepared or freed. */
ox_status ox_module_add_const(ox_module*, int32_t dtype, const uint64_t* dims, int32_t rank,
                              const void* bytes, size_t nbytes, int32_t borrow, int32_t* out_value);
/* ≙ GraphBuilder::input (builder.rs:115-124). */
ox_status ox_module_add_input(ox_module*, const char* name, int32_t dtype, const ox_dimexpr* dims,
                              int32_t rank, int32_t* out_value);
/* ≙ GraphBuilder::prim (builder.rs:152-191): infers the output type. */
ox_status ox_module_add_prim(ox_module*, const ox_prim_desc*, const int32_t* inputs, int32_t n_in,
                             int32_t* out_value);
/* ≙ GraphBuilder::composite (builder.rs:196-234). */
ox_status ox_module_add_composite(ox_module*, const char* name, const ox_attr* attrs, int32_t n_attrs,
                                  const int32_t* inputs, int32_t n_in, const ox_tensor_type* outs,
                                  int32_t n_out, int32_t* out_values);
/* ≙ GraphBuilder::output (builder.rs:237-242). */
ox_status ox_module_add_output(ox_module*, const char* name, int32_t value);
/* ≙ GraphBuilder::constrain (builder.rs:102-112). */
ox_status ox_module_add_constraint(ox_module*, const ox_dimexpr* left, const ox_dimexpr* right,
                                   const char* context);
/* ≙ GraphBuilder::set_loc (builder.rs:79-81); NULL clears. */
void ox_module_set_loc(ox_module*, const char* node_name, const char* op_type);
/* ≙ validate::validate (crates/onyxia-ir/src/validate.rs:15). */
ox_status ox_module_validate(const ox_module*);
/* ≙ decomp::inline_composites (crates/onyxia-ir/src/decomp.rs:73-133) with
 * `supports(name) = name ∈ keep`. Rewrites the module in place. */
ox_status ox_module_inline_composites(ox_module*, const char* const* keep, int32_t n_keep);
/* ≙ fold::fold_transpose_into_matmul followed by eliminate_dead (crates/onyxia-ir/src/fold.rs:129-204): a
 * Transpose of the last two axes feeding a MatMul operand becomes the MatMul's trans flag. Returns 1 when
 * something was folded, 0 when not, -1 on an internal error. */
int32_t ox_module_fold_transposes(ox_module*);

/* Introspection used by callers such as LlmSession (crates/onyxia-cli/src/llm.rs:47-61,232-246). */
int32_t ox_module_num_nodes(const ox_module*);
int32_t ox_module_num_values(const ox_module*);
int32_t ox_module_num_inputs(const ox_module*);
int32_t ox_module_num_outputs(const ox_module*);
const char* ox_module_input_name(const ox_module*, int32_t i);
const char* ox_module_output_name(const ox_module*, int32_t i);
/* dtype and rank of input i. */
ox_status ox_module_input_desc(const ox_module*, int32_t i, int32_t* dtype, int32_t* rank);
/* Evaluate input i's declared shape under symbol bindings given by name. */
ox_status ox_module_eval_input_shape(const ox_module*, int32_t i, const char* const* sym_names,
                                     const uint64_t* sym_values, int32_t n_syms, uint64_t* out_dims);
/* Name of node i's operation ("matmul", "com.microsoft.MatMulNBits", …). */
const char* ox_module_node_op(const ox_module*, int32_t i);
/* Type of a value rendered as text, e.g. "f16[batch_size, 1, 1152]". The
 * pointer is valid until the next call on this thread. */
const char* ox_module_value_type_str(const ox_module*, int32_t value);

/* ── Backend ≙ impl Backend (crates/onyxia-backend-wgpu/src/session.rs:107-242) ── */
/* Options for ox_backend_create_ex; zero-initialise for defaults. */
typedef struct ox_backend_options {
    int32_t without_fused_kernels; /* ≙ WgpuBackend::without_fused_kernels (session.rs:125-134) */
    int32_t disable_graphs;        /* launch kernels one by one instead of replaying CUDA graphs */
    int32_t disable_pattern_fusion;/* keep every node its own launch (no cross-node fusion) */
    int32_t disable_persistent_step; /* one launch per operation of a decode step instead of the persistent step kernel */
    int32_t reserved[4];
} ox_backend_options;

/* One backend per process and device set. `device_ordinals` lists the CUDA
 * devices. A backend drives ONE device — the first of the list; further entries are checked for
 * validity and otherwise unused. Several GPUs are used by running one process (one backend) per
 * GPU and joining them into a tensor-parallel group, see below. */
ox_status ox_backend_create(const int32_t* device_ordinals, int32_t n_devices, ox_backend** out);
ox_status ox_backend_create_ex(const int32_t* device_ordinals, int32_t n_devices,
                               const ox_backend_options* options, ox_backend** out);
void ox_backend_free(ox_backend*);
/* Tensor parallelism (no counterpart in the reference). One process per GPU: rank 0 obtains an
 * id with ox_tp_unique_id and distributes its 128 bytes by whatever channel the host has; every
 * rank then calls ox_backend_join_tp on its backend (a collective call: it returns when all
 * `world` ranks have joined). A joined backend executes the `onyxia.AllReduce` composites that
 * ox_module_tp_partition inserts as NCCL all-reduces on the session's stream.
 * `nccl_library_path` names libnccl.so.2 when the process has not loaded NCCL yet (NULL: search
 * the loader path); the library is opened at run time, so nothing here is needed on one GPU.
 * The group's communicator lives until the process exits: ox_backend_free on a joined backend
 * does not tear it down (destroying or aborting an NCCL communicator while the host language's
 * runtime shuts down was seen to block). */
ox_status ox_tp_unique_id(const char* nccl_library_path, uint8_t out[128]);
ox_status ox_backend_join_tp(ox_backend*, int32_t rank, int32_t world, const uint8_t id[128], const char* nccl_library_path);
/* 1 when the joined group reduces f16 messages of up to 1 MiB with the library's own kernel over peer memory
 * (regions exchanged with CUDA IPC at join time, ordinary peer loads, bounded waits), 0 when every all-reduce
 * goes to ncclAllReduce (no group, more than 8 ranks, the mapping failed, or ONYXIA_DISABLE_PEER_ALLREDUCE=1). */
int32_t ox_backend_peer_allreduce(const ox_backend*);
/* ≙ Backend::supports (backend.rs:28-31): 1 if a fused kernel is registered under this name. */
int32_t ox_backend_supports(const ox_backend*, const char* composite_name);
/* ≙ Backend::prepare (backend.rs:33-34). Consumes `module` (also on failure). */
ox_status ox_backend_prepare(ox_backend*, ox_module* module, ox_session** out);

/* ── Session ≙ impl Session (backend.rs:37-54; wgpu session.rs:510-649) ── */
void ox_session_free(ox_session*);
/* ≙ Session::upload. Host layout = interp::Tensor (crates/onyxia-ir/src/interp.rs:29-49). */
ox_status ox_session_upload(ox_session*, int32_t dtype, const uint64_t* shape, int32_t rank,
                            const void* bytes, size_t nbytes, ox_tensor** out);
/* ≙ Session::run: inputs matched by name against the module signature; all
 * module outputs are returned in signature order. `out_names[i]` points into
 * session-owned storage; `out_tensors[i]` are new handles the caller releases. */
ox_status ox_session_run(ox_session*, const char* const* names, ox_tensor* const* inputs, int32_t n_in,
                         const char** out_names, ox_tensor** out_tensors, int32_t out_cap, int32_t* n_out);
/* Number of module outputs = how many entries a run returns (≙ module.outputs.len(), graph.rs:267). */
int32_t ox_session_num_outputs(const ox_session*);
/* ≙ Session::download: blocks until the tensor's producer has finished. */
ox_status ox_session_download(ox_session*, const ox_tensor*, void* dst, size_t cap, size_t* written);

/* Device tensor handles: cheap to clone (≙ `type Tensor: Clone`, backend.rs:41-42). */
ox_tensor* ox_tensor_clone(const ox_tensor*);
void ox_tensor_release(ox_tensor*);
ox_status ox_tensor_describe(const ox_tensor*, int32_t* dtype, uint64_t* shape, int32_t shape_cap, int32_t* rank);
size_t ox_tensor_nbytes(const ox_tensor*);

/* Inherent session methods of the reference GPU backend
 * (crates/onyxia-backend-wgpu/src/session.rs:280-340). */
ox_status ox_session_wait_idle(ox_session*);
uint64_t ox_session_resident_bytes(const ox_session*);
uint64_t ox_session_peak_resident_bytes(const ox_session*);
void ox_session_pool_stats(const ox_session*, uint64_t* fresh_allocations, uint64_t* reuses);
/* Per-launch device timing ≙ enable_profiling / take_timings
 * (crates/onyxia-backend-wgpu/src/profile.rs:18-28). */
typedef struct ox_kernel_timing {
    const char* kernel; /* kernel label */
    const char* node;   /* IR node name or op */
    uint64_t time_ns;
} ox_kernel_timing;
int32_t ox_session_enable_profiling(ox_session*, int32_t on);
/* Copies up to `cap` records; returns the number available. Strings stay valid
 * until the next take. */
int32_t ox_session_take_timings(ox_session*, ox_kernel_timing* out, int32_t cap);
/* Device-side stopwatch on the session's stream: `start` records an event
 * behind the work queued so far, `stop` records a second one, waits for it and
 * returns the elapsed milliseconds between the two. */
ox_status ox_session_timer_start(ox_session*);
ox_status ox_session_timer_stop(ox_session*, float* elapsed_ms);
/* Number of kernel launches (graph nodes included) issued since prepare. */
uint64_t ox_session_launch_count(const ox_session*);
/* Planner counters since prepare: out[0] plans built from scratch, out[1] plans
 * patched in place for a changed symbol binding, out[2] plans reused unchanged,
 * out[3] CUDA-graph launches, out[4] graph kernel nodes whose parameters were
 * rewritten, out[5] runs, out[6..8] host microseconds summed over those runs
 * spent binding inputs, planning, and patching + launching. */
void ox_session_plan_stats(const ox_session*, uint64_t out[9]);
/* Greedy sampling on the device: index of the maximum over the last axis of
 * `logits`, highest index among equal maxima (≙ sampling::sample_greedy,
 * crates/onyxia-cli/src/sampling.rs:71-80, which keeps the last maximum).
 * Returns an I64 tensor shaped like `logits` without its last axis. */
ox_status ox_session_argmax_last(ox_session*, const ox_tensor* logits, ox_tensor** out);
/* Temperature / top-k / top-p sampling on the device ≙ sampling::sample
 * (crates/onyxia-cli/src/sampling.rs:36-195): the logits of every row are divided
 * by `temperature`; `top_k` > 0 keeps the k largest (k at or above the vocabulary:
 * all of them), otherwise 0 < `top_p` < 1 keeps the shortest prefix of the
 * descending order whose cumulative probability reaches p, otherwise all are kept;
 * the token is the first index at which the running sum of exp(l - max) over the
 * kept entries reaches uniform[row] * sum. The random generator stays with the
 * caller: `uniform` holds one number in [0, 1] per row (the reference uses
 * next_u32 / u32::MAX). A temperature at or below 1e-6 selects greedily, like the
 * reference. Sums are exact and ties among equal logits are kept in index order,
 * so a draw is reproducible; it can differ from the reference's f32 running sums
 * only when uniform * sum falls within rounding of a boundary between two tokens.
 * Rows without a finite logit are reported as OX_ERR_RUNTIME at the next
 * synchronising call. Returns an I64 tensor shaped like `logits` without its last axis. */
ox_status ox_session_sample_last(ox_session*, const ox_tensor* logits, float temperature, int64_t top_k, float top_p,
                                 const float* uniform, size_t n_uniform, ox_tensor** out);
/* The same argmax written into a tensor the caller already holds, without
 * allocating anything: no device allocation, no buffer from the session's pool,
 * no new tensor handle. One kernel is enqueued on the session's stream; its
 * scratch is a fixed array inside the library's device image. This entry point
 * has no counterpart in the reference; it exists for callers that must not
 * allocate at the point where they sample (a serving loop running against a
 * device-memory budget it has already committed in full, or a section that
 * cannot tolerate the device-wide synchronisation an allocation may cause).
 *   - `logits`: F32 or F16, densely packed, at most 64 rows (the product of all
 *     axes but the last); more rows fail with OX_ERR_RUNTIME and a message that
 *     names the limit. `out`: an I64 tensor with exactly one element per row.
 *   - The first call on a device looks up the scratch array's address while that
 *     device is current; make it before starting any stream capture.
 *   - All calls on one device share the scratch array: calls that could execute
 *     concurrently (other sessions, other host threads) race and must be ordered
 *     by the caller. Calls on one session are ordered by its stream. */
ox_status ox_session_argmax_last_into(ox_session*, const ox_tensor* logits, ox_tensor* out);

/* The KV-cache generation loop as one call per step ≙ LlmSession (crates/onyxia-cli/src/llm.rs:26-246):
 * `present.N.*` outputs are fed back as `past_key_values.N.*` inputs, the cache starts empty, masks are
 * all ones, `position_ids` (if the module has them) continue from the current length. `ox_llm_step` runs
 * `n_ids` new tokens (a prompt, or one token); with `token_out` the greedy choice (highest logit of the last
 * position, last index among equals ≙ sampling.rs:71-80) is made on the device and 8 bytes come back; with
 * `logits_out` the last position's logits are copied out in their stored dtype. The session is borrowed and
 * must outlive the loop object; one thread at a time. */
typedef struct ox_llm ox_llm;
ox_status ox_llm_create(ox_session*, int64_t max_seq_len, ox_llm** out);
void ox_llm_free(ox_llm*);
int64_t ox_llm_sequence_length(const ox_llm*);
int32_t ox_llm_logits_dtype(const ox_llm*); /* ox_dtype code of the logits `ox_llm_step` copies out */
void ox_llm_reset(ox_llm*);
ox_status ox_llm_step(ox_llm*, const int64_t* ids, int32_t n_ids, int64_t* token_out, void* logits_out, size_t logits_cap,
                      size_t* logits_written);
/* `n_new` greedy tokens in one call: the first step runs `ids` (a prompt, or one token), every later step takes its
 * input id from the previous step's argmax on the device. Every step still uploads its attention mask from host
 * memory and sends its token id to (pinned) host memory, but the host does not wait in between: the steps are
 * enqueued back to back and the call returns when `tokens_out[0 .. n_new)` is complete. It does not stop at an
 * end-of-sequence id; the caller truncates. ≙ the decode loop of crates/onyxia-cli/src/bench.rs:152-174 without
 * its per-token host round trip. */
ox_status ox_llm_generate(ox_llm*, const int64_t* ids, int32_t n_ids, int32_t n_new, int64_t* tokens_out);
/* The same step with the next token drawn on the device from the last position's logits by temperature /
 * top-k / top-p sampling (see ox_session_sample_last; crates/onyxia-cli/src/sampling.rs:36-65); `uniform` is
 * the caller's random number in [0, 1]. */
ox_status ox_llm_step_sampled(ox_llm*, const int64_t* ids, int32_t n_ids, float temperature, int64_t top_k, float top_p, float uniform,
                              int64_t* token_out);

#ifdef __cplusplus
}
#endif
#endif /* ONYXIA_CUDA_H */
