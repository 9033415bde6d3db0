// Host-side interface to the CUDA kernels: one `emit_*` function per kernel
// family. An emit function does not launch; it appends launch records
// ({function, grid, block, shared memory, parameter bytes, pointer
// relocations}) to an Emitter. The session replays the records — directly, or
// as nodes of a CUDA graph — after patching pointer fields with the current
// buffer addresses.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <algorithm>
#include <cmath>
#include <initializer_list>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace oxk {

// Error codes written to the error word (first writer wins).
enum : int {
    ERR_NONE = 0,
    ERR_GATHER_OOB = 1,
    ERR_SCATTER_OOB = 2,
    ERR_INT_DIV_ZERO = 3,
    ERR_INT_POW_NEG = 4,
    ERR_SLICE_OOB = 5,
    ERR_WAIT_TIMEOUT = 6,
    ERR_SAMPLE_NO_FINITE = 7,
};

struct ErrWord {
    int code;
    int node;      // launch tag (IR node index)
    long long a;   // offending value
    long long b;   // bound
};

// A device address known only at execution time: a runtime value slot plus a
// byte offset into it.
struct Buf {
    uint32_t slot = 0xFFFFFFFFu;
    int64_t off = 0;
    Buf at(int64_t bytes) const { return Buf{slot, off + bytes}; }
    bool valid() const { return slot != 0xFFFFFFFFu; }
};
// Reserved slots resolved by the session.
constexpr uint32_t kSlotErr = 0xFFFFFFF0u;      // the session's ErrWord
constexpr uint32_t kSlotScratch = 0xFFFFFFF1u;  // the plan's scratch area (offset = position in it)
constexpr uint32_t kSlotNull = 0xFFFFFFF2u;     // resolves to nullptr
// A session-lifetime array of kCounterWords zeroed 32-bit arrival counters;
// kernels that use it leave every word zero again when they finish.
constexpr uint32_t kSlotCounters = 0xFFFFFFF3u;
constexpr size_t kCounterWords = 1 << 16;
// The plan's block of per-run scalars (int64 each; offset = byte position).
// Values that change from run to run without changing the launch geometry —
// the KV length of a decode step — are read from here by the kernels, so the
// parameter bytes of their launches stay identical and a CUDA graph replays
// unmodified. The session refreshes the block before every run.
constexpr uint32_t kSlotDyn = 0xFFFFFFF4u;
constexpr int kDynPerNode = 4;

struct Reloc {
    uint32_t field_off;  // byte offset of a pointer field inside the parameter struct
    Buf buf;
};

// A 2-D tiled tensor map over f16 elements that has to be encoded into the parameter bytes once the
// address of its tensor is known (TMA loads: `cp.async.bulk.tensor`).
struct TmapReloc {
    uint32_t field_off;      // byte offset of the 128-byte map inside the parameter struct (64-byte aligned there)
    Buf buf;                 // base of the tensor
    uint64_t dim0, dim1;     // extents in elements: contiguous axis, outer axis
    uint64_t stride1_bytes;  // bytes between outer rows (a multiple of 16)
    uint32_t box0, box1;     // tile extents in elements (box0·2 ≤ 128 bytes with the 128-byte swizzle)
    // Byte offset of an int32 field of the parameter struct that the kernel reads as "use the map"; it is
    // cleared when the tensor's address in a run turns out not to be 16-byte aligned (the kernel then takes
    // its plain-load path). 0xFFFFFFFF: no such field, a misaligned tensor is an error.
    uint32_t enable_off = 0xFFFFFFFFu;
};

struct PersistOp;  // persist.hpp

struct LaunchRec {
    const void* func = nullptr;
    dim3 grid{1, 1, 1}, block{1, 1, 1};
    dim3 cluster{0, 0, 0};  // thread-block cluster shape; x = 0 launches without clusters
    unsigned smem = 0;
    std::vector<uint8_t> params;
    std::vector<Reloc> relocs;
    std::vector<TmapReloc> tmaps;
    const char* label = "";
    int node = -1;  // IR node index, for error messages and profiling
    // The kernel executes `griddepcontrol.wait` before it reads anything an
    // earlier launch wrote and before it writes anything at all, on every path
    // to its exit. Such a kernel may be launched while its predecessor in the
    // stream is still running (programmatic dependent launch): its prologue —
    // barrier set-up, prefetch of constant weights — overlaps the predecessor.
    // Every such kernel triggers its own dependents at entry, so the section
    // before its wait may overlap not only the launch before it but several
    // earlier ones: it may read only memory that NO launch of the same run
    // writes (constants, rows of a KV cache below the step's first new row).
    bool pdl = false;
    // Not a kernel of this library: a collective the session enqueues itself. The parameter bytes
    // are a CollP (with the usual pointer relocations); `func` is null.
    int coll = 0;  // 1 = sum over the tensor-parallel ranks
    // The grid's CTAs wait on one another: the launch must be cooperative (all CTAs co-resident).
    bool cooperative = false;
    // What this launch does, in the form the persistent step kernel executes: a run of consecutive
    // launches that all carry one can be replaced by a single launch of that kernel.
    std::shared_ptr<const PersistOp> pop;
};

struct CollP {
    const void* send;
    void* recv;
    unsigned long long count;
    int dtype;
};

class Emitter {
public:
    std::vector<LaunchRec> recs;
    int node = -1;
    size_t scratch_bytes = 0;  // high-water mark of scratch requested by this plan

    // Reserve `bytes` of scratch that lives for the duration of one node.
    Buf scratch(size_t bytes, size_t align = 256) {
        size_t off = (scratch_cursor_ + align - 1) / align * align;
        scratch_cursor_ = off + bytes;
        if (scratch_cursor_ > scratch_bytes) scratch_bytes = scratch_cursor_;
        return Buf{kSlotScratch, (int64_t)off};
    }
    void begin_node(int n) {
        node = n;
        scratch_cursor_ = 0;
        dyn_vals.clear();
    }
    // Register a per-run scalar of the current node; kernels read it through
    // the returned address instead of from their parameter bytes.
    std::vector<int64_t> dyn_vals;
    Buf dyn(int64_t value) {
        if ((int)dyn_vals.size() >= kDynPerNode) throw std::runtime_error("too many per-run scalars for one node");
        dyn_vals.push_back(value);
        return Buf{kSlotDyn, (int64_t)((node * kDynPerNode + (int)dyn_vals.size() - 1) * 8)};
    }

    template <class P>
    LaunchRec& launch(void (*kernel)(const P), dim3 grid, dim3 block, unsigned smem, const P& p,
                std::initializer_list<std::pair<const void*, Buf>> ptrs, const char* label, bool pdl = false) {
        static_assert(sizeof(P) <= 4000, "kernel parameter struct too large");
        LaunchRec r;
        r.func = (const void*)kernel;
        r.grid = grid;
        r.block = block;
        r.smem = smem;
        r.params.resize(sizeof(P));
        std::memcpy(r.params.data(), &p, sizeof(P));
        for (auto& pr : ptrs) {
            Reloc rl;
            rl.field_off = (uint32_t)((const char*)pr.first - (const char*)&p);
            rl.buf = pr.second;
            r.relocs.push_back(rl);
        }
        r.label = label;
        r.node = node;
        r.pdl = pdl;
        recs.push_back(std::move(r));
        return recs.back();
    }

private:
    size_t scratch_cursor_ = 0;
};

// A tensor operand at lowering time: symbolic address, dtype code, concrete dims.
struct TRef {
    Buf buf;
    int dtype = 0;
    std::vector<int64_t> shape;
    // Physical row capacity of axis 2 for KV-cache tensors ([B, KV, T, D] whose
    // buffer holds `cap` rows per head); 0 = densely packed.
    int64_t cap = 0;
    int64_t numel() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
};

// Streaming multiprocessors of the current device (cached per device; thread-safe).
int sm_count();
// Raises a kernel's dynamic shared-memory limit on the current device once (thread-safe); throws on failure.
void ensure_max_dynamic_smem(const void* func, int bytes);

inline unsigned grid_for(int64_t n, int block, int64_t max_blocks = 0) {
    if (max_blocks <= 0) max_blocks = (int64_t)sm_count() * 16;
    int64_t g = (n + block - 1) / block;
    if (g < 1) g = 1;
    if (g > max_blocks) g = max_blocks;
    return (unsigned)g;
}

// ── primitives (one kernel family per IR primitive) ─────────────────────
void emit_unary(Emitter&, int op, const TRef& x, const TRef& y);
void emit_binary(Emitter&, int op, const TRef& a, const TRef& b, const TRef& y);
void emit_compare(Emitter&, int op, const TRef& a, const TRef& b, const TRef& y);
void emit_select(Emitter&, const TRef& c, const TRef& a, const TRef& b, const TRef& y);
void emit_cast(Emitter&, const TRef& x, const TRef& y);
void emit_matmul(Emitter&, const TRef& a, const TRef& b, const TRef& y, bool trans_a, bool trans_b);
void emit_reduce(Emitter&, int op, const TRef& x, const TRef& y, const std::vector<size_t>& axes);
void emit_reshape_copy(Emitter&, const TRef& x, const TRef& y);
void emit_transpose(Emitter&, const TRef& x, const TRef& y, const std::vector<size_t>& perm);
void emit_broadcast(Emitter&, const TRef& x, const TRef& y);
void emit_concat(Emitter&, const std::vector<TRef>& xs, const TRef& y, size_t axis);
void emit_slice(Emitter&, const TRef& x, const TRef& y, const std::vector<int64_t>& starts,
                const std::vector<int64_t>& steps);
void emit_gather(Emitter&, const TRef& data, const TRef& idx, const TRef& y, size_t axis);
void emit_scatter(Emitter&, const TRef& data, const TRef& idx, const TRef& upd, const TRef& y);
void emit_iota(Emitter&, const TRef& y);
void emit_dim_values(Emitter&, const std::vector<int64_t>& vals, const TRef& y);
void emit_dequantize(Emitter&, const TRef& q, const TRef& scales, const TRef* zp, const TRef& y, int64_t block_size);

// ── fused composites ────────────────────────────────────────────────────
void emit_softmax(Emitter&, const TRef& x, const TRef& y);  // last axis
// y = x · rsqrt(mean(x²) + eps) · w over the last axis; with `res` the input is
// x + res and the sum is also written to `sum_out`.
void emit_rmsnorm(Emitter&, const TRef& x, const TRef& w, const TRef& y, double eps, const TRef* res,
                  const TRef* sum_out);
void emit_gelu(Emitter&, const TRef& x, const TRef& y, bool tanh_approx, const TRef* mul);  // optional ·mul (GeGLU)
void emit_rotary(Emitter&, const TRef& x, const TRef& pos, const TRef& cos, const TRef& sin, const TRef& y,
                 int64_t heads, int64_t half);

struct GqaDesc {
    int64_t batch, seq, heads, kv_heads, head_dim, past;  // past = P (logical rows of the past tensors)
    double scale;
    int64_t window;        // -1 = none
    int64_t rot_half;      // 0 = no rotary
    int64_t cache_rows;    // rows of cos/sin
    bool has_bias;
    int64_t bias_b, bias_h;  // bias batch/head extents (1 = broadcast)
    bool in_place;         // present aliases past: only new rows are written
    // > 0: size the key split for this many rows (a bucket ≥ past + seq) and let
    // the kernels read the true length from the plan's per-run scalars, so a
    // decode step changes no launch parameter until the bucket is outgrown.
    int64_t t_bucket;
};
void emit_gqa(Emitter&, const GqaDesc&, const TRef& q, const TRef& k, const TRef& v, const TRef& past_k,
              const TRef& past_v, const TRef& seqlens, const TRef* cos, const TRef* sin, const TRef* bias,
              const TRef& out, const TRef& present_k, const TRef& present_v);

// The decode step (S = 1) over an in-place cache as one launch of thread-block
// clusters; false when the shape is outside what that kernel handles. `t_size`
// bounds the present length the launch is sized for; the true length is read
// from `dyn_t` at run time.
// One token per row of `logits` by temperature / top-k / top-p sampling (crates/onyxia-cli/src/sampling.rs:36-195);
// `u` holds one uniform number in [0, 1] per row.
void emit_sample_rows(Emitter&, const TRef& logits, const TRef& out, Buf u, float temperature, long long top_k, float top_p);
// Attention over many new positions on the tensor cores (f16, no bias; after gqa_prepare). False = shape not taken.
bool emit_gqa_prefill_tc(Emitter&, const GqaDesc&, Buf q_rot, const TRef& seqlens, const TRef& out, const TRef& present_k,
                         const TRef& present_v, Buf dyn_t, long long T, long long cap);
bool emit_gqa_decode(Emitter&, const GqaDesc&, const TRef& q, const TRef& k, const TRef& v, const TRef& seqlens,
                     const TRef* cos, const TRef* sin, const TRef& out, const TRef& present_k, const TRef& present_v,
                     Buf dyn_t, long long t_size);

struct NBitsDesc {
    int64_t m, k, n, block_size, n_blocks;
    int act_dtype, scale_dtype;
    bool has_zp;
    // The weight constant was re-laid out by emit_nbits_interleave (backend-
    // private layout for the tensor-core decode kernel).
    bool interleaved;
    // The weight constant was replaced by tile records holding nibbles, scales
    // and zero points together (emit_nbits_pack_tiles); `scales` and `zp` are
    // not read by the kernel.
    bool tiled;
};
// y[m, n] = a[m, :] · dequant(w)[n, :]ᵀ for packed u4 weights [N, n_blocks, bs].
void emit_matmul_nbits(Emitter&, const NBitsDesc&, const TRef& a, const TRef& w, const TRef& scales,
                       const TRef* zp, const TRef& y);

// Tensor-core decode kernel for f16 activations and scales over interleaved weights.
void emit_matmul_nbits_mma(Emitter&, const NBitsDesc&, const TRef& a, const TRef& w, const TRef& scales,
                           const TRef* zp, const TRef& y);
// One-time re-layout of a packed u4 weight constant: within each 32-bit word,
// nibble j moves to position (j >> 1) + 4·(j & 1).
void emit_nbits_interleave(Emitter&, Buf src, Buf dst, long long bytes);

// Streaming decode kernel over tile-major weight records (f16 activations and scales).
void emit_matmul_nbits_stream(Emitter&, const NBitsDesc&, const TRef& a, const TRef& tiles, const TRef& y);
// One-time gathering of a packed u4 weight [N, n_blocks, 32], its f16 scales
// and optional u4 zero points into tile records; `dst` needs nbits_tiled_bytes.
// Row tile rt of the matrix becomes row tile rt·rt_mul + rt_add of the
// destination stream, so several matrices can share one stream (one after the
// other, or interleaved row tile by row tile).
size_t nbits_tiled_bytes(long long n, long long n_blocks, bool has_zp);
void emit_nbits_pack_tiles(Emitter&, Buf w, Buf scales, Buf zp, Buf dst, long long n, long long n_blocks, bool has_zp,
                           long long rt_mul = 1, long long rt_add = 0);

// Several MatMulNBits over the same activations as one launch of the streaming
// kernel, optionally with a prologue on the activations and a GeGLU epilogue:
//   v = a;  [v = rmsnorm(v, eps1)·w1;]  [v = res + v, also stored to sum_out;]  [v = rmsnorm(v, eps2)·w2;]
//   plain:  y[i] = v · W_iᵀ for each segment i (the stream holds W_0's row tiles, then W_1's, …)
//   geglu:  y[0] = gelu(v · W_0ᵀ) · (v · W_1ᵀ), the stream alternating row tiles of W_0 and W_1
// Every step rounds where the primitives of the corresponding decompositions store a tensor.
struct NBitsGroup {
    long long m, k;
    bool has_zp;
    int n_seg;            // 1..3
    long long seg_n[3];
    TRef y[3];
    int geglu;            // 0 none, 1 tanh form, 2 erf form
    const TRef* w1;
    double eps1;
    const TRef* res;
    const TRef* sum_out;
    const TRef* w2;
    double eps2;
};
void emit_nbits_group(Emitter&, const NBitsGroup&, const TRef& a, const TRef& tiles);
// The tcgen05 GEMM form of a group's matrices (any number of activation rows, in passes of up to
// 256): no prologue, no epilogue. `interleave2`: the stream alternates row tiles of segments 0 and 1.
void emit_nbits_gemm_tc(Emitter&, const NBitsGroup&, const TRef& x, const TRef& tiles, bool interleave2);

// y = Σ over the tensor-parallel ranks of x (executed by the session through its communicator).
void emit_allreduce(Emitter&, const TRef& x, const TRef& y);

// argmax over the last axis, highest index among equal maxima → i64.
// `part` is scratch of argmax_scratch_bytes(rows) bytes, `counters` the zeroed arrival counters.
constexpr int kArgmaxMaxBlocks = 128;
inline size_t argmax_scratch_bytes(int64_t rows) { return (size_t)rows * kArgmaxMaxBlocks * 12 + 64; }
void emit_argmax_last(Emitter&, const TRef& x, const TRef& y, Buf part, Buf counters);

// The same argmax with its scratch in a fixed array of the module's global
// data: launches one kernel on `stream` and allocates nothing. At most
// kStaticArgmaxMaxRows rows per call; calls on one device share the array and
// must not overlap. Returns nullptr, or a message describing the failure.
constexpr int kStaticArgmaxMaxRows = 64;
const char* argmax_last_static(int device, cudaStream_t stream, const void* x, int dtype, long long rows,
                               long long cols, long long* y);

// Clear the error word (one tiny launch at the head of a plan is not needed:
// the session clears it with a memset when it reads it).
}  // namespace oxk
