// Host runtime of the CUDA backend: device tensors, the buffer pool, the
// fused-kernel registry, the session (prepare / upload / run / download).
//
// Behavioural model: the reference GPU backend's session
// (crates/onyxia-backend-wgpu/src/session.rs:137-242 prepare, :532-611 run,
// gpu.rs:400-448 pool), rewritten around CUDA streams and graphs.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../ir/ir.hpp"
#include "../kernels/kernels.hpp"

namespace oxrt {

using ox::DType;
using ox::Module;
using ox::Node;
using ox::ValueId;

[[noreturn]] void cuda_fail(cudaError_t e, const char* what);
#define OX_CUDA(expr)                                   \
    do {                                                \
        cudaError_t _e = (expr);                        \
        if (_e != cudaSuccess) ::oxrt::cuda_fail(_e, #expr); \
    } while (0)

class Pool;

// A device allocation, returned to its pool when the last reference goes.
struct DeviceBuffer {
    void* ptr = nullptr;
    size_t bytes = 0;
    // Shared ownership: a tensor handle may outlive the session that made it.
    std::shared_ptr<Pool> pool;
    // For KV-cache buffers: rows written so far per head (−1 = not a cache).
    // Only the view that ends at this row may be appended to in place.
    int64_t kv_rows = -1;
    ~DeviceBuffer();
};
using BufferRef = std::shared_ptr<DeviceBuffer>;

// Size-bucketed caching allocator with live/peak accounting
// (≙ BufferPool + MemCounter, gpu.rs:266-448). Buffers are recycled only once
// nothing references them; all work of a session is ordered on one stream, so
// a recycled buffer is never written before its previous readers ran.
class Pool : public std::enable_shared_from_this<Pool> {
public:
    explicit Pool(int device) : device_(device) {}
    ~Pool();
    BufferRef alloc(size_t bytes);
    void release(void* ptr, size_t bytes);
    void trim();
    uint64_t live_bytes() const { return live_; }
    uint64_t peak_bytes() const { return peak_; }
    uint64_t fresh_allocations = 0, reuses = 0;

private:
    int device_;
    std::multimap<size_t, void*> free_;
    std::unordered_map<void*, size_t> real_size_;
    uint64_t live_ = 0, peak_ = 0, cached_ = 0;
};

// A device-resident tensor handle (≙ GpuTensor, session.rs:23-30).
struct DTensor {
    DType dtype = DType::F32;
    std::vector<int64_t> shape;
    BufferRef buf;
    size_t offset = 0;
    // Rows per head the buffer has room for when this is a KV cache
    // [B, KV, T, D] with T ≤ cap; 0 = densely packed.
    int64_t cap = 0;
    int64_t numel() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
    size_t nbytes() const { return ox::dtype_storage_bytes(dtype, (uint64_t)numel()); }
    void* ptr() const { return buf ? (char*)buf->ptr + offset : nullptr; }
};

struct Options {
    bool without_fused = false;
    bool disable_graphs = false;
    bool disable_pattern_fusion = false;
    bool disable_pdl = false;  // launch every kernel fully serialised
    bool disable_persist = false;  // one launch per operation instead of the persistent step kernel
};

class Session;

// What a fused kernel sees when it is lowered for one concrete binding.
struct FusedCtx {
    oxk::Emitter& em;
    const Node& node;
    const std::vector<oxk::TRef>& ins;
    const std::vector<oxk::TRef>& outs;
    bool kv_in_place = false;
    // MatMulNBits: layout of the weight constant (input 1): 0 as uploaded,
    // 1 nibble-interleaved, 2 tile records with scales and zero points inside.
    int weights_layout = 0;
    // Set by a kernel that sized its launch for a bucket of a growing dimension
    // and reads the true value from the per-run scalars: the launch stays valid
    // while the value stays in (bucket − bucket_step, bucket].
    int64_t bucket = 0, bucket_step = 0;
};

// A hand-written kernel for one composite (≙ CompositeKernel, fused.rs:27-41).
struct FusedKernel {
    std::string name;
    // Whether this node's operand types are ones the kernel handles; other
    // instances of the composite fall back to the decomposition.
    bool (*accepts)(const Module&, const Node&);
    void (*lower)(FusedCtx&);
};

// ≙ KernelRegistry / standard_kernels (fused.rs:43-86).
class KernelRegistry {
public:
    void add(FusedKernel k) { map_[k.name] = std::move(k); }
    bool contains(const std::string& name) const { return map_.count(name) > 0; }
    const FusedKernel* get(const std::string& name) const {
        auto it = map_.find(name);
        return it == map_.end() ? nullptr : &it->second;
    }

private:
    std::unordered_map<std::string, FusedKernel> map_;
};
const KernelRegistry& standard_kernels();

struct Timing {
    std::string kernel, node;
    uint64_t time_ns;
};

// One rank's end of a tensor-parallel group (NCCL underneath, loaded on first use).
class Communicator {
public:
    Communicator(int device, int rank, int world, const uint8_t id_bytes[128], const char* nccl_path);
    ~Communicator();
    Communicator(const Communicator&) = delete;
    Communicator& operator=(const Communicator&) = delete;
    int rank() const { return rank_; }
    int world() const { return world_; }
    // Enqueues the sum over all ranks on `stream` (capturable into a CUDA graph). f16 messages that fit a
    // staging slot run as one kernel over peer memory (each rank copies its addend into a buffer its peers
    // have mapped, raises a flag in their memory, waits — bounded — for theirs, and adds all addends in rank
    // order in f32); everything else goes to ncclAllReduce. `err_word` / `node` tell the kernel where to
    // report a wait that ran out.
    void allreduce_sum(const void* send, void* recv, size_t count, DType dtype, cudaStream_t stream, void* err_word = nullptr,
                       int node = -1);
    bool peer_path_ready() const { return peer_ok_; }
    const std::string& peer_path_note() const { return peer_note_; }
    static constexpr int kMaxPeers = 8;

private:
    void setup_peer_path(int device);
    void* comm_ = nullptr;
    int rank_, world_;
    // peer path: one region per rank (flags, counters, staging slots), mapped into every other rank
    bool peer_ok_ = false;
    std::string peer_note_;
    char* region_ = nullptr;
    char* peer_region_[kMaxPeers] = {};
};
// The id rank 0 creates and hands to every rank of a new group (by whatever channel the host has).
void tp_unique_id(const char* nccl_path, uint8_t out[128]);

class Backend {
public:
    Backend(std::vector<int> devices, Options opt);
    bool supports(const std::string& name) const {
        if (name == "onyxia.AllReduce") return comm_ != nullptr;
        return !opt_.without_fused && standard_kernels().contains(name);
    }
    void join(std::shared_ptr<Communicator> c) { comm_ = std::move(c); }
    Communicator* communicator() const { return comm_.get(); }
    std::unique_ptr<Session> prepare(Module m);
    const Options& options() const { return opt_; }
    int device() const { return devices_[0]; }

private:
    std::vector<int> devices_;
    Options opt_;
    std::shared_ptr<Communicator> comm_;
};

}  // namespace oxrt
