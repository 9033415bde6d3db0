// Tensor-parallel plumbing: a communicator over NCCL, loaded at run time so that
// the library itself has no link-time dependency on it (single-GPU users, and
// machines without a GPU, never touch NCCL).
#include <dlfcn.h>

#include <mutex>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../kernels/common.cuh"
#include "../kernels/kernels.hpp"
#include "runtime.hpp"

namespace oxrt {

using namespace ox;

namespace {

// The handful of NCCL entry points in use, with the ABI of nccl.h 2.x.
struct NcclApi {
    using Comm = void*;
    struct UniqueId {
        char internal[128];
    };
    int (*GetUniqueId)(UniqueId*) = nullptr;
    int (*CommInitRank)(Comm*, int, UniqueId, int) = nullptr;
    int (*CommAbort)(Comm) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, Comm, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    void* lib = nullptr;
};

NcclApi& nccl(const char* path) {
    static NcclApi api;
    static std::mutex mu;  // two backends may join from different host threads
    std::lock_guard<std::mutex> lock(mu);
    if (api.lib) return api;
    // a process that already loaded NCCL (torch does) shares that copy
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!lib && path && *path) lib = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) {
        const char* why = dlerror();  // the call clears the message: read it once
        fail(ErrKind::Runtime, std::string("cannot load NCCL: ") + (why ? why : "libnccl.so.2 not found"));
    }
    auto sym = [&](const char* name) {
        void* p = dlsym(lib, name);
        if (!p) fail(ErrKind::Runtime, std::string("NCCL symbol missing: ") + name);
        return p;
    };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.lib = lib;
    return api;
}

void nccl_check(NcclApi& api, int rc, const char* what) {
    if (rc != 0) fail(ErrKind::Runtime, std::string("NCCL error in ") + what + ": " + (api.GetErrorString ? api.GetErrorString(rc) : "?"));
}

constexpr int kNcclFloat16 = 6, kNcclFloat32 = 7, kNcclSum = 0, kNcclInt8 = 0;

// ── all-reduce over peer memory ──────────────────────────────────────────
// Layout of a rank's region (the same on every rank):
//   [0, 8 KB)        arrival words: word (source rank · kArCtas + cta) holds the number of the latest
//                    all-reduce whose addend that CTA of that rank has published; written by the peers
//   [8 KB, 12 KB)    this rank's own counters: [0] number of all-reduces finished, [1] CTAs done
//   [12 KB, …)       kArSlots staging slots of kArSlotBytes; all-reduce q uses slot q mod kArSlots
// A thread owns one 16-byte vector of the message, so its loads from all peers are in flight together
// (a load over NVLink takes ≈ 2 µs; a thread that walked several vectors paid that once per vector).
// Why a slot is free when it is used again: CTA c of a rank leaves all-reduce q only after it has seen
// every peer's arrival word c reach q, and a peer publishes q only after its all-reduce q − 1 has
// finished as a whole (launches are ordered on its stream), i.e. after it stopped reading everybody's
// slot of q − 1. So when a rank starts q + 1 nobody reads its slots of q − 1 and older: two slots would
// do; four are kept.
constexpr int kArCtas = 256, kArThreads = 256, kArSlots = 4;
constexpr size_t kArSlotBytes = 1 << 20, kArCounterOff = 8192, kArSlotOff = 12288;
static_assert(kArSlotBytes / 16 <= (size_t)kArCtas * kArThreads, "one 16-byte vector per thread");
static_assert((size_t)Communicator::kMaxPeers * kArCtas * 4 <= kArCounterOff, "arrival words overlap the counters");
constexpr size_t kArRegionBytes = kArSlotOff + kArSlots * kArSlotBytes;
constexpr long long kArWaitCycles = 1000000000LL;  // ≈ 0.5 s

struct PeerArP {
    const uint4* in;
    uint4* out;
    char* region;                              // this rank's
    char* peer[Communicator::kMaxPeers];       // every rank's region as mapped here (own entry = region)
    oxk::ErrWord* err;
    unsigned long long n_vec;                  // 16-byte vectors in the message
    int rank, world, node;
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_peer(const uint4* p) {  // never from a stale L1 line: the slot is rewritten every few launches
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kArThreads) peer_allreduce_f16(const PeerArP p) {
    __shared__ int gave_up;
    unsigned* counters = reinterpret_cast<unsigned*>(p.region + kArCounterOff);
    const unsigned q = *reinterpret_cast<volatile unsigned*>(counters) + 1u;  // this all-reduce's number (1, 2, …)
    const unsigned slot = q % kArSlots;
    const unsigned long long i = (unsigned long long)blockIdx.x * kArThreads + threadIdx.x;
    const bool has = i < p.n_vec;
    uint4* mine = reinterpret_cast<uint4*>(p.region + kArSlotOff + (size_t)slot * kArSlotBytes);
    if (threadIdx.x == 0) gave_up = 0;
    // 1. publish this rank's addend
    uint4 own = make_uint4(0u, 0u, 0u, 0u);
    if (has) {
        own = p.in[i];
        mine[i] = own;
    }
    __syncthreads();  // the CTA's stores happen before the release below (cumulative at system scope)
    if (threadIdx.x < (unsigned)p.world && (int)threadIdx.x != p.rank)
        st_release_sys(reinterpret_cast<unsigned*>(p.peer[threadIdx.x]) + p.rank * kArCtas + blockIdx.x, q);
    // 2. wait (bounded) for the same chunk of every peer
    if (threadIdx.x < (unsigned)p.world && (int)threadIdx.x != p.rank) {
        const unsigned* w = reinterpret_cast<const unsigned*>(p.region) + threadIdx.x * kArCtas + blockIdx.x;
        const long long t0 = clock64();
        while ((int)(ld_acquire_sys(w) - q) < 0) {
            if (clock64() - t0 > kArWaitCycles) {
                gave_up = 1;
                oxk::report(p.err, oxk::ERR_WAIT_TIMEOUT, p.node, (long long)threadIdx.x, (long long)q);
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    // 3. add the addends in rank order (f32), one rounding
    if (!gave_up && has) {
        uint4 part[Communicator::kMaxPeers];
#pragma unroll
        for (int r = 0; r < Communicator::kMaxPeers; r++)
            if (r < p.world)
                part[r] = r == p.rank ? own : ld_peer(reinterpret_cast<const uint4*>(p.peer[r] + kArSlotOff + (size_t)slot * kArSlotBytes) + i);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < Communicator::kMaxPeers; r++)
            if (r < p.world) {
                const __half2* h = reinterpret_cast<const __half2*>(&part[r]);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = __half22float2(h[e]);
                    acc[2 * e] += f.x;
                    acc[2 * e + 1] += f.y;
                }
            }
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int e = 0; e < 4; e++) oh[e] = __floats2half2_rn(acc[2 * e], acc[2 * e + 1]);
        p.out[i] = o;
    }
    // 4. the last CTA to finish closes the all-reduce
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(counters + 1, 1u) == gridDim.x - 1) {
            counters[1] = 0u;
            __threadfence();
            *reinterpret_cast<volatile unsigned*>(counters) = q;
        }
    }
}

}  // namespace

void tp_unique_id(const char* nccl_path, uint8_t out[128]) {
    NcclApi& api = nccl(nccl_path);
    NcclApi::UniqueId id;
    nccl_check(api, api.GetUniqueId(&id), "ncclGetUniqueId");
    std::memcpy(out, id.internal, 128);
}

Communicator::Communicator(int device, int rank, int world, const uint8_t id_bytes[128], const char* nccl_path)
    : rank_(rank), world_(world) {
    if (world < 1 || rank < 0 || rank >= world) fail(ErrKind::Attribute, "tensor-parallel rank out of range");
    NcclApi& api = nccl(nccl_path);
    OX_CUDA(cudaSetDevice(device));
    NcclApi::UniqueId id;
    std::memcpy(id.internal, id_bytes, 128);
    nccl_check(api, api.CommInitRank(&comm_, world, id, rank), "ncclCommInitRank");
    const char* off = std::getenv("ONYXIA_DISABLE_PEER_ALLREDUCE");
    if (world > 1 && world <= kMaxPeers && !(off && std::atoi(off) != 0)) {
        try {
            setup_peer_path(device);
        } catch (const std::exception& e) {
            peer_ok_ = false;
            peer_note_ = e.what();
        }
    } else {
        peer_note_ = world > kMaxPeers ? "more ranks than the peer path maps" : "switched off";
    }
    if (const char* dbg = std::getenv("ONYXIA_TP_DEBUG"))
        if (std::atoi(dbg) != 0) std::fprintf(stderr, "rank %d: peer all-reduce %s%s%s\n", rank, peer_ok_ ? "ready" : "not used", peer_note_.empty() ? "" : ": ", peer_note_.c_str());
}

// Every rank allocates its region, exports it with CUDA IPC, learns the others' handles through an
// ncclAllGather (which is also the barrier that orders every rank's zero-fill before any peer's first
// flag) and maps them.
void Communicator::setup_peer_path(int device) {
    NcclApi& api = nccl(nullptr);
    OX_CUDA(cudaSetDevice(device));
    OX_CUDA(cudaMalloc((void**)&region_, kArRegionBytes));
    OX_CUDA(cudaMemset(region_, 0, kArRegionBytes));
    cudaIpcMemHandle_t mine;
    OX_CUDA(cudaIpcGetMemHandle(&mine, region_));
    char* d_handles = nullptr;
    OX_CUDA(cudaMalloc((void**)&d_handles, sizeof(cudaIpcMemHandle_t) * (size_t)(world_ + 1)));
    OX_CUDA(cudaMemcpy(d_handles + sizeof(cudaIpcMemHandle_t) * (size_t)world_, &mine, sizeof(mine), cudaMemcpyHostToDevice));
    cudaStream_t st;
    OX_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    nccl_check(api, api.AllGather(d_handles + sizeof(cudaIpcMemHandle_t) * (size_t)world_, d_handles, sizeof(cudaIpcMemHandle_t), kNcclInt8, comm_, st),
               "ncclAllGather");
    OX_CUDA(cudaStreamSynchronize(st));
    std::vector<cudaIpcMemHandle_t> all((size_t)world_);
    OX_CUDA(cudaMemcpy(all.data(), d_handles, sizeof(cudaIpcMemHandle_t) * (size_t)world_, cudaMemcpyDeviceToHost));
    OX_CUDA(cudaStreamDestroy(st));
    OX_CUDA(cudaFree(d_handles));
    for (int r = 0; r < world_; r++) {
        if (r == rank_) {
            peer_region_[r] = region_;
            continue;
        }
        void* ptr = nullptr;
        OX_CUDA(cudaIpcOpenMemHandle(&ptr, all[(size_t)r], cudaIpcMemLazyEnablePeerAccess));
        peer_region_[r] = static_cast<char*>(ptr);
    }
    peer_ok_ = true;
}

// A backend is usually dropped while the process exits, in no particular order across ranks and
// often during interpreter shutdown, when NCCL's own helper threads may already be gone: both
// ncclCommDestroy and ncclCommAbort were seen to block there. The communicator is therefore left
// to process teardown; a rank that wants to leave a group and go on working should end the process
// that owns the backend.
Communicator::~Communicator() { comm_ = nullptr; }

void Communicator::allreduce_sum(const void* send, void* recv, size_t count, DType dtype, cudaStream_t stream, void* err_word, int node) {
    const size_t bytes = count * 2;
    if (peer_ok_ && dtype == DType::F16 && err_word && bytes <= kArSlotBytes && bytes % 16 == 0 && ((uintptr_t)send % 16) == 0 &&
        ((uintptr_t)recv % 16) == 0) {
        PeerArP p{};
        p.in = static_cast<const uint4*>(send);
        p.out = static_cast<uint4*>(recv);
        p.region = region_;
        for (int r = 0; r < world_; r++) p.peer[r] = peer_region_[r];
        p.err = static_cast<oxk::ErrWord*>(err_word);
        p.n_vec = bytes / 16;
        p.rank = rank_;
        p.world = world_;
        p.node = node;
        // the same grid on every rank: CTA c of one rank pairs with CTA c of the others
        const unsigned ctas = (unsigned)((p.n_vec + kArThreads - 1) / kArThreads);  // ≤ kArCtas: one vector per thread
        peer_allreduce_f16<<<ctas, kArThreads, 0, stream>>>(p);
        OX_CUDA(cudaGetLastError());
        return;
    }
    int dt;
    switch (dtype) {
        case DType::F16: dt = kNcclFloat16; break;
        case DType::F32: dt = kNcclFloat32; break;
        default: fail(ErrKind::DType, "all-reduce of this dtype is not supported");
    }
    NcclApi& api = nccl(nullptr);
    nccl_check(api, api.AllReduce(send, recv, count, dt, kNcclSum, comm_, stream), "ncclAllReduce");
}

}  // namespace oxrt
