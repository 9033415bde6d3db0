// Tensor-parallel plumbing: a communicator over NCCL, loaded at run time so that
// the library itself has no link-time dependency on it (single-GPU users, and
// machines without a GPU, never touch NCCL).
#include <dlfcn.h>

#include <mutex>

#include <cstring>

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
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.lib = lib;
    return api;
}

void nccl_check(NcclApi& api, int rc, const char* what) {
    if (rc != 0) fail(ErrKind::Runtime, std::string("NCCL error in ") + what + ": " + (api.GetErrorString ? api.GetErrorString(rc) : "?"));
}

constexpr int kNcclFloat16 = 6, kNcclFloat32 = 7, kNcclSum = 0;

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
}

// A backend is usually dropped while the process exits, in no particular order across ranks and
// often during interpreter shutdown, when NCCL's own helper threads may already be gone: both
// ncclCommDestroy and ncclCommAbort were seen to block there. The communicator is therefore left
// to process teardown; a rank that wants to leave a group and go on working should end the process
// that owns the backend.
Communicator::~Communicator() { comm_ = nullptr; }

void Communicator::allreduce_sum(const void* send, void* recv, size_t count, DType dtype, cudaStream_t stream) {
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
