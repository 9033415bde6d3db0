// Per-device facts and one-time kernel attributes, shared by the emit functions. Several sessions on
// different GPUs may lower plans from different host threads of one process: both caches are keyed
// by the current device and guarded by a mutex.
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>

#include "kernels.hpp"

namespace oxk {

int sm_count() {
    static std::mutex mu;
    static std::map<int, int> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(dev);
    if (it != cache.end()) return it->second;
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = 148;  // the part this library is written for
    }
    cache[dev] = n;
    return n;
}

void ensure_max_dynamic_smem(const void* func, int bytes) {
    static std::mutex mu;
    static std::map<std::pair<int, const void*>, int> done;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    int& have = done[{dev, func}];
    if (have >= bytes) return;
    cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    }
    have = bytes;
}

}  // namespace oxk
