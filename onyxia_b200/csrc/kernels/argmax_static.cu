// Greedy-sampling argmax that allocates nothing.
//
// The multi-block argmax needs a little scratch (one best value and index per
// CTA, one arrival counter per row). Here that scratch is a fixed array in the
// module's global data instead of pool memory, so a call consists of one kernel
// launch and no allocation of any kind — not from the device, not from the
// session's pool. The price is a fixed capacity (kStaticArgmaxMaxRows rows per
// call) and a single shared scratch per device: two calls whose kernels could
// overlap on one device (different streams, or different host threads) race on
// it and must be ordered by the caller.
//
// The first call on a device looks the array's address up with
// cudaGetSymbolAddress while that device is current. The lookup may initialise
// the module on the device, so make that first call outside any stream capture.
#include <mutex>

#include "common.cuh"
#include "kernels.hpp"

namespace oxk {

namespace {

constexpr int kBlocksMax = 128;  // CTAs per row
constexpr size_t kPartV = 0;                                                             // float [rows][128]
constexpr size_t kPartI = kPartV + (size_t)kStaticArgmaxMaxRows * kBlocksMax * 4;        // int64 [rows][128]
constexpr size_t kCount = kPartI + (size_t)kStaticArgmaxMaxRows * kBlocksMax * 8;        // u32   [rows]
constexpr size_t kScratchBytes = kCount + (size_t)kStaticArgmaxMaxRows * 4;

// Zero when the module is loaded. Only the counters have to be zero when a call
// starts; the kernel puts every counter it used back to zero before it ends.
// The partial results are written before they are read within one call.
static __device__ __align__(256) unsigned char g_argmax_scratch[kScratchBytes];

struct StaticArgmaxP {
    const void* x;
    long long* y;
    unsigned char* scratch;
    long long rows, cols;
    int blocks;
};

// Larger value wins; among equal values the higher index wins; an index < 0 is "nothing yet".
__device__ __forceinline__ bool beats(float v, long long i, float bv, long long bi) {
    return bi < 0 || (i >= 0 && (v > bv || (v == bv && i > bi)));
}

__device__ __forceinline__ void cta_best(float& v, long long& i, float* sv, long long* si) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        long long oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (beats(ov, oi, v, i)) v = ov, i = oi;
    }
    __syncthreads();
    if (lane == 0) sv[w] = v, si[w] = i;
    __syncthreads();
    v = lane < nw ? sv[lane] : -INFINITY;
    i = lane < nw ? si[lane] : -1;
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        long long oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (beats(ov, oi, v, i)) v = ov, i = oi;
    }
}

template <int DT> __global__ void __launch_bounds__(256) sample_argmax_static(const StaticArgmaxP p) {
    __shared__ float sv[8];
    __shared__ long long si[8];
    __shared__ unsigned order;
    float* part_v = reinterpret_cast<float*>(p.scratch + kPartV);
    long long* part_i = reinterpret_cast<long long*>(p.scratch + kPartI);
    unsigned* counters = reinterpret_cast<unsigned*>(p.scratch + kCount);

    const long long row = blockIdx.y, base = row * p.cols;
    const long long per = (p.cols + p.blocks - 1) / p.blocks;
    const long long c0 = blockIdx.x * per, c1 = c0 + per < p.cols ? c0 + per : p.cols;
    float v = -INFINITY;
    long long i = -1;
    for (long long c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        float e = ld<DT>(p.x, base + c);
        if (i < 0 || e >= v) v = e, i = c;  // ascending columns: >= keeps the last maximum
    }
    cta_best(v, i, sv, si);
    if (p.blocks > 1) {
        if (threadIdx.x == 0) {
            part_v[row * kBlocksMax + blockIdx.x] = v;
            part_i[row * kBlocksMax + blockIdx.x] = i;
            __threadfence();
            order = atomicAdd(counters + row, 1u);
            if (order == (unsigned)p.blocks - 1) counters[row] = 0;
        }
        __syncthreads();
        if (order != (unsigned)p.blocks - 1) return;  // the last CTA of the row merges
        __threadfence();
        v = -INFINITY;
        i = -1;
        for (int k = threadIdx.x; k < p.blocks; k += blockDim.x) {
            float ov = __ldcg(part_v + row * kBlocksMax + k);
            long long oi = __ldcg(part_i + row * kBlocksMax + k);
            if (beats(ov, oi, v, i)) v = ov, i = oi;
        }
        cta_best(v, i, sv, si);
    }
    if (threadIdx.x == 0) p.y[row] = i < 0 ? 0 : i;
}

// Address of g_argmax_scratch on each device, looked up on first use.
std::mutex g_setup_mutex;
unsigned char* g_scratch_ptr[64] = {};

}  // namespace

const char* argmax_last_static(int device, cudaStream_t stream, const void* x, int dtype, long long rows,
                               long long cols, long long* y) {
    if (device < 0 || device >= 64) return "argmax (static scratch): device ordinal out of range";
    if (dtype != DT_F32 && dtype != DT_F16) return "argmax (static scratch): logits must be f32 or f16";
    if (rows < 1 || cols < 1) return "argmax (static scratch): empty input";
    if (rows > kStaticArgmaxMaxRows)
        return "argmax (static scratch): more rows than the fixed scratch holds (limit 64 rows per call)";
    unsigned char* scratch;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!g_scratch_ptr[device]) {
            int current = -1;
            if (cudaGetDevice(&current) != cudaSuccess || current != device)
                return "argmax (static scratch): the session's device must be current for the first call";
            unsigned char* ptr = nullptr;
            cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_argmax_scratch);
            if (e != cudaSuccess || !ptr) return cudaGetErrorString(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
            g_scratch_ptr[device] = ptr;
        }
        scratch = g_scratch_ptr[device];
    }
    StaticArgmaxP p{};
    p.x = x;
    p.y = y;
    p.scratch = scratch;
    p.rows = rows;
    p.cols = cols;
    p.blocks = (int)std::max<long long>(1, std::min<long long>(kBlocksMax, cols / 2048));
    dim3 grid((unsigned)p.blocks, (unsigned)rows), block(256);
    if (dtype == DT_F32)
        sample_argmax_static<DT_F32><<<grid, block, 0, stream>>>(p);
    else
        sample_argmax_static<DT_F16><<<grid, block, 0, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace oxk
