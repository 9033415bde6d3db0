// Device-side conventions shared by every kernel.
//
// * Every kernel takes ONE parameter struct by value (`__global__ void k(const P p)`),
//   so a launch is fully described by {function, grid, block, smem, bytes of P}.
//   The runtime records those, patches the pointer fields when a buffer moves and
//   replays them from a CUDA graph.
// * Element types follow crates/onyxia-ir/src/types.rs:13-26; the *working*
//   type mirrors the interpreter's domains (interp.rs:193-199): floats compute in
//   f32 (f64 for transcendentals in the generic path), integers in wrapping
//   int64, bools as bool.
// * A kernel that meets a condition the interpreter reports as an error
//   (gather/scatter index out of range, integer division by zero, negative
//   integer power) records it in the session's error word and keeps going with
//   a harmless value; nothing traps.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.hpp"

namespace oxk {

constexpr int kMaxRank = 8;

// dtype codes = ox::DType / ox_dtype
enum : int { DT_F32 = 0, DT_F16, DT_I64, DT_I32, DT_U32, DT_U8, DT_I8, DT_BOOL, DT_U4, DT_I4 };

__device__ __forceinline__ void report(ErrWord* e, int code, int node, long long a, long long b) {
    if (e && atomicCAS(&e->code, 0, code) == 0) {
        e->node = node;
        e->a = a;
        e->b = b;
    }
}

// ── dtype traits ────────────────────────────────────────────────────────
template <int DT> struct Ty;
template <> struct Ty<DT_F32> { using S = float; using W = float; static constexpr bool is_float = true; };
template <> struct Ty<DT_F16> { using S = __half; using W = float; static constexpr bool is_float = true; };
template <> struct Ty<DT_I64> { using S = long long; using W = long long; static constexpr bool is_float = false; };
template <> struct Ty<DT_I32> { using S = int; using W = long long; static constexpr bool is_float = false; };
template <> struct Ty<DT_U32> { using S = unsigned; using W = long long; static constexpr bool is_float = false; };
template <> struct Ty<DT_U8> { using S = unsigned char; using W = long long; static constexpr bool is_float = false; };
template <> struct Ty<DT_I8> { using S = signed char; using W = long long; static constexpr bool is_float = false; };
template <> struct Ty<DT_BOOL> { using S = unsigned char; using W = bool; static constexpr bool is_float = false; };

template <int DT> __device__ __forceinline__ typename Ty<DT>::W ld(const void* p, long long i) {
    using S = typename Ty<DT>::S;
    if constexpr (DT == DT_F16) return __half2float(((const __half*)p)[i]);
    else if constexpr (DT == DT_BOOL) return ((const unsigned char*)p)[i] != 0;
    else return (typename Ty<DT>::W)((const S*)p)[i];
}

template <int DT> __device__ __forceinline__ void st(void* p, long long i, typename Ty<DT>::W v) {
    using S = typename Ty<DT>::S;
    if constexpr (DT == DT_F16) ((__half*)p)[i] = __float2half_rn(v);
    else if constexpr (DT == DT_BOOL) ((unsigned char*)p)[i] = v ? 1 : 0;
    else if constexpr (Ty<DT>::is_float) ((S*)p)[i] = v;
    else ((S*)p)[i] = (S)(unsigned long long)v;  // two's-complement truncation, like Rust `as`
}

// Packed nibble read (low nibble = earlier element, interp.rs:174-188).
__device__ __forceinline__ long long ld_u4(const void* p, long long i) {
    return (((const unsigned char*)p)[i >> 1] >> ((i & 1) * 4)) & 0xF;
}
__device__ __forceinline__ long long ld_i4(const void* p, long long i) {
    int nib = (((const unsigned char*)p)[i >> 1] >> ((i & 1) * 4)) & 0xF;
    return (long long)((nib ^ 8) - 8);
}

// ── N-d index helpers ───────────────────────────────────────────────────
// Output shape plus, per operand, strides expressed over output coordinates
// (0 on broadcast dims; may be negative for reversed slices).
struct NdShape {
    int rank;
    long long dim[kMaxRank];
};
struct NdStride {
    long long s[kMaxRank];
};

__device__ __forceinline__ long long nd_offset(long long linear, const NdShape& shp, const NdStride& st) {
    long long off = 0;
#pragma unroll
    for (int d = kMaxRank - 1; d >= 0; d--) {
        if (d < shp.rank) {
            long long c = linear % shp.dim[d];
            linear /= shp.dim[d];
            off += c * st.s[d];
        }
    }
    return off;
}

// Developer tracing, compiled in with -DOX_TRACE only: thread 0 of block 0 appends
// (id, global timer) to a log that follows the error word in device memory.
#ifdef OX_TRACE
__device__ __forceinline__ void ox_trace(ErrWord* e, int id) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        unsigned long long* t = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(e) + 256);
        const unsigned i = atomicAdd(reinterpret_cast<unsigned*>(t), 1u);
        if (i < 8000) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            t[1 + i] = ((unsigned long long)id << 56) | (now & 0x00FFFFFFFFFFFFFFull);
        }
    }
}
// the same for a thread other than thread 0 (the caller picks one thread of block 0)
__device__ __forceinline__ void ox_trace_here(ErrWord* e, int id) {
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        unsigned long long* t = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(e) + 256);
        const unsigned i = atomicAdd(reinterpret_cast<unsigned*>(t), 1u);
        if (i < 8000) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            t[1 + i] = ((unsigned long long)id << 56) | (now & 0x00FFFFFFFFFFFFFFull);
        }
    }
}
#else
#define ox_trace(e, id) ((void)0)
#define ox_trace_here(e, id) ((void)0)
#endif

// Programmatic dependent launch. `pdl_trigger` lets the next kernel in the
// stream start its prologue once every CTA of this grid has called it;
// `pdl_wait` returns when all earlier grids have completed and their writes are
// visible. Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
    pdl_trigger();
    pdl_wait();
}

__device__ __forceinline__ long long global_tid() {
    return (long long)blockIdx.x * blockDim.x + threadIdx.x;
}
__device__ __forceinline__ long long global_threads() { return (long long)gridDim.x * blockDim.x; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum / max over up to 1024 threads; `red` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
    if (w == 0) t = warp_sum(t);
    if (threadIdx.x == 0) red[0] = t;
    __syncthreads();
    return red[0];
}
__device__ __forceinline__ float block_max(float v, float* red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float t = (threadIdx.x < nw) ? red[threadIdx.x] : -INFINITY;
    if (w == 0) t = warp_max(t);
    if (threadIdx.x == 0) red[0] = t;
    __syncthreads();
    return red[0];
}

}  // namespace oxk
