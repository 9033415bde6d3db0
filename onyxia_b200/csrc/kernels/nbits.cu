// com.microsoft.MatMulNBits: y[m, n] = Σ_k a[m, k] · w[n, k] with
// w[n, k] = (q[n, k] − zp[n, k/bs]) · scale[n, k/bs] for 4-bit weights packed
// 32 to a 16-byte block (decomposition: crates/onyxia-ir/src/decomp.rs:615-663;
// lowering and wire layout: crates/onyxia-lower/src/rules.rs:890-940).
//
// Rounding follows the decomposition: each dequantised weight is rounded to
// the scales' dtype (exact here, see below), then to the activations' dtype if
// that differs, and the f32 dot product is rounded once to the activations'
// dtype on store. The interpreter accumulates in f64; f32 accumulation differs
// from it only by rounding.
//
// Generic path (`nbits_gemv_simt`, any float dtype mix; the f16 decode path is nbits_mma.cu): Each lane streams whole 16-byte
// blocks of nibbles with 128-bit loads (one scale per block), keeps the
// matching activation slice in registers, and rows are finished with warp
// shuffles. Algorithmic bytes per weight: 0.5 (nibbles) + 2/32 or 4/32
// (scale) = 0.5625 / 0.625 B.
#include "common.cuh"
#include "kernels.hpp"

namespace oxk {

struct NBitsGemvP {
    const void* a;        // [M, K] activations
    const uint4* w;       // [N, n_blocks] 16-byte blocks of 32 nibbles
    const void* scales;   // [N, n_blocks]
    const unsigned char* zp;  // [N, n_blocks] packed nibbles, or null
    void* y;              // [M, N]
    long long m0;         // first activation row handled by this launch
    long long m_total;
    long long k, n, n_blocks;
};

// (q − zp)·scale rounded to the scales' dtype, then widened to f32. For f16
// scales the product is formed by one f16 multiply (single rounding); for f32
// scales by one f32 multiply. Both equal the interpreter's f64 product rounded
// once, because an integer of ≤ 5 bits times one scale is exact in f64.
template <int SDT> struct ScaleOps;
template <> struct ScaleOps<DT_F16> {
    using S = __half;
    static __device__ __forceinline__ S load(const void* p, long long i) { return ((const __half*)p)[i]; }
    static __device__ __forceinline__ float deq(int qmz, S s) { return __half2float(__hmul(__int2half_rn(qmz), s)); }
};
template <> struct ScaleOps<DT_F32> {
    using S = float;
    static __device__ __forceinline__ S load(const void* p, long long i) { return ((const float*)p)[i]; }
    static __device__ __forceinline__ float deq(int qmz, S s) { return (float)qmz * s; }
};

// One warp per weight row; MT activation rows share every weight read.
template <int ADT, int SDT, int MT> __global__ void __launch_bounds__(256) nbits_gemv_simt(const NBitsGemvP p) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    using SO = ScaleOps<SDT>;
    for (long long row = warp; row < p.n; row += nwarps) {
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = 0.f;
        const uint4* wrow = p.w + row * p.n_blocks;
        for (long long blk = lane; blk < p.n_blocks; blk += 32) {
            uint4 packed = __ldg(wrow + blk);
            typename SO::S s = SO::load(p.scales, row * p.n_blocks + blk);
            int z = 8;
            if (p.zp) {
                long long zi = row * p.n_blocks + blk;
                z = (p.zp[zi >> 1] >> ((zi & 1) * 4)) & 0xF;
            }
            const unsigned words[4] = {packed.x, packed.y, packed.z, packed.w};
            const long long k0 = blk * 32;
#pragma unroll
            for (int wd = 0; wd < 4; wd++) {
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    long long kk = k0 + wd * 8 + e;
                    if (kk < p.k) {  // the last block may be padding beyond K
                        int q = (words[wd] >> (4 * e)) & 0xF;
                        float wv = SO::deq(q - z, s);
                        if constexpr (ADT == DT_F16 && SDT == DT_F32) wv = __half2float(__float2half_rn(wv));
#pragma unroll
                        for (int m = 0; m < MT; m++) {
                            if (p.m0 + m < p.m_total) acc[m] = fmaf(ld<ADT>(p.a, (p.m0 + m) * p.k + kk), wv, acc[m]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; m++) {
            float v = warp_sum(acc[m]);
            if (lane == 0 && p.m0 + m < p.m_total) st<ADT>(p.y, (p.m0 + m) * p.n + row, v);
        }
    }
}

template <int ADT, int SDT> static void launch_gemv(Emitter& em, NBitsGemvP p, const TRef& a, const TRef& w,
                                                    const TRef& scales, const TRef* zp, const TRef& y) {
    Buf zb = zp ? zp->buf : Buf{kSlotNull, 0};
    long long warps = p.n;
    dim3 g((unsigned)std::min<long long>((warps + 7) / 8, sm_count() * 8LL)), b(256);
    for (long long m0 = 0; m0 < p.m_total; m0 += 8) {
        p.m0 = m0;
        long long left = p.m_total - m0;
#define GO(MT) \
    em.launch(nbits_gemv_simt<ADT, SDT, MT>, g, b, 0, p, {{&p.a, a.buf}, {&p.w, w.buf}, {&p.scales, scales.buf}, {&p.zp, zb}, {&p.y, y.buf}}, "nbits_gemv_simt")
        if (left >= 8) GO(8);
        else if (left > 4) GO(8);
        else if (left > 2) GO(4);
        else if (left == 2) GO(2);
        else GO(1);
#undef GO
    }
}

void emit_matmul_nbits(Emitter& em, const NBitsDesc& d, const TRef& a, const TRef& w, const TRef& scales,
                       const TRef* zp, const TRef& y) {
    if (d.block_size != 32) throw std::runtime_error("nbits kernels need block_size 32");
    if (d.m == 0 || d.n == 0) return;
    if (d.tiled) {
        emit_matmul_nbits_stream(em, d, a, w, y);
        return;
    }
    if (d.interleaved) {
        emit_matmul_nbits_mma(em, d, a, w, scales, zp, y);
        return;
    }
    NBitsGemvP p{};
    p.m_total = d.m;
    p.k = d.k;
    p.n = d.n;
    p.n_blocks = d.n_blocks;
    if (d.act_dtype == DT_F16 && d.scale_dtype == DT_F16) launch_gemv<DT_F16, DT_F16>(em, p, a, w, scales, zp, y);
    else if (d.act_dtype == DT_F32 && d.scale_dtype == DT_F32) launch_gemv<DT_F32, DT_F32>(em, p, a, w, scales, zp, y);
    else if (d.act_dtype == DT_F16 && d.scale_dtype == DT_F32) launch_gemv<DT_F16, DT_F32>(em, p, a, w, scales, zp, y);
    else launch_gemv<DT_F32, DT_F16>(em, p, a, w, scales, zp, y);
}

}  // namespace oxk
