// Device helpers shared by the kernels that consume int4 tile records
// (1024 B of interleaved nibbles, 128 B of f16 scales, optionally 64 B of zero
// points per 16-row × 128-column tile): mbarrier / bulk-copy wrappers, the
// nibble → f16 widening step and the m16n8k16 MMA the tiles are fed to.
#pragma once
#include "common.cuh"

namespace oxk {
namespace tile {

constexpr int kTileW = 1024;  // nibble bytes per tile record
constexpr int kTileS = 128;   // scale bytes per tile record
constexpr int kTileZ = 64;    // zero-point bytes per tile record (when present)

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar, unsigned count) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the barrier did not complete within `cycles`.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, long long cycles) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (clock64() - t0 < cycles)
        if (mbar_try(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_load(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
    asm(  // a pure function of its operands: the compiler may schedule it among independent chains
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned hu(__half2 h) { return *reinterpret_cast<unsigned*>(&h); }
__device__ __forceinline__ __half2 uh(unsigned u) { return *reinterpret_cast<__half2*>(&u); }

// (a & b) | c in one instruction.
__device__ __forceinline__ unsigned and_or(unsigned a, unsigned b, unsigned c) {
    unsigned d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// One 32-bit word (8 interleaved nibbles) → four scaled f16 pairs {k0,k1} {k2,k3} {k4,k5} {k6,k7}.
// The low nibble of each half-word becomes the f16 1024 + q, the next one 1024 + 16·q;
// (q − zp)·s is rounded to f16 once, like the interpreter's Dequantize.
__device__ __forceinline__ void widen_word(unsigned w, __half2 sub_lo, __half2 add_hi, __half2 s2, unsigned (&out)[4]) {
    const __half2 sixteenth = __float2half2_rn(0.0625f);
    const unsigned magic = 0x64006400u, m_lo = 0x000F000Fu, m_hi = 0x00F000F0u;
    const unsigned lo = and_or(w, m_lo, magic), hi = and_or(w, m_hi, magic);
    const unsigned w8 = w >> 8;
    const unsigned lo2 = and_or(w8, m_lo, magic), hi2 = and_or(w8, m_hi, magic);
    out[0] = hu(__hmul2(__hsub2(uh(lo), sub_lo), s2));
    out[1] = hu(__hmul2(__hfma2(uh(hi), sixteenth, add_hi), s2));
    out[2] = hu(__hmul2(__hsub2(uh(lo2), sub_lo), s2));
    out[3] = hu(__hmul2(__hfma2(uh(hi2), sixteenth, add_hi), s2));
}

__device__ __forceinline__ float r16(float v) { return __half2float(__float2half_rn(v)); }
__device__ __forceinline__ float r16d(double v) { return __half2float(__double2half(v)); }

// Gelu constants rounded to f16, as the decomposition's scalar constants are.
struct GeluConsts {
    float c_half, c_one, c_coef, c_k, c_inv_sqrt2;
};

// gelu(gate)·up with the rounding points of the Gelu decomposition followed by Mul
// (crates/onyxia-ir/src/decomp.rs:185-213); the caller rounds the product when it stores it.
// form 1: tanh approximation; form 2: erf by Abramowitz–Stegun 7.1.26 (interp.rs:860-872).
__device__ __forceinline__ float geglu_value(const GeluConsts& p, int form, float x, float up) {
    float inner;
    if (form == 1) {
        const float x2 = r16(x * x), x3 = r16(x2 * x), cx3 = r16(p.c_coef * x3), s = r16(x + cx3), sc = r16(p.c_k * s);
        inner = r16d(tanh((double)sc));
    } else {
        double z = (double)r16(x * p.c_inv_sqrt2);
        const double sign = z < 0.0 ? -1.0 : 1.0;
        z = fabs(z);
        const double tt = 1.0 / (1.0 + 0.3275911 * z);
        const double e = 1.0 - (((((1.061405429 * tt - 1.453152027) * tt) + 1.421413741) * tt - 0.284496736) * tt + 0.254829592) * tt * exp(-z * z);
        inner = r16d(sign * e);
    }
    const float one_plus = r16(p.c_one + inner), hx = r16(p.c_half * x);
    return r16(hx * one_plus) * up;
}

// One tile record against one activation row: lane (g, t) widens the 32 nibbles of rows g and g + 8 at
// block t and feeds eight MMAs on two accumulator chains. `ap` points at the lane's 16-byte activation
// chunk of this k tile (chunks of the four 8-element sub-blocks m follow at `step` uint4s).
__device__ __forceinline__ void tile_mma_zp8(const unsigned char* rec, const uint4* ap, int step, int lane, float (&ca)[4], float (&cb)[4]) {
    const uint4* wq = reinterpret_cast<const uint4*>(rec);
    const uint4 wl = wq[lane], wh = wq[32 + lane];
    const __half2 s2 = reinterpret_cast<const __half2*>(rec + kTileW)[lane];  // {row g, row g+8}
    const __half2 s2l = __low2half2(s2), s2h = __high2half2(s2);
    const __half2 sub_c = __float2half2_rn(1032.f), add_c = __float2half2_rn(-72.f);  // zero point 8
    const uint4 av0 = ap[0], av1 = ap[step], av2 = ap[2 * step], av3 = ap[3 * step];
    unsigned al[4], ah[4];
    widen_word(wl.x, sub_c, add_c, s2l, al);
    widen_word(wh.x, sub_c, add_c, s2h, ah);
    mma16816(ca, al[0], ah[0], al[1], ah[1], av0.x, av0.y);
    mma16816(cb, al[2], ah[2], al[3], ah[3], av0.z, av0.w);
    widen_word(wl.y, sub_c, add_c, s2l, al);
    widen_word(wh.y, sub_c, add_c, s2h, ah);
    mma16816(ca, al[0], ah[0], al[1], ah[1], av1.x, av1.y);
    mma16816(cb, al[2], ah[2], al[3], ah[3], av1.z, av1.w);
    widen_word(wl.z, sub_c, add_c, s2l, al);
    widen_word(wh.z, sub_c, add_c, s2h, ah);
    mma16816(ca, al[0], ah[0], al[1], ah[1], av2.x, av2.y);
    mma16816(cb, al[2], ah[2], al[3], ah[3], av2.z, av2.w);
    widen_word(wl.w, sub_c, add_c, s2l, al);
    widen_word(wh.w, sub_c, add_c, s2h, ah);
    mma16816(ca, al[0], ah[0], al[1], ah[1], av3.x, av3.y);
    mma16816(cb, al[2], ah[2], al[3], ah[3], av3.z, av3.w);
}

// Two tile records at once, their four accumulator chains interleaved.
__device__ __forceinline__ void tile_mma2_zp8(const unsigned char* rec1, const uint4* ap1, const unsigned char* rec2, const uint4* ap2,
                                              int step, int lane, float (&ca)[4], float (&cb)[4], float (&cc)[4], float (&cd)[4]) {
    const uint4* wq1 = reinterpret_cast<const uint4*>(rec1);
    const uint4* wq2 = reinterpret_cast<const uint4*>(rec2);
    const uint4 wl1 = wq1[lane], wh1 = wq1[32 + lane], wl2 = wq2[lane], wh2 = wq2[32 + lane];
    const __half2 s1 = reinterpret_cast<const __half2*>(rec1 + kTileW)[lane], s2 = reinterpret_cast<const __half2*>(rec2 + kTileW)[lane];
    const __half2 s1l = __low2half2(s1), s1h = __high2half2(s1), s2l = __low2half2(s2), s2h = __high2half2(s2);
    const __half2 sub_c = __float2half2_rn(1032.f), add_c = __float2half2_rn(-72.f);  // zero point 8
    const unsigned w1l[4] = {wl1.x, wl1.y, wl1.z, wl1.w}, w1h[4] = {wh1.x, wh1.y, wh1.z, wh1.w};
    const unsigned w2l[4] = {wl2.x, wl2.y, wl2.z, wl2.w}, w2h[4] = {wh2.x, wh2.y, wh2.z, wh2.w};
#pragma unroll
    for (int m = 0; m < 4; m++) {
        const uint4 a1 = ap1[m * step], a2 = ap2[m * step];
        unsigned l1[4], h1[4], l2[4], h2[4];
        widen_word(w1l[m], sub_c, add_c, s1l, l1);
        widen_word(w1h[m], sub_c, add_c, s1h, h1);
        widen_word(w2l[m], sub_c, add_c, s2l, l2);
        widen_word(w2h[m], sub_c, add_c, s2h, h2);
        mma16816(ca, l1[0], h1[0], l1[1], h1[1], a1.x, a1.y);
        mma16816(cc, l2[0], h2[0], l2[1], h2[1], a2.x, a2.y);
        mma16816(cb, l1[2], h1[2], l1[3], h1[3], a1.z, a1.w);
        mma16816(cd, l2[2], h2[2], l2[3], h2[3], a2.z, a2.w);
    }
}

}  // namespace tile
}  // namespace oxk
