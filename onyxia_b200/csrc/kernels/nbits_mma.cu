// Decode-path MatMulNBits for f16 activations and f16 scales:
// y[m, n] = Σ_k a[m, k] · round_f16((q[n, k] − zp)·s[n, k/32]),  m ≤ 8 per pass.
//
// HBM-bound. Design:
//  * A warp owns a 16-row × 128-column tile of the weight matrix per step.
//    Lane (g = lane/4, t = lane%4) streams the 16-byte block (32 nibbles) of
//    rows g and g+8 at block column 4·tile + t with two 128-bit loads, plus the
//    two matching scales: every byte of the weight stream is read exactly once,
//    coalesced as 64-byte row segments.
//  * Nibbles are widened two at a time with the 0x6400 trick: (w & 0x000F000F) |
//    0x64006400 is the f16 pair {1024+q_lo, 1024+q_hi}; subtracting 1024+zp is
//    exact, and one f16 multiply by the block scale rounds exactly like the
//    interpreter's dequantisation. ≈1.6 ALU instructions per weight.
//  * The multiply-accumulate runs on the tensor cores as m16n8k16 MMAs with f32
//    accumulators: the 16×16 A fragment is the dequantised tile, the 16×8 B
//    fragment holds up to 8 activation rows, so batches of up to 8 tokens share
//    one pass over the weights and no cross-lane reduction is needed.
//  * The weight constant is re-laid out once at prepare time so that the two
//    nibbles a widening step extracts together are neighbours in k (see
//    `nbits_interleave`); activations are then read in their natural order.
//  * Small matrices are split along K across CTAs; partial tiles go to scratch
//    and the last CTA to arrive (a counter per row tile) adds them in split
//    order, so the result does not depend on scheduling.
//
// Algorithmic bytes: N·⌈K/32⌉·(16 + 2) + zero points + activations in/out.
#include <cstdlib>

#include "common.cuh"
#include "kernels.hpp"

namespace oxk {

// Within every 32-bit word, nibble j (k-offset j) moves to position
// (j >> 1) + 4·(j & 1): the pairs {p, p+4} a widening step extracts then hold
// k-neighbours {2p, 2p+1}.
struct InterleaveP {
    const unsigned* src;
    unsigned* dst;
    long long words;
};
__global__ void nbits_interleave(const InterleaveP p) {
    for (long long i = global_tid(); i < p.words; i += global_threads()) {
        unsigned w = p.src[i], o = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) o |= ((w >> (4 * j)) & 0xFu) << (4 * ((j >> 1) + 4 * (j & 1)));
        p.dst[i] = o;
    }
}

void emit_nbits_interleave(Emitter& em, Buf src, Buf dst, long long bytes) {
    InterleaveP p{};
    p.words = bytes / 4;
    em.launch(nbits_interleave, dim3(grid_for(p.words, 256)), dim3(256), 0, p, {{&p.src, src}, {&p.dst, dst}}, "nbits_interleave");
}

struct NBitsMmaP {
    const __half* a;
    const uint4* w;
    const __half* scales;
    const unsigned char* zp;
    __half* y;
    double* part;         // [ksplit][row_tiles][128] when ksplit > 1
    unsigned* counters;   // [row_tiles], zero between launches
    long long m0, m_total, k, n, n_blocks;
    int ksplit, tiles_per_split, k_tiles, row_tiles;
};

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned h2u(__half2 h) { return *reinterpret_cast<unsigned*>(&h); }
__device__ __forceinline__ __half2 u2h(unsigned u) { return *reinterpret_cast<__half2*>(&u); }

// One 32-bit word (8 interleaved nibbles) → four scaled f16 pairs {k0,k1} {k2,k3} {k4,k5} {k6,k7}.
__device__ __forceinline__ void widen8(unsigned w, __half2 sub_lo, __half2 add_hi, __half2 s2, unsigned (&out)[4]) {
    const __half2 sixteenth = __float2half2_rn(0.0625f);
    unsigned lo = (w & 0x000F000Fu) | 0x64006400u;
    unsigned hi = (w & 0x00F000F0u) | 0x64006400u;
    unsigned w8 = w >> 8;
    unsigned lo2 = (w8 & 0x000F000Fu) | 0x64006400u;
    unsigned hi2 = (w8 & 0x00F000F0u) | 0x64006400u;
    out[0] = h2u(__hmul2(__hsub2(u2h(lo), sub_lo), s2));
    out[1] = h2u(__hmul2(__hfma2(u2h(hi), sixteenth, add_hi), s2));
    out[2] = h2u(__hmul2(__hsub2(u2h(lo2), sub_lo), s2));
    out[3] = h2u(__hmul2(__hfma2(u2h(hi2), sixteenth, add_hi), s2));
}

__global__ void __launch_bounds__(128) nbits_gemv(const NBitsMmaP p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rt = blockIdx.x % p.row_tiles, split = blockIdx.x / p.row_tiles;
    const long long nb = p.n_blocks;
    const long long row_lo = (long long)rt * 16 + g, row_hi = row_lo + 8;
    const long long rl = row_lo < p.n ? row_lo : p.n - 1, rh = row_hi < p.n ? row_hi : p.n - 1;  // clamp loads
    const bool full_k = (p.k & 31) == 0;
    const long long mrow = p.m0 + g;
    const bool has_act = mrow < p.m_total;

    // Each 128-column tile is summed by the tensor cores in f32 from a zero
    // accumulator; tiles are then added in f64, so the only rounding that matters
    // is the final one to f16 (the interpreter accumulates in f64).
    double acc[4] = {0.0, 0.0, 0.0, 0.0};
    const int kt_begin = split * p.tiles_per_split;
    int kt_end = kt_begin + p.tiles_per_split;
    if (kt_end > p.k_tiles) kt_end = p.k_tiles;

    // One tile of weights (two 16-byte blocks, their scales and zero points) per
    // lane, fetched one iteration ahead so the loads of tile i+1 are in flight
    // while tile i is widened and multiplied.
    struct Tile {
        uint4 wl, wh;
        __half sl, sh;
        int zl, zh;
    };
    auto fetch = [&](int kt) {
        Tile tl;
        tl.wl = make_uint4(0, 0, 0, 0);
        tl.wh = tl.wl;
        tl.sl = __float2half(0.f);
        tl.sh = tl.sl;
        tl.zl = 8;
        tl.zh = 8;
        const long long kb = (long long)kt * 4 + t;
        if (kt < kt_end && kb < nb) {
            tl.wl = __ldg(p.w + rl * nb + kb);
            tl.wh = __ldg(p.w + rh * nb + kb);
            tl.sl = p.scales[rl * nb + kb];
            tl.sh = p.scales[rh * nb + kb];
            if (p.zp) {
                long long il = rl * nb + kb, ih = rh * nb + kb;
                tl.zl = (p.zp[il >> 1] >> ((il & 1) * 4)) & 0xF;
                tl.zh = (p.zp[ih >> 1] >> ((ih & 1) * 4)) & 0xF;
            }
        }
        return tl;
    };
    Tile next = fetch(kt_begin + warp);
    for (int kt = kt_begin + warp; kt < kt_end; kt += 4) {
        const long long kb = (long long)kt * 4 + t;
        const Tile cur = next;
        next = fetch(kt + 4);
        const uint4 wl = cur.wl, wh = cur.wh;
        const __half sl = cur.sl, sh = cur.sh;
        const int zl = cur.zl, zh = cur.zh;
        // activations of batch row g for block kb: 32 halves = four 16-byte words
        uint4 av[4];
#pragma unroll
        for (int m = 0; m < 4; m++) av[m] = make_uint4(0, 0, 0, 0);
        if (has_act && kb < nb) {
            const __half* ap = p.a + mrow * p.k + kb * 32;
            if (full_k && ((reinterpret_cast<uintptr_t>(ap) & 15) == 0)) {
#pragma unroll
                for (int m = 0; m < 4; m++) av[m] = *reinterpret_cast<const uint4*>(ap + 8 * m);
            } else {
                __half tmp[32];
#pragma unroll
                for (int e = 0; e < 32; e++) tmp[e] = (kb * 32 + e < p.k) ? ap[e] : __float2half(0.f);
#pragma unroll
                for (int m = 0; m < 4; m++) av[m] = *reinterpret_cast<uint4*>(&tmp[8 * m]);
            }
        }
        const __half2 s2l = __half2half2(sl), s2h = __half2half2(sh);
        const __half2 subl = __float2half2_rn(1024.f + (float)zl), subh = __float2half2_rn(1024.f + (float)zh);
        const __half2 addl = __float2half2_rn(-64.f - (float)zl), addh = __float2half2_rn(-64.f - (float)zh);
        const unsigned wls[4] = {wl.x, wl.y, wl.z, wl.w}, whs[4] = {wh.x, wh.y, wh.z, wh.w};
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int m = 0; m < 4; m++) {
            unsigned al[4], ah[4];
            widen8(wls[m], subl, addl, s2l, al);
            widen8(whs[m], subh, addh, s2h, ah);
            const unsigned bx = av[m].x, by = av[m].y, bz = av[m].z, bw = av[m].w;
            mma16816(c, al[0], ah[0], al[1], ah[1], bx, by);
            mma16816(c, al[2], ah[2], al[3], ah[3], bz, bw);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) acc[i] += (double)c[i];
    }

    // fold the four warps (fixed order), then finish or hand the partial tile on
    __shared__ double red[4][32][4];
#pragma unroll
    for (int i = 0; i < 4; i++) red[warp][lane][i] = acc[i];
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int i = 0; i < 4; i++) acc[i] = red[0][lane][i] + red[1][lane][i] + red[2][lane][i] + red[3][lane][i];

    if (p.ksplit > 1) {
        double2* mine = reinterpret_cast<double2*>(p.part + ((long long)split * p.row_tiles + rt) * 128) + 2 * lane;
        mine[0] = make_double2(acc[0], acc[1]);
        mine[1] = make_double2(acc[2], acc[3]);
        __threadfence();
        unsigned arrived = 0;
        if (lane == 0) arrived = atomicAdd(p.counters + rt, 1u);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived != (unsigned)p.ksplit - 1) return;
        __threadfence();
        acc[0] = acc[1] = acc[2] = acc[3] = 0.0;
        for (int s = 0; s < p.ksplit; s++) {
            const double2* src = reinterpret_cast<const double2*>(p.part + ((long long)s * p.row_tiles + rt) * 128) + 2 * lane;
            double2 v0 = __ldcg(src), v1 = __ldcg(src + 1);
            acc[0] += v0.x;
            acc[1] += v0.y;
            acc[2] += v1.x;
            acc[3] += v1.y;
        }
        if (lane == 0) p.counters[rt] = 0;  // ready for the next launch
    }
    // c0:(row g, col 2t) c1:(row g, col 2t+1) c2:(row g+8, col 2t) c3:(row g+8, col 2t+1); col = batch row
#pragma unroll
    for (int i = 0; i < 4; i++) {
        long long row = (i < 2) ? row_lo : row_hi;
        long long col = p.m0 + 2 * t + (i & 1);
        if (row < p.n && col < p.m_total) p.y[col * p.n + row] = __double2half(acc[i]);
    }
}

void emit_matmul_nbits_mma(Emitter& em, const NBitsDesc& d, const TRef& a, const TRef& w, const TRef& scales,
                           const TRef* zp, const TRef& y) {
    NBitsMmaP p{};
    p.m_total = d.m;
    p.k = d.k;
    p.n = d.n;
    p.n_blocks = d.n_blocks;
    p.row_tiles = (int)((d.n + 15) / 16);
    p.k_tiles = (int)((d.n_blocks + 3) / 4);
    // enough CTAs for ~4 per SM, at least one k-tile per warp
    static const int ctas_per_sm = [] {
        const char* e = std::getenv("ONYXIA_GEMV_CTAS_PER_SM");  // tuning knob
        int v = e ? std::atoi(e) : 4;
        return v < 1 ? 1 : v;
    }();
    long long want = ((long long)sm_count() * ctas_per_sm + p.row_tiles - 1) / p.row_tiles;
    long long max_split = (p.k_tiles + 3) / 4;
    p.ksplit = (int)std::max<long long>(1, std::min<long long>(want, max_split));
    p.tiles_per_split = (p.k_tiles + p.ksplit - 1) / p.ksplit;
    p.ksplit = (p.k_tiles + p.tiles_per_split - 1) / p.tiles_per_split;
    Buf part{kSlotNull, 0}, counters{kSlotNull, 0};
    if (p.ksplit > 1) {
        part = em.scratch((size_t)p.ksplit * p.row_tiles * 128 * sizeof(double));
        counters = Buf{kSlotCounters, 0};
        if ((size_t)p.row_tiles > kCounterWords) throw std::runtime_error("nbits split-K: too many row tiles");
    }
    Buf zb = zp ? zp->buf : Buf{kSlotNull, 0};
    dim3 g((unsigned)(p.row_tiles * p.ksplit)), b(128);
    for (long long m0 = 0; m0 < d.m; m0 += 8) {
        p.m0 = m0;
        em.launch(nbits_gemv, g, b, 0, p,
                  {{&p.a, a.buf}, {&p.w, w.buf}, {&p.scales, scales.buf}, {&p.zp, zb}, {&p.y, y.buf}, {&p.part, part},
                   {&p.counters, counters}},
                  "nbits_gemv");
    }
}

}  // namespace oxk
