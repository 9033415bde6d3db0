// MatMulNBits for more than 8 activation rows (prefill, batched decode): a
// tcgen05 GEMM with the accumulator in tensor memory.
//
//   Yᵀ[n, m] = Σ_k W[n, k] · X[m, k],   W = round_f16((q − zp)·s) from the tile records
//
// The weights are the MMA's A operand (128 rows of W per CTA = 8 row tiles), the
// activations its B operand (MB = 16 … 256 rows of X per pass), so the weight
// stream is read once per MB activation rows. Per step of 128 k:
//   * eight producer warps each widen one tile record (the streaming GEMV's
//     nibble arithmetic, exact (q − zp)·s rounding) into the A panel in shared
//     memory — K-major, 128-byte rows, 128-byte swizzle; one of their threads asks the
//     TMA unit for the matching activation columns (two tiled loads of 64 k × MB rows
//     through a tensor map with the same swizzle, zero-filled outside the matrix), which
//     land in the B panel and complete the stage's barrier by byte count;
//   * one thread of a ninth warp issues eight tcgen05.mma (M 128 × N MB × K 16,
//     f16 inputs, f32 accumulation in TMEM) and commits them to the mbarrier that
//     frees the stage.
// Stages form a ring (full / empty mbarriers). After the last step the first four
// warps read the accumulator with tcgen05.ld (a warp reads the 32 TMEM lanes of
// its quarter), round to f16 and store Y, consecutive threads on consecutive n.
//
// Every wait is bounded; on expiry the kernel records ERR_WAIT_TIMEOUT, lets the
// remaining phases run out and frees its tensor memory before it exits.
//
// Accuracy: the tensor core adds into its f32 accumulator without rounding to nearest, so a long chain of
// MMAs drifts. Consecutive steps therefore rotate over up to four accumulators side by side in tensor
// memory, which the epilogue adds: chains a quarter as long, at no cost in the main loop.
//
// Split K: a matrix with few row blocks (or a few more than a whole wave of CTAs) would leave SMs idle,
// so the k range of the row blocks beyond the last whole wave (all of them when there is less than one
// wave) can be cut into `splits` pieces, each CTA writing its f32 partial
// accumulator to scratch; a second kernel adds the pieces in fixed order and rounds once.
//
// FLOPs 2·M·N·K; bytes as for the GEMV (0.5625 per weight) once per MB rows.
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "kernels.hpp"

namespace oxk {

namespace {

constexpr int kProducerWarps = 8;         // warps that widen the weights (A panels), one per row tile
constexpr int kMmaWarp = kProducerWarps;  // the warp that issues the MMAs
constexpr int kThreadsTc = (kMmaWarp + 1) * 32;
constexpr int kTileWt = 1024, kTileSt = 128, kTileZt = 64;
constexpr int kPanelA = 128 * 128;  // bytes: 128 rows × 64 k of f16
constexpr long long kWaitCyclesTc = 2000000000LL;

struct TcP {
    alignas(64) unsigned char xmap[128];  // tensor map over the activations [M, K] (box 64 k × mb rows), when use_tma
    const __half* x;             // activations [M, K]
    const unsigned char* tiles;  // tile records, row tile by row tile
    __half* y[3];                // outputs per segment [M, seg_n]
    ErrWord* err;
    long long m0, m_total, k;
    long long seg_n[3];
    int seg_rt0[4];
    int n_seg, interleave2;      // interleave2: row tiles alternate between segment 0 and 1
    int k_tiles, row_tiles, mb, stages, tile_bytes, has_zp, node;
    int use_tma;                 // 0: K is not a multiple of 8 (or x is not 16-byte aligned) — plain loads
    int n_acc;                   // accumulators in tensor memory that the steps rotate over (1, 2 or 4)
    int n_full;                  // row blocks (CTAs) that take all of K; the blocks after them are cut along k
    int splits;                  // pieces of the k range of those tail blocks; > 1: partial sums go to `partial`
    float* partial;              // [splits][mb][n_pad] f32, rows counted from the first tail block
    long long n_pad;             // weight rows of the tail blocks (128 per block)
};

__device__ __forceinline__ unsigned s_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool bar_try_tc(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool bar_wait_tc(unsigned bar, unsigned parity) {
    if (bar_try_tc(bar, parity)) return true;
    const long long t0 = clock64();
    while (clock64() - t0 < kWaitCyclesTc)
        if (bar_try_tc(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ unsigned and_or_tc(unsigned a, unsigned b, unsigned c) {
    unsigned d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ unsigned h2u_tc(__half2 h) { return *reinterpret_cast<unsigned*>(&h); }
__device__ __forceinline__ __half2 u2h_tc(unsigned u) { return *reinterpret_cast<__half2*>(&u); }
// One 32-bit word (8 interleaved nibbles) → 8 consecutive k as four f16 pairs.
__device__ __forceinline__ uint4 widen_tc(unsigned w, __half2 sub_lo, __half2 add_hi, __half2 s2) {
    const __half2 sixteenth = __float2half2_rn(0.0625f);
    const unsigned magic = 0x64006400u, m_lo = 0x000F000Fu, m_hi = 0x00F000F0u;
    const unsigned lo = and_or_tc(w, m_lo, magic), hi = and_or_tc(w, m_hi, magic);
    const unsigned w8 = w >> 8;
    const unsigned lo2 = and_or_tc(w8, m_lo, magic), hi2 = and_or_tc(w8, m_hi, magic);
    uint4 o;
    o.x = h2u_tc(__hmul2(__hsub2(u2h_tc(lo), sub_lo), s2));
    o.y = h2u_tc(__hmul2(__hfma2(u2h_tc(hi), sixteenth, add_hi), s2));
    o.z = h2u_tc(__hmul2(__hsub2(u2h_tc(lo2), sub_lo), s2));
    o.w = h2u_tc(__hmul2(__hfma2(u2h_tc(hi2), sixteenth, add_hi), s2));
    return o;
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1 024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc(unsigned smem_byte_addr) {
    return (unsigned long long)((smem_byte_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__global__ void __launch_bounds__(kThreadsTc, 2) nbits_gemm_tc(const __grid_constant__ TcP p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the swizzle pattern repeats every 1 024 bytes: panels start on that boundary
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int mb = p.mb, S = p.stages;
    const int panel_b = mb * 128;                       // bytes of one 64-k activation panel
    const int stage_bytes = 2 * kPanelA + 2 * panel_b;  // A panels, then B panels
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + (size_t)S * stage_bytes);  // full[S], empty[S], done
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * S + 1);

    pdl_enter();

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            // a stage is full when every producer warp has arrived, and so has the thread that posted the
            // activation bytes, and those bytes have landed
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_addr(bars + s)), "r"(kProducerWarps + 1) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_addr(bars + S + s)) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_addr(bars + 2 * S)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    int tmem_cols = 32;
    while (tmem_cols < mb * p.n_acc) tmem_cols <<= 1;
    if (warp == kMmaWarp) {  // the MMA warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = *tmem_slot;

    // CTAs 0 … n_full − 1 own a whole row block; the ones after them share the tail blocks, `splits` CTAs each
    const int tail_j = (int)blockIdx.x - p.n_full;
    const int block = tail_j < 0 ? (int)blockIdx.x : p.n_full + tail_j / p.splits;
    const int splits = tail_j < 0 ? 1 : p.splits, split = tail_j < 0 ? 0 : tail_j % p.splits;
    const int rt0 = block * 8;  // first row tile of this CTA
    const int kt_lo = (int)((long long)p.k_tiles * split / splits);  // this CTA's piece of the k range, in 128-k steps
    const int steps = (int)((long long)p.k_tiles * (split + 1) / splits) - kt_lo;
    bool ok = true;

    if (warp < kProducerWarps) {
        // ── producers: warp w widens row tile rt0 + w ──
        const int g = lane >> 2, t = lane & 3;
        const int rt = rt0 + warp;
        const bool rt_live = rt < p.row_tiles;
        const unsigned char* rec = p.tiles + (size_t)(rt_live ? rt : 0) * p.k_tiles * p.tile_bytes;
        // this warp's record of a step: two 16-byte words of nibbles per lane, the two rows' scales (and zero points)
        struct Rec {
            uint4 wl, wh;
            __half2 s2;
            uchar2 z;
        };
        auto fetch = [&](int i) {
            Rec r;
            r.wl = make_uint4(0, 0, 0, 0);
            r.wh = r.wl;
            r.s2 = __float2half2_rn(0.f);
            r.z = make_uchar2(8, 8);
            if (rt_live && i < steps) {
                const unsigned char* q = rec + (size_t)(kt_lo + i) * p.tile_bytes;
                r.wl = __ldg(reinterpret_cast<const uint4*>(q) + lane);
                r.wh = __ldg(reinterpret_cast<const uint4*>(q) + 32 + lane);
                r.s2 = *reinterpret_cast<const __half2*>(q + kTileWt + lane * 4);
                if (p.has_zp) r.z = *reinterpret_cast<const uchar2*>(q + kTileWt + kTileSt + lane * 2);
            }
            return r;
        };
        Rec next = fetch(0);
        for (int i = 0; i < steps; i++) {
            const int s = i % S;
            if (i >= S && ok && !bar_wait_tc(s_addr(bars + S + s), ((i / S) - 1) & 1)) ok = false;
            unsigned char* stage = smem + (size_t)s * stage_bytes;
            ox_trace(p.err, 41);
            if (p.use_tma) {
                // B: activation rows m0 … m0 + mb, columns 128·i … + 128, as two 64-k panels
                if (tid == 0) {
                    const unsigned bar = s_addr(bars + s), dst = s_addr(stage + 2 * kPanelA);
                    const unsigned long long map = reinterpret_cast<unsigned long long>(&p.xmap);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2u * (unsigned)panel_b) : "memory");
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                        "l"(map), "r"((kt_lo + i) * 128), "r"((int)p.m0), "r"(bar)
                        : "memory");
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                            dst + (unsigned)panel_b),
                        "l"(map), "r"((kt_lo + i) * 128 + 64), "r"((int)p.m0), "r"(bar)
                        : "memory");
                }
            } else {
                // plain loads, element by element: thread c fills chunk `c & 15` of rows (c >> 4) + 16·j
                const int ch = tid & 15, r0 = tid >> 4;
                unsigned char* bpan = stage + 2 * kPanelA;
                const long long k0 = (long long)(kt_lo + i) * 128 + ch * 8;
                const unsigned dst0 = s_addr(bpan + (ch >> 3) * panel_b + r0 * 128 + (((ch & 7) ^ (r0 & 7)) << 4));
                for (int j = 0; j * 16 < mb; j++) {
                    const long long row = p.m0 + r0 + 16 * j;
                    __half tmp[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) tmp[e] = (row < p.m_total && k0 + e < p.k) ? p.x[row * p.k + k0 + e] : __float2half(0.f);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst0 + j * 2048), "r"(reinterpret_cast<unsigned*>(tmp)[0]),
                                 "r"(reinterpret_cast<unsigned*>(tmp)[1]), "r"(reinterpret_cast<unsigned*>(tmp)[2]),
                                 "r"(reinterpret_cast<unsigned*>(tmp)[3])
                                 : "memory");
                }
                if (tid == 0) bar_arrive(s_addr(bars + s));  // stands for the byte-count arrival; the warp's own arrival below orders the stores
            }
            // A: rows 16·warp + g and + 8, k = 32·t + 8·m … + 8 of this 128-k step; the next record is already on its way
            const Rec cur = next;
            next = fetch(i + 1);
            const __half2 s2l = __low2half2(cur.s2), s2h = __high2half2(cur.s2);
            const float zl = (float)cur.z.x, zh = (float)cur.z.y;
            const __half2 subl = __float2half2_rn(1024.f + zl), subh = __float2half2_rn(1024.f + zh);
            const __half2 addl = __float2half2_rn(-64.f - zl), addh = __float2half2_rn(-64.f - zh);
            const unsigned wls[4] = {cur.wl.x, cur.wl.y, cur.wl.z, cur.wl.w}, whs[4] = {cur.wh.x, cur.wh.y, cur.wh.z, cur.wh.w};
            const int row_l = warp * 16 + g, row_h = row_l + 8;
            unsigned char* panel = stage + (t >> 1) * kPanelA;  // blocks 0,1 → first 64 k; 2,3 → second
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const int chunk = (t & 1) * 4 + m;  // 16-byte chunk of the 128-byte row
                *reinterpret_cast<uint4*>(panel + row_l * 128 + ((chunk ^ (row_l & 7)) << 4)) = widen_tc(wls[m], subl, addl, s2l);
                *reinterpret_cast<uint4*>(panel + row_h * 128 + ((chunk ^ (row_h & 7)) << 4)) = widen_tc(whs[m], subh, addh, s2h);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // make the stores visible to the tensor core
            __syncwarp();
            if (lane == 0) bar_arrive(s_addr(bars + s));
            ox_trace(p.err, 43);
        }
    } else {
        // ── MMA issuer ──
        const unsigned idesc = (1u << 4) | ((unsigned)(mb >> 3) << 17) | (8u << 24);  // f16 × f16 → f32, K-major, N = mb, M = 128
        for (int i = 0; i < steps; i++) {
            const int s = i % S;
            if (ok && !bar_wait_tc(s_addr(bars + s), (i / S) & 1)) ok = false;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the asynchronous copies landed through the generic proxy
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                ox_trace_here(p.err, 44);
                const unsigned a0 = s_addr(smem + (size_t)s * stage_bytes), b0 = a0 + 2 * kPanelA;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const unsigned long long da = umma_desc(a0 + (j >> 2) * kPanelA + (j & 3) * 32);
                    const unsigned long long db = umma_desc(b0 + (j >> 2) * panel_b + (j & 3) * 32);
                    const unsigned accumulate = (i >= p.n_acc || j > 0) ? 1u : 0u;  // the first step of each accumulator overwrites it
                    asm volatile(
                        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n" ::"r"(tmem + (unsigned)((i % p.n_acc) * mb)),
                        "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
                        : "memory");
                }
                // the stage is free once these MMAs have read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_addr(bars + S + s)) : "memory");
                ox_trace_here(p.err, 45);
                if (i == steps - 1)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_addr(bars + 2 * S)) : "memory");
            }
            __syncwarp();
        }
    }

    // ── epilogue: warps 0-3 read their quarter of the 128 accumulator lanes ──
    if (warp < 4) {
        if (ok && steps > 0 && !bar_wait_tc(s_addr(bars + 2 * S), 0)) ok = false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int row_in_cta = warp * 32 + lane;           // weight row = accumulator lane
        const int rtg = rt0 + (row_in_cta >> 4);
        int seg = 0;
        long long row;
        if (p.interleave2) {
            seg = rtg & 1;
            row = (long long)(rtg >> 1) * 16 + (row_in_cta & 15);
        } else {
            if (p.n_seg > 1 && rtg >= p.seg_rt0[1]) seg = 1;
            if (p.n_seg > 2 && rtg >= p.seg_rt0[2]) seg = 2;
            row = (long long)(rtg - p.seg_rt0[seg]) * 16 + (row_in_cta & 15);
        }
        const bool row_ok = rtg < p.row_tiles && row < p.seg_n[seg];
        __half* yout = p.y[seg];
        const int acc_used = min(p.n_acc, steps);
        for (int c0 = 0; c0 < mb; c0 += 16) {
            float sum[16];  // adding two to four f32 partial sums rounds to nearest: three roundings at 2^-24
#pragma unroll
            for (int j = 0; j < 16; j++) sum[j] = 0.f;
            for (int a = 0; a < acc_used; a++) {
                unsigned v[16];
                const unsigned addr = tmem + ((unsigned)(warp * 32) << 16) + (unsigned)(a * mb + c0);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                      "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                    : "r"(addr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; j++) sum[j] += __uint_as_float(v[j]);
            }
            if (splits > 1) {
                float* part = p.partial + ((size_t)split * mb + c0) * p.n_pad + (size_t)(block - p.n_full) * 128 + row_in_cta;
#pragma unroll
                for (int j = 0; j < 16; j++)
                    if (ok && p.m0 + c0 + j < p.m_total) part[(size_t)j * p.n_pad] = sum[j];
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const long long mrow = p.m0 + c0 + j;
                    if (ok && row_ok && mrow < p.m_total) yout[mrow * p.seg_n[seg] + row] = __float2half_rn(sum[j]);
                }
            }
        }
    }
    if (!ok && lane == 0) report(p.err, ERR_WAIT_TIMEOUT, p.node, (long long)blockIdx.x, (long long)warp);

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
}

// Adds the pieces of a split-K pass in fixed order and stores the f16 outputs.
struct TcReduceP {
    const float* partial;
    __half* y[3];
    long long m0, m_total, n_pad;
    long long seg_n[3];
    int seg_rt0[4];
    int n_seg, interleave2, row_tiles, mb, splits;
    long long row0;  // first weight row (in stream order) of the tail blocks
};

// Adds the pieces of the row blocks that were cut along K, in piece order, in f64; one rounding. blockIdx.y is the
// activation row, a thread owns four consecutive weight rows (one 16-byte load per piece, the loads of four pieces in
// flight together).
__global__ void __launch_bounds__(256) nbits_gemm_reduce(const TcReduceP p) {
    pdl_enter();
    const int rows = (int)((long long)p.row_tiles * 16 - p.row0);  // a multiple of 16
    const int m = (int)blockIdx.y;
    const int rl = (int)(blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (rl >= rows) return;
    const float4* src = reinterpret_cast<const float4*>(p.partial + (size_t)m * p.n_pad + rl);
    const size_t piece = (size_t)p.mb * p.n_pad / 4;  // float4s between two pieces
    double acc[4] = {0.0, 0.0, 0.0, 0.0};
    int sp = 0;
    for (; sp + 4 <= p.splits; sp += 4) {
        const float4 a = src[(size_t)sp * piece], b = src[(size_t)(sp + 1) * piece], c = src[(size_t)(sp + 2) * piece], d = src[(size_t)(sp + 3) * piece];
        acc[0] = (((acc[0] + (double)a.x) + (double)b.x) + (double)c.x) + (double)d.x;
        acc[1] = (((acc[1] + (double)a.y) + (double)b.y) + (double)c.y) + (double)d.y;
        acc[2] = (((acc[2] + (double)a.z) + (double)b.z) + (double)c.z) + (double)d.z;
        acc[3] = (((acc[3] + (double)a.w) + (double)b.w) + (double)c.w) + (double)d.w;
    }
    for (; sp < p.splits; sp++) {
        const float4 a = src[(size_t)sp * piece];
        acc[0] += (double)a.x;
        acc[1] += (double)a.y;
        acc[2] += (double)a.z;
        acc[3] += (double)a.w;
    }
    const long long r = p.row0 + rl;
    const int rtg = (int)(r >> 4);
    int seg = 0;
    long long row;
    if (p.interleave2) {
        seg = rtg & 1;
        row = (long long)(rtg >> 1) * 16 + (r & 15);
    } else {
        if (p.n_seg > 1 && rtg >= p.seg_rt0[1]) seg = 1;
        if (p.n_seg > 2 && rtg >= p.seg_rt0[2]) seg = 2;
        row = (long long)(rtg - p.seg_rt0[seg]) * 16 + (r & 15);
    }
    __half* y = p.y[seg] + (size_t)(p.m0 + m) * p.seg_n[seg];
#pragma unroll
    for (int e = 0; e < 4; e++)
        if (row + e < p.seg_n[seg]) y[row + e] = __double2half(acc[e]);
}

}  // namespace

// The GEMM form of a MatMulNBits group (no prologue, no epilogue: the caller runs those as
// separate launches). `interleave2`: the stream alternates row tiles of segment 0 and 1.
void emit_nbits_gemm_tc(Emitter& em, const NBitsGroup& gr, const TRef& x, const TRef& tiles, bool interleave2) {
    if (gr.m == 0) return;
    TcP p{};
    p.m_total = gr.m;
    p.k = gr.k;
    p.k_tiles = (int)(((gr.k + 31) / 32 + 3) / 4);
    p.n_seg = gr.n_seg;
    p.interleave2 = interleave2 ? 1 : 0;
    int rt = 0;
    for (int i = 0; i < gr.n_seg; i++) {
        p.seg_n[i] = gr.seg_n[i];
        p.seg_rt0[i] = rt;
        rt += (int)((gr.seg_n[i] + 15) / 16);
    }
    p.seg_rt0[gr.n_seg] = rt;
    p.row_tiles = rt;
    p.has_zp = gr.has_zp ? 1 : 0;
    p.tile_bytes = kTileWt + kTileSt + (gr.has_zp ? kTileZt : 0);
    p.node = em.node;
    // activation rows per pass: the smallest MMA N that holds them all, at most 256
    int mb = 16;
    while (mb < gr.m && mb < 256) mb <<= 1;
    p.mb = mb;
    const size_t stage = 2 * (size_t)kPanelA + 2 * (size_t)mb * 128;
    // two CTAs per SM where two stages of each fit in half the shared memory, else one CTA with up to 4
    const size_t half_sm = 110 * 1024, whole_sm = 216 * 1024;
    p.stages = (int)std::min<size_t>(4, (2 * stage <= half_sm ? half_sm : whole_sm) / stage);
    if (p.stages < 2) p.stages = 2;
    p.n_acc = mb <= 128 ? 4 : 2;  // 512 columns of tensor memory per SM; two CTAs share it when mb ≤ 64
    p.use_tma = (gr.k % 8 == 0 && x.buf.off % 16 == 0) ? 1 : 0;
    const size_t smem = stage * p.stages + 1024 /*alignment slack*/ + (2 * p.stages + 1) * 8 + 16;
    ensure_max_dynamic_smem((const void*)nbits_gemm_tc, 220 * 1024);
    const Buf null{kSlotNull, 0};
    const unsigned grid = (unsigned)((p.row_tiles + 7) / 8);
    // Whole waves of row blocks take all of K. The blocks left over (all of them when there is less than one
    // wave) are cut into the number of pieces that minimises, in units of one 128-k step (≈ 1.3 µs),
    // waves × (steps per piece + about four steps of set-up and drain per CTA) + the second kernel's launch
    // and the partial sums' trip to memory and back; at least two steps per piece.
    const long long slots = (long long)sm_count() * (2 * stage <= half_sm ? 2 : 1);
    long long n_full = (long long)grid / slots * slots, tail = grid - n_full;
    if (tail * 10 >= slots * 6) {  // the last wave is well filled as it is
        n_full = grid;
        tail = 0;
    }
    int splits = 1;
    if (tail > 0) {
        double best = 1e300;
        for (int sp = 1; sp <= 8 && sp * 2 <= std::max(p.k_tiles, 2); sp++) {
            const long long waves = (tail * sp + slots - 1) / slots;
            double cost = (double)waves * ((double)p.k_tiles / sp + 4.0);
            if (sp > 1) cost += 2.5 + (double)sp * mb * (double)tail * 128 * 8.0 / 3.9e6;
            if (cost < best * 0.97) {  // a larger count has to earn its extra pass over the partial sums
                best = cost;
                splits = sp;
            }
        }
    }
    if (const char* e = std::getenv("ONYXIA_GEMM_SPLITS")) {  // diagnostics: every row block cut into that many pieces
        splits = std::max(1, std::min({std::atoi(e), 8, std::max(p.k_tiles, 1)}));
        n_full = 0;
        tail = grid;
    }
    if (splits == 1) {
        n_full = grid;
        tail = 0;
    }
    static const bool debug = std::getenv("ONYXIA_GEMM_DEBUG") != nullptr;  // diagnostics
    if (debug) std::fprintf(stderr, "nbits_gemm_tc: m %lld k_tiles %d grid %u mb %d: %d pieces over %lld of the row blocks\n", gr.m, p.k_tiles, grid, mb, splits, tail);
    p.n_full = (int)n_full;
    p.splits = splits;
    p.n_pad = tail * 128;
    const Buf partial = splits > 1 ? em.scratch((size_t)splits * mb * p.n_pad * sizeof(float)) : null;
    for (long long m0 = 0; m0 < gr.m; m0 += mb) {
        p.m0 = m0;
        LaunchRec& rec = em.launch(nbits_gemm_tc, dim3((unsigned)(n_full + tail * splits)), dim3(kThreadsTc), (unsigned)smem, p,
                  {{&p.x, x.buf}, {&p.tiles, tiles.buf}, {&p.err, Buf{kSlotErr, 0}}, {&p.partial, partial}, {&p.y[0], gr.y[0].buf},
                   {&p.y[1], gr.n_seg > 1 ? gr.y[1].buf : null}, {&p.y[2], gr.n_seg > 2 ? gr.y[2].buf : null}},
                  "nbits_gemm_tc", /*pdl=*/true);
        if (p.use_tma)
            rec.tmaps.push_back(TmapReloc{(uint32_t)offsetof(TcP, xmap), x.buf, (uint64_t)gr.k, (uint64_t)gr.m, (uint64_t)gr.k * 2, 64u, (uint32_t)mb,
                                          (uint32_t)offsetof(TcP, use_tma)});
        if (splits > 1) {
            TcReduceP q{};
            q.m0 = m0;
            q.m_total = gr.m;
            q.n_pad = p.n_pad;
            q.n_seg = p.n_seg;
            q.interleave2 = p.interleave2;
            q.row_tiles = p.row_tiles;
            q.mb = mb;
            q.splits = splits;
            q.row0 = n_full * 128;
            for (int i = 0; i < 3; i++) q.seg_n[i] = p.seg_n[i];
            for (int i = 0; i < 4; i++) q.seg_rt0[i] = p.seg_rt0[i];
            const long long rows = (long long)p.row_tiles * 16 - q.row0, m_here = std::min<long long>(mb, gr.m - m0);
            em.launch(nbits_gemm_reduce, dim3((unsigned)((rows / 4 + 255) / 256), (unsigned)m_here), dim3(256), 0, q,
                      {{&q.partial, partial}, {&q.y[0], gr.y[0].buf}, {&q.y[1], gr.n_seg > 1 ? gr.y[1].buf : null},
                       {&q.y[2], gr.n_seg > 2 ? gr.y[2].buf : null}},
                      "nbits_gemm_reduce", /*pdl=*/true);
        }
    }
}

}  // namespace oxk
