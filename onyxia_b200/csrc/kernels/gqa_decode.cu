// com.microsoft.GroupQueryAttention for one new token per sequence (S = 1) over
// a KV cache that is appended in place: one launch does rotary on q and k, the
// cache append, the causal / sliding-window mask, softmax and P·V.
// Specification: the decomposition crates/onyxia-ir/src/decomp.rs:357-613.
//
// One thread-block cluster works on one (batch row, KV head, group of query
// heads); its CTAs split the visible keys into contiguous ranges.
//   1. Every CTA rotates the group's q rows into shared memory; the CTA whose
//      range ends at the newest position also rotates the new k row and writes
//      it and the new v row into the cache.
//   2. K rows of the CTA's range arrive in shared memory as bulk asynchronous
//      copies (rows of one head are contiguous in the cache), a block of keys per
//      copy through a small ring; one warp per key forms q·k in f64 for all
//      heads of the group. Scores are rounded where the decomposition stores
//      them (product, scaled product).
//   3. Row maximum: CTA-local, then across the cluster through distributed
//      shared memory. Exponentials are rounded like the interpreter's; their sum
//      is exact in f64 (multiples of 2⁻²⁴ not above 1), so the cluster-wide sum
//      does not depend on the order of addition.
//   4. V rows stream through the same ring; p = round(e / Σ) and Σ p·v in f64 per
//      CTA; the partial outputs are added across the cluster in rank order by the
//      CTA that owns a slice of the head dimension, rounded and stored.
// Three kernels share these phases: gqa_decode (any dtype, f64 products; described
// above), gqa_decode_h (f16, head size 256: 64-key blocks staged by the whole CTA,
// tensor-core products) and gqa_decode_s (f16, head size 64 / 128: every warp
// streams its own 16-key tiles; see its own comment).
// Nothing spins on memory: CTAs meet at hardware cluster barriers; the generic
// kernel's waits on bulk-copy completion are bounded (an expired wait sets the
// error word and the CTA carries on to the barriers, so the cluster always
// drains), and the f16 kernels wait only on their own asynchronous copies.
#include <cooperative_groups.h>

#include <cstdlib>
#include <map>
#include <mutex>

#include "common.cuh"
#include "kernels.hpp"
#include "persist.hpp"

namespace oxk {

namespace cg = cooperative_groups;

namespace {

constexpr int kThreads = 256;
constexpr int kKeyBlock = 32;   // keys per bulk copy
constexpr int kRing = 6;        // copies in flight
constexpr long long kWaitCycles = 2000000000LL;

template <int DT> __device__ __forceinline__ float rndf(float v) {
    if constexpr (DT == DT_F16) return __half2float(__float2half_rn(v));
    else return v;
}
template <int DT> __device__ __forceinline__ float rndd(double v) {
    if constexpr (DT == DT_F16) return __half2float(__double2half(v));
    else return (float)v;
}

__device__ __forceinline__ unsigned sm_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool bar_try(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool bar_wait(unsigned bar, unsigned parity) {
    if (bar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (clock64() - t0 < kWaitCycles)
        if (bar_try(bar, parity)) return true;
    return false;
}

struct GqaDecP {
    const void* q;        // [B,1,H,D]
    const void* k;        // [B,1,KV,D] new key
    const void* v;        // [B,1,KV,D] new value
    void* cache_k;        // [B,KV,cap,D], appended in place
    void* cache_v;
    const int* seqlens;
    const void* cos;
    const void* sin;
    void* out;            // [B,1,H·D]
    ErrWord* err;
    const long long* dyn_t;  // present length T (rows valid after this step), refreshed per run
    long long H, KV, cap, window, half, cache_rows;
    float scale;          // rounded to the tensor dtype
    int groups;           // query-head groups per KV head
    int chunk_max;        // keys a CTA may be given (sizes the score rows in shared memory)
    int l2_ahead;         // streaming kernel: tiles (of this warp) by which K / V rows are asked into L2 ahead of their loads; 0: none
    int node;
};

// DPL = head-dim elements per lane (D = 32·DPL), GT = query heads per cluster, CX = CTAs per cluster.
template <int DT, int DPL, int GT> __global__ void __launch_bounds__(kThreads, 1) gqa_decode(const GqaDecP p) {
    using E = typename Ty<DT>::S;
    constexpr int D = 32 * DPL;
    constexpr int ESZ = (int)sizeof(E);
    constexpr int kBlockBytes = kKeyBlock * D * ESZ;
    cg::cluster_group cluster = cg::this_cluster();
    const int CX = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* ring = smem;                                                   // kRing blocks of keys
    float* q_s = reinterpret_cast<float*>(ring + kRing * kBlockBytes);            // [GT][D] rotated q
    float* sc = q_s + GT * D;                                                     // [GT][chunk_max] scores → exponentials → probabilities
    double* part = reinterpret_cast<double*>(sc + GT * ((p.chunk_max + 3) & ~3)); // [2][GT][D] partial outputs of the two key halves
    double* red = part + 2 * GT * D;                                              // [GT][8] per-warp partial sums
    float* cmax = reinterpret_cast<float*>(red + GT * 8);                         // [GT] this CTA's maxima (read by the cluster)
    double* csum = reinterpret_cast<double*>(cmax + 8);                           // [GT] this CTA's sums   (read by the cluster)
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(csum + 8);   // [kRing]

    pdl_enter();

    const long long b = blockIdx.z;
    const long long kvh = blockIdx.y / p.groups, gc = blockIdx.y % p.groups;
    const long long G = p.H / p.KV, h0 = kvh * G + gc * GT;
    const int live = (int)(G - gc * GT < GT ? G - gc * GT : GT);  // heads of this group that exist
    const long long T = *p.dyn_t;
    const long long tot = (long long)p.seqlens[b] + 1, qpos = tot - 1 > 0 ? tot - 1 : 0;
    const long long hi = qpos < T - 1 ? qpos : T - 1;
    const long long lo = (p.window >= 0 && qpos - p.window > 0) ? qpos - p.window : 0;
    const long long n = hi >= lo ? hi - lo + 1 : 0;
    const long long chunk = (n + CX - 1) / CX;
    const long long my_lo = lo + rank * chunk;
    long long my_n = n - rank * chunk;
    my_n = my_n < 0 ? 0 : (my_n > chunk ? chunk : my_n);
    if (my_n > p.chunk_max) {  // cannot happen for a launch sized by the host; never index past the rows
        if (tid == 0) report(p.err, ERR_SLICE_OOB, p.node, my_n, p.chunk_max);
        my_n = p.chunk_max;
    }
    const int n_blocks = (int)((my_n + kKeyBlock - 1) / kKeyBlock);
    const long long head_base = (b * p.KV + kvh) * p.cap * D;  // element offset of this head's rows
    E* ck = reinterpret_cast<E*>(p.cache_k) + head_base;
    E* cv = reinterpret_cast<E*>(p.cache_v) + head_base;
    const bool owns_new = qpos <= T - 1 && n > 0 && (hi - lo) / chunk == rank;  // the newest key is in this CTA's range

    long long rope_row = qpos;
    if (p.half && rope_row >= p.cache_rows) {
        if (tid == 0 && rank == 0) report(p.err, ERR_GATHER_OOB, p.node, rope_row, p.cache_rows);
        rope_row = 0;
    }
    auto rope = [&](const void* x, long long base, int e) -> float {
        if (e >= 2 * p.half) return ld<DT>(x, base + e);
        const bool first = e < p.half;
        const long long j = first ? e : e - p.half;
        const float c = ld<DT>(p.cos, rope_row * p.half + j), s = ld<DT>(p.sin, rope_row * p.half + j);
        const float x1 = ld<DT>(x, base + j), x2 = ld<DT>(x, base + j + p.half);
        return first ? rndf<DT>(x1 * c) - rndf<DT>(x2 * s) : rndf<DT>(x2 * c) + rndf<DT>(x1 * s);
    };

    // copies: block i of 2·n_blocks — K blocks first, then V blocks — goes to ring slot i % kRing
    auto issue = [&](int i) {  // one thread
        const bool is_v = i >= n_blocks;
        const int blk = is_v ? i - n_blocks : i;
        long long rows = my_n - (long long)blk * kKeyBlock;
        rows = rows > kKeyBlock ? kKeyBlock : rows;
        const unsigned bytes = (unsigned)(rows * D * ESZ);
        const unsigned bar = sm_addr(bars + i % kRing);
        const E* src = (is_v ? cv : ck) + (my_lo + (long long)blk * kKeyBlock) * D;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         sm_addr(ring + (i % kRing) * kBlockBytes)),
                     "l"(src), "r"(bytes), "r"(bar)
                     : "memory");
    };
    if (tid == 0) {
        for (int s = 0; s < kRing; s++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sm_addr(bars + s)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int i = 0; i < kRing && i < 2 * n_blocks; i++) issue(i);
    }

    // 1. rotated q (every CTA), new k / v rows (the owner)
    for (int i = tid; i < GT * D; i += kThreads) {
        const int g = i / D, e = i % D;
        float v = 0.f;
        if (g < live) {
            const long long base = (b * p.H + h0 + g) * D;
            v = p.half ? rope(p.q, base, e) : ld<DT>(p.q, base + e);
        }
        q_s[i] = rndf<DT>(v);
    }
    float new_k = 0.f, new_v = 0.f;  // element tid of the new rows (D ≤ kThreads)
    if (owns_new && tid < D && gc == 0) {
        const long long base = (b * p.KV + kvh) * D;
        new_k = p.half ? rope(p.k, base, tid) : ld<DT>(p.k, base + tid);
        new_v = ld<DT>(p.v, base + tid);
        st<DT>(ck, qpos * D + tid, new_k);
        st<DT>(cv, qpos * D + tid, new_v);
        // a row shorter than the batch's longest: clear what lies beyond its newest key
        for (long long z = qpos + 1; z < T; z++) {
            st<DT>(ck, z * D + tid, 0.f);
            st<DT>(cv, z * D + tid, 0.f);
        }
    } else if (owns_new && tid < D) {
        const long long base = (b * p.KV + kvh) * D;
        new_k = p.half ? rope(p.k, base, tid) : ld<DT>(p.k, base + tid);
        new_v = ld<DT>(p.v, base + tid);
    }
    __syncthreads();

    bool ok = true;
    // 2. scores of this CTA's keys: one warp per key, lanes across the head dimension
    double qv[GT][DPL];
#pragma unroll
    for (int g = 0; g < GT; g++)
#pragma unroll
        for (int e = 0; e < DPL; e++) qv[g][e] = (double)q_s[g * D + lane * DPL + e];
    const int row_stride = (p.chunk_max + 3) & ~3;
    for (int blk = 0; blk < n_blocks; blk++) {
        const int i = blk, slot = i % kRing;
        if (ok && !bar_wait(sm_addr(bars + slot), (i / kRing) & 1)) ok = false;
        E* rows = reinterpret_cast<E*>(ring + slot * kBlockBytes);
        const long long first = my_lo + (long long)blk * kKeyBlock;
        // the newest key's row was fetched before it was written: patch it in shared memory
        if (owns_new && qpos >= first && qpos < first + kKeyBlock && tid < D) st<DT>(rows, (qpos - first) * D + tid, new_k);
        __syncthreads();
        const int here = (int)(my_n - (long long)blk * kKeyBlock < kKeyBlock ? my_n - (long long)blk * kKeyBlock : kKeyBlock);
        for (int r = warp; r < here; r += kThreads / 32) {
            double kx[DPL];
#pragma unroll
            for (int e = 0; e < DPL; e++) kx[e] = (double)ld<DT>(rows, (long long)r * D + lane * DPL + e);
#pragma unroll
            for (int g = 0; g < GT; g++) {
                double dot = 0.0;
#pragma unroll
                for (int e = 0; e < DPL; e++) dot += qv[g][e] * kx[e];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                if (lane == 0) sc[g * row_stride + blk * kKeyBlock + r] = rndf<DT>(rndd<DT>(dot) * p.scale);
            }
        }
        __syncthreads();  // the block is consumed: its slot may take the next copy
        if (tid == 0 && i + kRing < 2 * n_blocks) issue(i + kRing);
    }

    // 3. softmax statistics across the cluster
    auto warp_max_f = [&](float v) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
        return v;
    };
    for (int g = warp; g < GT; g += kThreads / 32) {
        float m = -INFINITY;
        for (int i = lane; i < (int)my_n; i += 32) m = fmaxf(m, sc[g * row_stride + i]);
        m = warp_max_f(m);
        if (lane == 0) cmax[g] = m;
    }
    cluster.sync();
    float gmax[GT];
#pragma unroll
    for (int g = 0; g < GT; g++) {
        float m = -INFINITY;
        for (int r = 0; r < CX; r++) m = fmaxf(m, *cluster.map_shared_rank(cmax + g, r));
        gmax[g] = m;
    }
    // exponentials, rounded like the decomposition's Sub → Exp; their sum is exact in f64
    {
        double local[GT];
#pragma unroll
        for (int g = 0; g < GT; g++) local[g] = 0.0;
        for (int i = tid; i < (int)my_n; i += kThreads) {
#pragma unroll
            for (int g = 0; g < GT; g++) {
                const float e = rndd<DT>(exp((double)rndd<DT>((double)sc[g * row_stride + i] - (double)gmax[g])));
                sc[g * row_stride + i] = e;
                local[g] += (double)e;
            }
        }
#pragma unroll
        for (int g = 0; g < GT; g++) {
            double v = local[g];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) red[g * 8 + warp] = v;
        }
        __syncthreads();
        if (tid < GT) {
            double v = 0.0;
            for (int w = 0; w < kThreads / 32; w++) v += red[tid * 8 + w];
            csum[tid] = v;
        }
    }
    cluster.sync();
    float total[GT];
#pragma unroll
    for (int g = 0; g < GT; g++) {
        double v = 0.0;
        for (int r = 0; r < CX; r++) v += *cluster.map_shared_rank(csum + g, r);
        total[g] = rndd<DT>(v);
    }
    // probabilities, rounded like the decomposition's Div
    for (int i = tid; i < (int)my_n; i += kThreads)
#pragma unroll
        for (int g = 0; g < GT; g++) sc[g * row_stride + i] = rndd<DT>((double)sc[g * row_stride + i] / (double)total[g]);
    __syncthreads();

    // 4. P·V: thread (half, c) adds the keys of its half of each block for dims c·DPH … of every head
    constexpr int DPH = D / (kThreads / 2);  // dims per thread (2 at D = 256)
    constexpr int DPT = DPH >= 1 ? DPH : 1;
    const int half_id = tid / (kThreads / 2), c0 = (tid % (kThreads / 2)) * DPT;
    const bool has_dims = c0 < D;
    double acc[GT][DPT];
#pragma unroll
    for (int g = 0; g < GT; g++)
#pragma unroll
        for (int e = 0; e < DPT; e++) acc[g][e] = 0.0;
    for (int blk = 0; blk < n_blocks; blk++) {
        const int i = n_blocks + blk, slot = i % kRing;
        if (ok && !bar_wait(sm_addr(bars + slot), (i / kRing) & 1)) ok = false;
        E* rows = reinterpret_cast<E*>(ring + slot * kBlockBytes);
        const long long first = my_lo + (long long)blk * kKeyBlock;
        if (owns_new && qpos >= first && qpos < first + kKeyBlock && tid < D) st<DT>(rows, (qpos - first) * D + tid, new_v);
        __syncthreads();
        const int here = (int)(my_n - (long long)blk * kKeyBlock < kKeyBlock ? my_n - (long long)blk * kKeyBlock : kKeyBlock);
        if (has_dims) {
            for (int r = half_id; r < here; r += 2) {
                float vx[DPT];
#pragma unroll
                for (int e = 0; e < DPT; e++) vx[e] = ld<DT>(rows, (long long)r * D + c0 + e);
#pragma unroll
                for (int g = 0; g < GT; g++) {
                    const double pr = (double)sc[g * row_stride + blk * kKeyBlock + r];
#pragma unroll
                    for (int e = 0; e < DPT; e++) acc[g][e] += pr * (double)vx[e];
                }
            }
        }
        __syncthreads();
        if (tid == 0 && i + kRing < 2 * n_blocks) issue(i + kRing);
    }
    if (has_dims)
#pragma unroll
        for (int g = 0; g < GT; g++)
#pragma unroll
            for (int e = 0; e < DPT; e++) part[(half_id * GT + g) * D + c0 + e] = acc[g][e];
    if (!ok) {
        // a copy did not land in time: record it and give what is still in flight a last bounded chance
        if (tid == 0) {
            report(p.err, ERR_WAIT_TIMEOUT, p.node, (long long)blockIdx.x, (long long)n_blocks);
            for (int i = 2 * n_blocks - kRing < 0 ? 0 : 2 * n_blocks - kRing; i < 2 * n_blocks; i++)
                bar_wait(sm_addr(bars + i % kRing), (i / kRing) & 1);
        }
        __syncthreads();
    }
    cluster.sync();

    // each CTA finishes a slice of the head dimension: partial outputs added in rank order
    const int slice = (D + CX - 1) / CX;
    for (int i = tid; i < GT * slice; i += kThreads) {
        const int g = i / slice, c = rank * slice + i % slice;
        if (g >= live || c >= D) continue;
        double v = 0.0;
        for (int r = 0; r < CX; r++) {
            const double* rp = cluster.map_shared_rank(part, r);
            v += rp[g * D + c] + rp[(GT + g) * D + c];
        }
        st<DT>(p.out, (b * p.H + h0 + g) * D + c, rndd<DT>(v));
    }
    cluster.sync();  // nobody leaves while its shared memory may still be read
}


// ── f16 variant: the two contractions run on the tensor cores ────────────
// Scores: per 16 keys, m16n8k16 MMAs with the K rows as A (keys × head dim) and
// the rotated q rows as B (head dim × heads, up to 8 heads). P·V: the rounded
// probabilities as A (heads × keys) and V rows as B (keys × 8 dims, read
// transposed). Products of two f16 values are exact; sums are f32. K/V rows are
// copied one row per bulk copy into rows padded by 16 bytes, so that the 8×8
// matrix loads touch every bank once.
constexpr int kRowPad = 8;  // f16 elements
// Keys per staged block and blocks in flight. A block is consumed between two CTA barriers and the score
// pass gives a warp 16 keys: with 32-key blocks two of the eight warps worked and a 1 024-key range paid 64
// barrier pairs; 64-key blocks halve both (batched decode at a 2 048-token context: the kernel is the layer).
constexpr int kKeyBlockH = 64;
constexpr int kRingH = 4;

// round_f16(exp(−|d|)) for every f16 argument (the softmax argument is ≤ 0; NaN patterns give NaN), filled once per
// device: the decomposition's Exp computes exp in f64 and rounds once, which for an f16 argument is a function of
// its 15 magnitude bits.
__device__ __half g_dec_exp_lut[32768];

__global__ void gqa_decode_fill_lut() {
    for (int i = (int)global_tid(); i < 32768; i += (int)global_threads())
        g_dec_exp_lut[i] = __double2half(exp(-(double)__half2float(__ushort_as_half((unsigned short)i))));
}

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int DPL, int GT> __global__ void __launch_bounds__(kThreads, 2) gqa_decode_h(const GqaDecP p) {
    constexpr int DT = DT_F16;
    constexpr int D = 32 * DPL, RS = D + kRowPad;      // row stride in elements
    constexpr int kBlockBytes = kKeyBlockH * RS * 2;
    constexpr int NW = kThreads / 32;
    cg::cluster_group cluster = cg::this_cluster();
    const int CX = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int kpad = (p.chunk_max + 15) & ~15;  // keys per CTA rounded up to whole MMA tiles

    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* ring = smem;                                             // kRingH blocks of kKeyBlockH padded rows
    __half* q_h = reinterpret_cast<__half*>(ring + kRingH * kBlockBytes);    // [8][RS] rotated q, zero rows beyond the group
    float* sc = reinterpret_cast<float*>(q_h + 8 * RS);                     // [GT][kpad] scores → exponentials
    __half* p_h = reinterpret_cast<__half*>(sc + GT * kpad);                // [8][kpad + 8] probabilities (A operand of P·V)
    float* part = reinterpret_cast<float*>(p_h + 8 * (kpad + 8));           // [GT][D] this CTA's partial output (read by the cluster)
    double* red = reinterpret_cast<double*>(part + GT * D);                 // [GT][NW]
    float* xmax = reinterpret_cast<float*>(red + GT * NW);                  // [8 ranks][GT] maxima, written by every CTA of the cluster
    double* xsum = reinterpret_cast<double*>(xmax + 8 * GT);                // [8 ranks][GT] sums,   written by every CTA of the cluster
    float* xpart = reinterpret_cast<float*>(xsum + 8 * GT);                 // [8 ranks][GT][slice] partial outputs of this CTA's slice

    ox_trace(p.err, 11);
    pdl_trigger();

    const long long b = blockIdx.z;
    const long long kvh = blockIdx.y / p.groups, gc = blockIdx.y % p.groups;
    const long long G = p.H / p.KV, h0 = kvh * G + gc * GT;
    const int live = (int)(G - gc * GT < GT ? G - gc * GT : GT);
    const long long head_base = (b * p.KV + kvh) * p.cap * D;
    __half* ck = reinterpret_cast<__half*>(p.cache_k) + head_base;
    __half* cv = reinterpret_cast<__half*>(p.cache_v) + head_base;
    // The present length comes with the launch (written before the graph started), so the key range can
    // be guessed — newest key at T − 1, the dense case — and the fetch of the old cache rows, which no
    // kernel of this step writes, started before the wait for the predecessor. The per-row length
    // (seqlens, produced inside this step) is checked after the wait; a ragged row fetches again.
    const long long T = *p.dyn_t;
    long long qpos, lo, my_lo;
    int n, chunk, my_n, n_blocks;
    bool owns_new;
    auto set_range = [&](long long q) {
        qpos = q;
        const long long hi = qpos < T - 1 ? qpos : T - 1;
        lo = (p.window >= 0 && qpos - p.window > 0) ? qpos - p.window : 0;
        n = (int)(hi >= lo ? hi - lo + 1 : 0);
        chunk = (n + CX - 1) / CX;
        my_lo = lo + (long long)rank * chunk;
        my_n = n - rank * chunk;
        my_n = my_n < 0 ? 0 : (my_n > chunk ? chunk : my_n);
        if (my_n > p.chunk_max) {  // a launch whose cluster shape and key capacity disagree: say so, never index past the rows
            if (tid == 0) report(p.err, ERR_SLICE_OOB, p.node, my_n, p.chunk_max);
            my_n = p.chunk_max;
        }
        n_blocks = (my_n + kKeyBlockH - 1) / kKeyBlockH;
        owns_new = qpos <= T - 1 && n > 0 && (int)((hi - lo) / chunk) == rank;
    };
    set_range(T - 1 > 0 ? T - 1 : 0);

    // Block i of 2·n_blocks (K blocks, then V blocks) → ring slot i % kRingH, as 16-byte asynchronous
    // copies into padded rows; every thread commits one group per block (empty beyond the last block).
    // The newest key's row is not fetched: its owner writes it into the slot directly.
    auto fetch = [&](int i) {
        if (i < 2 * n_blocks) {
            const bool is_v = i >= n_blocks;
            const int blk = is_v ? i - n_blocks : i;
            int rows = my_n - blk * kKeyBlockH;
            rows = rows > kKeyBlockH ? kKeyBlockH : rows;
            // thread → 16-byte column tid % (D/8) of rows tid / (D/8) + j·(threads / (D/8)): one address pair per
            // block, the rest are constant offsets
            constexpr int CPR = D / 8, RPP = kThreads / CPR;  // chunks per row, rows per pass of the CTA
            const int r0 = tid / CPR, col = tid % CPR;
            const __half* src = (is_v ? cv : ck) + (my_lo + (long long)blk * kKeyBlockH + r0) * D + col * 8;
            const unsigned dst = sm_addr(ring + (i % kRingH) * kBlockBytes) + (unsigned)(r0 * RS + col * 8) * 2;
            const int skip = owns_new ? (int)(qpos - (my_lo + (long long)blk * kKeyBlockH)) - r0 : -1 - r0;
#pragma unroll
            for (int j = 0; j < kKeyBlockH / RPP; j++)
                if (r0 + j * RPP < rows && j * RPP != skip)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (unsigned)(j * RPP * RS * 2)), "l"(src + (long long)j * RPP * D)
                                 : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int i = 0; i < kRingH; i++) fetch(i);
    ox_trace(p.err, 13);
    pdl_wait();
    ox_trace(p.err, 12);
    {
        const long long tot = (long long)p.seqlens[b] + 1, q = tot - 1 > 0 ? tot - 1 : 0;
        if (q != qpos) {  // a row shorter than the batch's longest: drop what was fetched for the guess
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
            set_range(q);
            for (int i = 0; i < kRingH; i++) fetch(i);
        }
    }
    long long rope_row = qpos;
    if (p.half && rope_row >= p.cache_rows) {
        if (tid == 0 && rank == 0) report(p.err, ERR_GATHER_OOB, p.node, rope_row, p.cache_rows);
        rope_row = 0;
    }

    // 1. rotated q for the heads of the group (zero rows up to 8), the new k / v rows, zeroed padding.
    // Thread e owns element e of every row, so all its loads are independent and issued together.
    float new_k = 0.f, new_v = 0.f;  // element tid of the new rows (D ≤ kThreads)
    if (tid < D) {
        const int e = tid;
        const bool rot = e < 2 * p.half, first = e < p.half;
        const int j = first ? e : e - (int)p.half, e2 = first ? e + (int)p.half : e - (int)p.half;  // partner element
        // unconditional loads from clamped addresses, all issued before any is used
        const int jc = rot ? j : 0;
        const long long kbase = (b * p.KV + kvh) * D;
        const __half* hq = reinterpret_cast<const __half*>(p.q);
        const __half* hk = reinterpret_cast<const __half*>(p.k);
        const __half* hv = reinterpret_cast<const __half*>(p.v);
        const __half* hcos = p.half ? reinterpret_cast<const __half*>(p.cos) : hq;
        const __half* hsin = p.half ? reinterpret_cast<const __half*>(p.sin) : hq;
        const __half rc = hcos[p.half ? rope_row * p.half + jc : 0], rsn = hsin[p.half ? rope_row * p.half + jc : 0];
        __half rx[GT + 1], ry[GT + 1];
#pragma unroll
        for (int hh = 0; hh < GT; hh++) {
            const long long base = (b * p.H + h0 + (hh < live ? hh : 0)) * D;
            rx[hh] = hq[base + e];
            ry[hh] = hq[base + (rot ? e2 : e)];
        }
        rx[GT] = hk[kbase + e];
        ry[GT] = hk[kbase + (rot ? e2 : e)];
        const __half rv = hv[kbase + e];
        const float c = rot ? __half2float(rc) : 1.f, s = rot ? __half2float(rsn) : 0.f;
        float x[GT + 1], y[GT + 1];  // rows: the group's q heads, then the new k
#pragma unroll
        for (int hh = 0; hh <= GT; hh++) {
            x[hh] = __half2float(rx[hh]);
            y[hh] = rot ? __half2float(ry[hh]) : 0.f;
        }
        if (owns_new) new_v = __half2float(rv);
        // first half: x1·cos − x2·sin; second half: x2·cos + x1·sin, with x the own element and y the partner
        auto turn = [&](float own, float partner) {
            if (!rot) return own;
            return first ? rndf<DT>(own * c) - rndf<DT>(partner * s) : rndf<DT>(own * c) + rndf<DT>(partner * s);
        };
#pragma unroll
        for (int hh = 0; hh < 8; hh++) q_h[hh * RS + e] = __float2half_rn(hh < GT && hh < live ? turn(x[hh < GT ? hh : 0], y[hh < GT ? hh : 0]) : 0.f);
        new_k = turn(x[GT], y[GT]);
        if (owns_new && gc == 0) {
            st<DT>(ck, qpos * D + e, new_k);
            st<DT>(cv, qpos * D + e, new_v);
            for (long long z = qpos + 1; z < T; z++) {  // a row shorter than the batch's longest
                st<DT>(ck, z * D + e, 0.f);
                st<DT>(cv, z * D + e, 0.f);
            }
        }
    }
    for (int i = tid; i < 8 * (kpad + 8); i += kThreads) p_h[i] = __float2half(0.f);
    cluster.sync();  // also: every CTA of the cluster has started, so its shared memory may be written remotely
    ox_trace(p.err, 14);

    // 2. scores: q as the B operand (head dim × heads), kept in registers
    unsigned qb[D / 16][2];
#pragma unroll
    for (int j = 0; j < D / 16; j++) {
        qb[j][0] = *reinterpret_cast<const unsigned*>(q_h + g * RS + 16 * j + 2 * t);
        qb[j][1] = *reinterpret_cast<const unsigned*>(q_h + g * RS + 16 * j + 2 * t + 8);
    }
    for (int blk = 0; blk < n_blocks; blk++) {
        const int slot = blk % kRingH;
        asm volatile("cp.async.wait_group %0;" ::"n"(kRingH - 1) : "memory");  // this thread's copies of the oldest block landed
        __half* rows = reinterpret_cast<__half*>(ring + slot * kBlockBytes);
        const int first = blk * kKeyBlockH;  // index within this CTA's keys
        const long long first_pos = my_lo + first;
        if (owns_new && qpos >= first_pos && qpos < first_pos + kKeyBlockH && tid < D)
            rows[(qpos - first_pos) * RS + tid] = __float2half_rn(new_k);
        __syncthreads();
        int here = my_n - first;
        here = here > kKeyBlockH ? kKeyBlockH : here;
        for (int kt = warp; kt * 16 < here; kt += NW) {  // 16 keys per MMA tile
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const int m = lane >> 3, r = lane & 7;
            const unsigned a_addr = sm_addr(rows + (kt * 16 + (m & 1) * 8 + r) * RS + (m >> 1) * 8);
#pragma unroll
            for (int j = 0; j < D / 16; j++) {
                unsigned a[4];
                ldsm_x4(a, a_addr + j * 32);
                mma_f16(c, a[0], a[1], a[2], a[3], qb[j][0], qb[j][1]);
            }
            // c0: (key g, head 2t)  c1: (key g, head 2t+1)  c2: (key g+8, head 2t)  c3: (key g+8, head 2t+1)
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int key = first + kt * 16 + g + (q >= 2 ? 8 : 0), head = 2 * t + (q & 1);
                if (head < GT && key < my_n) sc[head * kpad + key] = rndf<DT>(rndf<DT>(c[q]) * p.scale);
            }
        }
        __syncthreads();  // the block is consumed: its slot takes the next one
        fetch(blk + kRingH);
    }

    ox_trace(p.err, 15);
    // 3. softmax statistics: every CTA stores its maxima (then its sums) into slot `rank` of every
    // CTA's exchange area through distributed shared memory; after the cluster barrier each reads its own copy.
    for (int hh = warp; hh < GT; hh += NW) {
        float m = -INFINITY;
        for (int i = lane; i < my_n; i += 32) m = fmaxf(m, sc[hh * kpad + i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane < CX) cluster.map_shared_rank(xmax, lane)[rank * GT + hh] = m;
    }
    cluster.sync();
    ox_trace(p.err, 16);
    float gmax[GT];
#pragma unroll
    for (int hh = 0; hh < GT; hh++) {
        float m = -INFINITY;
        for (int r = 0; r < CX; r++) m = fmaxf(m, xmax[r * GT + hh]);
        gmax[hh] = m;
    }
    {
        double local[GT];
#pragma unroll
        for (int hh = 0; hh < GT; hh++) local[hh] = 0.0;
        for (int i = tid; i < my_n; i += kThreads) {
#pragma unroll
            for (int hh = 0; hh < GT; hh++) {
                // scores and maxima are f16 values: the rounded difference is one half subtraction, its exponential a table entry
                const __half dlt = __hsub(__float2half_rn(sc[hh * kpad + i]), __float2half_rn(gmax[hh]));
                const float e = __half2float(g_dec_exp_lut[__half_as_ushort(dlt) & 0x7FFF]);
                sc[hh * kpad + i] = e;
                local[hh] += (double)e;
            }
        }
#pragma unroll
        for (int hh = 0; hh < GT; hh++) {
            double v = local[hh];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) red[hh * NW + warp] = v;
        }
        __syncthreads();
        if (warp == 0) {
            for (int hh = 0; hh < GT; hh++) {
                double v = 0.0;
                for (int w = 0; w < NW; w++) v += red[hh * NW + w];
                if (lane < CX) cluster.map_shared_rank(xsum, lane)[rank * GT + hh] = v;
            }
        }
    }
    cluster.sync();
    ox_trace(p.err, 17);
    float total[GT];
#pragma unroll
    for (int hh = 0; hh < GT; hh++) {
        double v = 0.0;
        for (int r = 0; r < CX; r++) v += xsum[r * GT + hh];
        total[hh] = rndd<DT>(v);
    }
    for (int i = tid; i < my_n; i += kThreads)
#pragma unroll
        // e and Σ are f16 values: their f32 quotient rounds to the same f16 as the exact one would
        // (a quotient of two 11-bit integers is never within 2⁻²⁴ of a 12-bit rounding boundary unless it is on it)
        for (int hh = 0; hh < GT; hh++) p_h[hh * (kpad + 8) + i] = __float2half_rn(sc[hh * kpad + i] / total[hh]);
    __syncthreads();

    ox_trace(p.err, 18);
    // 4. P·V: warp w owns dims [w·D/NW, (w+1)·D/NW) in n-tiles of 8; A = probabilities (heads × keys)
    constexpr int NT = D / 8 / NW;  // n-tiles per warp
    float o[NT > 0 ? NT : 1][4];
#pragma unroll
    for (int i = 0; i < (NT > 0 ? NT : 1); i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    for (int blk = 0; blk < n_blocks; blk++) {
        const int i = n_blocks + blk, slot = i % kRingH;
        asm volatile("cp.async.wait_group %0;" ::"n"(kRingH - 1) : "memory");
        __half* rows = reinterpret_cast<__half*>(ring + slot * kBlockBytes);
        const int first = blk * kKeyBlockH;
        const long long first_pos = my_lo + first;
        int here = my_n - first;
        here = here > kKeyBlockH ? kKeyBlockH : here;
        if (owns_new && qpos >= first_pos && qpos < first_pos + kKeyBlockH && tid < D)
            rows[(qpos - first_pos) * RS + tid] = __float2half_rn(new_v);
        // rows beyond the last key of a partly filled tile hold stale bytes: clear them (their p is 0, but 0·NaN is NaN)
        for (int z = here * D + tid; z < ((here + 15) & ~15) * D; z += kThreads) rows[(z / D) * RS + z % D] = __float2half(0.f);
        __syncthreads();
        if (NT > 0) {
            for (int kt = 0; kt * 16 < here; kt++) {
                const unsigned a0 = *reinterpret_cast<const unsigned*>(p_h + g * (kpad + 8) + first + kt * 16 + 2 * t);
                const unsigned a2 = *reinterpret_cast<const unsigned*>(p_h + g * (kpad + 8) + first + kt * 16 + 2 * t + 8);
                const int m = lane >> 3, r = lane & 7;
#pragma unroll
                for (int nt = 0; nt < NT; nt += 2) {
                    // matrices: (keys 0-7, dims n0..), (keys 8-15, dims n0..), (keys 0-7, dims n0+8..), (keys 8-15, dims n0+8..)
                    const int n0 = (warp * NT + nt) * 8;
                    unsigned bm[4];
                    ldsm_x4_t(bm, sm_addr(rows + (kt * 16 + (m & 1) * 8 + r) * RS + n0 + (m >> 1) * 8));
                    mma_f16(o[nt], a0, 0u, a2, 0u, bm[0], bm[1]);
                    if (nt + 1 < NT) mma_f16(o[nt + 1], a0, 0u, a2, 0u, bm[2], bm[3]);
                }
            }
        }
        __syncthreads();
        fetch(i + kRingH);
    }
    ox_trace(p.err, 19);
    // c0: (head g, dim n0 + 2t)  c1: (head g, dim n0 + 2t + 1); rows 8-15 of the tile are padding.
    // Dim c belongs to the CTA c / slice, which adds the CX partial values in rank order.
    const int slice = (D + CX - 1) / CX;
    if (NT > 0 && g < GT)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const int c = (warp * NT + nt) * 8 + 2 * t + q, owner = c / slice;
                cluster.map_shared_rank(xpart, owner)[(rank * GT + g) * slice + c - owner * slice] = o[nt][q];
            }
    cluster.sync();
    for (int i = tid; i < GT * slice; i += kThreads) {
        const int hh = i / slice, c = rank * slice + i % slice;
        if (hh >= live || c >= D) continue;
        float v = 0.f;
        for (int r = 0; r < CX; r++) v += xpart[(r * GT + hh) * slice + i % slice];
        st<DT>(p.out, (b * p.H + h0 + hh) * D + c, v);
    }
    ox_trace(p.err, 20);
}

template <int DPL, int GT> size_t decode_h_smem(int chunk_max) {
    constexpr int D = 32 * DPL, RS = D + kRowPad;
    const int kpad = (chunk_max + 15) & ~15;
    return (size_t)kRingH * kKeyBlockH * RS * 2 + (size_t)8 * RS * 2 + (size_t)GT * kpad * 4 + (size_t)8 * (kpad + 8) * 2 +
           (size_t)GT * D * 4 + (size_t)GT * (kThreads / 32) * 8 + (size_t)8 * GT * 4 + (size_t)8 * GT * 8 +
           (size_t)8 * GT * D * 4 + 128;
}


// ── f16, D ≤ 128: the streaming form ────────────────────────────────────────
// Same phases and rounding points as gqa_decode_h, but no CTA-wide staging: a warp owns every eighth 16-key tile
// of the CTA's key range.
//   * Scores: the lane reads 16 bytes of key rows g and g + 8 per 32-dim chunk straight from the cache into
//     registers (next tile's loads in flight while this one is multiplied). A dot product does not care in which
//     order the dimensions are visited, so the eight dims a lane holds serve as the k slots (2t, 2t+1, 2t+8, 2t+9)
//     of two MMAs, against the same eight dims of q read with one 16-byte load from shared memory.
//   * P·V needs V transposed: each warp streams its tiles through a private two-stage ring in shared memory
//     (cp.async, warp-level waits only), reads them with ldmatrix.trans, and keeps a partial output over its
//     keys for all D dims; the eight partial outputs are added in warp order, then across the cluster in rank
//     order as before.
// The newest key's row is not read from the cache (its writer may belong to another cluster): every CTA forms it
// from the step's k / v inputs and patches it into the tile that holds its position.
template <int DPL, int GT, int NW> __global__ void __launch_bounds__(NW * 32, 16 / NW) gqa_decode_s(const GqaDecP p) {
    constexpr int kT = NW * 32;  // threads: 8 warps, or 4 (twice as many CTAs per SM: their fixed phases overlap better on short key ranges)
    constexpr int DT = DT_F16;
    constexpr int D = 32 * DPL, RS = D + kRowPad;
    constexpr int NCH = D / 32;
    constexpr int kStageBytes = 16 * RS * 2;  // one 16-key tile of padded rows
    cg::cluster_group cluster = cg::this_cluster();
    const int CX = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int kpad = (p.chunk_max + 15) & ~15;

    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* vring = smem;                                             // [NW][2] tiles; later [NW][GT][D] partial outputs
    __half* q_h = reinterpret_cast<__half*>(vring + NW * 2 * kStageBytes);   // [8][RS] rotated q, zero rows beyond the group
    __half* newk_h = q_h + 8 * RS;                                           // [D] rotated new key
    __half* newv_h = newk_h + D;                                             // [D] new value
    __half* sp = newv_h + D;                                                // [GT][kpad + 8] scores → exponentials → probabilities (f16 values throughout)
    double* red = reinterpret_cast<double*>(sp + GT * (kpad + 8));          // [GT][NW]
    float* xmax = reinterpret_cast<float*>(red + GT * NW);                  // [8 ranks][GT]
    double* xsum = reinterpret_cast<double*>(xmax + 8 * GT);                // [8 ranks][GT]
    float* xpart = reinterpret_cast<float*>(xsum + 8 * GT);                 // [CX ranks][GT][slice], slice = ⌈D / CX⌉

    pdl_trigger();

    const long long b = blockIdx.z;
    const long long kvh = blockIdx.y / p.groups, gc = blockIdx.y % p.groups;
    const long long G = p.H / p.KV, h0 = kvh * G + gc * GT;
    const int live = (int)(G - gc * GT < GT ? G - gc * GT : GT);
    const long long head_base = (b * p.KV + kvh) * p.cap * D;
    __half* ck = reinterpret_cast<__half*>(p.cache_k) + head_base;
    __half* cv = reinterpret_cast<__half*>(p.cache_v) + head_base;
    const long long T = *p.dyn_t;
    long long qpos, lo, my_lo;
    int n, chunk, my_n, n_tiles, new_rel;  // new_rel: index of the newest key within this CTA's keys, or −1
    auto set_range = [&](long long q) {
        qpos = q;
        const long long hi = qpos < T - 1 ? qpos : T - 1;
        lo = (p.window >= 0 && qpos - p.window > 0) ? qpos - p.window : 0;
        n = (int)(hi >= lo ? hi - lo + 1 : 0);
        chunk = (n + CX - 1) / CX;
        my_lo = lo + (long long)rank * chunk;
        my_n = n - rank * chunk;
        my_n = my_n < 0 ? 0 : (my_n > chunk ? chunk : my_n);
        if (my_n > p.chunk_max) {
            if (tid == 0) report(p.err, ERR_SLICE_OOB, p.node, my_n, p.chunk_max);
            my_n = p.chunk_max;
        }
        n_tiles = (my_n + 15) >> 4;
        const bool owns_new = qpos <= T - 1 && n > 0 && (int)((hi - lo) / chunk) == rank;
        new_rel = owns_new && qpos - my_lo < my_n ? (int)(qpos - my_lo) : -1;
    };
    set_range(T - 1 > 0 ? T - 1 : 0);

    // K rows g and g + 8 of a tile, the lane's 16 bytes of every 32-dim chunk (rows past the range read the last valid row)
    uint4 kl[NCH], kh[NCH];
    auto load_k = [&](int tile, uint4 (&l)[NCH], uint4 (&h)[NCH]) {
        if (tile < n_tiles) {
            const int r_lo = min(tile * 16 + g, my_n - 1), r_hi = min(tile * 16 + g + 8, my_n - 1);
            const uint4* pl = reinterpret_cast<const uint4*>(ck + (my_lo + r_lo) * D + 8 * t);
            const uint4* ph = reinterpret_cast<const uint4*>(ck + (my_lo + r_hi) * D + 8 * t);
#pragma unroll
            for (int c = 0; c < NCH; c++) {
                l[c] = __ldcs(pl + 4 * c);
                h[c] = __ldcs(ph + 4 * c);
            }
        }
    };
    // A tile's 16 rows are contiguous in the cache: one 128-byte line per lane asks them into L2, so
    // that the loads issued one tile ahead find them there instead of waiting for memory.
    auto prefetch_tile = [&](const __half* base, int tile) {
        if (p.l2_ahead > 0 && tile < n_tiles) {
            const char* row0 = reinterpret_cast<const char*>(base + (my_lo + (long long)tile * 16) * D);
            const int valid = min(16, my_n - tile * 16) * D * 2;  // bytes of the tile inside the key range
            for (int off = lane * 128; off < valid; off += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(row0 + off));
        }
    };
    load_k(warp, kl, kh);  // old cache rows: no kernel of this step writes them
    pdl_wait();
    {
        const long long tot = (long long)p.seqlens[b] + 1, q = tot - 1 > 0 ? tot - 1 : 0;
        if (q != qpos) {  // a row shorter than the batch's longest
            set_range(q);
            load_k(warp, kl, kh);
        }
    }
    long long rope_row = qpos;
    if (p.half && rope_row >= p.cache_rows) {
        if (tid == 0 && rank == 0) report(p.err, ERR_GATHER_OOB, p.node, rope_row, p.cache_rows);
        rope_row = 0;
    }

    // 1. rotated q rows, the new k / v rows (every CTA keeps them in shared memory; the owner of the newest
    // position in group 0 also appends them to the cache)
    if (tid < D) {
        const int e = tid;
        const bool rot = e < 2 * p.half, first = e < p.half;
        const int j = first ? e : e - (int)p.half, e2 = first ? e + (int)p.half : e - (int)p.half;
        const int jc = rot ? j : 0;
        const long long kbase = (b * p.KV + kvh) * D;
        const __half* hq = reinterpret_cast<const __half*>(p.q);
        const __half* hk = reinterpret_cast<const __half*>(p.k);
        const __half* hv = reinterpret_cast<const __half*>(p.v);
        const __half* hcos = p.half ? reinterpret_cast<const __half*>(p.cos) : hq;
        const __half* hsin = p.half ? reinterpret_cast<const __half*>(p.sin) : hq;
        const __half rc = hcos[p.half ? rope_row * p.half + jc : 0], rsn = hsin[p.half ? rope_row * p.half + jc : 0];
        __half rx[GT + 1], ry[GT + 1];
#pragma unroll
        for (int hh = 0; hh < GT; hh++) {
            const long long base = (b * p.H + h0 + (hh < live ? hh : 0)) * D;
            rx[hh] = hq[base + e];
            ry[hh] = hq[base + (rot ? e2 : e)];
        }
        rx[GT] = hk[kbase + e];
        ry[GT] = hk[kbase + (rot ? e2 : e)];
        const __half rv = hv[kbase + e];
        const float c = rot ? __half2float(rc) : 1.f, s = rot ? __half2float(rsn) : 0.f;
        auto turn = [&](float own, float partner) {
            if (!rot) return own;
            return first ? rndf<DT>(own * c) - rndf<DT>(partner * s) : rndf<DT>(own * c) + rndf<DT>(partner * s);
        };
#pragma unroll
        for (int hh = 0; hh < 8; hh++)
            q_h[hh * RS + e] = __float2half_rn(hh < GT && hh < live ? turn(__half2float(rx[hh < GT ? hh : 0]), rot ? __half2float(ry[hh < GT ? hh : 0]) : 0.f) : 0.f);
        const __half nk = __float2half_rn(turn(__half2float(rx[GT]), rot ? __half2float(ry[GT]) : 0.f));
        newk_h[e] = nk;
        newv_h[e] = rv;
        if (new_rel >= 0 && gc == 0) {
            ck[qpos * D + e] = nk;
            cv[qpos * D + e] = rv;
            for (long long z = qpos + 1; z < T; z++) {  // a row shorter than the batch's longest
                ck[z * D + e] = __float2half(0.f);
                cv[z * D + e] = __float2half(0.f);
            }
        }
    }
    for (int i = tid; i < GT * (kpad + 8); i += kT) sp[i] = __float2half(0.f);  // keys past the range keep probability 0
    cluster.sync();  // also: every CTA of the cluster has started, so its shared memory may be written remotely

    // 2. scores
    {
        uint4 qb[NCH];  // q[head g][dims 32c + 8t … + 8]
#pragma unroll
        for (int c = 0; c < NCH; c++) qb[c] = *reinterpret_cast<const uint4*>(q_h + g * RS + 32 * c + 8 * t);
        for (int tile = warp; tile < n_tiles; tile += NW) {
            uint4 nl[NCH], nh[NCH];
#pragma unroll
            for (int c = 0; c < NCH; c++) nl[c] = nh[c] = make_uint4(0, 0, 0, 0);
            load_k(tile + NW, nl, nh);
            prefetch_tile(ck, tile + (1 + p.l2_ahead) * NW);
            if (new_rel >= 0 && (new_rel >> 4) == tile) {  // the newest key's row comes from this step's input
                const int r = new_rel & 15;
#pragma unroll
                for (int c = 0; c < NCH; c++) {
                    const uint4 nv = *reinterpret_cast<const uint4*>(newk_h + 32 * c + 8 * t);
                    if (r == g) kl[c] = nv;
                    if (r == g + 8) kh[c] = nv;
                }
            }
            float c4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < NCH; c++) {
                mma_f16(c4, kl[c].x, kh[c].x, kl[c].y, kh[c].y, qb[c].x, qb[c].y);
                mma_f16(c4, kl[c].z, kh[c].z, kl[c].w, kh[c].w, qb[c].z, qb[c].w);
            }
            // c0: (key g, head 2t)  c1: (key g, head 2t+1)  c2: (key g+8, head 2t)  c3: (key g+8, head 2t+1)
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int key = tile * 16 + g + (q >= 2 ? 8 : 0), head = 2 * t + (q & 1);
                if (head < GT && key < my_n) sp[head * (kpad + 8) + key] = __float2half_rn(rndf<DT>(c4[q]) * p.scale);
            }
#pragma unroll
            for (int c = 0; c < NCH; c++) {
                kl[c] = nl[c];
                kh[c] = nh[c];
            }
        }
    }

    // V tile → stage `s` of this warp's ring: lane → 16-byte column lane % (D/8) of rows lane / (D/8) + j·(32 / (D/8)).
    // Rows past the range are zeroed (their probability is 0, but 0·NaN is NaN); always commits one group.
    auto fetch_v = [&](int tile, int s) {
        if (tile < n_tiles) {
            constexpr int CPR = D / 8, RPP = 32 / CPR;
            const int r0 = lane / CPR, col = lane % CPR;
            unsigned char* stage = vring + (warp * 2 + s) * kStageBytes;
            const __half* src = cv + (my_lo + tile * 16 + r0) * D + col * 8;
            const unsigned dst = sm_addr(stage) + (unsigned)(r0 * RS + col * 8) * 2;
#pragma unroll
            for (int j = 0; j < 16 / RPP; j++) {
                const int key = tile * 16 + r0 + j * RPP;
                if (key == new_rel)
                    *reinterpret_cast<uint4*>(stage + ((r0 + j * RPP) * RS + col * 8) * 2) = *reinterpret_cast<const uint4*>(newv_h + col * 8);
                else if (key < my_n)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (unsigned)(j * RPP * RS * 2)), "l"(src + (long long)j * RPP * D) : "memory");
                else
                    *reinterpret_cast<uint4*>(stage + ((r0 + j * RPP) * RS + col * 8) * 2) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch_v(warp, 0);       // on their way while the softmax statistics are exchanged
    fetch_v(warp + NW, 1);
    __syncthreads();        // every warp's scores are in shared memory

    // 3. softmax statistics (as in gqa_decode_h)
    for (int hh = warp; hh < GT; hh += NW) {
        float m = -INFINITY;
        for (int i = lane; i < my_n; i += 32) m = fmaxf(m, __half2float(sp[hh * (kpad + 8) + i]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane < CX) cluster.map_shared_rank(xmax, lane)[rank * GT + hh] = m;
    }
    cluster.sync();
    float gmax[GT];
#pragma unroll
    for (int hh = 0; hh < GT; hh++) {
        float m = -INFINITY;
        for (int r = 0; r < CX; r++) m = fmaxf(m, xmax[r * GT + hh]);
        gmax[hh] = m;
    }
    {
        double local[GT];
#pragma unroll
        for (int hh = 0; hh < GT; hh++) local[hh] = 0.0;
        for (int i = tid; i < my_n; i += kT) {
#pragma unroll
            for (int hh = 0; hh < GT; hh++) {
                const __half dlt = __hsub(sp[hh * (kpad + 8) + i], __float2half_rn(gmax[hh]));
                const __half e = g_dec_exp_lut[__half_as_ushort(dlt) & 0x7FFF];
                sp[hh * (kpad + 8) + i] = e;
                local[hh] += (double)__half2float(e);
            }
        }
#pragma unroll
        for (int hh = 0; hh < GT; hh++) {
            double v = local[hh];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) red[hh * NW + warp] = v;
        }
        __syncthreads();
        if (warp == 0) {
            for (int hh = 0; hh < GT; hh++) {
                double v = 0.0;
                for (int w = 0; w < NW; w++) v += red[hh * NW + w];
                if (lane < CX) cluster.map_shared_rank(xsum, lane)[rank * GT + hh] = v;
            }
        }
    }
    cluster.sync();
    float total[GT];
#pragma unroll
    for (int hh = 0; hh < GT; hh++) {
        double v = 0.0;
        for (int r = 0; r < CX; r++) v += xsum[r * GT + hh];
        total[hh] = rndd<DT>(v);
    }
    for (int i = tid; i < my_n; i += kT)
#pragma unroll
        for (int hh = 0; hh < GT; hh++) sp[hh * (kpad + 8) + i] = __float2half_rn(__half2float(sp[hh * (kpad + 8) + i]) / total[hh]);
    __syncthreads();

    // 4. P·V over this warp's tiles, all D dims
    constexpr int NT = D / 8;
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    {
        int it = 0;
        for (int tile = warp; tile < n_tiles; tile += NW, it++) {
            asm volatile("cp.async.wait_group 1;" ::: "memory");  // all but the newest group: this tile has landed
            __syncwarp();
            const __half* rows = reinterpret_cast<const __half*>(vring + (warp * 2 + (it & 1)) * kStageBytes);
            // rows of the A operand are heads: the ones past the group are zero
            const unsigned a0 = g < GT ? *reinterpret_cast<const unsigned*>(sp + g * (kpad + 8) + tile * 16 + 2 * t) : 0u;
            const unsigned a2 = g < GT ? *reinterpret_cast<const unsigned*>(sp + g * (kpad + 8) + tile * 16 + 2 * t + 8) : 0u;
            const int m = lane >> 3, r = lane & 7;
#pragma unroll
            for (int nt = 0; nt < NT; nt += 2) {
                unsigned bm[4];
                ldsm_x4_t(bm, sm_addr(rows + ((m & 1) * 8 + r) * RS + nt * 8 + (m >> 1) * 8));
                mma_f16(o[nt], a0, 0u, a2, 0u, bm[0], bm[1]);
                mma_f16(o[nt + 1], a0, 0u, a2, 0u, bm[2], bm[3]);
            }
            __syncwarp();  // every lane has read the stage before it is refilled
            fetch_v(tile + 2 * NW, it & 1);
            prefetch_tile(cv, tile + (2 + p.l2_ahead) * NW);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // the rings are free: they take the warps' partial outputs
    float* part = reinterpret_cast<float*>(vring);  // [NW][GT][D]
    if (g < GT)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            part[(warp * GT + g) * D + nt * 8 + 2 * t] = o[nt][0];
            part[(warp * GT + g) * D + nt * 8 + 2 * t + 1] = o[nt][1];
        }
    __syncthreads();
    // Dim c belongs to the CTA c / slice, which adds the CX partial values in rank order.
    const int slice = (D + CX - 1) / CX;
    for (int i = tid; i < GT * D; i += kT) {
        const int hh = i / D, c = i % D, owner = c / slice;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) v += part[(w * GT + hh) * D + c];  // warp order
        cluster.map_shared_rank(xpart, owner)[(rank * GT + hh) * slice + c - owner * slice] = v;
    }
    cluster.sync();
    for (int i = tid; i < GT * slice; i += kT) {
        const int hh = i / slice, c = rank * slice + i % slice;
        if (hh >= live || c >= D) continue;
        float v = 0.f;
        for (int r = 0; r < CX; r++) v += xpart[(r * GT + hh) * slice + i % slice];
        st<DT>(p.out, (b * p.H + h0 + hh) * D + c, v);
    }
}

template <int DPL, int GT> size_t decode_s_smem(int chunk_max, int cx, int nw) {
    constexpr int D = 32 * DPL, RS = D + kRowPad;
    const int kpad = (chunk_max + 15) & ~15, slice = (D + cx - 1) / cx;
    return (size_t)nw * 2 * 16 * RS * 2 + (size_t)8 * RS * 2 + (size_t)2 * D * 2 + (size_t)GT * (kpad + 8) * 2 +
           (size_t)GT * nw * 8 + (size_t)8 * GT * 4 + (size_t)8 * GT * 8 + (size_t)cx * GT * slice * 4 + 128;
}

}  // namespace

namespace {

template <int DT, int DPL, int GT> size_t decode_smem(int chunk_max) {
    constexpr int D = 32 * DPL;
    const size_t esz = DT == DT_F16 ? 2 : 4;
    return (size_t)kRing * kKeyBlock * D * esz + (size_t)GT * D * 4 + (size_t)GT * ((chunk_max + 3) & ~3) * 4 +
           (size_t)2 * GT * D * 8 + (size_t)GT * 8 * 8 + 32 + 64 + (size_t)kRing * 8;
}

template <int DT, int DPL, int GT>
bool launch_decode(Emitter& em, const GqaDecP& p0, dim3 grid, int cx, const Buf (&bufs)[11], int stream_warps) {
    int nw = kThreads / 32;
    size_t smem = decode_smem<DT, DPL, GT>(p0.chunk_max);
    void (*fn)(const GqaDecP) = gqa_decode<DT, DPL, GT>;
    if constexpr (DT == DT_F16 && DPL >= 2) {  // D ≥ 64: whole n-tiles per warp
        smem = decode_h_smem<DPL, GT>(p0.chunk_max);
        fn = gqa_decode_h<DPL, GT>;
        if constexpr (DPL <= 4) {  // D ≤ 128: the streaming form (its P·V accumulators for all of D fit in registers)
            static const bool off = std::getenv("ONYXIA_DISABLE_GQA_STREAM") && std::atoi(std::getenv("ONYXIA_DISABLE_GQA_STREAM")) != 0;  // diagnostics
            if (!off) {
                nw = stream_warps;
                smem = decode_s_smem<DPL, GT>(p0.chunk_max, cx, nw);
                fn = nw == 4 ? gqa_decode_s<DPL, GT, 4> : gqa_decode_s<DPL, GT, 8>;
            }
        }
    }
    if (smem > 224 * 1024) return false;
    if (smem > 48 * 1024) ensure_max_dynamic_smem((const void*)fn, 224 * 1024);  // cached per device and kernel
    GqaDecP p = p0;
    em.launch(fn, grid, dim3((unsigned)nw * 32), (unsigned)smem, p,
              {{&p.q, bufs[0]}, {&p.k, bufs[1]}, {&p.v, bufs[2]}, {&p.cache_k, bufs[3]}, {&p.cache_v, bufs[4]},
               {&p.seqlens, bufs[5]}, {&p.cos, bufs[6]}, {&p.sin, bufs[7]}, {&p.out, bufs[8]}, {&p.err, bufs[9]},
               {&p.dyn_t, bufs[10]}},
              "gqa_decode", /*pdl=*/true);
    em.recs.back().cluster = dim3((unsigned)cx, 1, 1);
    return true;
}

template <int DT, int GT>
bool launch_decode_d(Emitter& em, const GqaDecP& p, dim3 grid, int cx, const Buf (&bufs)[11], long long D, int sw) {
    switch (D) {
        case 32: return launch_decode<DT, 1, GT>(em, p, grid, cx, bufs, sw);
        case 64: return launch_decode<DT, 2, GT>(em, p, grid, cx, bufs, sw);
        case 128: return launch_decode<DT, 4, GT>(em, p, grid, cx, bufs, sw);
        case 256: return launch_decode<DT, 8, GT>(em, p, grid, cx, bufs, sw);
        default: return false;
    }
}

template <int DT> bool launch_decode_g(Emitter& em, const GqaDecP& p, dim3 grid, int cx, const Buf (&bufs)[11], long long D, int gt, int sw) {
    if (gt == 4) return launch_decode_d<DT, 4>(em, p, grid, cx, bufs, D, sw);
    if (gt == 2) return launch_decode_d<DT, 2>(em, p, grid, cx, bufs, D, sw);
    return launch_decode_d<DT, 1>(em, p, grid, cx, bufs, D, sw);
}

}  // namespace

// Emits the single-launch decode kernel when the node is a decode step over an
// in-place cache (S = 1, no bias, present aliases past, length read per run);
// returns false when the shape is outside what the kernel handles.
bool emit_gqa_decode(Emitter& em, const GqaDesc& d, const TRef& q, const TRef& k, const TRef& v, const TRef& seqlens,
                     const TRef* cos, const TRef* sin, const TRef& out, const TRef& present_k, const TRef& present_v,
                     Buf dyn_t, long long t_size) {
    const long long B = d.batch, H = d.heads, KV = d.kv_heads, D = d.head_dim;
    if (d.seq != 1 || !d.in_place || d.has_bias || B == 0 || B > 65535) return false;
    if (q.dtype != DT_F16 && q.dtype != DT_F32) return false;
    const long long G = H / KV;
    const int GT = G >= 4 ? 4 : (G >= 2 ? 2 : 1);
    const int groups = (int)((G + GT - 1) / GT);
    if (KV * groups > 65535) return false;
    const long long span = (d.window >= 0 && d.window + 1 < t_size) ? d.window + 1 : t_size;
    // CTAs per cluster: as many as the key range is worth splitting into, but no more than it takes to
    // fill the machine — with many (batch row, KV head) pairs each CTA should rather own more keys than
    // pay the cluster exchanges for a handful.
    const long long pairs = B * KV * groups;
    int cx = span > 128 ? 8 : span > 64 ? 4 : span > 32 ? 2 : 1;
    int cx_fill = 1;
    while (cx_fill < 8 && pairs * cx_fill * 2 <= 2 * sm_count()) cx_fill <<= 1;
    int cx_long = 1;  // a single CTA streams a long key range slowly: at most ≈ 1 024 keys each
    static const long long keys_per_cta = [] {
        const char* e = std::getenv("ONYXIA_GQA_KEYS_PER_CTA");  // diagnostics
        return e && std::atoll(e) >= 64 ? std::atoll(e) : 1024LL;
    }();
    while (cx_long < 8 && span > keys_per_cta * cx_long) cx_long <<= 1;
    if (cx > std::max(cx_fill, cx_long)) cx = std::max(cx_fill, cx_long);
    // … unless a CTA's share of the scores would not fit in shared memory
    while (cx < 8 && (span + cx - 1) / cx > 6144) cx <<= 1;
    // For the streaming f16 kernel (D ≤ 128) the cluster size and the CTA's warp count are chosen by cost: a CTA takes
    // a fixed ≈ 10 µs (start, four cluster barriers, the dependent loads of the prologue) plus its keys at the rate
    // its warps' two-deep pipelines sustain — measured ≈ 33 GB/s for 8 warps alone on an SM (17 for 4), and an SM
    // gives its resident CTAs ≈ 40 GB/s together; clusters of 8 / 4 leave 32 / 8 of the 296 CTA slots unused; a few
    // waves count whole, many waves overlap their ends. Fewer, longer CTAs win as soon as the (batch row, KV head)
    // pairs alone fill the machine; CTAs of 4 warps (four per SM) overlap their fixed phases better on short ranges.
    static const bool model_off = std::getenv("ONYXIA_GQA_KEYS_PER_CTA") != nullptr;
    static const int warps_env = [] {
        const char* e = std::getenv("ONYXIA_GQA_WARPS");  // diagnostics: 4 or 8 forces the warp count
        return e ? std::atoi(e) : 0;
    }();
    int stream_warps = 8;
    if (q.dtype == DT_F16 && (D == 64 || D == 128) && !model_off) {
        const double row_bytes = (double)D * 2 * 2;
        const int sms = sm_count();
        double best = 1e300;
        int best_cx = cx, best_nw = 8;
        for (int nw = 8; nw >= 4; nw >>= 1) {
            if (warps_env == 4 || warps_env == 8) {
                if (nw != warps_env) continue;
            }
            for (int c = 1; c <= 8; c <<= 1) {
                const long long chunk = (span + c - 1) / c;
                if (c > 1 && chunk < 16) break;
                if (nw == 4 && chunk > 1536) continue;  // measured: long ranges stream faster through 8-warp CTAs
                const size_t bytes = (size_t)nw * 8960 + 6 * 1024 + (size_t)GT * (chunk + 24) * 2;  // upper bound of the kernel's shared memory
                if (bytes > 220 * 1024) continue;
                const int per_sm = (int)std::min<size_t>(16 / nw, (228 * 1024) / (bytes + 1024));
                const long long ctas = pairs * c;
                long long slots = (long long)sms * per_sm;
                if (c == 8) slots = slots * 264 / 296;
                if (c == 4) slots = slots * 288 / 296;
                const double waves = ctas <= 4 * slots ? (double)((ctas + slots - 1) / slots) : (double)ctas / (double)slots;
                const long long together = std::min<long long>(per_sm, (ctas + sms - 1) / sms);  // CTAs that share an SM
                const double rate = std::min(nw == 8 ? 33e3 : 17e3, 40e3 / (double)together);   // bytes per µs and CTA
                const double t = waves * (10.0 + (double)chunk * row_bytes / rate);
                if (t < best) {
                    best = t;
                    best_cx = c;
                    best_nw = nw;
                }
            }
        }
        cx = best_cx;
        stream_warps = best_nw;
    }

    GqaDecP p{};
    p.H = H;
    p.KV = KV;
    p.cap = present_k.cap ? present_k.cap : t_size;
    p.window = d.window;
    p.half = d.rot_half;
    p.cache_rows = d.cache_rows;
    p.scale = q.dtype == DT_F16 ? __half2float(__double2half(d.scale)) : (float)d.scale;
    p.groups = groups;
    p.chunk_max = (int)((span + cx - 1) / cx);
    static const int l2_ahead = [] {
        const char* e = std::getenv("ONYXIA_GQA_L2_AHEAD");  // diagnostics
        return e ? std::max(0, std::min(std::atoi(e), 8)) : 2;
    }();
    p.l2_ahead = l2_ahead;
    p.node = em.node;
    const Buf null{kSlotNull, 0};
    const Buf bufs[11] = {q.buf, k.buf, v.buf, present_k.buf, present_v.buf, seqlens.buf, cos ? cos->buf : null,
                          sin ? sin->buf : null, out.buf, Buf{kSlotErr, 0}, dyn_t};
    dim3 grid((unsigned)cx, (unsigned)(KV * groups), (unsigned)B);
    if (q.dtype == DT_F16 && D >= 64) {  // the f16 kernel's exponential table, once per device
        static std::mutex mu;
        static std::map<int, bool> done;
        int dev = 0;
        cudaGetDevice(&dev);
        std::lock_guard<std::mutex> lock(mu);
        if (!done[dev]) {
            gqa_decode_fill_lut<<<32, 256>>>();
            if (cudaDeviceSynchronize() != cudaSuccess) {
                cudaGetLastError();
                return false;
            }
            done[dev] = true;
        }
    }
    const bool ok = q.dtype == DT_F16 ? launch_decode_g<DT_F16>(em, p, grid, cx, bufs, D, GT, stream_warps)
                                      : launch_decode_g<DT_F32>(em, p, grid, cx, bufs, D, GT, stream_warps);
    // A single sequence in f16: the launch can also run as an operation of the persistent step kernel.
    if (ok && B == 1 && q.dtype == DT_F16 && D >= 64 && G <= 8 && p.cap < (1LL << 31) && d.cache_rows < (1LL << 31)) {
        auto op = std::make_shared<PersistOp>();
        op->kind = POP_ATTN;
        op->node = em.node;
        op->q = q.buf;
        op->kx = k.buf;
        op->vx = v.buf;
        op->cache_k = present_k.buf;
        op->cache_v = present_v.buf;
        op->seqlens = seqlens.buf;
        if (cos) op->cos = cos->buf;
        if (sin) op->sin = sin->buf;
        op->out = out.buf;
        op->dyn_t = dyn_t;
        op->H = H;
        op->KV = KV;
        op->D = D;
        op->cap = p.cap;
        op->window = d.window;
        op->half = d.rot_half;
        op->cache_rows = d.cache_rows;
        op->span = span;
        op->scale = p.scale;
        em.recs.back().pop = std::move(op);
    }
    return ok;
}

}  // namespace oxk
