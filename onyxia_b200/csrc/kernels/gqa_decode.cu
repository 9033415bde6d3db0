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
// Nothing spins on memory: CTAs meet at hardware cluster barriers, and waits on
// copy completion are bounded (an expired wait sets the error word and the CTA
// carries on to the barriers, so the cluster always drains).
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.hpp"

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

}  // namespace

namespace {

template <int DT, int DPL, int GT> size_t decode_smem(int chunk_max) {
    constexpr int D = 32 * DPL;
    const size_t esz = DT == DT_F16 ? 2 : 4;
    return (size_t)kRing * kKeyBlock * D * esz + (size_t)GT * D * 4 + (size_t)GT * ((chunk_max + 3) & ~3) * 4 +
           (size_t)2 * GT * D * 8 + (size_t)GT * 8 * 8 + 32 + 64 + (size_t)kRing * 8;
}

template <int DT, int DPL, int GT>
bool launch_decode(Emitter& em, const GqaDecP& p0, dim3 grid, int cx, const Buf (&bufs)[11]) {
    const size_t smem = decode_smem<DT, DPL, GT>(p0.chunk_max);
    if (smem > 200 * 1024) return false;
    auto fn = gqa_decode<DT, DPL, GT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) throw std::runtime_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    }
    GqaDecP p = p0;
    em.launch(fn, grid, dim3(kThreads), (unsigned)smem, p,
              {{&p.q, bufs[0]}, {&p.k, bufs[1]}, {&p.v, bufs[2]}, {&p.cache_k, bufs[3]}, {&p.cache_v, bufs[4]},
               {&p.seqlens, bufs[5]}, {&p.cos, bufs[6]}, {&p.sin, bufs[7]}, {&p.out, bufs[8]}, {&p.err, bufs[9]},
               {&p.dyn_t, bufs[10]}},
              "gqa_decode", /*pdl=*/true);
    em.recs.back().cluster = dim3((unsigned)cx, 1, 1);
    return true;
}

template <int DT, int GT>
bool launch_decode_d(Emitter& em, const GqaDecP& p, dim3 grid, int cx, const Buf (&bufs)[11], long long D) {
    switch (D) {
        case 32: return launch_decode<DT, 1, GT>(em, p, grid, cx, bufs);
        case 64: return launch_decode<DT, 2, GT>(em, p, grid, cx, bufs);
        case 128: return launch_decode<DT, 4, GT>(em, p, grid, cx, bufs);
        case 256: return launch_decode<DT, 8, GT>(em, p, grid, cx, bufs);
        default: return false;
    }
}

template <int DT> bool launch_decode_g(Emitter& em, const GqaDecP& p, dim3 grid, int cx, const Buf (&bufs)[11], long long D, int gt) {
    if (gt == 4) return launch_decode_d<DT, 4>(em, p, grid, cx, bufs, D);
    if (gt == 2) return launch_decode_d<DT, 2>(em, p, grid, cx, bufs, D);
    return launch_decode_d<DT, 1>(em, p, grid, cx, bufs, D);
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
    const int cx = span > 128 ? 8 : span > 64 ? 4 : span > 32 ? 2 : 1;

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
    p.node = em.node;
    const Buf null{kSlotNull, 0};
    const Buf bufs[11] = {q.buf, k.buf, v.buf, present_k.buf, present_v.buf, seqlens.buf, cos ? cos->buf : null,
                          sin ? sin->buf : null, out.buf, Buf{kSlotErr, 0}, dyn_t};
    dim3 grid((unsigned)cx, (unsigned)(KV * groups), (unsigned)B);
    return q.dtype == DT_F16 ? launch_decode_g<DT_F16>(em, p, grid, cx, bufs, D, GT)
                             : launch_decode_g<DT_F32>(em, p, grid, cx, bufs, D, GT);
}

}  // namespace oxk
