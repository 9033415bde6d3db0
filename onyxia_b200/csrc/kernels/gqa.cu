// com.microsoft.GroupQueryAttention, fused: rotary on q/k, KV-cache append,
// causal + sliding-window mask, softmax, P·V.
// Specification: the decomposition crates/onyxia-ir/src/decomp.rs:357-613
// (operand layout from crates/onyxia-lower/src/rules.rs:777-888).
//
// Per batch row b: tot = seqlens_k[b] + 1, past_b = max(tot − S, 0); query j
// sits at position past_b + j; present = valid past rows ++ new rows ++ zeros;
// a query sees keys col ≤ qpos and, with a window w ≥ 0, col ≥ qpos − w.
//
// The kernels round where the decomposition's primitives store a tensor
// (scores, scaled scores, shifted scores, exponentials, their sum, the
// probabilities, the output) and add in f64 in between, like the interpreter,
// so for f16 tensors they reproduce its rounding noise instead of adding their
// own.
//
// Three launches, the key range split over CTAs in the last two:
//   gqa_prepare  rotates q into scratch and writes the new K (rotated) / V rows
//                into the present cache (copying the valid past unless the
//                present buffer *is* the past buffer)
//   gqa_scores   one warp per key: q·k for the heads of one KV group, scaled,
//                biased, stored as f32 rows of scratch; the last CTA of a query
//                to finish reduces the row to (max, Σ exp)
//   gqa_pv       one warp per key again: p = exp(s − max)/Σ, acc += p·v; the
//                last CTA to finish adds the partial accumulators in split order
//                and stores the output row
// "Last CTA" is decided by an arrival counter per query; nothing ever waits.
//
// KV tensors are [B, KV, T, D] views of buffers that hold `cap ≥ T` rows per
// head, so an append never moves the rows already there.
#include "common.cuh"
#include "kernels.hpp"

namespace oxk {

template <int DT> __device__ __forceinline__ float rnd(float v) {
    if constexpr (DT == DT_F16) return __half2float(__float2half_rn(v));
    else return v;
}
template <int DT> __device__ __forceinline__ float rnd_d(double v) {
    if constexpr (DT == DT_F16) return __half2float(__double2half(v));
    else return (float)v;
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct GqaPrepP {
    const void* q;
    const void* k;
    const void* v;
    const void* past_k;
    const void* past_v;
    const int* seqlens;
    const void* cos;
    const void* sin;
    void* q_rot;  // [B,S,H,D], only with rotary
    void* present_k;
    void* present_v;
    ErrWord* err;
    const long long* dyn_t;  // when set, the present length T is read from here
    long long B, S, H, KV, D, P, T, past_cap, pres_cap, half, cache_rows;
    long long nq;    // threads that rotate q (0 without rotary)
    long long nkv;   // threads that build the present caches
    int in_place, node;
};

template <int DT>
__device__ __forceinline__ float rope_elem(const void* x, long long base, long long e, long long half, const void* cos,
                                           const void* sin, long long row) {
    if (e >= 2 * half) return ld<DT>(x, base + e);
    bool first = e < half;
    long long j = first ? e : e - half;
    float c = ld<DT>(cos, row * half + j), s = ld<DT>(sin, row * half + j);
    float x1 = ld<DT>(x, base + j), x2 = ld<DT>(x, base + j + half);
    return first ? rnd<DT>(x1 * c) - rnd<DT>(x2 * s) : rnd<DT>(x2 * c) + rnd<DT>(x1 * s);
}

template <int DT> __global__ void gqa_prepare(const GqaPrepP p) {
    pdl_enter();
    const long long total = p.nq + p.nkv;
    const long long T = p.dyn_t ? *p.dyn_t : p.T;
    for (long long i = global_tid(); i < total; i += global_threads()) {
        if (i < p.nq) {
            // q rotation: i over [B,S,H,D]
            long long e = i % p.D, bs = i / (p.D * p.H), b = bs / p.S, j = bs % p.S;
            long long tot = (long long)p.seqlens[b] + 1, past_b = tot - p.S > 0 ? tot - p.S : 0;
            long long row = past_b + j;
            if (row >= p.cache_rows) {
                report(p.err, ERR_GATHER_OOB, p.node, row, p.cache_rows);
                row = 0;
            }
            st<DT>(p.q_rot, i, rope_elem<DT>(p.q, i - e, e, p.half, p.cos, p.sin, row));
            continue;
        }
        long long r = i - p.nq;
        long long rows = p.in_place ? p.S : T;  // rows visited per (b, kv head)
        long long e = r % p.D, t0 = (r / p.D) % rows, kvh = (r / (p.D * rows)) % p.KV, b = r / (p.D * rows * p.KV);
        long long tot = (long long)p.seqlens[b] + 1, past_b = tot - p.S > 0 ? tot - p.S : 0;
        long long pres_base = (b * p.KV + kvh) * p.pres_cap * p.D, past_base = (b * p.KV + kvh) * p.past_cap * p.D;
        auto new_k = [&](long long j) -> float {
            long long base = ((b * p.S + j) * p.KV + kvh) * p.D;
            if (p.half == 0) return ld<DT>(p.k, base + e);
            long long row = past_b + j;
            if (row >= p.cache_rows) {
                report(p.err, ERR_GATHER_OOB, p.node, row, p.cache_rows);
                row = 0;
            }
            return rope_elem<DT>(p.k, base, e, p.half, p.cos, p.sin, row);
        };
        auto new_v = [&](long long j) -> float { return ld<DT>(p.v, ((b * p.S + j) * p.KV + kvh) * p.D + e); };
        if (p.in_place) {
            // the buffer already holds the valid past; write the new rows ...
            long long j = t0, t = past_b + j;
            if (t < T) {
                st<DT>(p.present_k, pres_base + t * p.D + e, new_k(j));
                st<DT>(p.present_v, pres_base + t * p.D + e, new_v(j));
            }
            // ... and, for a ragged row, clear what lies beyond them
            if (j == p.S - 1)
                for (long long z = past_b + p.S; z < T; z++) {
                    st<DT>(p.present_k, pres_base + z * p.D + e, 0.f);
                    st<DT>(p.present_v, pres_base + z * p.D + e, 0.f);
                }
        } else {
            long long t = t0;
            float kv = 0.f, vv = 0.f;
            if (t < p.P && t < past_b) {
                kv = ld<DT>(p.past_k, past_base + t * p.D + e);
                vv = ld<DT>(p.past_v, past_base + t * p.D + e);
            } else if (t >= past_b && t < past_b + p.S) {
                kv = new_k(t - past_b);
                vv = new_v(t - past_b);
            }
            st<DT>(p.present_k, pres_base + t * p.D + e, kv);
            st<DT>(p.present_v, pres_base + t * p.D + e, vv);
        }
    }
}

struct GqaAttnP {
    const void* q;  // [B,S,H,D]
    const void* pk;
    const void* pv;
    const int* seqlens;
    const void* bias;
    float* scores;      // [B,S,H,span]: scaled, biased, rounded scores of the visible keys (−inf beyond
                        // them); turned into exp(score − max) by the last CTA of gqa_scores
    float* stats;       // [B,S,H,2]: row max, Σ exp (rounded)
    double* part;       // [B,S,H,nsplit,D] partial P·V accumulators
    unsigned* counters; // [2][B·S·KV·groups]
    void* out;          // [B,S,H·D]
    const long long* dyn_t;  // when set, the present length T is read from here
    long long B, S, H, KV, D, T, cap, window, chunk, span;
    long long bias_sb, bias_sh;
    float scale;  // rounded to the tensor dtype
    int nsplit, groups;  // groups = head-group chunks per kv head
};

struct GqaWho {
    long long b, s, kvh, gc, h0, G, lo, hi, n;  // visible keys are lo..hi (n of them)
    long long query;                            // linear id of (b, s, kvh, gc) for counters
};

__device__ __forceinline__ GqaWho gqa_who(const GqaAttnP& p, int GT) {
    GqaWho w;
    w.b = blockIdx.z;
    w.G = p.H / p.KV;
    long long y = blockIdx.y;
    w.s = y % p.S;
    y /= p.S;
    w.gc = y % p.groups;
    w.kvh = y / p.groups;
    w.h0 = w.kvh * w.G + w.gc * GT;
    long long tot = (long long)p.seqlens[w.b] + 1, past_b = tot - p.S > 0 ? tot - p.S : 0;
    long long qpos = past_b + w.s;
    const long long T = p.dyn_t ? *p.dyn_t : p.T;
    w.hi = qpos < T - 1 ? qpos : T - 1;
    w.lo = (p.window >= 0 && qpos - p.window > 0) ? qpos - p.window : 0;
    w.n = w.hi >= w.lo ? w.hi - w.lo + 1 : 0;
    w.query = ((w.b * p.S + w.s) * p.KV + w.kvh) * p.groups + w.gc;
    return w;
}

// True in exactly one CTA per query: the one whose arrival completes the count.
__device__ __forceinline__ bool last_cta(unsigned* counter, int expected) {
    __shared__ unsigned arrived;
    __syncthreads();
    if (expected <= 1) return true;
    __threadfence();
    if (threadIdx.x == 0) {
        arrived = atomicAdd(counter, 1u);
        if (arrived == (unsigned)expected - 1) *counter = 0;  // leave it zero for the next launch
    }
    __syncthreads();
    bool last = arrived == (unsigned)expected - 1;
    if (last) __threadfence();
    return last;
}

// DPL = head-dim elements per lane (D = 32·DPL), GT = query heads per CTA.
template <int DT, int DPL, int GT> __global__ void __launch_bounds__(128) gqa_scores(const GqaAttnP p) {
    constexpr int NW = 4;
    pdl_enter();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long split = blockIdx.x;
    const GqaWho w = gqa_who(p, GT);

    float qv[GT][DPL];
#pragma unroll
    for (int g = 0; g < GT; g++) {
        bool live = w.gc * GT + g < w.G;
#pragma unroll
        for (int i = 0; i < DPL; i++)
            qv[g][i] = live ? ld<DT>(p.q, ((w.b * p.S + w.s) * p.H + w.h0 + g) * p.D + lane * DPL + i) : 0.f;
    }
    const long long kv_base = (w.b * p.KV + w.kvh) * p.cap * p.D + lane * DPL;
    const long long i_begin = split * p.chunk;
    long long i_end = i_begin + p.chunk;
    if (i_end > p.span) i_end = p.span;
    for (long long i = i_begin + warp; i < i_end; i += NW) {
        const long long t = w.lo + i;
        const bool visible = i < w.n;
        float kx[DPL];
#pragma unroll
        for (int e = 0; e < DPL; e++) kx[e] = visible ? ld<DT>(p.pk, kv_base + t * p.D + e) : 0.f;
#pragma unroll
        for (int g = 0; g < GT; g++) {
            if (w.gc * GT + g >= w.G) continue;
            double dot = 0.0;
#pragma unroll
            for (int e = 0; e < DPL; e++) dot += (double)qv[g][e] * (double)kx[e];
            dot = warp_sum_d(dot);
            float sc = rnd<DT>(rnd_d<DT>(dot) * p.scale);
            if (p.bias && visible) sc = rnd<DT>(sc + ld<DT>(p.bias, w.b * p.bias_sb + (w.h0 + g) * p.bias_sh + w.s * p.T + t));
            if (lane == 0) p.scores[((w.b * p.S + w.s) * p.H + w.h0 + g) * p.span + i] = visible ? sc : -INFINITY;
        }
    }
    if (!last_cta(p.counters + w.query, p.nsplit)) return;

    // Row statistics of the decomposition's Softmax (decomp.rs:174-183), one warp
    // per head: the scores are replaced by their rounded exponentials and the
    // rounded sum is kept for the P·V pass.
    for (int g = warp; g < GT; g += NW) {
        if (w.gc * GT + g >= w.G) continue;
        float* row = p.scores + ((w.b * p.S + w.s) * p.H + w.h0 + g) * p.span;
        float mx = -INFINITY;
        for (long long i = lane; i < w.n; i += 32) mx = fmaxf(mx, __ldcg(row + i));
        mx = warp_max(mx);
        double sum = 0.0;
        for (long long i = lane; i < w.n; i += 32) {
            float e = rnd_d<DT>(exp((double)rnd<DT>(__ldcg(row + i) - mx)));
            row[i] = e;
            sum += (double)e;
        }
        sum = warp_sum_d(sum);
        if (lane == 0) {
            float* st_ = p.stats + ((w.b * p.S + w.s) * p.H + w.h0 + g) * 2;
            st_[0] = mx;
            st_[1] = rnd_d<DT>(sum);
        }
    }
}

template <int DT, int DPL, int GT> __global__ void __launch_bounds__(128) gqa_pv(const GqaAttnP p) {
    constexpr int NW = 4;
    pdl_enter();
    constexpr int D = 32 * DPL;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long split = blockIdx.x;
    const GqaWho w = gqa_who(p, GT);

    float sum[GT];
    double acc[GT][DPL];
#pragma unroll
    for (int g = 0; g < GT; g++) {
        bool live = w.gc * GT + g < w.G;
        const float* st_ = p.stats + ((w.b * p.S + w.s) * p.H + w.h0 + g) * 2;
        sum[g] = live ? st_[1] : 1.f;
#pragma unroll
        for (int i = 0; i < DPL; i++) acc[g][i] = 0.0;
    }
    const long long kv_base = (w.b * p.KV + w.kvh) * p.cap * p.D + lane * DPL;
    const long long i_begin = split * p.chunk;
    long long i_end = i_begin + p.chunk;
    if (i_end > w.n) i_end = w.n;
    for (long long i = i_begin + warp; i < i_end; i += NW) {
        const long long t = w.lo + i;
        float vx[DPL];
#pragma unroll
        for (int e = 0; e < DPL; e++) vx[e] = ld<DT>(p.pv, kv_base + t * p.D + e);
#pragma unroll
        for (int g = 0; g < GT; g++) {
            if (w.gc * GT + g >= w.G) continue;
            float e = p.scores[((w.b * p.S + w.s) * p.H + w.h0 + g) * p.span + i];  // exponentials by now
            float pr = rnd<DT>(e / sum[g]);
#pragma unroll
            for (int k = 0; k < DPL; k++) acc[g][k] += (double)pr * (double)vx[k];
        }
    }
    // fold the four warps in order
    __shared__ double sh[NW][GT][D];
#pragma unroll
    for (int g = 0; g < GT; g++)
#pragma unroll
        for (int k = 0; k < DPL; k++) sh[warp][g][lane * DPL + k] = acc[g][k];
    __syncthreads();
    for (int idx = threadIdx.x; idx < GT * D; idx += blockDim.x) {
        int g = idx / D, c = idx % D;
        if (w.gc * GT + g >= w.G) continue;
        double v = sh[0][g][c] + sh[1][g][c] + sh[2][g][c] + sh[3][g][c];
        long long head = (w.b * p.S + w.s) * p.H + w.h0 + g;
        if (p.nsplit == 1) st<DT>(p.out, head * D + c, rnd_d<DT>(v));
        else p.part[(head * p.nsplit + split) * D + c] = v;
    }
    if (p.nsplit == 1) return;
    if (!last_cta(p.counters + (long long)gridDim.y * gridDim.z + w.query, p.nsplit)) return;
    for (int idx = threadIdx.x; idx < GT * D; idx += blockDim.x) {
        int g = idx / D, c = idx % D;
        if (w.gc * GT + g >= w.G) continue;
        long long head = (w.b * p.S + w.s) * p.H + w.h0 + g;
        double v = 0.0;
        for (int s = 0; s < p.nsplit; s++) v += __ldcg(p.part + (head * p.nsplit + s) * D + c);
        st<DT>(p.out, head * D + c, rnd_d<DT>(v));
    }
}

template <int DT> static void emit_gqa_t(Emitter& em, const GqaDesc& d, const TRef& q, const TRef& k, const TRef& v,
                                         const TRef& past_k, const TRef& past_v, const TRef& seqlens, const TRef* cos,
                                         const TRef* sin, const TRef* bias, const TRef& out, const TRef& present_k,
                                         const TRef& present_v) {
    const long long B = d.batch, S = d.seq, H = d.heads, KV = d.kv_heads, D = d.head_dim, P = d.past, T = P + S;
    if (B == 0 || S == 0) return;
    const int esz = DT == DT_F16 ? 2 : 4;
    Buf null{kSlotNull, 0};

    GqaPrepP pp{};
    pp.B = B; pp.S = S; pp.H = H; pp.KV = KV; pp.D = D; pp.P = P; pp.T = T;
    pp.past_cap = past_k.cap ? past_k.cap : P;
    pp.pres_cap = present_k.cap ? present_k.cap : T;
    // With a bucket the true length travels through the plan's per-run scalars.
    const bool dyn = d.t_bucket > 0 && d.in_place && !bias;
    const long long Tsz = dyn ? d.t_bucket : T;
    Buf dyn_t = dyn ? em.dyn(T) : null;
    if (dyn && S == 1 && emit_gqa_decode(em, d, q, k, v, seqlens, cos, sin, out, present_k, present_v, dyn_t, Tsz)) return;
    if (dyn) pp.P = pp.T = 0;
    pp.half = d.rot_half;
    pp.cache_rows = d.cache_rows;
    pp.in_place = d.in_place ? 1 : 0;
    pp.node = em.node;
    pp.nq = d.rot_half ? B * S * H * D : 0;
    pp.nkv = B * KV * (d.in_place ? S : T) * D;
    Buf qrot = d.rot_half ? em.scratch((size_t)(B * S * H * D * esz)) : null;
    em.launch(gqa_prepare<DT>, dim3(grid_for(pp.nq + pp.nkv, 256)), dim3(256), 0, pp,
              {{&pp.q, q.buf}, {&pp.k, k.buf}, {&pp.v, v.buf}, {&pp.past_k, past_k.buf}, {&pp.past_v, past_v.buf},
               {&pp.seqlens, seqlens.buf}, {&pp.cos, cos ? cos->buf : null}, {&pp.sin, sin ? sin->buf : null},
               {&pp.q_rot, qrot}, {&pp.present_k, present_k.buf}, {&pp.present_v, present_v.buf}, {&pp.err, Buf{kSlotErr, 0}},
               {&pp.dyn_t, dyn_t}},
              "gqa_prepare", /*pdl=*/true);

    if constexpr (DT == DT_F16) {
        // many new positions: scores and P·V on the tensor cores
        if (!bias && emit_gqa_prefill_tc(em, d, d.rot_half ? qrot : q.buf, seqlens, out, present_k, present_v, dyn_t, dyn ? 0 : T, pp.pres_cap))
            return;
    }

    GqaAttnP ap{};
    ap.B = B; ap.S = S; ap.H = H; ap.KV = KV; ap.D = D; ap.T = dyn ? 0 : T;
    ap.cap = pp.pres_cap;
    ap.window = d.window;
    ap.scale = DT == DT_F16 ? __half2float(__double2half(d.scale)) : (float)d.scale;
    if (bias) {
        ap.bias_sb = d.bias_b == 1 ? 0 : d.bias_h * S * T;
        ap.bias_sh = d.bias_h == 1 ? 0 : S * T;
    }
    const long long G = H / KV;
    const int GT = G >= 4 ? 4 : (G >= 2 ? 2 : 1);
    ap.groups = (int)((G + GT - 1) / GT);
    ap.span = (d.window >= 0 && d.window + 1 < Tsz) ? d.window + 1 : Tsz;
    // Split the visible key range so that the launch fills the machine; the
    // arrival counters bound the number of queries a split launch may have.
    long long queries = B * KV * ap.groups * S;
    long long want = (sm_count() * 4LL + queries - 1) / queries;   // ≈ 4 CTAs per SM
    long long max_split = (ap.span + 7) / 8;              // ≥ 8 keys per CTA (two per warp)
    long long nsplit = std::max<long long>(1, std::min<long long>(want, max_split));
    if (2 * queries > (long long)kCounterWords) nsplit = 1;
    nsplit = std::min<long long>(nsplit, 1024);
    ap.chunk = (ap.span + nsplit - 1) / nsplit;
    ap.nsplit = (int)((ap.span + ap.chunk - 1) / ap.chunk);
    Buf scores = em.scratch((size_t)(B * S * H * ap.span * 4));
    Buf stats = em.scratch((size_t)(B * S * H * 2 * 4));
    Buf part = ap.nsplit > 1 ? em.scratch((size_t)(B * S * H * ap.nsplit * D * 8)) : null;
    if (KV * ap.groups * S > 65535 || B > 65535) throw std::runtime_error("fused GQA: grid dimension exceeds 65535");
    dim3 g((unsigned)ap.nsplit, (unsigned)(KV * ap.groups * S), (unsigned)B), blk(128);
    Buf qsrc = d.rot_half ? qrot : q.buf;
#define PTRS                                                                                                       \
    {{&ap.q, qsrc}, {&ap.pk, present_k.buf}, {&ap.pv, present_v.buf}, {&ap.seqlens, seqlens.buf},                  \
     {&ap.bias, bias ? bias->buf : null}, {&ap.scores, scores}, {&ap.stats, stats}, {&ap.part, part},              \
     {&ap.counters, Buf{kSlotCounters, 0}}, {&ap.out, out.buf}, {&ap.dyn_t, dyn_t}}
#define GO(K, LABEL, DPL, GTT) em.launch(K<DT, DPL, GTT>, g, blk, 0, ap, PTRS, LABEL, /*pdl=*/true)
#define GO_D(K, LABEL, GTT)                  \
    switch (D / 32) {                        \
        case 1: GO(K, LABEL, 1, GTT); break; \
        case 2: GO(K, LABEL, 2, GTT); break; \
        case 4: GO(K, LABEL, 4, GTT); break; \
        default: GO(K, LABEL, 8, GTT); break; \
    }
#define GO_G(K, LABEL)                                  \
    if (GT == 4) { GO_D(K, LABEL, 4) }                  \
    else if (GT == 2) { GO_D(K, LABEL, 2) }             \
    else { GO_D(K, LABEL, 1) }
    GO_G(gqa_scores, "gqa_scores")
    GO_G(gqa_pv, "gqa_pv")
#undef GO_G
#undef GO_D
#undef GO
#undef PTRS
}

void emit_gqa(Emitter& em, const GqaDesc& d, const TRef& q, const TRef& k, const TRef& v, const TRef& past_k,
              const TRef& past_v, const TRef& seqlens, const TRef* cos, const TRef* sin, const TRef* bias,
              const TRef& out, const TRef& present_k, const TRef& present_v) {
    if (q.dtype == DT_F16) emit_gqa_t<DT_F16>(em, d, q, k, v, past_k, past_v, seqlens, cos, sin, bias, out, present_k, present_v);
    else emit_gqa_t<DT_F32>(em, d, q, k, v, past_k, past_v, seqlens, cos, sin, bias, out, present_k, present_v);
}

}  // namespace oxk
