// com.microsoft.GroupQueryAttention, fused: rotary on q/k, KV-cache append,
// causal + sliding-window mask, split-K online softmax, P·V.
// Specification: the decomposition crates/onyxia-ir/src/decomp.rs:357-613
// (operand layout from crates/onyxia-lower/src/rules.rs:777-888).
//
// Per batch row b: tot = seqlens_k[b] + 1, past_b = max(tot − S, 0); query j
// sits at position past_b + j; present = valid past rows ++ new rows ++ zeros;
// a query sees keys col ≤ qpos and, with a window w ≥ 0, col ≥ qpos − w.
//
// Three launches:
//   gqa_prepare   rotates q into scratch and writes the new K (rotated) / V rows
//                 into the present cache (copying the valid past unless the
//                 present buffer *is* the past buffer)
//   gqa_partial   one CTA per (key split, kv head × head group × query, batch):
//                 each warp streams K/V rows, lanes hold a slice of the head
//                 dim, scores are finished with warp shuffles; writes
//                 (max, sum, acc[D]) per split to scratch
//   gqa_combine   merges the splits and stores the output row
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
    const long long total = p.nq + p.nkv;
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
        long long rows = p.in_place ? p.S : p.T;  // rows visited per (b, kv head)
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
            if (t < p.T) {
                st<DT>(p.present_k, pres_base + t * p.D + e, new_k(j));
                st<DT>(p.present_v, pres_base + t * p.D + e, new_v(j));
            }
            // ... and, for a ragged row, clear what lies beyond them
            if (j == p.S - 1)
                for (long long z = past_b + p.S; z < p.T; z++) {
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
    float* part;  // [B,S,H,nsplit,D+2]
    void* out;    // [B,S,H·D]
    long long B, S, H, KV, D, T, cap, window, chunk;
    long long bias_sb, bias_sh;
    float scale;  // rounded to the tensor dtype
    int nsplit, groups;  // groups = head-group chunks per kv head
};

// DPL = head-dim elements per lane (D = 32·DPL), GT = query heads per CTA.
template <int DT, int DPL, int GT> __global__ void __launch_bounds__(128) gqa_partial(const GqaAttnP p) {
    constexpr int NW = 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long b = blockIdx.z, split = blockIdx.x;
    const long long G = p.H / p.KV;
    long long y = blockIdx.y;
    const long long s = y % p.S;
    y /= p.S;
    const long long gc = y % p.groups, kvh = y / p.groups;
    const long long h0 = kvh * G + gc * GT;

    const long long tot = (long long)p.seqlens[b] + 1, past_b = tot - p.S > 0 ? tot - p.S : 0;
    long long qpos = past_b + s;
    long long hi = qpos < p.T - 1 ? qpos : p.T - 1;                      // last visible key
    long long lo = (p.window >= 0 && qpos - p.window > 0) ? qpos - p.window : 0;  // first visible key
    long long t_begin = lo + split * p.chunk, t_end = t_begin + p.chunk - 1;
    if (t_end > hi) t_end = hi;

    float qv[GT][DPL], acc[GT][DPL], mx[GT], sum[GT];
#pragma unroll
    for (int g = 0; g < GT; g++) {
        mx[g] = -INFINITY;
        sum[g] = 0.f;
        bool live = gc * GT + g < G;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            acc[g][i] = 0.f;
            qv[g][i] = live ? ld<DT>(p.q, ((b * p.S + s) * p.H + h0 + g) * p.D + lane * DPL + i) : 0.f;
        }
    }
    const long long kv_base = (b * p.KV + kvh) * p.cap * p.D + lane * DPL;
    for (long long t = t_begin + warp; t <= t_end; t += NW) {
        float kx[DPL], vx[DPL];
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            kx[i] = ld<DT>(p.pk, kv_base + t * p.D + i);
            vx[i] = ld<DT>(p.pv, kv_base + t * p.D + i);
        }
#pragma unroll
        for (int g = 0; g < GT; g++) {
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < DPL; i++) dot = fmaf(qv[g][i], kx[i], dot);
            dot = warp_sum(dot);
            float sc = rnd<DT>(rnd<DT>(dot) * p.scale);
            if (p.bias) sc = rnd<DT>(sc + ld<DT>(p.bias, b * p.bias_sb + (h0 + g) * p.bias_sh + s * p.T + t));
            float m_new = fmaxf(mx[g], sc);
            float corr = __expf(mx[g] - m_new), pr = __expf(sc - m_new);
            if (m_new == -INFINITY) {
                corr = 1.f;
                pr = 0.f;
            }
            sum[g] = sum[g] * corr + pr;
#pragma unroll
            for (int i = 0; i < DPL; i++) acc[g][i] = acc[g][i] * corr + pr * vx[i];
            mx[g] = m_new;
        }
    }
    // merge the four warps through shared memory
    __shared__ float sh[NW][GT][32 * DPL + 2];
#pragma unroll
    for (int g = 0; g < GT; g++) {
#pragma unroll
        for (int i = 0; i < DPL; i++) sh[warp][g][lane * DPL + i] = acc[g][i];
        if (lane == 0) {
            sh[warp][g][32 * DPL] = mx[g];
            sh[warp][g][32 * DPL + 1] = sum[g];
        }
    }
    __syncthreads();
    const int D = 32 * DPL;
    for (int idx = threadIdx.x; idx < GT * (D + 2); idx += blockDim.x) {
        int g = idx / (D + 2), c = idx % (D + 2);
        if (gc * GT + g >= G) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; w++) M = fmaxf(M, sh[w][g][D]);
        float val;
        if (c == D) {
            val = M;
        } else {
            val = 0.f;
#pragma unroll
            for (int w = 0; w < NW; w++) {
                float f = (sh[w][g][D] == -INFINITY) ? 0.f : __expf(sh[w][g][D] - M);
                val += f * (c == D + 1 ? sh[w][g][D + 1] : sh[w][g][c]);
            }
        }
        p.part[((((b * p.S + s) * p.H + h0 + g) * p.nsplit) + split) * (D + 2) + c] = val;
    }
}

template <int DT> __global__ void gqa_combine(const GqaAttnP p) {
    const long long b = blockIdx.y, sh_ = blockIdx.x;  // sh_ = s·H + h
    const int D = (int)p.D;
    const float* part = p.part + ((b * p.S * p.H + sh_) * p.nsplit) * (D + 2);
    float M = -INFINITY;
    for (int i = 0; i < p.nsplit; i++) M = fmaxf(M, part[i * (D + 2) + D]);
    float L = 0.f;
    for (int i = 0; i < p.nsplit; i++) {
        float m = part[i * (D + 2) + D];
        if (m != -INFINITY) L += part[i * (D + 2) + D + 1] * __expf(m - M);
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.f;
        for (int i = 0; i < p.nsplit; i++) {
            float m = part[i * (D + 2) + D];
            if (m != -INFINITY) o += part[i * (D + 2) + d] * __expf(m - M);
        }
        st<DT>(p.out, (b * p.S * p.H + sh_) * D + d, o / L);
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
               {&pp.q_rot, qrot}, {&pp.present_k, present_k.buf}, {&pp.present_v, present_v.buf}, {&pp.err, Buf{kSlotErr, 0}}},
              "gqa_prepare");

    GqaAttnP ap{};
    ap.B = B; ap.S = S; ap.H = H; ap.KV = KV; ap.D = D; ap.T = T;
    ap.cap = pp.pres_cap;
    ap.window = d.window;
    ap.scale = DT == DT_F16 ? __half2float(__double2half(d.scale)) : (float)d.scale;
    if (bias) {
        ap.bias_sb = d.bias_b == 1 ? 0 : d.bias_h * S * T;
        ap.bias_sh = d.bias_h == 1 ? 0 : S * T;
    }
    // Split the visible key range so that the launch fills the machine.
    const long long G = H / KV;
    const int GT = G >= 4 ? 4 : (G >= 2 ? 2 : 1);
    ap.groups = (int)((G + GT - 1) / GT);
    long long span = (d.window >= 0 && d.window + 1 < T) ? d.window + 1 : T;
    long long ctas_per_split = B * KV * ap.groups * S;
    long long want = (148 * 4 + ctas_per_split - 1) / ctas_per_split;  // ≈ 4 CTAs per SM
    long long max_split = (span + 15) / 16;                           // ≥ 16 keys per CTA
    long long nsplit = std::max<long long>(1, std::min<long long>(want, max_split));
    nsplit = std::min<long long>(nsplit, 1024);
    ap.chunk = (span + nsplit - 1) / nsplit;
    ap.nsplit = (int)((span + ap.chunk - 1) / ap.chunk);
    Buf part = em.scratch((size_t)(B * S * H * ap.nsplit * (D + 2) * 4));
    if (KV * ap.groups * S > 65535 || B > 65535) throw std::runtime_error("fused GQA: grid dimension exceeds 65535");
    dim3 g((unsigned)ap.nsplit, (unsigned)(KV * ap.groups * S), (unsigned)B), blk(128);
    Buf qsrc = d.rot_half ? qrot : q.buf;
#define GO(DPL, GTT)                                                                                              \
    em.launch(gqa_partial<DT, DPL, GTT>, g, blk, 0, ap,                                                            \
              {{&ap.q, qsrc}, {&ap.pk, present_k.buf}, {&ap.pv, present_v.buf}, {&ap.seqlens, seqlens.buf},        \
               {&ap.bias, bias ? bias->buf : null}, {&ap.part, part}, {&ap.out, out.buf}},                         \
              "gqa_partial")
#define GO_D(GTT)                  \
    switch (D / 32) {              \
        case 1: GO(1, GTT); break; \
        case 2: GO(2, GTT); break; \
        case 4: GO(4, GTT); break; \
        default: GO(8, GTT); break; \
    }
    if (GT == 4) { GO_D(4) } else if (GT == 2) { GO_D(2) } else { GO_D(1) }
#undef GO_D
#undef GO
    em.launch(gqa_combine<DT>, dim3((unsigned)(S * H), (unsigned)B), dim3((unsigned)std::min<long long>(D, 256)), 0, ap,
              {{&ap.q, qsrc}, {&ap.pk, present_k.buf}, {&ap.pv, present_v.buf}, {&ap.seqlens, seqlens.buf},
               {&ap.bias, bias ? bias->buf : null}, {&ap.part, part}, {&ap.out, out.buf}},
              "gqa_combine");
}

void emit_gqa(Emitter& em, const GqaDesc& d, const TRef& q, const TRef& k, const TRef& v, const TRef& past_k,
              const TRef& past_v, const TRef& seqlens, const TRef* cos, const TRef* sin, const TRef* bias,
              const TRef& out, const TRef& present_k, const TRef& present_v) {
    if (q.dtype == DT_F16) emit_gqa_t<DT_F16>(em, d, q, k, v, past_k, past_v, seqlens, cos, sin, bias, out, present_k, present_v);
    else emit_gqa_t<DT_F32>(em, d, q, k, v, past_k, past_v, seqlens, cos, sin, bias, out, present_k, present_v);
}

}  // namespace oxk
