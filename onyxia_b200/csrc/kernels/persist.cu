// persist_step: a whole batch-1 decode step (the chain of int4 GEMVs with their
// norm / residual / GeGLU fusions and the attention of every layer) as ONE
// launch of one CTA per SM. See persist.hpp for the design; this file holds the
// kernel and the host code that lays out its operation table.
//
// Arithmetic follows the interpreter's primitive sequence exactly where it
// rounds (crates/onyxia-ir/src/decomp.rs:241-257 SimplifiedLayerNormalization,
// :185-213 Gelu, :357-613 GroupQueryAttention, :615-663 MatMulNBits;
// interp.rs:6-12 "round when a primitive stores"): every intermediate that the
// decompositions store as an f16 tensor is rounded to f16 here too, sums that
// the interpreter forms in f64 are formed in f64 (or exactly), and the int4
// inner products are summed in f32 per 128-column tile and in f64 across tiles.
#include <cstdlib>
#include <map>
#include <mutex>

#include "common.cuh"
#include "nbits_tile.cuh"
#include "persist.hpp"

namespace oxk {

namespace {

using namespace tile;

#ifndef OX_CW
#define OX_CW 16
#endif
constexpr int kCW = OX_CW;                 // consumer warps
constexpr int kCT = kCW * 32;              // consumer threads
constexpr int kPT = kCT + 32;              // + the producer warp
constexpr int kStTiles = 3;                // tile records per ring stage
constexpr int kTileB = kTileW + kTileS;    // 1152: records without zero points
constexpr int kStageB = kStTiles * kTileB; // 3456
constexpr int kPassTiles = 128;            // tiles a CTA multiplies between two reductions
constexpr int kMaxOps = 160;
constexpr int kMaxPrologueK = 2048;        // the norm / residual prologue keeps ≤ 8 f16 pairs per thread, in registers
constexpr long long kWaitP = 1000000000LL; // ≈ 0.5 s: how long any wait may last before the CTA gives up
// Arrival words (one per producing CTA, polled by a single warp before the data is read) cut the polling
// traffic but cost a second L2 round trip per link: measured 1.4 µs slower per link than polling the tagged
// data directly, while the traffic they save never was the bottleneck. Kept for experiments.
constexpr bool kUseArrivalWords = false;
constexpr unsigned kPollPauseNs = 40;      // pause between two reads of a word that has not arrived yet
#ifndef OX_POLL_SPIN
#define OX_POLL_SPIN 40
#endif
constexpr int kPollSpinCycles = OX_POLL_SPIN;  // > 0: pause by watching the clock for this many cycles instead of nanosleep
constexpr int kRowPad = 8;                 // f16 elements of padding per staged K row (bank spread for ldmatrix)
// Copies of every tagged vector that other CTAs wait for. All 148 CTAs poll the words of one small vector: with one
// copy, a cache line is read by 148 × 16 threads in a loop and both their loads and the producer's store queue
// in that line's L2 slice — a link of the chain took 2.5–5 µs in situ against ≈ 1 µs on an idle GPU.
#ifndef OX_REPS
#define OX_REPS 1
#endif
constexpr int kReps = OX_REPS;
constexpr int kRepMaxEntries = 8192;       // longer vectors (an lm_head's) are not copied: nothing in the run waits for them

enum : int {
    PF_SRC_TAGGED = 1,   // activations arrive as tagged pairs (else a plain f16 array)
    PF_SRC_RESID = 2,    // activations are the residual this CTA keeps in shared memory
    PF_W1 = 4,
    PF_RES = 8,
    PF_RES_SMEM = 16,    // the residual operand is the one kept in shared memory
    PF_W2 = 32,
    PF_SUM_OUT = 64,
    PF_GEGLU_TANH = 128,
    PF_GEGLU_ERF = 256,
    PF_Q_TAGGED = 512,   // attention: q / k / v arrive as tagged pairs
};

struct PGemvDev {
    const unsigned char* tiles;  // tile records, row tile by row tile
    const void* src;             // activations [K]: plain f16 or tagged pairs
    const __half* w1;
    const __half* w2;
    const __half* res;
    __half* sum_out;
    unsigned long long* xout;    // tagged results, entry = padded output row / 2
    unsigned* xflag;             // one arrival word per producing CTA of this operation (index: CTA counted from `rot`)
    const unsigned* src_flag;    // arrival words of the operation that produces `src` (tagged sources)
    __half* y[3];                // plain results per segment
    int seg_n[3];
    int seg_rt0[4];
    int k, k_tiles, row_tiles, sub, rot;  // sub: row tiles per unit (2: gate/up pairs)
    int src_nflag;
    float eps1, eps2;
    // Tagged vectors exist in several copies (entries apart by the stride): CTA c reads copy c mod reps, so the
    // CTAs that poll one cache line are 1 / reps of the grid.
    int src_reps, src_rstride, out_reps, out_rstride;
};

struct PAttnDev {
    const void* q;               // [H·D]: plain f16 or tagged pairs
    const void* k;               // [KV·D]
    const void* v;               // [KV·D]
    __half* cache_k;             // [KV][cap][D], appended in place
    __half* cache_v;
    const int* seqlens;
    const __half* cos;
    const __half* sin;
    __half* out;                 // plain [H·D]
    unsigned long long* xout;    // tagged [H·D / 2]
    unsigned long long* xsc;     // tagged scores of all visible keys: [KV][ceil(G/2)][n_cap]
    unsigned* xflag_sc;          // arrival words of the scores, one per attention CTA
    unsigned* xflag;             // arrival words of the results, one per attention CTA
    const unsigned* src_flag;    // arrival words of the operation that produces q, k and v (tagged sources)
    const long long* dyn_t;      // present length after this step
    int H, KV, D, half, window, cache_rows, n_cap, cap;
    float scale;
    int next_attn;               // index of the next attention operation of the run, or −1
    int src_nflag;
    int src_reps, src_rstride;   // copies of q / k / v (see PGemvDev)
    int out_reps, out_rstride;   // copies of the tagged output
    int pad;
};

struct POpDev {
    int kind, flags, node, pad;
    union {
        PGemvDev g;
        PAttnDev a;
    };
};

struct PersistP {
    ErrWord* err;
    const long long* epoch;
    int n_ops, ring_stages;
    // byte offsets into dynamic shared memory
    int off_bars, off_acts, off_resid, off_part, off_red, off_attn, off_params, params_bytes;
    // attention staging: rows of keys per CTA, padded key count of the longest visible span
    int att_chunk_pad, att_npad, first_attn, pad2;
    GeluConsts gc;
    POpDev ops[kMaxOps];
};

#ifndef OX_LD_MODE
#define OX_LD_MODE 0
#endif
__device__ __forceinline__ unsigned long long ld_tagged(const unsigned long long* p) {
    unsigned long long v;
#if OX_LD_MODE == 1
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
#elif OX_LD_MODE == 2
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
#elif OX_LD_MODE == 3
    asm volatile("ld.global.cv.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
#elif OX_LD_MODE == 4
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
#elif OX_LD_MODE == 5
    asm volatile("atom.relaxed.gpu.global.or.b64 %0, [%1], 0;" : "=l"(v) : "l"(p) : "memory");
#else
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
#endif
    return v;
}
__device__ __forceinline__ void st_tagged(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCT) : "memory"); }

// What every consumer thread carries through the operations.
struct Ctx {
    const PersistP* p;
    unsigned char* smem;
    volatile int* dead;   // set when a wait of this CTA expired
    unsigned epoch;
    int tid, lane, warp;
    int op_index;         // the operation being executed (tracing)
    ErrWord* err;
    int* trace_n;
};

// Developer tracing (-DOX_TRACE): thread 0 of every 20th CTA logs (id, operation, time) into its own
// slots after the error word (no atomics, one store per event).
#ifdef OX_TRACE
__device__ __forceinline__ void ptrace(const Ctx& c, int id) {
    if (c.tid == 0 && blockIdx.x % 20 == 0) {
        unsigned long long* t = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(c.err) + 256) + 1 + (blockIdx.x / 20) * 990;
        const int k = *c.trace_n;
        if (k < 989) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            t[k] = ((unsigned long long)id << 56) | ((unsigned long long)c.op_index << 40) | (now & 0xFFFFFFFFFFull);
            *c.trace_n = k + 1;
        }
    }
}
#else
#define ptrace(c, id) ((void)0)
#endif

// Completes the poll of one tagged word whose first read was `v`.
__device__ __forceinline__ unsigned long long poll_finish(const Ctx& c, const unsigned long long* src, unsigned long long v, int node) {
    if ((unsigned)(v >> 32) == c.epoch) return v;
    const long long t0 = clock64();
    for (;;) {
        // Thousands of threads poll a handful of cache lines: without a pause between the reads the
        // producer's store queues behind them in the L2 slice and every link of the chain slows down.
        if (kPollSpinCycles > 0) {
            const long long s0 = clock64();
            while (clock64() - s0 < kPollSpinCycles) {
            }
        } else {
            __nanosleep(kPollPauseNs);
        }
        v = ld_tagged(src);
        if ((unsigned)(v >> 32) == c.epoch) return v;
        if (*c.dead) return v;
        if (clock64() - t0 > kWaitP) {
            *c.dead = 1;
            report(c.p->err, ERR_WAIT_TIMEOUT, node, (long long)blockIdx.x, (long long)(v >> 32));
            return v;
        }
    }
}

__device__ __forceinline__ bool wait_bar(const Ctx& c, unsigned bar, unsigned parity, int node) {
    if (mbar_try(bar, parity)) return true;
    ptrace(c, 60);  // the data was not there yet
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try(bar, parity)) return true;
        if (*c.dead) return false;
        if (clock64() - t0 > kWaitP) {
            *c.dead = 1;
            report(c.p->err, ERR_WAIT_TIMEOUT, node, (long long)blockIdx.x, -1);
            return false;
        }
    }
}

__device__ __forceinline__ unsigned ld_flag(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_flag(unsigned* p, unsigned v) { asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

// Waits until the `n` producing CTAs of an operation have announced their results. Only one warp
// reads the arrival words (a few cache lines, with a pause between rounds); the other warps wait at
// the barrier, so thousands of idle threads do not flood the L2 with polls while producers still
// work. The words are hints — a producer writes its word right after its results, without a fence —
// and the results themselves are validated by their tags when they are read.
__device__ __forceinline__ void wait_flags(const Ctx& c, const unsigned* flags, int n, int node) {
    if (!kUseArrivalWords) return;
    if (c.warp == 0 && flags) {
        const long long t0 = clock64();
        for (;;) {
            bool ok = true;
            for (int i = c.lane; i < n; i += 32) ok = ok && ld_flag(flags + i) == c.epoch;
            if (__all_sync(0xffffffffu, ok)) break;
            if (*c.dead) break;
            if (clock64() - t0 > kWaitP) {
                if (c.lane == 0) {
                    *c.dead = 1;
                    report(c.p->err, ERR_WAIT_TIMEOUT, node, (long long)blockIdx.x, -2);
                }
                break;
            }
            __nanosleep(kPollPauseNs);
        }
    }
    consumer_sync();
}

// Position of activation element k in the B-fragment layout (one activation row): chunk (kt·4 + m)·4 + t
// holds elements kt·128 + t·32 + m·8 … + 8.
__device__ __forceinline__ int frag_index(int k) { return ((((k >> 7) * 4 + ((k >> 3) & 3)) * 4 + ((k >> 5) & 3)) << 3) + (k & 7); }

__device__ __forceinline__ unsigned pack_h2(float lo, float hi) {
    const __half2 h = __halves2half2(__float2half_rn(lo), __float2half_rn(hi));
    return hu(h);
}

// Sum of one double per consumer thread; every thread gets the total. `red` holds kCW doubles and
// must not be reused before another consumer_sync has passed.
__device__ __forceinline__ double consumer_sum(const Ctx& c, double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (c.lane == 0) red[c.warp] = v;
    consumer_sync();
    double tot = 0.0;
#pragma unroll
    for (int w = 0; w < kCW; w++) tot += red[w];
    return tot;
}

// U units over G CTAs: CTA `cp` (counted from the operation's rotation) takes ⌊U/G⌋ units, the first
// U mod G CTAs one more — so an operation with fewer units than CTAs occupies one contiguous block of them.
__host__ __device__ __forceinline__ void share_units(int cp, int U, int G, int* u0, int* n) {
    const int base = U / G, extra = U - base * G;
    *u0 = cp * base + (cp < extra ? cp : extra);
    *n = base + (cp < extra ? 1 : 0);
}

// The CTA's share of a GEMV: units of `sub` row tiles each.
__device__ __forceinline__ void gemv_share(const PGemvDev& g, int* rt_first, int* my_rts) {
    const int G = (int)gridDim.x, U = g.row_tiles / g.sub;
    int cp = (int)blockIdx.x - g.rot;
    if (cp < 0) cp += G;
    int u0, n;
    share_units(cp, U, G, &u0, &n);
    *rt_first = u0 * g.sub;
    *my_rts = n * g.sub;
}

// Tables over all f16 arguments of the three transcendental steps of the chain, each entry computed the way
// the interpreter does (f64 function, one rounding to f16): a lookup replaces ~100 f64 instructions that
// every thread would otherwise execute on the critical path of a phase.
//   g_exp_lut[|d| bits]  = round_f16(exp(−|d|))          (softmax: the argument is ≤ 0)
//   g_tanh_lut[x bits]   = round_f16(tanh(x))            (Gelu, tanh form)
//   g_erf_lut[z bits]    = round_f16(erf_A&S-7.1.26(z))  (Gelu, exact form; interp.rs:860-872)
__device__ __half g_exp_lut[32768];
__device__ __half g_tanh_lut[65536];
__device__ __half g_erf_lut[65536];

__global__ void persist_fill_luts() {
    for (int i = (int)global_tid(); i < 65536; i += (int)global_threads()) {
        const double x = (double)__half2float(__ushort_as_half((unsigned short)i));
        g_tanh_lut[i] = __double2half(tanh(x));
        double z = x;
        const double sign = z < 0.0 ? -1.0 : 1.0;
        z = fabs(z);
        const double tt = 1.0 / (1.0 + 0.3275911 * z);
        const double e = 1.0 - (((((1.061405429 * tt - 1.453152027) * tt) + 1.421413741) * tt - 0.284496736) * tt + 0.254829592) * tt * exp(-z * z);
        g_erf_lut[i] = __double2half(sign * e);
        if (i < 32768) g_exp_lut[i] = __double2half(exp(-x));
    }
}

// gelu(gate)·up with the rounding points of the Gelu decomposition followed by Mul (decomp.rs:185-213).
__device__ __forceinline__ float geglu_lut(const GeluConsts& p, int form, float x, float up) {
    float inner;
    if (form == 1) {
        const float x2 = r16(x * x), x3 = r16(x2 * x), cx3 = r16(p.c_coef * x3), sv = r16(x + cx3);
        inner = __half2float(g_tanh_lut[__half_as_ushort(__float2half_rn(p.c_k * sv))]);
    } else {
        inner = __half2float(g_erf_lut[__half_as_ushort(__float2half_rn(x * p.c_inv_sqrt2))]);
    }
    const float one_plus = r16(p.c_one + inner), hx = r16(p.c_half * x);
    return r16(hx * one_plus) * up;
}

// ── GEMV operation (consumer side) ──────────────────────────────────────
// The serial parts of an operation — the norm / residual prologue over a few hundred f16 pairs, the row
// sums, the epilogue — are bound by the latency of each warp's dependent instructions, not by issue slots:
// measured on the 1B decode step, the prologue on 4 / 8 / 16 warps gives 1032 / 933 / 902 µs per step, so it
// runs on all of them (more loads in flight while the tagged words are polled). Warps without rows skip the
// row sums and the epilogue.
#ifndef OX_PW
#define OX_PW OX_CW
#endif
constexpr int kPW = OX_PW;          // warps that run a prologue
constexpr int kPTh = kPW * 32;
constexpr int kEP = (kMaxPrologueK / 2 + kPTh - 1) / kPTh;  // f16 pairs per prologue thread

__device__ __forceinline__ void prologue_sync() { asm volatile("bar.sync 2, %0;" ::"n"(kPTh) : "memory"); }

// Sum of one double per prologue thread; every prologue thread gets the total.
__device__ __forceinline__ double prologue_sum(const Ctx& c, double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (c.lane == 0) red[c.warp] = v;
    prologue_sync();
    double tot = 0.0;
#pragma unroll
    for (int w = 0; w < kPW; w++) tot += red[w];
    return tot;
}

__device__ void run_gemv(const Ctx& c, const POpDev& op, unsigned& stage_q) {
    const PersistP& p = *c.p;
    const PGemvDev& g = op.g;
    const int flags = op.flags;
    int rt_first, my_rts;
    gemv_share(g, &rt_first, &my_rts);
    if (my_rts == 0 && !(flags & PF_SUM_OUT)) return;

    __half* acts = reinterpret_cast<__half*>(c.smem + p.off_acts);
    float* resid = reinterpret_cast<float*>(c.smem + p.off_resid);
    float* part = reinterpret_cast<float*>(c.smem + p.off_part);
    double* red = reinterpret_cast<double*>(c.smem + p.off_red);
    const int K = g.k, ne = K >> 1, kpad = g.k_tiles * 128;
    const int tid = c.tid;

    // ── activations → shared memory in fragment order ──
    if (flags & PF_SRC_TAGGED) wait_flags(c, g.src_flag, g.src_nflag, op.node);
    ptrace(c, 34);
    if (!(flags & (PF_W1 | PF_RES | PF_W2))) {
        for (int i = K + tid; i < kpad; i += kCT) acts[frag_index(i)] = __float2half(0.f);
        if (flags & PF_SRC_TAGGED) {
            const unsigned long long* src = reinterpret_cast<const unsigned long long*>(g.src) + (size_t)((int)blockIdx.x % g.src_reps) * g.src_rstride;
            for (int base = 0; base < ne; base += 4 * kCT) {
                unsigned long long v[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int idx = base + e * kCT + tid;
                    v[e] = ld_tagged(src + (idx < ne ? idx : ne - 1));
                }
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int idx = base + e * kCT + tid;
                    if (idx < ne) {
                        v[e] = poll_finish(c, src + idx, v[e], op.node);
                        *reinterpret_cast<unsigned*>(acts + frag_index(2 * idx)) = (unsigned)v[e];
                    }
                }
            }
        } else if (flags & PF_SRC_RESID) {
            for (int i = tid; i < ne; i += kCT)
                *reinterpret_cast<unsigned*>(acts + frag_index(2 * i)) = pack_h2(resid[2 * i], resid[2 * i + 1]);
        } else {
            const unsigned* src = reinterpret_cast<const unsigned*>(g.src);
            for (int i = tid; i < ne; i += kCT) *reinterpret_cast<unsigned*>(acts + frag_index(2 * i)) = src[i];
        }
    } else if (tid < kPTh) {
        // Prologue: [RMS norm ·w1] [+ residual → sum_out] [RMS norm ·w2], up to kEP pairs per thread in
        // registers. Constant operands are fetched first so that they are in flight while the activations are polled.
        for (int i = K + tid; i < kpad; i += kPTh) acts[frag_index(i)] = __float2half(0.f);
        const __half2 zero2 = __float2half2_rn(0.f);
        __half2 hw1[kEP], hw2[kEP], hres[kEP];
        unsigned long long v[kEP];
        const unsigned long long* tsrc = reinterpret_cast<const unsigned long long*>(g.src) +
                                         ((flags & PF_SRC_TAGGED) ? (size_t)((int)blockIdx.x % g.src_reps) * g.src_rstride : 0);
#pragma unroll
        for (int e = 0; e < kEP; e++) {
            const int idx = tid + e * kPTh;
            const int ic = idx < ne ? idx : 0;
            hw1[e] = (flags & PF_W1) ? reinterpret_cast<const __half2*>(g.w1)[ic] : zero2;
            hw2[e] = (flags & PF_W2) ? reinterpret_cast<const __half2*>(g.w2)[ic] : zero2;
            hres[e] = ((flags & PF_RES) && !(flags & PF_RES_SMEM)) ? reinterpret_cast<const __half2*>(g.res)[ic] : zero2;
            if (flags & PF_SRC_TAGGED) v[e] = ld_tagged(tsrc + ic);
            else if (flags & PF_SRC_RESID) v[e] = 0;
            else v[e] = reinterpret_cast<const unsigned*>(g.src)[ic];
        }
        float x[kEP][2];
#pragma unroll
        for (int e = 0; e < kEP; e++) {
            const int idx = tid + e * kPTh;
            const bool in = idx < ne;
            if (flags & PF_SRC_RESID) {
                x[e][0] = in ? resid[2 * idx] : 0.f;
                x[e][1] = in ? resid[2 * idx + 1] : 0.f;
            } else {
                if ((flags & PF_SRC_TAGGED) && in)
                    v[e] = poll_finish(c, tsrc + idx, v[e], op.node);
                const float2 f = __half22float2(uh((unsigned)v[e]));
                x[e][0] = in ? f.x : 0.f;
                x[e][1] = in ? f.y : 0.f;
            }
        }
        const double inv_k = 1.0 / (double)K;
        ptrace(c, 35);
#ifdef OX_TRACE
        if (c.lane == 0 && blockIdx.x == 60 && c.op_index >= 50 && c.op_index < 55) {  // when each warp of one CTA had its words
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(c.err) + 256)[1 + 8 * 990 + (c.op_index - 50) * 16 + c.warp] = now;
        }
#endif
        if (flags & PF_W1) {
            double ss = 0.0;
#pragma unroll
            for (int e = 0; e < kEP; e++) ss += (double)r16(x[e][0] * x[e][0]) + (double)r16(x[e][1] * x[e][1]);
            ptrace(c, 37);
            const double tot = prologue_sum(c, ss, red);
            ptrace(c, 38);
            const float msq = r16d(tot * inv_k), denom = r16(msq + g.eps1), inv = r16d(rsqrt((double)denom));
#pragma unroll
            for (int e = 0; e < kEP; e++) {
                const float2 w = __half22float2(hw1[e]);
                x[e][0] = r16(r16(x[e][0] * inv) * w.x);
                x[e][1] = r16(r16(x[e][1] * inv) * w.y);
            }
        }
        ptrace(c, 36);
        if (flags & PF_RES) {
#pragma unroll
            for (int e = 0; e < kEP; e++) {
                const int idx = tid + e * kPTh;
                if (idx >= ne) continue;
                float r0, r1;
                if (flags & PF_RES_SMEM) {
                    r0 = resid[2 * idx];
                    r1 = resid[2 * idx + 1];
                } else {
                    const float2 f = __half22float2(hres[e]);
                    r0 = f.x;
                    r1 = f.y;
                }
                x[e][0] = r16(x[e][0] + r0);
                x[e][1] = r16(x[e][1] + r1);
                if (flags & PF_SUM_OUT) {
                    resid[2 * idx] = x[e][0];
                    resid[2 * idx + 1] = x[e][1];
                    if (blockIdx.x == 0) reinterpret_cast<unsigned*>(g.sum_out)[idx] = pack_h2(x[e][0], x[e][1]);
                }
            }
        }
        if (flags & PF_W2) {
            double ss = 0.0;
#pragma unroll
            for (int e = 0; e < kEP; e++) ss += (double)r16(x[e][0] * x[e][0]) + (double)r16(x[e][1] * x[e][1]);
            const double tot = prologue_sum(c, ss, red + kPW);
            const float msq = r16d(tot * inv_k), denom = r16(msq + g.eps2), inv = r16d(rsqrt((double)denom));
#pragma unroll
            for (int e = 0; e < kEP; e++) {
                const float2 w = __half22float2(hw2[e]);
                x[e][0] = r16(x[e][0] * inv) * w.x;  // the product is rounded when it is stored below
                x[e][1] = r16(x[e][1] * inv) * w.y;
            }
        }
#pragma unroll
        for (int e = 0; e < kEP; e++) {
            const int idx = tid + e * kPTh;
            if (idx < ne) *reinterpret_cast<unsigned*>(acts + frag_index(2 * idx)) = pack_h2(x[e][0], x[e][1]);
        }
    }
    consumer_sync();
    ptrace(c, 31);
#ifdef OX_TRACE
    unsigned t_acts = 0;
    if (c.tid == 0 && c.op_index == 52) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        t_acts = (unsigned)now;
    }
#endif
    if (my_rts == 0) return;

    // ── tiles ──
    const int kt_n = g.k_tiles, spr = (kt_n + kStTiles - 1) / kStTiles;
    int rt_per_pass = (kPassTiles / kt_n) / g.sub * g.sub;
    if (rt_per_pass < g.sub) rt_per_pass = g.sub;
    const int R = p.ring_stages;
    const unsigned bars = smem_addr(c.smem + p.off_bars);
    const int lane = c.lane, gq = lane >> 2, t = lane & 3;
    const uint4* ap0 = reinterpret_cast<const uint4*>(acts) + t;  // the one activation row sits at g = 0
    const unsigned long long tag = (unsigned long long)c.epoch << 32;
    const int geglu = (flags & PF_GEGLU_TANH) ? 1 : ((flags & PF_GEGLU_ERF) ? 2 : 0);
    const unsigned slot_q = stage_q % (unsigned)R, par_q = (stage_q / (unsigned)R) & 1u;  // ring position of this operation's first stage

    for (int rt0 = 0; rt0 < my_rts; rt0 += rt_per_pass) {
        const int rts = my_rts - rt0 < rt_per_pass ? my_rts - rt0 : rt_per_pass;
        const int ntile = rts * kt_n;
        // A warp takes tiles warp, warp + kCW, …, two at a time while there are two (their independent
        // accumulator chains overlap). Row tile, k tile, ring slot and phase of the warp's next tile are
        // carried along incrementally: no division in the loop.
        struct Cursor {
            int r, kt, sg;      // row tile within the pass, k tile, stage within the row tile (kt / kStTiles)
            unsigned slot, par; // ring slot of that stage and the phase parity to wait for
        };
        auto seek = [&](int j) {
            Cursor q;
            q.r = j / kt_n;
            q.kt = j - q.r * kt_n;
            q.sg = q.kt / kStTiles;
            const unsigned off = (unsigned)((rt0 + q.r) * spr + q.sg);
            const unsigned s0 = slot_q + off % (unsigned)R;
            q.slot = s0 >= (unsigned)R ? s0 - (unsigned)R : s0;
            q.par = (par_q + off / (unsigned)R + (s0 >= (unsigned)R ? 1u : 0u)) & 1u;
            return q;
        };
        auto advance = [&](Cursor& q, int by) {  // by < kt_n + kStTiles is not required: loops handle any step
            q.kt += by;
            while (q.kt >= kt_n) {
                q.kt -= kt_n;
                q.r++;
                // to the first stage of the next row tile
                const unsigned step = (unsigned)(spr - q.sg);
                q.sg = 0;
                q.slot += step;
                while (q.slot >= (unsigned)R) {
                    q.slot -= (unsigned)R;
                    q.par ^= 1u;
                }
            }
            const int sg = q.kt / kStTiles;
            const unsigned step = (unsigned)(sg - q.sg);
            q.sg = sg;
            q.slot += step;
            while (q.slot >= (unsigned)R) {
                q.slot -= (unsigned)R;
                q.par ^= 1u;
            }
        };
        auto record = [&](const Cursor& q) {
            wait_bar(c, bars + q.slot * 8, q.par, op.node);
            return c.smem + (size_t)q.slot * kStageB + (q.kt - q.sg * kStTiles) * kTileB;
        };
        auto finish = [&](int j, const Cursor& q, const float (&ca)[4], const float (&cb)[4]) {
            if (t == 0) {  // column 0 of the fragment is the activation row
                part[j * 16 + gq] = ca[0] + cb[0];
                part[j * 16 + gq + 8] = ca[2] + cb[2];
            }
            __syncwarp();
            if (lane == 0) {
                const int first = q.sg * kStTiles;
                const int cnt = kt_n - first < kStTiles ? kt_n - first : kStTiles;
                // the warp that takes the last tile of a partly filled stage also arrives for the missing tiles
                mbar_arrive(bars + (unsigned)(R + (int)q.slot) * 8, q.kt - first == cnt - 1 ? 1u + (unsigned)(kStTiles - cnt) : 1u);
            }
        };
        int j = c.warp;
        if (j < ntile) {
            Cursor q1 = seek(j);
#ifdef OX_NO_PAIR
            for (; j < ntile; j += kCW) {
                const unsigned char* rec = record(q1);
                float ca[4] = {0.f, 0.f, 0.f, 0.f}, cb[4] = {0.f, 0.f, 0.f, 0.f};
                tile_mma_zp8(rec, ap0 + q1.kt * 16, 4, lane, ca, cb);
                finish(j, q1, ca, cb);
                if (j + kCW < ntile) advance(q1, kCW);
            }
#endif
            for (; j + kCW < ntile; j += 2 * kCW) {
                Cursor q2 = q1;
                advance(q2, kCW);
                const unsigned char* rec1 = record(q1);
                const unsigned char* rec2 = record(q2);
                float ca[4] = {0.f, 0.f, 0.f, 0.f}, cb[4] = {0.f, 0.f, 0.f, 0.f}, cc[4] = {0.f, 0.f, 0.f, 0.f}, cd[4] = {0.f, 0.f, 0.f, 0.f};
                tile_mma2_zp8(rec1, ap0 + q1.kt * 16, rec2, ap0 + q2.kt * 16, 4, lane, ca, cb, cc, cd);
                finish(j, q1, ca, cb);
                finish(j + kCW, q2, cc, cd);
                q1 = q2;
                if (j + 2 * kCW < ntile) advance(q1, kCW);
            }
            if (j < ntile) {
                const unsigned char* rec = record(q1);
                float ca[4] = {0.f, 0.f, 0.f, 0.f}, cb[4] = {0.f, 0.f, 0.f, 0.f};
                tile_mma_zp8(rec, ap0 + q1.kt * 16, 4, lane, ca, cb);
                finish(j, q1, ca, cb);
            }
        }
        consumer_sync();
        ptrace(c, 32);
        // Row sums over the k tiles in f64, rounded once; the result replaces the row's first partial. Four
        // threads share a row: each adds every fourth tile, two exchanges combine them. Only the warps that
        // have rows take part.
        const int nrow = rts * 16;
        for (int base = 0; base < nrow * 4; base += kCT) {
            if (base + (c.warp << 5) >= nrow * 4) break;  // warp-uniform: this warp has no rows (left)
            const int i = (base + tid) >> 2, q4 = tid & 3;
            const bool in = i < nrow;
            float y = 0.f;
            const int r = i >> 4, row = i & 15;
            double sum = 0.0;
            if (in) {
                const float* pr = part + (r * kt_n) * 16 + row;
                for (int kt = q4; kt < kt_n; kt += 4) sum += (double)pr[kt * 16];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if (in) {
                y = r16d(sum);
                if (q4 == 0) part[(r * kt_n) * 16 + row] = y;
            }
            if (!geglu) {
                const float yo = __shfl_down_sync(0xffffffffu, y, 4);
                if (in && q4 == 0) {
                    const int rtg = rt_first + rt0 + r;
                    int seg = 0;
                    if (rtg >= g.seg_rt0[1]) seg = 1;
                    if (rtg >= g.seg_rt0[2]) seg = 2;
                    const int rowg = (rtg - g.seg_rt0[seg]) * 16 + row;
                    if (rowg < g.seg_n[seg]) g.y[seg][rowg] = __float2half_rn(y);
                    if (!(row & 1)) {
                        const unsigned long long word = tag | pack_h2(y, yo);
                        for (int r = 0; r < g.out_reps; r++) st_tagged(g.xout + (size_t)r * g.out_rstride + ((rtg * 16 + row) >> 1), word);
                    }
                }
            }
        }
        if (geglu) {
            consumer_sync();
            const int npair = (rts >> 1) * 16;
            for (int base = 0; base < npair; base += kCT) {
                if (base + (c.warp << 5) >= npair) break;  // warp-uniform
                const int i = base + tid;
                const bool in = i < npair;
                const int pj = i >> 4, row = i & 15;
                float h = 0.f;
                if (in) {
                    const float gate = part[((2 * pj) * kt_n) * 16 + row], up = part[((2 * pj + 1) * kt_n) * 16 + row];
                    h = r16(geglu_lut(p.gc, geglu, gate, up));
                }
                const float ho = __shfl_down_sync(0xffffffffu, h, 1);
                if (in) {
                    const int rowg = (((rt_first + rt0) >> 1) + pj) * 16 + row;
                    if (rowg < g.seg_n[0]) g.y[0][rowg] = __float2half_rn(h);
                    if (!(row & 1)) {
                        const unsigned long long word = tag | pack_h2(h, ho);
                        for (int r = 0; r < g.out_reps; r++) st_tagged(g.xout + (size_t)r * g.out_rstride + (rowg >> 1), word);
                    }
                }
            }
        }
        if (rt0 + rt_per_pass < my_rts) consumer_sync();  // the partial sums are rewritten by the next pass
    }
    stage_q += (unsigned)(my_rts * spr);
    if (tid == 0) {
        int cp = (int)blockIdx.x - g.rot;
        if (cp < 0) cp += (int)gridDim.x;
        st_flag(g.xflag + cp, c.epoch);
    }
    ptrace(c, 33);
#ifdef OX_TRACE
    if (c.tid == 0 && c.op_index == 52) {  // every producer of one operation: when it had its inputs, when it was done
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(c.err) + 256)[1 + 8 * 990 + 100 + blockIdx.x] = (now << 32) | t_acts;
    }
#endif
}

// ── attention operation ─────────────────────────────────────────────────
struct AttGeo {
    long long qpos, lo, T;
    int n, chunk, my0, my_n, kvh, dt;
    bool active, has_new, owns_new;
};

__device__ __forceinline__ AttGeo att_geometry(const PAttnDev& a) {
    AttGeo ge;
    const int NC = a.D >> 3;  // CTAs per KV head: one per 8 head-dim columns
    const int cta = (int)blockIdx.x;
    ge.active = cta < a.KV * NC;
    ge.kvh = cta / NC;
    ge.dt = cta - ge.kvh * NC;
    ge.T = *a.dyn_t;
    const long long tot = (long long)a.seqlens[0] + 1;
    ge.qpos = tot - 1 > 0 ? tot - 1 : 0;
    const long long hi = ge.qpos < ge.T - 1 ? ge.qpos : ge.T - 1;
    ge.lo = (a.window >= 0 && ge.qpos - a.window > 0) ? ge.qpos - a.window : 0;
    long long n = hi >= ge.lo ? hi - ge.lo + 1 : 0;
    if (n > a.n_cap) n = a.n_cap;  // cannot happen for a launch sized by the host; never index past the staging rows
    ge.n = (int)n;
    ge.chunk = (ge.n + NC - 1) / NC;
    ge.my0 = ge.dt * ge.chunk;
    int my_n = ge.n - ge.my0;
    ge.my_n = my_n < 0 ? 0 : (my_n > ge.chunk ? ge.chunk : my_n);
    ge.has_new = ge.qpos <= ge.T - 1 && ge.n > 0;  // the newest key (this step's) is the last visible one
    ge.owns_new = ge.has_new && (ge.n - 1) / ge.chunk == ge.dt;
    return ge;
}

struct AttSmem {
    __half* raw;    // [(G + 2)][D] q heads, new k, new v as they arrived
    __half* q_h;    // [8][D + pad] rotated q, zero rows beyond the group
    __half* Ks;     // [chunk_pad][D + pad] this CTA's keys
    __half* Vs;     // [npad][8] every visible key, this CTA's 8 columns
    __half* p_s;    // [8][npad + 8] scores → exponentials → probabilities, zero rows beyond the group
    float* pv;      // [kCW][8][8]
    int* imax;                  // [8] row maxima (order-preserving integer image of the float)
    unsigned long long* isum;   // [8] row sums of the exponentials in units of 2⁻²⁴
};

__device__ __forceinline__ AttSmem att_smem(const PersistP& p, unsigned char* smem, int D) {
    AttSmem s;
    unsigned char* b = smem + p.off_attn;
    const int RS = D + kRowPad, PS = p.att_npad + 8;
    s.raw = reinterpret_cast<__half*>(b);
    b += 10 * D * 2;
    s.q_h = reinterpret_cast<__half*>(b);
    b += 8 * RS * 2;
    s.Ks = reinterpret_cast<__half*>(b);
    b += (size_t)p.att_chunk_pad * RS * 2;
    s.Vs = reinterpret_cast<__half*>(b);
    b += (size_t)p.att_npad * 16;
    s.p_s = reinterpret_cast<__half*>(b);
    b += (size_t)8 * PS * 2;
    s.pv = reinterpret_cast<float*>(b);
    b += kCW * 64 * 4;
    s.isum = reinterpret_cast<unsigned long long*>(b);
    b += 8 * 8;
    s.imax = reinterpret_cast<int*>(b);
    return s;
}

// Starts the copies of the old cache rows an attention operation will read (rows no kernel of this
// step writes) and clears the padding of its staging arrays. Called well before the operation runs.
__device__ void att_prefetch(const Ctx& c, const POpDev& op, bool first) {
    const PersistP& p = *c.p;
    const PAttnDev& a = op.a;
    const AttGeo ge = att_geometry(a);
    if (ge.active) {
        const int D = a.D, RS = D + kRowPad, PS = p.att_npad + 8, cpr = D >> 3;
        const AttSmem s = att_smem(p, c.smem, D);
        if (first) {  // rows of the probability array beyond the group's heads stay zero for the whole launch
            const int G = a.H / a.KV;
            for (int i = G * PS + c.tid; i < 8 * PS; i += kCT) s.p_s[i] = __float2half(0.f);
        }
        const __half* ck = a.cache_k + (size_t)ge.kvh * a.cap * D;
        const __half* cv = a.cache_v + (size_t)ge.kvh * a.cap * D;
        for (int i = c.tid; i < ge.my_n * cpr; i += kCT) {
            const int r = i / cpr, col = i - r * cpr;
            const long long pos = ge.lo + ge.my0 + r;
            if (ge.has_new && pos == ge.qpos) continue;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(s.Ks + r * RS + col * 8)), "l"(ck + pos * D + col * 8) : "memory");
        }
        for (int i = c.tid; i < ge.n; i += kCT) {
            const long long pos = ge.lo + i;
            if (ge.has_new && pos == ge.qpos) continue;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(s.Vs + i * 8)), "l"(cv + pos * D + ge.dt * 8) : "memory");
        }
        // the last, partly filled tile of 16 keys: V rows and probabilities beyond the keys are zero;
        // the softmax statistics start from their neutral values
        const int pad = ((ge.n + 15) & ~15) - ge.n;
        const uint4 z = make_uint4(0, 0, 0, 0);
        if (c.tid < pad) reinterpret_cast<uint4*>(s.Vs)[ge.n + c.tid] = z;
        if (c.tid < 8 * pad) s.p_s[(c.tid / pad) * PS + ge.n + c.tid % pad] = __float2half(0.f);
        if (c.tid < 8) {
            s.imax[c.tid] = (int)0x80000000;
            s.isum[c.tid] = 0ull;
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

__device__ __forceinline__ void ldsm_x2_t(unsigned (&r)[2], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// One new token against the cache (decomp.rs:357-613 for S = 1): rotary on q and the new k, append,
// scores of the visible keys, softmax, P·V. CTA (kv head, dt) computes the scores of its slice of the
// keys, publishes them, reads everybody's scores, forms every probability itself and multiplies them
// with its 8 columns of V — so each CTA owns 8 finished output columns and nothing has to be reduced
// across CTAs.
template <int D> __device__ void run_attn(const Ctx& c, const POpDev& op) {
    const PersistP& p = *c.p;
    const PAttnDev& a = op.a;
    const AttGeo ge = att_geometry(a);
    if (!ge.active) return;
    constexpr int RS = D + kRowPad;
    const int PS = p.att_npad + 8;
    const AttSmem s = att_smem(p, c.smem, D);
    const int tid = c.tid, lane = c.lane, warp = c.warp, gq = lane >> 2, t = lane & 3;
    const int G = a.H / a.KV, h0 = ge.kvh * G, HP = (G + 1) >> 1;
    const unsigned long long tag = (unsigned long long)c.epoch << 32;
    __half* ck = a.cache_k + (size_t)ge.kvh * a.cap * D;
    __half* cv = a.cache_v + (size_t)ge.kvh * a.cap * D;

    long long rope_row = ge.qpos;
    if (a.half && rope_row >= a.cache_rows) {
        if (tid == 0 && blockIdx.x == 0) report(p.err, ERR_GATHER_OOB, op.node, rope_row, a.cache_rows);
        rope_row = 0;
    }
    // rotary factors of element tid (loaded before the polls; constants)
    float rc = 1.f, rs = 0.f;
    const bool rot = tid < 2 * a.half, first = tid < a.half;
    if (tid < D && rot) {
        const int j = first ? tid : tid - a.half;
        rc = __half2float(a.cos[rope_row * a.half + j]);
        rs = __half2float(a.sin[rope_row * a.half + j]);
    }

    // 1. q heads of the group, the new k and v rows → raw[(G + 2)][D]
    if (op.flags & PF_Q_TAGGED) wait_flags(c, a.src_flag, a.src_nflag, op.node);
    {
        const int nq = G * (D / 2), nk = D / 2;
        const int total = nq + 2 * nk;
        for (int base = 0; base < total; base += 2 * kCT) {
            unsigned long long v[2];
            const void* src[2];
            int dst[2];
            bool in[2];
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int i = base + e * kCT + tid;
                in[e] = i < total;
                const int ic = in[e] ? i : 0;
                int elem;  // pair index within its source array
                const void* b;
                if (ic < nq) {
                    b = a.q;
                    elem = h0 * (D / 2) + ic;
                    dst[e] = ic;
                } else if (ic < nq + nk) {
                    b = a.k;
                    elem = ge.kvh * (D / 2) + ic - nq;
                    dst[e] = ic;
                } else {
                    b = a.v;
                    elem = ge.kvh * (D / 2) + ic - nq - nk;
                    dst[e] = ic;
                }
                if (op.flags & PF_Q_TAGGED) {
                    src[e] = reinterpret_cast<const unsigned long long*>(b) + (size_t)((int)blockIdx.x % a.src_reps) * a.src_rstride + elem;
                    v[e] = ld_tagged(reinterpret_cast<const unsigned long long*>(src[e]));
                } else {
                    src[e] = nullptr;
                    v[e] = reinterpret_cast<const unsigned*>(b)[elem];
                }
            }
#pragma unroll
            for (int e = 0; e < 2; e++) {
                if (!in[e]) continue;
                if (op.flags & PF_Q_TAGGED) v[e] = poll_finish(c, reinterpret_cast<const unsigned long long*>(src[e]), v[e], op.node);
                reinterpret_cast<unsigned*>(s.raw)[dst[e]] = (unsigned)v[e];
            }
        }
    }
    consumer_sync();
    ptrace(c, 41);

    // 2. rotary (decomp.rs:259-355: x1·cos − x2·sin | x2·cos + x1·sin, products rounded), append
    if (tid < D) {
        const int e = tid, e2 = first ? e + a.half : e - a.half;
        auto turn = [&](const __half* row) {
            const float own = __half2float(row[e]);
            if (!rot) return own;
            const float partner = __half2float(row[e2]);
            return first ? r16(own * rc) - r16(partner * rs) : r16(own * rc) + r16(partner * rs);
        };
#pragma unroll
        for (int hh = 0; hh < 8; hh++) s.q_h[hh * RS + e] = __float2half_rn(hh < G ? turn(s.raw + hh * D) : 0.f);
        if (ge.owns_new) {
            const __half nk = __float2half_rn(turn(s.raw + G * D));
            const __half nv = s.raw[(G + 1) * D + e];
            s.Ks[(ge.n - 1 - ge.my0) * RS + e] = nk;
            ck[ge.qpos * D + e] = nk;
            cv[ge.qpos * D + e] = nv;
            for (long long z = ge.qpos + 1; z < ge.T; z++) {  // a row shorter than the present length: clear the rest
                ck[z * D + e] = __float2half(0.f);
                cv[z * D + e] = __float2half(0.f);
            }
        }
        if (ge.has_new && e < 8) s.Vs[(ge.n - 1) * 8 + e] = s.raw[(G + 1) * D + ge.dt * 8 + e];
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    consumer_sync();
    ptrace(c, 42);

    // 3. scores of this CTA's keys: one warp per 16 keys; K rows as A, rotated q as B
    {
        const int n_kt = (ge.my_n + 15) >> 4;
        for (int kt = warp; kt < n_kt; kt += kCW) {
            float cacc[4] = {0.f, 0.f, 0.f, 0.f};
            const int m = lane >> 3, r = lane & 7;
            const unsigned a_addr = smem_addr(s.Ks + (kt * 16 + (m & 1) * 8 + r) * RS + (m >> 1) * 8);
#pragma unroll
            for (int j = 0; j < D / 16; j++) {
                unsigned af[4];
                ldsm_x4(af, a_addr + j * 32);
                const unsigned b0 = *reinterpret_cast<const unsigned*>(s.q_h + gq * RS + 16 * j + 2 * t);
                const unsigned b1 = *reinterpret_cast<const unsigned*>(s.q_h + gq * RS + 16 * j + 2 * t + 8);
                mma16816(cacc, af[0], af[1], af[2], af[3], b0, b1);
            }
            // c0: (key g, head 2t)  c1: (key g, head 2t+1)  c2, c3: key g + 8
            if (2 * t < G) {
#pragma unroll
                for (int hf = 0; hf < 2; hf++) {
                    const int key = kt * 16 + gq + hf * 8;
                    if (key < ge.my_n) {
                        const float s0 = r16(r16(cacc[2 * hf]) * a.scale), s1 = r16(r16(cacc[2 * hf + 1]) * a.scale);
                        st_tagged(a.xsc + ((size_t)(ge.kvh * HP + t) * a.n_cap + ge.my0 + key), tag | pack_h2(s0, s1));
                    }
                }
            }
        }
    }

    if (tid == 0) st_flag(a.xflag_sc + blockIdx.x, c.epoch);
    ptrace(c, 43);
    wait_flags(c, a.xflag_sc + ge.kvh * (D / 8), D / 8, op.node);
    // 4. everybody's scores → p_s rows (head pair hp → rows 2hp, 2hp + 1)
    {
        const int total = HP * ge.n;
        const unsigned long long* src = a.xsc + (size_t)ge.kvh * HP * a.n_cap;
        for (int base = 0; base < total; base += 2 * kCT) {
            unsigned long long v[2];
            int hp[2], key[2];
            bool in[2];
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int i = base + e * kCT + tid;
                in[e] = i < total;
                const int ic = in[e] ? i : 0;
                hp[e] = ic / ge.n;
                key[e] = ic - hp[e] * ge.n;
                v[e] = ld_tagged(src + (size_t)hp[e] * a.n_cap + key[e]);
            }
#pragma unroll
            for (int e = 0; e < 2; e++) {
                if (!in[e]) continue;
                v[e] = poll_finish(c, src + (size_t)hp[e] * a.n_cap + key[e], v[e], op.node);
                const __half2 h2 = uh((unsigned)v[e]);
                s.p_s[(2 * hp[e]) * PS + key[e]] = __low2half(h2);
                if (2 * hp[e] + 1 < G) s.p_s[(2 * hp[e] + 1) * PS + key[e]] = __high2half(h2);
            }
        }
    }
    consumer_sync();
    ptrace(c, 44);

    // 5. softmax over the visible keys (decomp.rs:174-183): max, exp of the rounded difference, the
    // exact sum of the rounded exponentials, rounded quotient. A thread works on one head (lane mod G)
    // and every (kCT / G)-th key; the lanes of a warp that share a head reduce among themselves.
    // Exponentials are multiples of 2⁻²⁴ not above 1: summed exactly as integers, which is what the
    // interpreter's f64 sum gives.
    {
        const int hh = lane & (G - 1);  // G is a power of two
        const unsigned peers = (0x01010101u * ((G == 1) ? 0xFFu : (G == 2) ? 0x55u : (G == 4) ? 0x11u : 0x01u)) << hh;
        const int k0 = tid / G, kstep = kCT / G;
        __half* row = s.p_s + hh * PS;
        float m = -INFINITY;
        for (int i = k0; i < ge.n; i += kstep) m = fmaxf(m, __half2float(row[i]));
        {
            // order-preserving map of the float bits to a signed integer
            const int bits = __float_as_int(m), key = bits >= 0 ? bits : bits ^ 0x7FFFFFFF;
            const int wmax = __reduce_max_sync(peers, key);
            if (lane < G) atomicMax(s.imax + hh, wmax);
        }
        consumer_sync();
        ptrace(c, 51);
        const int key = s.imax[hh];
        const __half gmax = __float2half_rn(__int_as_float(key >= 0 ? key : key ^ 0x7FFFFFFF));  // an f16 value: exact
        unsigned acc = 0u;  // a thread meets at most ⌈n·G / kCT⌉ ≤ 64 keys: below 2³⁰
        for (int i = k0; i < ge.n; i += kstep) {
            const __half d = __hsub(row[i], gmax);  // one rounding of the exact difference, as in the f64 domain
            const __half e = g_exp_lut[__half_as_ushort(d) & 0x7FFF];
            row[i] = e;
            acc += (unsigned)(__half2float(e) * 16777216.f);
        }
        {
            const unsigned lo = __reduce_add_sync(peers, acc & 0xFFFFu), hi = __reduce_add_sync(peers, acc >> 16);
            if (lane < G) atomicAdd(s.isum + hh, ((unsigned long long)hi << 16) + lo);
        }
        consumer_sync();
        ptrace(c, 52);
        const unsigned long long tot = s.isum[hh];
        const double totd = (double)(unsigned)(tot >> 32) * 4294967296.0 + (double)(unsigned)tot;
        const float total = r16d(totd * 5.9604644775390625e-08);
        // e and Σ are f16 values: their f32 quotient rounds to the same f16 as the exact one
        for (int i = k0; i < ge.n; i += kstep) row[i] = __float2half_rn(__half2float(row[i]) / total);
    }
    consumer_sync();
    ptrace(c, 45);

    // 6. P·V for this CTA's 8 columns: probabilities as A (heads × keys), V rows as B (keys × 8)
    {
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        const int n_kt = (ge.n + 15) >> 4;
        for (int kt = warp; kt < n_kt; kt += kCW) {
            const unsigned a0 = *reinterpret_cast<const unsigned*>(s.p_s + gq * PS + kt * 16 + 2 * t);
            const unsigned a2 = *reinterpret_cast<const unsigned*>(s.p_s + gq * PS + kt * 16 + 2 * t + 8);
            unsigned bm[2];
            ldsm_x2_t(bm, smem_addr(s.Vs + (kt * 16 + (lane & 15)) * 8));
            mma16816(o, a0, 0u, a2, 0u, bm[0], bm[1]);
        }
        // c0: (head g, column 2t)  c1: (head g, column 2t + 1); rows 8-15 are padding
        s.pv[(warp * 8 + gq) * 8 + 2 * t] = o[0];
        s.pv[(warp * 8 + gq) * 8 + 2 * t + 1] = o[1];
    }
    consumer_sync();
    if (warp == 0) {
        const int hh = lane >> 3, col = lane & 7;  // 4 heads per round
        for (int hb = 0; hb < G; hb += 4) {
            const int head = hb + hh;
            float v = 0.f;
            if (head < G)
                for (int w = 0; w < kCW; w++) v += s.pv[(w * 8 + head) * 8 + col];
            v = r16(v);
            const float vo = __shfl_down_sync(0xffffffffu, v, 1);
            if (head < G) {
                const int idx = (h0 + head) * D + ge.dt * 8 + col;
                a.out[idx] = __float2half_rn(v);
                if (!(col & 1)) {
                    const unsigned long long word = tag | pack_h2(v, vo);
                    for (int r = 0; r < a.out_reps; r++) st_tagged(a.xout + (size_t)r * a.out_rstride + (idx >> 1), word);
                }
            }
        }
    }
    if (tid == 0) st_flag(a.xflag + blockIdx.x, c.epoch);
    consumer_sync();  // the staging arrays are free again
    ptrace(c, 46);
}

__global__ void __launch_bounds__(kPT, 1) persist_step(const __grid_constant__ PersistP pk) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int dead_flag;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // The operation table moves to shared memory first: read through a pointer, kernel parameters are
    // ordinary global loads (an L2 round trip each with no L1 left beside 220 KB of shared memory), and
    // the operations consult their descriptors all the time.
    {
        const unsigned* src = reinterpret_cast<const unsigned*>(&pk);
        unsigned* dst = reinterpret_cast<unsigned*>(smem + pk.off_params);
        for (int i = tid; i < pk.params_bytes / 4; i += kPT) dst[i] = src[i];
    }
    const PersistP& p = *reinterpret_cast<const PersistP*>(smem + pk.off_params);
    const int R = pk.ring_stages;
    const unsigned bars = smem_addr(smem + pk.off_bars);
    if (tid == 0) {
        dead_flag = 0;
        for (int s = 0; s < R; s++) {
            mbar_init(bars + s * 8, 1);               // full: one arrival (the producer's expect) + the bytes
            mbar_init(bars + (R + s) * 8, kStTiles);  // empty: one arrival per tile of the stage
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    Ctx c;
    c.p = &p;
    c.smem = smem;
    c.dead = &dead_flag;
    c.epoch = (unsigned)*p.epoch;
    c.tid = tid;
    c.lane = lane;
    c.warp = warp;
    c.op_index = 0;
    c.err = pk.err;
    __shared__ int trace_count;
    if (tid == 0) trace_count = 0;
    c.trace_n = &trace_count;

    if (warp == kCW) {
        // ── producer: this CTA's tile records of every GEMV, in execution order ──
        // Eight lanes issue eight consecutive stages at a time (a lane waits for its own slot to be free, arms the
        // slot's barrier and starts its copy): one lane alone spends ≈ 250 ns per stage on the slot arithmetic and
        // the barrier, which bounds an SM at 14 GB/s — enough for the layers, whose weights are resident long
        // before they are used, but not for the 170 MB of an lm_head. More lanes per round would shorten the
        // distance the ring runs ahead (a round waits for its last slot).
        constexpr int kIssue = 8;
        unsigned q = 0;
        bool ok = true;
        for (int i = 0; i < p.n_ops && ok; i++) {
            if (p.ops[i].kind != POP_GEMV) continue;
            const PGemvDev& g = p.ops[i].g;
            int rt_first, my_rts;
            gemv_share(g, &rt_first, &my_rts);
            const int kt_n = g.k_tiles, spr = (kt_n + kStTiles - 1) / kStTiles;
            const int n_st = my_rts * spr;
            const unsigned char* base = g.tiles + ((size_t)rt_first * kt_n) * kTileB;
            // The norm weights of the operation's prologue are read once per step: from HBM (≈ 2 µs) unless somebody
            // asked for them first. The producer is a layer or so ahead of the consumers: its idle lanes pull them into L2.
            if (lane >= kIssue) {
                const int lines = (g.k * 2 + 127) >> 7;
                for (int ln = lane - kIssue; ln < 2 * lines; ln += 32 - kIssue) {
                    const __half* w = ln < lines ? g.w1 : g.w2;
                    if (w) asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(w) + (size_t)(ln < lines ? ln : ln - lines) * 128));
                }
            }
            for (int i0 = 0; i0 < n_st && ok; i0 += kIssue) {
                const int idx = i0 + lane;
                bool mine_ok = true;
                if (lane < kIssue && idx < n_st) {
                    const int r = idx / spr, s = idx - r * spr;
                    const int cnt = kt_n - s * kStTiles < kStTiles ? kt_n - s * kStTiles : kStTiles;
                    const unsigned qq = q + (unsigned)idx, round = qq / (unsigned)R, slot = qq - round * (unsigned)R;
                    if (round == 0 || wait_bar(c, bars + (R + slot) * 8, (round - 1u) & 1u, p.ops[i].node)) {
                        mbar_expect(bars + slot * 8, (unsigned)cnt * kTileB);
                        bulk_load(smem_addr(smem + (size_t)slot * kStageB), base + ((size_t)r * kt_n + (size_t)s * kStTiles) * kTileB,
                                  (unsigned)cnt * kTileB, bars + slot * 8);
                    } else {
                        mine_ok = false;
                    }
                }
                ok = __all_sync(0xffffffffu, mine_ok);
                if (!ok) q += (unsigned)(i0 + kIssue < n_st ? i0 + kIssue : n_st);  // an upper bound of what was started
            }
            if (ok) q += (unsigned)n_st;
        }
        if (!ok && lane == 0) {
            // a consumer gave up: let the copies still in flight land before the ring goes away (a slot whose copy
            // was never started does not complete: the wait on it runs into its limit, once)
            const unsigned from = q > (unsigned)R ? q - (unsigned)R : 0u;
            for (unsigned s = from; s < q; s++)
                if (!mbar_wait(bars + (s % (unsigned)R) * 8, (s / (unsigned)R) & 1u, kWaitP)) break;
        }
    } else {
        unsigned stage_q = 0;
        ptrace(c, 30);
        if (p.first_attn >= 0) att_prefetch(c, p.ops[p.first_attn], true);
        for (int i = 0; i < p.n_ops; i++) {
            const POpDev& op = p.ops[i];
            c.op_index = i;
            if (op.kind == POP_GEMV) {
                run_gemv(c, op, stage_q);
            } else {
                if (op.a.D == 256) run_attn<256>(c, op);
                else if (op.a.D == 128) run_attn<128>(c, op);
                else run_attn<64>(c, op);
                if (op.a.next_attn >= 0) att_prefetch(c, p.ops[op.a.next_attn], false);
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
}

float to_f16(double v) { return __half2float(__double2half(v)); }

constexpr int kSmemTotal = 227 * 1024 - 1024;  // dynamic part; the kernel also has a few static words

}  // namespace

int persist_max_ops() { return kMaxOps; }

bool build_persist_launch(const std::vector<const PersistOp*>& ops, Buf epoch, PersistLaunch* out, std::string* why) {
    auto no = [&](const char* w) {
        if (why) *why = w;
        return false;
    };
    const int n = (int)ops.size();
    if (n < 2) return no("fewer than two operations");
    if (n > kMaxOps) return no("too many operations for one launch");
    const int G = sm_count();

    auto params = std::make_unique<PersistP>();
    PersistP& p = *params;
    std::memset(&p, 0, sizeof(p));
    std::vector<Reloc> relocs;
    auto field = [&](const void* f) { return (uint32_t)((const char*)f - (const char*)&p); };
    auto ptr = [&](const void* f, Buf b) { relocs.push_back(Reloc{field(f), b}); };
    const Buf null{kSlotNull, 0};

    // what the run has produced so far: value slot → (first tagged entry, elements)
    struct Made {
        size_t entry;
        long long elems;
        size_t flag_entry;  // the producing operation's arrival words
        int nflag;          // how many CTAs produce it
        int reps, rstride;  // copies of the vector and their distance in entries
    };
    // entries of one copy rounded to whole cache lines, so that two copies never share one
    auto rep_layout = [&](size_t entries, int* reps, int* rstride) {
        *reps = entries <= (size_t)kRepMaxEntries ? kReps : 1;
        *rstride = (int)((entries + 15) / 16 * 16);
        return (size_t)*reps * (size_t)*rstride;
    };
    std::map<uint32_t, Made> made;
    std::map<uint32_t, int> written;  // every slot some operation of the run stores to (plain)
    uint32_t resid_slot = 0xFFFFFFFFu;
    size_t xentries = 0;
    int k_tiles_max = 1, resid_k = 0, span_max = 0, att_d = 0, att_chunk = 0;
    int last_attn = -1;
    p.first_attn = -1;
    std::vector<long long> load(G, 0);

    auto external = [&](Buf b) {  // an operand read from plain memory must not be produced inside the run
        return !b.valid() || b.slot >= 0xFFFFFFF0u || !written.count(b.slot);
    };

    for (int i = 0; i < n; i++) {
        const PersistOp& o = *ops[i];
        POpDev& d = p.ops[i];
        d.kind = o.kind;
        d.node = o.node;
        if (o.kind == POP_GEMV) {
            PGemvDev& g = d.g;
            const bool prologue = o.has_w1 || o.has_res || o.has_w2;
            if (o.k <= 0 || (o.k & 1)) return no("odd K");
            if (prologue && o.k > kMaxPrologueK) return no("prologue width above what a thread keeps in registers");
            g.k = (int)o.k;
            g.k_tiles = (int)(((o.k + 31) / 32 + 3) / 4);
            g.sub = o.geglu ? 2 : 1;
            if (g.k_tiles * g.sub > kPassTiles) return no("K too long for one pass");
            int rt = 0;
            for (int s = 0; s < 3; s++) {
                g.seg_n[s] = s < o.n_seg ? (int)o.seg_n[s] : 0;
                g.seg_rt0[s] = rt;
                if (s < o.n_seg) rt += (int)((o.seg_n[s] + 15) / 16);
            }
            g.seg_rt0[3] = rt;
            for (int s = o.n_seg; s < 3; s++) g.seg_rt0[s] = 1 << 30;  // never selected
            g.row_tiles = rt;
            if (o.geglu && (o.n_seg != 2 || o.seg_n[0] != o.seg_n[1])) return no("GeGLU needs two equal segments");
            if (o.geglu) g.seg_rt0[1] = g.seg_rt0[2] = 1 << 30;  // results are indexed by pair, segment 0 only
            g.eps1 = to_f16(o.eps1);
            g.eps2 = to_f16(o.eps2);
            k_tiles_max = std::max(k_tiles_max, g.k_tiles);
            // activations
            if (!o.a.valid() || o.a.off != 0) return no("activation operand with an offset");
            auto it = made.find(o.a.slot);
            if (o.a.slot == resid_slot) {
                d.flags |= PF_SRC_RESID;
                ptr(&g.src, null);
            } else if (it != made.end()) {
                if (it->second.elems != o.k) return no("producer and consumer disagree on a vector's length");
                d.flags |= PF_SRC_TAGGED;
                g.src_reps = it->second.reps;
                g.src_rstride = it->second.rstride;
                ptr(&g.src, Buf{kSlotXbuf, (int64_t)(it->second.entry * 8)});
                ptr(&g.src_flag, Buf{kSlotXbuf, (int64_t)(it->second.flag_entry * 8)});
                g.src_nflag = it->second.nflag;
            } else {
                if (!external(o.a)) return no("activations produced inside the run in a form the kernel cannot read");
                ptr(&g.src, o.a);
            }
            if (o.has_w1) {
                d.flags |= PF_W1;
                if (!external(o.w1)) return no("norm weight produced inside the run");
            }
            if (o.has_w2) {
                d.flags |= PF_W2;
                if (!external(o.w2)) return no("norm weight produced inside the run");
            }
            ptr(&g.w1, o.has_w1 ? o.w1 : null);
            ptr(&g.w2, o.has_w2 ? o.w2 : null);
            if (o.has_res) {
                d.flags |= PF_RES;
                if (o.res.slot == resid_slot && o.res.off == 0) {
                    d.flags |= PF_RES_SMEM;
                    ptr(&g.res, null);
                } else {
                    if (!external(o.res)) return no("residual produced inside the run outside the residual chain");
                    ptr(&g.res, o.res);
                }
                if (!o.sum_out.valid()) return no("residual add without a destination");
                d.flags |= PF_SUM_OUT;
                ptr(&g.sum_out, o.sum_out);
                resid_slot = o.sum_out.slot;
                resid_k = std::max(resid_k, g.k);
                written[o.sum_out.slot] = 1;
            } else {
                ptr(&g.res, null);
                ptr(&g.sum_out, null);
            }
            if (o.geglu) d.flags |= o.geglu == 1 ? PF_GEGLU_TANH : PF_GEGLU_ERF;
            ptr(&g.tiles, o.tiles);
            // results
            const size_t entry0 = xentries;
            const int out_tiles = o.geglu ? rt / 2 : rt;
            xentries += rep_layout((size_t)out_tiles * 8, &g.out_reps, &g.out_rstride);
            if (g.src_reps < 1) g.src_reps = 1;
            ptr(&g.xout, Buf{kSlotXbuf, (int64_t)(entry0 * 8)});
            const size_t flag0 = xentries;
            xentries += (size_t)(G + 1) / 2;
            ptr(&g.xflag, Buf{kSlotXbuf, (int64_t)(flag0 * 8)});
            if (!(d.flags & PF_SRC_TAGGED)) ptr(&g.src_flag, null);
            const int n_units = g.row_tiles / g.sub;
            for (int s = 0; s < 3; s++) {
                const bool has = o.geglu ? s == 0 : s < o.n_seg;
                ptr(&g.y[s], has ? o.y[s] : null);
                if (!has) continue;
                if (o.y[s].off != 0) return no("result operand with an offset");
                made[o.y[s].slot] = Made{entry0 + (size_t)(o.geglu ? 0 : g.seg_rt0[s]) * 8, o.seg_n[s], flag0, std::min(n_units, G), g.out_reps, g.out_rstride};
                written[o.y[s].slot] = 1;
            }
            // spread the units over the CTAs: rotate the assignment to where the run has streamed least so far
            // The CTAs that ran an attention operation just before this one are still busy fetching the next
            // layer's keys: units placed on them would start late.
            const int U = g.row_tiles / g.sub;
            long long best_cost = -1;
            int best_rot = 0;
            const long long unit_tiles = (long long)g.k_tiles * g.sub;
            const int busy = (i > 0 && ops[i - 1]->kind == POP_ATTN) ? (int)(ops[i - 1]->KV * (ops[i - 1]->D / 8)) : 0;
            for (int rot = 0; rot < G; rot += 4) {
                long long worst = 0;
                for (int cta = 0; cta < G; cta++) {
                    int cp = cta - rot;
                    if (cp < 0) cp += G;
                    int u0, nu;
                    share_units(cp, U, G, &u0, &nu);
                    worst = std::max(worst, load[cta] + nu * unit_tiles + (cta < busy && nu ? (1LL << 20) : 0));
                }
                if (best_cost < 0 || worst < best_cost) {
                    best_cost = worst;
                    best_rot = rot;
                }
            }
            g.rot = best_rot;
            for (int cta = 0; cta < G; cta++) {
                int cp = cta - best_rot;
                if (cp < 0) cp += G;
                int u0, nu;
                share_units(cp, U, G, &u0, &nu);
                load[cta] += nu * unit_tiles;
            }
        } else if (o.kind == POP_ATTN) {
            PAttnDev& a = d.a;
            if (o.D != 64 && o.D != 128 && o.D != 256) return no("head dimension");
            if (o.KV <= 0 || o.H % o.KV != 0 || o.H / o.KV > 8) return no("more than 8 query heads per KV head");
            if (((o.H / o.KV) & (o.H / o.KV - 1)) != 0) return no("query heads per KV head not a power of two");
            if (o.KV * (o.D / 8) > G) return no("more (KV head, column tile) pairs than SMs");
            if (att_d && att_d != (int)o.D) return no("attention operations with different head dimensions");
            if (o.span <= 0 || o.span > 4096) return no("visible span too long");
            att_d = (int)o.D;
            a.H = (int)o.H;
            a.KV = (int)o.KV;
            a.D = (int)o.D;
            a.half = (int)o.half;
            a.window = (int)o.window;
            a.cache_rows = (int)o.cache_rows;
            a.cap = (int)o.cap;
            a.n_cap = (int)o.span;
            a.scale = o.scale;
            a.next_attn = -1;
            if (last_attn >= 0) p.ops[last_attn].a.next_attn = i;
            else p.first_attn = i;
            last_attn = i;
            span_max = std::max(span_max, (int)o.span);
            const int NC = (int)o.D / 8;
            att_chunk = std::max(att_chunk, ((int)o.span + NC - 1) / NC);
            // q, k, v: all tagged (from one earlier operation of the run) or all plain
            const Buf qkv[3] = {o.q, o.kx, o.vx};
            const long long want[3] = {o.H * o.D, o.KV * o.D, o.KV * o.D};
            int tagged = 0;
            for (int s = 0; s < 3; s++)
                if (made.count(qkv[s].slot) && qkv[s].off == 0 && made[qkv[s].slot].elems == want[s]) tagged++;
            const void* fields[3] = {&a.q, &a.k, &a.v};
            a.src_reps = 1;
            if (tagged == 3) {
                d.flags |= PF_Q_TAGGED;
                a.src_reps = made[qkv[0].slot].reps;
                a.src_rstride = made[qkv[0].slot].rstride;
                if (made[qkv[1].slot].reps != a.src_reps || made[qkv[2].slot].reps != a.src_reps || made[qkv[1].slot].rstride != a.src_rstride ||
                    made[qkv[2].slot].rstride != a.src_rstride)
                    return no("q, k and v copied differently");
                for (int s = 0; s < 3; s++) ptr(fields[s], Buf{kSlotXbuf, (int64_t)(made[qkv[s].slot].entry * 8)});
                // the three must come from one operation: its arrival words cover them all
                if (made[qkv[1].slot].flag_entry != made[qkv[0].slot].flag_entry || made[qkv[2].slot].flag_entry != made[qkv[0].slot].flag_entry)
                    return no("q, k and v produced by different operations of the run");
                ptr(&a.src_flag, Buf{kSlotXbuf, (int64_t)(made[qkv[0].slot].flag_entry * 8)});
                a.src_nflag = made[qkv[0].slot].nflag;
            } else {
                for (int s = 0; s < 3; s++) {
                    if (!external(qkv[s])) return no("attention operands produced inside the run in a form the kernel cannot read");
                    ptr(fields[s], qkv[s]);
                }
                ptr(&a.src_flag, null);
            }
            if (!external(o.seqlens) || !external(o.cos) || !external(o.sin)) return no("attention side operands produced inside the run");
            ptr(&a.cache_k, o.cache_k);
            ptr(&a.cache_v, o.cache_v);
            ptr(&a.seqlens, o.seqlens);
            ptr(&a.cos, o.half ? o.cos : null);
            ptr(&a.sin, o.half ? o.sin : null);
            ptr(&a.out, o.out);
            ptr(&a.dyn_t, o.dyn_t);
            const size_t entry0 = xentries;
            xentries += rep_layout((size_t)(o.H * o.D / 2), &a.out_reps, &a.out_rstride);
            ptr(&a.xout, Buf{kSlotXbuf, (int64_t)(entry0 * 8)});
            const int HP = (int)((o.H / o.KV + 1) / 2);
            ptr(&a.xsc, Buf{kSlotXbuf, (int64_t)(xentries * 8)});
            xentries += (size_t)o.KV * HP * (size_t)o.span;
            if (o.out.off != 0) return no("result operand with an offset");
            const size_t flag0 = xentries;
            xentries += (size_t)(G + 1) / 2 * 2;
            ptr(&a.xflag, Buf{kSlotXbuf, (int64_t)(flag0 * 8)});
            ptr(&a.xflag_sc, Buf{kSlotXbuf, (int64_t)((flag0 + (size_t)(G + 1) / 2) * 8)});
            made[o.out.slot] = Made{entry0, o.H * o.D, flag0, (int)(o.KV * (o.D / 8)), a.out_reps, a.out_rstride};
            written[o.out.slot] = 1;
            written[o.cache_k.slot] = 1;
            written[o.cache_v.slot] = 1;
        } else {
            return no("unknown operation");
        }
    }

    // shared memory: ring | barriers | activations | residual | partial sums | reductions | attention staging
    const int npad = (span_max + 15) & ~15, chunk_pad = (att_chunk + 15) & ~15;
    size_t attn_bytes = 0;
    if (att_d) {
        const size_t RS = (size_t)att_d + kRowPad;
        attn_bytes = (size_t)10 * att_d * 2 + 8 * RS * 2 + (size_t)chunk_pad * RS * 2 + (size_t)npad * 16 + (size_t)8 * (npad + 8) * 2 +
                     (size_t)kCW * 64 * 4 + 8 * 8 + 8 * 4;
        attn_bytes = (attn_bytes + 127) / 128 * 128;
    }
    const size_t acts_bytes = (size_t)k_tiles_max * 256, resid_bytes = ((size_t)resid_k * 4 + 127) / 128 * 128;
    const size_t part_bytes = (size_t)kPassTiles * 16 * 4, red_bytes = (size_t)2 * kCW * 8;
    const size_t params_bytes = (offsetof(PersistP, ops) + (size_t)n * sizeof(POpDev) + 127) / 128 * 128;
    const size_t fixed = acts_bytes + resid_bytes + part_bytes + red_bytes + attn_bytes + params_bytes + 256;
    if (fixed + 8 * (kStageB + 16) > (size_t)kSmemTotal) return no("shared memory does not fit");
    int stages = (int)(((size_t)kSmemTotal - fixed) / (kStageB + 16));
    if (stages > 60) stages = 60;
    p.ring_stages = stages;
    size_t off = (size_t)stages * kStageB;
    p.off_bars = (int)off;
    off += ((size_t)stages * 16 + 127) / 128 * 128;
    p.off_acts = (int)off;
    off += acts_bytes;
    p.off_resid = (int)off;
    off += resid_bytes;
    p.off_part = (int)off;
    off += part_bytes;
    p.off_red = (int)off;
    off += red_bytes;
    off = (off + 127) / 128 * 128;
    p.off_attn = (int)off;
    off += attn_bytes;
    p.off_params = (int)off;
    p.params_bytes = (int)(offsetof(PersistP, ops) + (size_t)n * sizeof(POpDev));
    off += params_bytes;
    if (off > (size_t)kSmemTotal) return no("shared memory does not fit");
    p.att_chunk_pad = chunk_pad;
    p.att_npad = npad;
    p.n_ops = n;
    p.gc.c_half = to_f16(0.5);
    p.gc.c_one = to_f16(1.0);
    p.gc.c_coef = to_f16(0.044715);
    p.gc.c_k = to_f16(std::sqrt(2.0 / 3.14159265358979323846));
    p.gc.c_inv_sqrt2 = to_f16(0.70710678118654752440);
    ptr(&p.err, Buf{kSlotErr, 0});
    ptr(&p.epoch, epoch);

    {
        static std::mutex mu;
        static std::map<int, bool> done;
        int dev = 0;
        cudaGetDevice(&dev);
        std::lock_guard<std::mutex> lock(mu);
        if (!done[dev]) {
            cudaError_t e = cudaFuncSetAttribute((const void*)persist_step, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
            if (e != cudaSuccess) {
                cudaGetLastError();
                return no("the device refuses the kernel's shared memory");
            }
            persist_fill_luts<<<64, 256>>>();
            if (cudaDeviceSynchronize() != cudaSuccess) {
                cudaGetLastError();
                return no("the lookup tables could not be filled");
            }
            done[dev] = true;
        }
    }

    LaunchRec& r = out->rec;
    r = LaunchRec{};
    r.func = (const void*)persist_step;
    r.grid = dim3((unsigned)G);
    r.block = dim3(kPT);
    r.smem = (unsigned)off;
    // only the used part of the operation table travels
    const size_t used = offsetof(PersistP, ops) + (size_t)n * sizeof(POpDev);
    r.params.resize(sizeof(PersistP));
    std::memcpy(r.params.data(), &p, sizeof(PersistP));
    (void)used;
    r.relocs = std::move(relocs);
    r.label = "persist_step";
    r.node = ops[0]->node;
    r.cooperative = true;
    out->xbuf_bytes = std::max<size_t>(xentries * 8, 8);
    return true;
}

}  // namespace oxk
