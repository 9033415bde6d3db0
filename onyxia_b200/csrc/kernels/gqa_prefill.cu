// GroupQueryAttention over many new positions at once (prefill), f16, on the tensor cores.
// Specification: the decomposition crates/onyxia-ir/src/decomp.rs:357-613 — scores q·k rounded, scaled,
// rounded; causal + sliding-window mask; Softmax of decomp.rs:174-183 (row max, exp of the rounded
// difference, rounded; exact sum, rounded; quotient, rounded); P·V rounded.
//
// Runs after gqa_prepare (rotated q in scratch, new rows appended to the present cache). One CTA of eight
// warps per (16 query positions, query head, batch row); the keys are walked in blocks of 64, the warps
// split a block's keys four ways and the head dimension of the output two ways (a single warp per
// scheduler cannot hide the latency of its own ldmatrix → MMA chains: 2 warps per CTA took 103 µs per
// 512-token layer of the 1B configuration). The softmax of the decomposition is not an online one — every
// probability is e / Σe with both already rounded to f16 — so the keys are walked three times, forming
// the score tiles on the tensor cores each time instead of keeping a [queries × keys] array anywhere:
//   pass 1  row maxima
//   pass 2  Σ round16(exp(round16(s − max))), exactly (every term is a multiple of 2⁻²⁴ ≤ 1: added as
//           integers, which is what the interpreter's f64 sum gives), then rounded once like its Reduce
//   pass 3  p = round16(e / Σ) becomes the A operand of the P·V product straight from the score
//           tile's accumulator registers; V rows are the B operand through ldmatrix.trans; the four
//           key groups' f32 partial outputs are added in group order through shared memory
// K (and V in pass 3) blocks of 64 keys are staged by cp.async into padded shared-memory rows, two
// stages deep. Products are exact f16 × f16 and are added in f32 by the tensor core (the interpreter
// adds in f64): results differ from it by an f16 spacing on a small share of the elements, like the
// int4 matrix products.
#include <cstdlib>
#include <map>
#include <mutex>

#include "common.cuh"
#include "kernels.hpp"
#include "nbits_tile.cuh"

namespace oxk {
using namespace oxk::tile;

namespace {

constexpr int kKB = 64;      // keys per block
constexpr int kPad = 8;      // f16 elements of padding per staged row (keeps ldmatrix conflict-free)

// round_f16(exp(−|d|)) for every f16 argument (the softmax argument is ≤ 0), filled once per device.
__device__ __half g_pf_exp_lut[32768];

__global__ void gqa_prefill_fill_lut() {
    for (int i = (int)global_tid(); i < 32768; i += (int)global_threads())
        g_pf_exp_lut[i] = __double2half(exp(-(double)__half2float(__ushort_as_half((unsigned short)i))));
}

struct PrefillP {
    const __half* q;    // [B,S,H,D] (rotated)
    const __half* pk;   // [B,KV,cap,D]
    const __half* pv;
    const int* seqlens;
    __half* out;        // [B,S,H·D]
    const long long* dyn_t;  // when set, the present length T is read from here
    long long B, S, H, KV, T, cap, window;
    float scale;        // rounded to f16
};

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(unsigned (&r)[2], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void cp16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// D = head dimension. 16 query positions per CTA, 8 warps: warp = (key group kg of 16 keys within the
// 64-key block, half wd of the head dimension).
constexpr int kBM = 16, kWarps = 8, kNT = kWarps * 32;

template <int D> __global__ void __launch_bounds__(kNT) gqa_prefill_tc(const PrefillP p) {
    constexpr int RS = D + kPad, CPR = D / 8;   // staged row stride; 16-byte chunks per row
    constexpr int DH = D / 2, NDT = DH / 8;     // this warp's output columns, in tiles of 8
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __half* Qs = reinterpret_cast<__half*>(smem_raw);          // [16][RS]
    __half* Ks = Qs + kBM * RS;                                // [2][kKB][RS]
    __half* Vs = Ks + 2 * kKB * RS;                            // [2][kKB][RS]
    __shared__ float row_max[kBM][kWarps];
    __shared__ unsigned long long row_sum[kBM][kWarps];
    pdl_enter();

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, kg = warp >> 1, wd = warp & 1;
    const int gq = lane >> 2, t = lane & 3;
    const long long b = blockIdx.z, h = blockIdx.y, G = p.H / p.KV, kvh = h / G;
    const long long s0 = (long long)blockIdx.x * kBM;
    const long long T = p.dyn_t ? *p.dyn_t : p.T;
    const long long tot = (long long)p.seqlens[b] + 1, past_b = tot - p.S > 0 ? tot - p.S : 0;
    const long long s_last = (s0 + kBM < p.S ? s0 + kBM : p.S) - 1;
    const long long hi_blk = past_b + s_last < T - 1 ? past_b + s_last : T - 1;
    const long long lo_blk = (p.window >= 0 && past_b + s0 - p.window > 0) ? past_b + s0 - p.window : 0;
    const long long n_blk = hi_blk >= lo_blk ? hi_blk - lo_blk + 1 : 0;
    const int nkb = (int)((n_blk + kKB - 1) / kKB);

    // the two query positions of this thread's accumulator rows and the keys they may see, as offsets from lo_blk
    int lo[2], hi[2];
    bool live[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const long long s = s0 + gq + r * 8;
        live[r] = s < p.S;
        const long long qpos = past_b + s;
        const long long h_ = qpos < T - 1 ? qpos : T - 1;
        const long long l_ = (p.window >= 0 && qpos - p.window > 0) ? qpos - p.window : 0;
        lo[r] = (int)(l_ - lo_blk);
        hi[r] = live[r] ? (int)(h_ - lo_blk) : -1;  // a row past S sees nothing
    }

    const __half* kbase = p.pk + (b * p.KV + kvh) * p.cap * D;
    const __half* vbase = p.pv + (b * p.KV + kvh) * p.cap * D;
    auto load_block = [&](int stage, int kb, bool with_v) {
        __half* kd = Ks + stage * kKB * RS;
        __half* vd = Vs + stage * kKB * RS;
        for (int i = tid; i < kKB * CPR; i += kNT) {
            const int r = i / CPR, c = i - r * CPR;
            long long tk = lo_blk + (long long)kb * kKB + r;
            if (tk > hi_blk) tk = hi_blk;  // rows past the range are masked; any valid row will do
            cp16(smem_addr(kd + r * RS + c * 8), kbase + tk * D + c * 8);
            if (with_v) cp16(smem_addr(vd + r * RS + c * 8), vbase + tk * D + c * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    if (nkb == 0) {  // nothing visible: the rows are zero (what the split kernels give for an empty range)
        for (int i = tid; i < kBM * D; i += kNT) {
            const long long s = s0 + i / D;
            if (s < p.S) p.out[((b * p.S + s) * p.H + h) * D + i % D] = __float2half(0.f);
        }
        return;
    }

    // Q tile (rows past S repeat the last one; they are never stored)
    for (int i = tid; i < kBM * CPR; i += kNT) {
        const int r = i / CPR, c = i - r * CPR;
        long long s = s0 + r;
        if (s > p.S - 1) s = p.S - 1;
        cp16(smem_addr(Qs + r * RS + c * 8), p.q + ((b * p.S + s) * p.H + h) * D + c * 8);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");

    const unsigned q_addr = smem_addr(Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * RS + ((lane >> 4) & 1) * 8);
    // The 16 × 8 score tile `n` of a staged key block. Every pass forms a tile with this one sequence of
    // MMAs, so the three passes see bit-identical scores.
    auto score_tile = [&](const __half* kd, int n, float (&acc)[4]) {
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        const unsigned k_addr = smem_addr(kd + (n * 8 + (lane & 7)) * RS + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int j = 0; j < D / 16; j++) {
            unsigned a[4], bf[2];
            ldsm_x4(a, q_addr + j * 32);
            ldsm_x2(bf, k_addr + j * 32);
            mma16816(acc, a[0], a[1], a[2], a[3], bf[0], bf[1]);
        }
    };
    // two neighbouring tiles at once (two independent accumulator chains), each summed exactly like score_tile
    auto score_pair = [&](const __half* kd, int n, float (&a0)[4], float (&a1)[4]) {
        a0[0] = a0[1] = a0[2] = a0[3] = 0.f;
        a1[0] = a1[1] = a1[2] = a1[3] = 0.f;
        const unsigned k_addr = smem_addr(kd + (n * 8 + (lane & 7) + ((lane >> 4) & 1) * 8) * RS + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int j = 0; j < D / 16; j++) {
            unsigned a[4], bf[4];
            ldsm_x4(a, q_addr + j * 32);
            ldsm_x4(bf, k_addr + j * 32);
            mma16816(a0, a[0], a[1], a[2], a[3], bf[0], bf[1]);
            mma16816(a1, a[0], a[1], a[2], a[3], bf[2], bf[3]);
        }
    };
    // visibility of accumulator element e of tile n in key block kb; the rounded, scaled score
    auto visible = [&](int kb, int n, int e) {
        const int tk = kb * kKB + n * 8 + 2 * t + (e & 1);
        return tk >= lo[e >> 1] && tk <= hi[e >> 1];
    };
    auto scaled = [&](float c) { return r16(r16(c) * p.scale); };
    auto stage_in = [&](int kb, bool with_v) {  // block kb is complete in its stage, block kb + 1 on its way
        if (kb + 1 < nkb) {
            load_block((kb + 1) & 1, kb + 1, with_v);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
    };

    // ── pass 1: row maxima; each warp takes one of the block's eight key tiles ──
    const int my_tile = kg * 2 + wd;
    float mx[2] = {-INFINITY, -INFINITY};
    load_block(0, 0, false);
    for (int kb = 0; kb < nkb; kb++) {
        stage_in(kb, false);
        float acc[4];
        score_tile(Ks + (kb & 1) * kKB * RS, my_tile, acc);
#pragma unroll
        for (int e = 0; e < 4; e++)
            if (visible(kb, my_tile, e)) mx[e >> 1] = fmaxf(mx[e >> 1], scaled(acc[e]));
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        if (t == 0) row_max[gq + r * 8][warp] = mx[r];
    }
    __syncthreads();
    __half hmax[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        float m = row_max[gq + r * 8][0];
#pragma unroll
        for (int w = 1; w < kWarps; w++) m = fmaxf(m, row_max[gq + r * 8][w]);
        hmax[r] = __float2half_rn(m);  // an f16 value already
    }
    auto exp_of = [&](float s, int r) {
        const __half d = __hsub(__float2half_rn(s), hmax[r]);  // one rounding of the exact difference; ≤ 0
        return g_pf_exp_lut[__half_as_ushort(d) & 0x7FFF];
    };

    // ── pass 2: Σ e, exact: every e is a multiple of 2⁻²⁴ not above 1, summed as integers ──
    unsigned long long sum[2] = {0ull, 0ull};
    load_block(0, 0, false);
    for (int kb = 0; kb < nkb; kb++) {
        stage_in(kb, false);
        float acc[4];
        score_tile(Ks + (kb & 1) * kKB * RS, my_tile, acc);
#pragma unroll
        for (int e = 0; e < 4; e++)
            if (visible(kb, my_tile, e)) sum[e >> 1] += (unsigned)(__half2float(exp_of(scaled(acc[e]), e >> 1)) * 16777216.f);
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        if (t == 0) row_sum[gq + r * 8][warp] = sum[r];
    }
    __syncthreads();
    float total[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        unsigned long long s_ = 0ull;
#pragma unroll
        for (int w = 0; w < kWarps; w++) s_ += row_sum[gq + r * 8][w];
        total[r] = r16d((double)s_ * 5.9604644775390625e-08);  // · 2⁻²⁴, one rounding like the interpreter's Reduce
    }

    // ── pass 3: probabilities × V over this warp's 16 keys of each block and its half of the head dimension ──
    float o[NDT][4];
#pragma unroll
    for (int n = 0; n < NDT; n++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[n][e] = 0.f;
    load_block(0, 0, true);
    for (int kb = 0; kb < nkb; kb++) {
        stage_in(kb, true);
        float acc[2][4];
        score_pair(Ks + (kb & 1) * kKB * RS, kg * 2, acc[0], acc[1]);
        unsigned pa[2][2];  // per key tile: probabilities of row gq and of row gq + 8 as f16 pairs
#pragma unroll
        for (int n = 0; n < 2; n++) {
            float pr[4];
#pragma unroll
            for (int e = 0; e < 4; e++)  // e and Σ are f16 values: their f32 quotient rounds to the same f16 as the exact one
                pr[e] = visible(kb, kg * 2 + n, e) ? __half2float(exp_of(scaled(acc[n][e]), e >> 1)) / total[e >> 1] : 0.f;
            pa[n][0] = hu(__halves2half2(__float2half_rn(pr[0]), __float2half_rn(pr[1])));
            pa[n][1] = hu(__halves2half2(__float2half_rn(pr[2]), __float2half_rn(pr[3])));
        }
        const __half* vd = Vs + (kb & 1) * kKB * RS;
        const unsigned v_addr = smem_addr(vd + (kg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * RS + wd * DH + ((lane >> 4) & 1) * 8);
#pragma unroll
        for (int nd = 0; nd < NDT; nd += 2) {
            unsigned bf[4];
            ldsm_x4_t(bf, v_addr + nd * 16);
            mma16816(o[nd], pa[0][0], pa[0][1], pa[1][0], pa[1][1], bf[0], bf[1]);
            mma16816(o[nd + 1], pa[0][0], pa[0][1], pa[1][0], pa[1][1], bf[2], bf[3]);
        }
        __syncthreads();
    }
    // the four key groups' partial outputs are added in group order; the staging area is free now
    float* part = reinterpret_cast<float*>(Ks);  // [4][16][D]
#pragma unroll
    for (int n = 0; n < NDT; n++)
#pragma unroll
        for (int e = 0; e < 4; e++)
            part[(kg * kBM + gq + (e >> 1) * 8) * D + wd * DH + n * 8 + 2 * t + (e & 1)] = o[n][e];
    __syncthreads();
    for (int i = tid; i < kBM * D / 2; i += kNT) {
        const int row = i / (D / 2), col = (i - row * (D / 2)) * 2;
        const long long s = s0 + row;
        if (s >= p.S) continue;
        float v0 = 0.f, v1 = 0.f;
#pragma unroll
        for (int g4 = 0; g4 < 4; g4++) {
            const float2 f = *reinterpret_cast<const float2*>(part + (g4 * kBM + row) * D + col);
            v0 += f.x;
            v1 += f.y;
        }
        *reinterpret_cast<__half2*>(p.out + ((b * p.S + s) * p.H + h) * D + col) = __halves2half2(__float2half_rn(v0), __float2half_rn(v1));
    }
}

template <int D> void launch_prefill(Emitter& em, PrefillP& p, long long B, long long S, long long H, Buf q, Buf pk, Buf pv, Buf seqlens,
                                     Buf out, Buf dyn_t) {
    constexpr int RS = D + kPad;
    const size_t smem = (size_t)(kBM + 4 * kKB) * RS * 2;
    static_assert((size_t)4 * kBM * D * 4 <= (size_t)2 * kKB * (D + kPad) * 2, "the partial outputs must fit the K staging area");
    auto fn = gqa_prefill_tc<D>;
    if (smem > 48 * 1024) ensure_max_dynamic_smem((const void*)fn, (int)smem);
    em.launch(fn, dim3((unsigned)((S + kBM - 1) / kBM), (unsigned)H, (unsigned)B), dim3(kNT), (unsigned)smem, p,
              {{&p.q, q}, {&p.pk, pk}, {&p.pv, pv}, {&p.seqlens, seqlens}, {&p.out, out}, {&p.dyn_t, dyn_t}}, "gqa_prefill_tc", /*pdl=*/true);
}

}  // namespace

// The attention part of a fused GroupQueryAttention over S new positions whose rotated q and present
// caches gqa_prepare has written. False when the shape is not one this kernel takes.
bool emit_gqa_prefill_tc(Emitter& em, const GqaDesc& d, Buf q_rot, const TRef& seqlens, const TRef& out, const TRef& present_k,
                         const TRef& present_v, Buf dyn_t, long long T, long long cap) {
    const long long B = d.batch, S = d.seq, H = d.heads, KV = d.kv_heads, D = d.head_dim;
    if (d.has_bias || (D != 64 && D != 128 && D != 256) || S < 16) return false;
    if (H > 65535 || B > 65535 || KV <= 0 || H % KV != 0) return false;
    static const bool off = std::getenv("ONYXIA_DISABLE_PREFILL_TC") && std::atoi(std::getenv("ONYXIA_DISABLE_PREFILL_TC")) != 0;  // diagnostics
    if (off) return false;
    {
        static std::mutex mu;
        static std::map<int, bool> done;
        int dev = 0;
        cudaGetDevice(&dev);
        std::lock_guard<std::mutex> lock(mu);
        if (!done[dev]) {
            gqa_prefill_fill_lut<<<32, 256>>>();
            if (cudaDeviceSynchronize() != cudaSuccess) {
                cudaGetLastError();
                return false;
            }
            done[dev] = true;
        }
    }
    PrefillP p{};
    p.B = B; p.S = S; p.H = H; p.KV = KV; p.T = T; p.cap = cap;
    p.window = d.window;
    p.scale = __half2float(__double2half(d.scale));
    if (D == 64) launch_prefill<64>(em, p, B, S, H, q_rot, present_k.buf, present_v.buf, seqlens.buf, out.buf, dyn_t);
    else if (D == 128) launch_prefill<128>(em, p, B, S, H, q_rot, present_k.buf, present_v.buf, seqlens.buf, out.buf, dyn_t);
    else launch_prefill<256>(em, p, B, S, H, q_rot, present_k.buf, present_v.buf, seqlens.buf, out.buf, dyn_t);
    return true;
}

}  // namespace oxk
