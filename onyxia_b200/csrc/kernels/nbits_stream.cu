// Streaming MatMulNBits for the decode path (f16 activations, f16 scales, up
// to 8 activation rows per pass):
//   y[m, n] = Σ_k a[m, k] · round_f16((q[n, k] − zp[n, k/32]) · s[n, k/32])
//
// The kernel is bound by the HBM read of the weights, so everything is built
// around keeping that read a long, contiguous, deeply pipelined stream.
//
//  * Tile-major weights. At prepare time the packed nibbles, the scales and the
//    zero points of every 16-row × 128-column tile are gathered into one
//    contiguous record (`nbits_pack_tiles`): 1024 B of nibbles in the order the
//    lanes consume them, 128 B of scales (a lane's two rows side by side), 64 B
//    of zero points when the matrix has them. Records follow each other row tile by row tile, k tile by k tile;
//    rows and blocks beyond the matrix are stored as zero weights with zero
//    scale, so the inner loop has no bounds checks.
//  * One stream per warp. The records are numbered 0 … row_tiles·k_tiles − 1
//    and cut into equal contiguous ranges, one per warp of the grid. A warp
//    moves its range through a private ring of shared-memory stages with bulk
//    asynchronous copies (`cp.async.bulk`, completion counted on an mbarrier per
//    stage), so each warp keeps several kilobytes in flight without holding
//    them in registers, and no block-wide barrier sits in the loop.
//  * Tensor-core inner product. Lane (g, t) widens the 32 nibbles of rows g and
//    g + 8 at block t of the tile (0x6400 trick, exact (q − zp)·s rounding) and
//    feeds them to m16n8k16 MMAs as the A operand; the B operand holds up to 8
//    activation rows, staged once per CTA in shared memory in fragment order.
//    Tiles are summed in f32 on two independent MMA chains; every few tiles
//    the f32 sums move to an f64 accumulator.
//  * Ranges ignore row-tile boundaries. A warp that covers all k tiles of a row
//    tile stores the result directly; the pieces of a row tile shared between
//    neighbouring warps go to scratch, and the last warp to arrive (one counter
//    per row tile) adds the pieces in range order, so results do not depend on
//    scheduling.
//
// Algorithmic bytes: N·⌈K/32⌉·(16 + 2) (+ N·⌈K/32⌉/2 zero points) + activations.
#include <cstdlib>

#include "common.cuh"
#include "kernels.hpp"
#include "persist.hpp"

namespace oxk {

namespace {

constexpr int kWarps = 8;           // warps per CTA, each with its own stream
constexpr int kTileW = 1024;        // nibble bytes per tile record
constexpr int kTileS = 128;         // scale bytes per tile record
constexpr int kTileZ = 64;          // zero-point bytes per tile record (when present)
constexpr int kStageTiles = 3;      // tile records per pipeline stage
constexpr int kStages = 3;          // pipeline depth per warp
constexpr int kFoldTiles = 4;       // tiles summed in f32 before the sum moves to the f64 accumulator
constexpr long long kWaitCycles = 2000000000LL;  // ≈ 1 s: how long a stage may take to land before giving up

// ── prepare-time packing ────────────────────────────────────────────────
struct PackP {
    const unsigned* w;           // [N][nb][4] words, natural nibble order
    const __half* scales;        // [N][nb]
    const unsigned char* zp;     // packed nibbles over [N][nb], or null
    unsigned char* dst;
    long long n, nb, row_tiles, k_tiles;
    long long rt_mul, rt_add;    // row tile rt of this matrix is row tile rt·rt_mul + rt_add of the destination stream
    int tile_bytes;
};

__device__ __forceinline__ unsigned interleave_word(unsigned w) {
    unsigned o = 0;
#pragma unroll
    for (int j = 0; j < 8; j++) o |= ((w >> (4 * j)) & 0xFu) << (4 * ((j >> 1) + 4 * (j & 1)));
    return o;
}

// One thread per (tile, half h, row g, block t): 16 B of nibbles, one scale, one zero point.
__global__ void nbits_pack_tiles(const PackP p) {
    const long long units = p.row_tiles * p.k_tiles * 64;
    for (long long u = global_tid(); u < units; u += global_threads()) {
        const int slot = (int)(u & 63);  // h·32 + g·4 + t
        const long long tile = u >> 6;
        const long long rt = tile / p.k_tiles, kt = tile % p.k_tiles;
        const long long row = rt * 16 + (slot >> 5) * 8 + ((slot >> 2) & 7), kb = kt * 4 + (slot & 3);
        unsigned char* rec = p.dst + ((rt * p.rt_mul + p.rt_add) * p.k_tiles + kt) * p.tile_bytes;
        uint4 q = make_uint4(0, 0, 0, 0);
        __half s = __float2half(0.f);
        unsigned char z = 8;
        if (row < p.n && kb < p.nb) {
            const unsigned* src = p.w + (row * p.nb + kb) * 4;
            q = make_uint4(interleave_word(src[0]), interleave_word(src[1]), interleave_word(src[2]), interleave_word(src[3]));
            s = p.scales[row * p.nb + kb];
            if (p.zp) {
                long long i = row * p.nb + kb;
                z = (p.zp[i >> 1] >> ((i & 1) * 4)) & 0xF;
            }
        }
        reinterpret_cast<uint4*>(rec)[slot] = q;
        // scales and zero points: the values of rows g and g + 8 side by side per lane
        const int pair = (slot & 31) * 2 + (slot >> 5);
        reinterpret_cast<__half*>(rec + kTileW)[pair] = s;
        if (p.zp) rec[kTileW + kTileS + pair] = z;
    }
}

// ── PTX helpers ─────────────────────────────────────────────────────────
__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// Bounded wait: false when the barrier did not complete within kWaitCycles.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (clock64() - t0 < kWaitCycles)
        if (mbar_try(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_load(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void mma16816s(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                          unsigned b1) {
    asm volatile(
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
// The low nibble of each half-word becomes the f16 1024 + q, the next one 1024 + 16·q.
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

}  // namespace

struct StreamP {
    const __half* a;            // activations [M, K] (before the prologue)
    const unsigned char* tiles; // tile records of all segments, row tile by row tile
    ErrWord* err;
    __half* y[3];               // one output [M, seg_n] per segment (GeGLU: only y[0], [M, seg_n[0]])
    // Prologue on the activations, each step optional:
    //   v = a;  v = rmsnorm(v)·w1;  v = res + v (also stored to sum_out);  v = rmsnorm(v)·w2
    const __half* w1;
    const __half* res;
    __half* sum_out;
    const __half* w2;
    float eps1, eps2;           // rounded to f16
    float c_half, c_one, c_coef, c_k, c_inv_sqrt2;  // Gelu constants rounded to f16
    long long m0, m_total, k;
    long long seg_n[3];
    int seg_rt0[4];             // first row tile of each segment, then the total
    int n_seg;
    int geglu;                  // 0: plain outputs; 1 / 2: out = gelu_tanh / gelu_erf(segment 0)·segment 1, row tiles interleaved
    int k_tiles, row_tiles, rts_per_cta, act_bytes, aux_bytes, node;
    int rts_extra, rts_step;  // the first rts_extra CTAs own rts_per_cta row tiles, the others rts_step fewer (0: all alike)
};

// Result fragment of one row tile → the CTA's staging area [row tile][16 rows][MR], rounded to f16.
// c0:(row g, col 2t) c1:(row g, col 2t+1) c2:(row g+8, col 2t) c3:(row g+8, col 2t+1); col = activation row.
template <int MR> __device__ __forceinline__ void stream_stage(float* ystage, const double (&acc)[4], int rt_local, int lane) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const int row = g + (q >= 2 ? 8 : 0), col = 2 * t + (q & 1);
        if (col < MR) ystage[(rt_local * 16 + row) * MR + col] = __half2float(__double2half(acc[q]));
    }
}

__device__ __forceinline__ float r16(float v) { return __half2float(__float2half_rn(v)); }
__device__ __forceinline__ float r16d(double v) { return __half2float(__double2half(v)); }

// gelu(gate)·up with the rounding points of the Gelu decomposition followed by Mul
// (crates/onyxia-ir/src/decomp.rs:185-213); the caller rounds the product when it stores it.
__device__ __forceinline__ float geglu_value(const StreamP& p, float x, float up) {
    float inner;
    if (p.geglu == 1) {
        const float x2 = r16(x * x), x3 = r16(x2 * x), cx3 = r16(p.c_coef * x3), s = r16(x + cx3), sc = r16(p.c_k * s);
        inner = r16d(tanh((double)sc));
    } else {
        // erf by Abramowitz–Stegun 7.1.26, as the interpreter evaluates it (interp.rs:860-872)
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

// ST tile records per pipeline stage, NS stages per warp: 3 × 3 by default; 1 × 3 (a third of the ring) where the
// staged activation rows would otherwise leave room for one CTA per SM only.
template <int MR, bool HAS_ZP, int ST = kStageTiles, int NS = kStages> __global__ void __launch_bounds__(kWarps * 32, 2) nbits_stream(const StreamP p) {
    constexpr int kTileBytes = kTileW + kTileS + (HAS_ZP ? kTileZ : 0);
    constexpr int kStageBytes = ST * kTileBytes;
    extern __shared__ __align__(128) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // activations | aux: scratch of the prologue, later the output staging | rings | barriers | pieces
    float* aux = reinterpret_cast<float*>(smem + p.act_bytes);
    unsigned char* ring_base = smem + p.act_bytes + p.aux_bytes;
    unsigned char* ring = ring_base + warp * (NS * kStageBytes);
    const unsigned bars = smem_addr(ring_base + kWarps * NS * kStageBytes) + warp * NS * 8;

    // pieces of row tiles shared between warps of this CTA: [warp][first / last piece][128]
    double* pieces = reinterpret_cast<double*>(ring_base + kWarps * NS * kStageBytes + kWarps * NS * 8);

    // This CTA owns `cta_rts` consecutive row tiles = cta_tiles consecutive tile
    // records, cut into equal ranges for its warps.
    const int b_x = (int)blockIdx.x, b_few = b_x > p.rts_extra ? b_x - p.rts_extra : 0;  // CTAs before this one with the smaller share
    const int cta_rt0 = b_x * p.rts_per_cta - b_few * p.rts_step;
    const int cta_want = p.rts_per_cta - (b_x >= p.rts_extra ? p.rts_step : 0);
    const int cta_rts = p.row_tiles - cta_rt0 < cta_want ? p.row_tiles - cta_rt0 : cta_want;
    const int cta_tiles = cta_rts * p.k_tiles;
    const int per = (cta_tiles + kWarps - 1) / kWarps;
    const int beg = warp * per;
    const int n_tiles = beg >= cta_tiles ? 0 : (cta_tiles - beg < per ? cta_tiles - beg : per);
    const int n_stages = (n_tiles + ST - 1) / ST;
    const unsigned char* src = p.tiles + ((long long)cta_rt0 * p.k_tiles + beg) * kTileBytes;

    auto issue = [&](int st, int slot) {  // lane 0 only
        int cnt = n_tiles - st * ST;
        if (cnt > ST) cnt = ST;
        const unsigned bytes = (unsigned)cnt * kTileBytes;
        mbar_expect(bars + slot * 8, bytes);
        bulk_load(smem_addr(ring + slot * kStageBytes), src + (size_t)st * kStageBytes, bytes, bars + slot * 8);
    };

    // The weights do not depend on the kernels before this one: start streaming
    // them before waiting for the producer of the activations.
    if (lane == 0) {
        for (int s = 0; s < NS; s++) mbar_init(bars + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int s = 0; s < NS && s < n_stages; s++) issue(s, s);
    }
    __syncwarp();
    ox_trace(p.err, 1);
    pdl_trigger();
    pdl_wait();
    ox_trace(p.err, 2);

    // Activations → shared memory in B-fragment order: chunk (kt·4 + m)·4·MR + g·4 + t
    // holds v[m0 + g][kt·128 + t·32 + m·8 … + 8], zero beyond the matrix.
    if (!p.w1 && !p.res && !p.w2) {
        uint4* as = reinterpret_cast<uint4*>(smem);
        const int chunks = p.k_tiles * 16 * MR;
        const bool vec = (p.k & 7) == 0 && (reinterpret_cast<uintptr_t>(p.a) & 15) == 0;
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
            const int ct = c & 3, cg = (c >> 2) % MR, cm = (c / (4 * MR)) & 3, ckt = c / (16 * MR);
            const long long row = p.m0 + cg, k0 = (long long)ckt * 128 + ct * 32 + cm * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < p.m_total) {
                const __half* src_a = p.a + row * p.k + k0;
                if (vec && k0 + 8 <= p.k) {
                    v = *reinterpret_cast<const uint4*>(src_a);
                } else {
                    __half tmp[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) tmp[e] = k0 + e < p.k ? src_a[e] : __float2half(0.f);
                    v = *reinterpret_cast<uint4*>(tmp);
                }
            }
            as[c] = v;
        }
        __syncthreads();
    } else {
        // The prologue: RMS norm, residual add, RMS norm — the primitive sequence and rounding
        // points of SimplifiedLayerNormalization (decomp.rs:241-257) and Add. Every CTA does it
        // for the MR rows of this pass; CTA 0 also stores the residual sum.
        __half* ah = reinterpret_cast<__half*>(smem);
        float* v = aux;                                                // [MR][K]
        double* red = reinterpret_cast<double*>(aux + (((size_t)MR * p.k + 1) & ~(size_t)1));  // [MR][kWarps], then [MR] totals
        const int K = (int)p.k;
        auto block_sums = [&](double (&part)[MR]) {  // per-row sums over the CTA, result in red[MR·kWarps + m]
#pragma unroll
            for (int m = 0; m < MR; m++) {
                double x = part[m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
                if (lane == 0) red[m * kWarps + warp] = x;
            }
            __syncthreads();
            if (threadIdx.x < MR) {
                double tot = 0.0;
                for (int w = 0; w < kWarps; w++) tot += red[threadIdx.x * kWarps + w];
                red[MR * kWarps + threadIdx.x] = tot;
            }
            __syncthreads();
        };
        auto inv_rms = [&](int m, float eps) {
            const float ms = r16d(red[MR * kWarps + m] / (double)K), denom = r16(ms + eps);
            return r16d(1.0 / sqrt((double)denom));
        };
        const int kpad = p.k_tiles * 128;
        constexpr int EPT = 8;  // elements per thread the fast path keeps in registers
        if (MR * K <= EPT * kWarps * 32) {
            // Fast path: every operand of the chain is fetched in one round of loads.
            // The loads are unconditional, from clamped (always valid) addresses, and nothing uses a
            // loaded value before all of them are issued: a use inside a branch would make each load
            // wait for the one before it.
            float xs[EPT], rs[EPT], w1s[EPT], w2s[EPT];
            int ms[EPT], ks[EPT];
            __half hx[EPT], hr[EPT], h1[EPT], h2[EPT];
            const __half* res_p = p.res ? p.res : p.a;
            const __half* w1_p = p.w1 ? p.w1 : p.a;
            const __half* w2_p = p.w2 ? p.w2 : p.a;
            const long long last_row = p.m_total - 1;
#pragma unroll
            for (int e = 0; e < EPT; e++) {
                const int i = threadIdx.x + e * (kWarps * 32);
                const bool in = i < MR * K;
                const int ic = in ? i : MR * K - 1;
                const int m = ic / K, kk = ic - m * K;
                const long long row = p.m0 + m < last_row ? p.m0 + m : last_row;
                ms[e] = in ? m : -1;
                ks[e] = kk;
                hx[e] = p.a[row * p.k + kk];
                hr[e] = res_p[row * p.k + kk];
                h1[e] = w1_p[kk];
                h2[e] = w2_p[kk];
            }
#pragma unroll
            for (int e = 0; e < EPT; e++) {
                const bool row_ok = ms[e] >= 0 && p.m0 + ms[e] < p.m_total;
                xs[e] = row_ok ? __half2float(hx[e]) : 0.f;
                rs[e] = row_ok && p.res ? __half2float(hr[e]) : 0.f;
                w1s[e] = __half2float(h1[e]);
                w2s[e] = __half2float(h2[e]);
            }
            double* red_a = red;
            double* red_b = red + MR * kWarps;
            const double inv_k = 1.0 / (double)K;
            auto sums = [&](double* buf, float (&inv)[MR], float eps) {  // Σ r16(x²) per row over the CTA → 1/rms
                double part[MR];
#pragma unroll
                for (int m = 0; m < MR; m++) part[m] = 0.0;
#pragma unroll
                for (int e = 0; e < EPT; e++)
#pragma unroll
                    for (int m = 0; m < MR; m++)
                        if (ms[e] == m) part[m] += (double)r16(xs[e] * xs[e]);
#pragma unroll
                for (int m = 0; m < MR; m++) {
                    double x = part[m];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
                    if (lane == 0) buf[m * kWarps + warp] = x;
                }
                __syncthreads();
#pragma unroll
                for (int m = 0; m < MR; m++) {
                    double tot = 0.0;
#pragma unroll
                    for (int w = 0; w < kWarps; w++) tot += buf[m * kWarps + w];
                    // tot·(1/K) and rsqrt instead of the divisions: within an ulp of f64 of the interpreter's
                    // values, i.e. the same f16 after rounding, and a good deal shorter on this latency path
                    const float msq = r16d(tot * inv_k), denom = r16(msq + eps);
                    inv[m] = r16d(rsqrt((double)denom));
                }
            };
            auto add_res = [&]() {
#pragma unroll
                for (int e = 0; e < EPT; e++) {
                    if (ms[e] < 0 || p.m0 + ms[e] >= p.m_total) continue;
                    xs[e] = r16(xs[e] + rs[e]);
                    if (p.sum_out && blockIdx.x == 0) p.sum_out[(p.m0 + ms[e]) * p.k + ks[e]] = __float2half_rn(xs[e]);
                }
            };
            if (p.w1) {
                float inv[MR];
                sums(red_a, inv, p.eps1);
#pragma unroll
                for (int e = 0; e < EPT; e++)
#pragma unroll
                    for (int m = 0; m < MR; m++)
                        if (ms[e] == m) xs[e] = r16(r16(xs[e] * inv[m]) * w1s[e]);
            }
            if (p.res) add_res();
            if (p.w2) {
                float inv[MR];
                sums(red_b, inv, p.eps2);
#pragma unroll
                for (int e = 0; e < EPT; e++)
#pragma unroll
                    for (int m = 0; m < MR; m++)
                        if (ms[e] == m) xs[e] = r16(xs[e] * inv[m]) * w2s[e];
            }
            // f16, fragment order; the tail of the last k tile is cleared first
            for (int i = K + threadIdx.x; i < kpad; i += blockDim.x) {
                const int kt = i >> 7, ct = (i >> 5) & 3, cm = (i >> 3) & 3, e8 = i & 7;
#pragma unroll
                for (int m = 0; m < MR; m++) ah[(((kt * 4 + cm) * MR + m) * 4 + ct) * 8 + e8] = __float2half(0.f);
            }
#pragma unroll
            for (int e = 0; e < EPT; e++) {
                if (ms[e] < 0) continue;
                const int kk = ks[e], kt = kk >> 7, ct = (kk >> 5) & 3, cm = (kk >> 3) & 3, e8 = kk & 7;
                ah[(((kt * 4 + cm) * MR + ms[e]) * 4 + ct) * 8 + e8] = __float2half_rn(xs[e]);
            }
            __syncthreads();  // the scratch becomes the output staging from here on
        } else {
        double part[MR];
#pragma unroll
        for (int m = 0; m < MR; m++) part[m] = 0.0;
        // pass A: fetch (with the residual already added when there is no first norm)
        for (int i = threadIdx.x; i < MR * K; i += blockDim.x) {
            const int m = i / K, kk = i - m * K;
            float x = 0.f;
            if (p.m0 + m < p.m_total) {
                x = __half2float(p.a[(p.m0 + m) * p.k + kk]);
                if (!p.w1 && p.res) {
                    x = r16(x + __half2float(p.res[(p.m0 + m) * p.k + kk]));
                    if (p.sum_out && blockIdx.x == 0) p.sum_out[(p.m0 + m) * p.k + kk] = __float2half_rn(x);
                }
            }
            v[i] = x;
#pragma unroll
            for (int mm = 0; mm < MR; mm++)
                if (mm == m) part[mm] += (double)r16(x * x);
        }
        if (p.w1) {
            block_sums(part);
            float inv[MR];
#pragma unroll
            for (int m = 0; m < MR; m++) {
                inv[m] = inv_rms(m, p.eps1);
                part[m] = 0.0;
            }
            // pass B: first norm, residual add
            for (int i = threadIdx.x; i < MR * K; i += blockDim.x) {
                const int m = i / K, kk = i - m * K;
                float iv = 0.f;
#pragma unroll
                for (int mm = 0; mm < MR; mm++)
                    if (mm == m) iv = inv[mm];
                float x = r16(r16(v[i] * iv) * __half2float(p.w1[kk]));
                if (p.res && p.m0 + m < p.m_total) {
                    x = r16(x + __half2float(p.res[(p.m0 + m) * p.k + kk]));
                    if (p.sum_out && blockIdx.x == 0) p.sum_out[(p.m0 + m) * p.k + kk] = __float2half_rn(x);
                }
                v[i] = x;
#pragma unroll
                for (int mm = 0; mm < MR; mm++)
                    if (mm == m) part[mm] += (double)r16(x * x);
            }
        }
        float inv2[MR];
#pragma unroll
        for (int m = 0; m < MR; m++) inv2[m] = 0.f;
        if (p.w2) {
            block_sums(part);
#pragma unroll
            for (int m = 0; m < MR; m++) inv2[m] = inv_rms(m, p.eps2);
        } else {
            __syncthreads();  // pass C reads what other threads wrote to v
        }
        // pass C: second norm, f16, fragment order (zero beyond K)
        for (int i = threadIdx.x; i < MR * kpad; i += blockDim.x) {
            const int m = i / kpad, kk = i - m * kpad;
            float x = 0.f;
            if (kk < K) {
                x = v[m * K + kk];
                if (p.w2) {
                    float iv = 0.f;
#pragma unroll
                    for (int mm = 0; mm < MR; mm++)
                        if (mm == m) iv = inv2[mm];
                    x = r16(x * iv) * __half2float(p.w2[kk]);
                }
            }
            const int kt = kk >> 7, ct = (kk >> 5) & 3, cm = (kk >> 3) & 3, e = kk & 7;
            ah[(((kt * 4 + cm) * MR + m) * 4 + ct) * 8 + e] = __float2half_rn(x);
        }
        __syncthreads();  // the scratch becomes the output staging from here on
        }
    }

    ox_trace(p.err, 3);
    // lanes without an activation row read chunk 0 and ignore it
    const bool has_b = g < MR;
    const uint4* as_lane = reinterpret_cast<const uint4*>(smem) + (has_b ? g * 4 + t : 0);
    int rt = beg / p.k_tiles;  // row tile within the CTA
    const int kt0 = beg - rt * p.k_tiles;
    const uint4* ap = as_lane + kt0 * (16 * MR);
    int seg_left = p.k_tiles - kt0 < n_tiles ? p.k_tiles - kt0 : n_tiles;  // tiles to the end of this row tile's piece
    int seg_len = seg_left, consumed = 0;
    bool first_seg = true;
    int remaining = n_tiles, group = 0;
    float ca[4] = {0.f, 0.f, 0.f, 0.f}, cb[4] = {0.f, 0.f, 0.f, 0.f};
    double acc[4] = {0.0, 0.0, 0.0, 0.0};
    const __half2 sub_c = __float2half2_rn(1032.f), add_c = __float2half2_rn(-72.f);  // zero point 8

    bool ok = true;
    int st = 0, slot = 0;
    unsigned parity = 0;
    for (; st < n_stages; st++) {
        if (!mbar_wait(bars + slot * 8, parity)) {
            ok = false;
            break;
        }
        const unsigned char* rec = ring + slot * kStageBytes;
        // one tile record against the staged activations: 8 widenings + 8 MMAs on the two chains
        auto tile_product = [&](int j) {
            const uint4* wq = reinterpret_cast<const uint4*>(rec + j * kTileBytes);
            const uint4 wl = wq[lane], wh = wq[32 + lane];
            const __half2 s2 = reinterpret_cast<const __half2*>(rec + j * kTileBytes + kTileW)[lane];  // {row g, row g+8}
            const __half2 s2l = __low2half2(s2), s2h = __high2half2(s2);
            __half2 subl = sub_c, subh = sub_c, addl = add_c, addh = add_c;
            if (HAS_ZP) {
                const uchar2 z = reinterpret_cast<const uchar2*>(rec + j * kTileBytes + kTileW + kTileS)[lane];
                subl = __float2half2_rn(1024.f + (float)z.x);
                subh = __float2half2_rn(1024.f + (float)z.y);
                addl = __float2half2_rn(-64.f - (float)z.x);
                addh = __float2half2_rn(-64.f - (float)z.y);
            }
            const uint4 av0 = ap[0], av1 = ap[4 * MR], av2 = ap[8 * MR], av3 = ap[12 * MR];
            unsigned al[4], ah[4];
            widen_word(wl.x, subl, addl, s2l, al);
            widen_word(wh.x, subh, addh, s2h, ah);
            mma16816s(ca, al[0], ah[0], al[1], ah[1], av0.x, av0.y);
            mma16816s(cb, al[2], ah[2], al[3], ah[3], av0.z, av0.w);
            widen_word(wl.y, subl, addl, s2l, al);
            widen_word(wh.y, subh, addh, s2h, ah);
            mma16816s(ca, al[0], ah[0], al[1], ah[1], av1.x, av1.y);
            mma16816s(cb, al[2], ah[2], al[3], ah[3], av1.z, av1.w);
            widen_word(wl.z, subl, addl, s2l, al);
            widen_word(wh.z, subh, addh, s2h, ah);
            mma16816s(ca, al[0], ah[0], al[1], ah[1], av2.x, av2.y);
            mma16816s(cb, al[2], ah[2], al[3], ah[3], av2.z, av2.w);
            widen_word(wl.w, subl, addl, s2l, al);
            widen_word(wh.w, subh, addh, s2h, ah);
            mma16816s(ca, al[0], ah[0], al[1], ah[1], av3.x, av3.y);
            mma16816s(cb, al[2], ah[2], al[3], ah[3], av3.z, av3.w);
            ap += 16 * MR;
        };
        auto fold = [&]() {  // f32 tile sums → f64 running sum
#pragma unroll
            for (int q = 0; q < 4; q++) {
                acc[q] += (double)(ca[q] + cb[q]);
                ca[q] = 0.f;
                cb[q] = 0.f;
            }
            group = 0;
        };
        auto end_of_piece = [&]() {  // the row tile's piece is complete: hand it over, start the next row tile
            if (seg_len == p.k_tiles) {
                stream_stage<MR>(aux, acc, rt, lane);
            } else {
                double2* mine = reinterpret_cast<double2*>(pieces + (warp * 2 + (first_seg ? 0 : 1)) * 128) + 2 * lane;
                mine[0] = make_double2(acc[0], acc[1]);
                mine[1] = make_double2(acc[2], acc[3]);
            }
            acc[0] = acc[1] = acc[2] = acc[3] = 0.0;
            rt++;
            ap = as_lane;
            first_seg = false;
            const int rest = n_tiles - consumed;
            seg_left = p.k_tiles < rest ? p.k_tiles : rest;
            seg_len = seg_left;
        };
        if (ST > 1 && remaining >= ST && seg_left >= ST) {
            // the whole stage lies inside one row tile's piece: no per-tile bookkeeping
#pragma unroll
            for (int j = 0; j < ST; j++) tile_product(j);
            seg_left -= ST;
            consumed += ST;
            fold();  // chains of ST tiles (never longer than kFoldTiles − 1 + ST with what the other path left)
            if (seg_left == 0) end_of_piece();
        } else {
#pragma unroll
            for (int j = 0; j < ST; j++) {
                if (j < remaining) {
                    tile_product(j);
                    group++;
                    seg_left--;
                    if (group >= kFoldTiles || seg_left == 0) fold();
                    consumed++;
                    if (seg_left == 0) end_of_piece();
                }
            }
        }
        remaining -= ST;
        __syncwarp();  // every lane is done with this stage before it is refilled
        if (lane == 0 && st + NS < n_stages) issue(st + NS, slot);
        if (++slot == NS) {
            slot = 0;
            parity ^= 1;
        }
    }
    if (!ok) {
        // A copy did not land in time. Record it, then give the copies still in
        // flight a last bounded chance to land before this warp's ring goes away.
        if (lane == 0) report(p.err, ERR_WAIT_TIMEOUT, p.node, (long long)blockIdx.x, (long long)st);
        const int issued = st + NS < n_stages ? st + NS : n_stages;
        for (int s = st; s < issued; s++) mbar_wait(bars + (s % NS) * 8, (s / NS) & 1);
    }

    ox_trace(p.err, 4);
    // Row tiles cut by a boundary between two warps' ranges: the warp after the
    // first boundary inside the row tile adds the pieces in range order.
    __syncthreads();
    const int b = warp * per;  // boundary before this warp's range
    if (warp > 0 && b < cta_tiles && b % p.k_tiles != 0) {
        const int r = b / p.k_tiles, t0 = r * p.k_tiles;
        if ((warp - 1) * per <= t0) {
            const int j0 = t0 / per, j1 = (t0 + p.k_tiles - 1) / per;
            double sum[4] = {0.0, 0.0, 0.0, 0.0};
            for (int w = j0; w <= j1; w++) {
                // a warp's first piece lies in the row tile its range starts in
                const double2* src2 = reinterpret_cast<const double2*>(pieces + (w * 2 + (w * per >= t0 ? 0 : 1)) * 128) + 2 * lane;
                const double2 v0 = src2[0], v1 = src2[1];
                sum[0] += v0.x;
                sum[1] += v0.y;
                sum[2] += v1.x;
                sum[3] += v1.y;
            }
            stream_stage<MR>(aux, sum, r, lane);
        }
    }
    __syncthreads();

    ox_trace(p.err, 5);
    // Staged results → global memory, consecutive threads on consecutive rows.
    if (p.geglu == 0) {
        for (int i = threadIdx.x; i < cta_rts * 16 * MR; i += blockDim.x) {
            const int col = i / (cta_rts * 16), rr = i - col * (cta_rts * 16);  // rr = row within the CTA
            const int rtg = cta_rt0 + (rr >> 4);
            int seg = 0;
            if (p.n_seg > 1 && rtg >= p.seg_rt0[1]) seg = 1;
            if (p.n_seg > 2 && rtg >= p.seg_rt0[2]) seg = 2;
            const long long row = (long long)(rtg - p.seg_rt0[seg]) * 16 + (rr & 15), mrow = p.m0 + col;
            if (row < p.seg_n[seg] && mrow < p.m_total) p.y[seg][mrow * p.seg_n[seg] + row] = __float2half_rn(aux[rr * MR + col]);
        }
    } else {
        // row tiles alternate gate, up: pair j of the CTA holds rows 16·(cta_rt0/2 + j) … of both
        const int pairs = cta_rts / 2;
        for (int i = threadIdx.x; i < pairs * 16 * MR; i += blockDim.x) {
            const int col = i / (pairs * 16), rr = i - col * (pairs * 16);
            const int pj = rr >> 4, r = rr & 15;
            const long long row = (long long)(cta_rt0 / 2 + pj) * 16 + r, mrow = p.m0 + col;
            if (row < p.seg_n[0] && mrow < p.m_total) {
                const float gate = aux[((2 * pj) * 16 + r) * MR + col], up = aux[((2 * pj + 1) * 16 + r) * MR + col];
                p.y[0][mrow * p.seg_n[0] + row] = __float2half_rn(geglu_value(p, gate, up));
            }
        }
    }
    ox_trace(p.err, 6);
}

size_t nbits_tiled_bytes(long long n, long long n_blocks, bool has_zp) {
    const long long row_tiles = (n + 15) / 16, k_tiles = (n_blocks + 3) / 4;
    return (size_t)(row_tiles * k_tiles) * (size_t)(kTileW + kTileS + (has_zp ? kTileZ : 0));
}

void emit_nbits_pack_tiles(Emitter& em, Buf w, Buf scales, Buf zp, Buf dst, long long n, long long n_blocks, bool has_zp,
                           long long rt_mul, long long rt_add) {
    PackP p{};
    p.n = n;
    p.nb = n_blocks;
    p.row_tiles = (n + 15) / 16;
    p.k_tiles = (n_blocks + 3) / 4;
    p.rt_mul = rt_mul;
    p.rt_add = rt_add;
    p.tile_bytes = kTileW + kTileS + (has_zp ? kTileZ : 0);
    em.launch(nbits_pack_tiles, dim3(grid_for(p.row_tiles * p.k_tiles * 64, 256)), dim3(256), 0, p,
              {{&p.w, w}, {&p.scales, scales}, {&p.zp, has_zp ? zp : Buf{kSlotNull, 0}}, {&p.dst, dst}}, "nbits_pack_tiles");
}

namespace {

int env_int(const char* name, int dflt, int lo, int hi) {
    const char* e = std::getenv(name);
    int v = e ? std::atoi(e) : dflt;
    return v < lo ? lo : (v > hi ? hi : v);
}

using StreamFn = void (*)(const StreamP);
constexpr int kSmallStageTiles = 1, kSmallStages = 3;
template <bool Z> StreamFn stream_fn(int mr, bool small_ring) {
    if (small_ring) {
        switch (mr) {
            case 2: return nbits_stream<2, Z, kSmallStageTiles, kSmallStages>;
            case 4: return nbits_stream<4, Z, kSmallStageTiles, kSmallStages>;
            case 8: return nbits_stream<8, Z, kSmallStageTiles, kSmallStages>;
            default: break;
        }
    }
    switch (mr) {
        case 1: return nbits_stream<1, Z>;
        case 2: return nbits_stream<2, Z>;
        case 4: return nbits_stream<4, Z>;
        default: return nbits_stream<8, Z>;
    }
}

constexpr size_t kSmemBudget = 200 * 1024;

float to_f16(double v) { return __half2float(__double2half(v)); }

}  // namespace

// More than 8 activation rows: the prologue and the epilogue run as their own launches around the
// tensor-core GEMM, which reads the weight stream once per 256 rows instead of once per 8.
static void emit_nbits_group_gemm(Emitter& em, const NBitsGroup& gr, const TRef& a, const TRef& tiles) {
    auto scratch_like = [&](long long rows, long long cols) {
        TRef t;
        t.buf = em.scratch((size_t)(rows * cols * 2));
        t.dtype = DT_F16;
        t.shape = {rows, cols};
        return t;
    };
    TRef cur = a;
    cur.shape = {gr.m, gr.k};
    if (gr.w1) {
        TRef t = scratch_like(gr.m, gr.k);
        emit_rmsnorm(em, cur, *gr.w1, t, gr.eps1, nullptr, nullptr);
        cur = t;
    }
    if (gr.res) {
        if (!gr.w2) throw std::runtime_error("MatMulNBits group: a residual add without the norm after it");
        TRef t = scratch_like(gr.m, gr.k);
        TRef res = *gr.res, sum = *gr.sum_out;
        res.shape = sum.shape = {gr.m, gr.k};
        emit_rmsnorm(em, cur, *gr.w2, t, gr.eps2, &res, &sum);
        cur = t;
    } else if (gr.w2) {
        TRef t = scratch_like(gr.m, gr.k);
        emit_rmsnorm(em, cur, *gr.w2, t, gr.eps2, nullptr, nullptr);
        cur = t;
    }
    NBitsGroup g2 = gr;
    g2.geglu = 0;
    g2.w1 = g2.w2 = g2.res = g2.sum_out = nullptr;
    if (gr.geglu) {
        g2.y[0] = scratch_like(gr.m, gr.seg_n[0]);
        g2.y[1] = scratch_like(gr.m, gr.seg_n[1]);
    }
    emit_nbits_gemm_tc(em, g2, cur, tiles, gr.geglu != 0);
    if (gr.geglu) emit_gelu(em, g2.y[0], gr.y[0], gr.geglu == 1, &g2.y[1]);
}

void emit_nbits_group(Emitter& em, const NBitsGroup& gr, const TRef& a, const TRef& tiles) {
    if (gr.m == 0) return;
    static const int gemm_from = env_int("ONYXIA_GEMM_FROM_ROWS", 9, 1, 1 << 30);  // diagnostics: rows at which the GEMM takes over
    if (gr.m >= gemm_from) {
        emit_nbits_group_gemm(em, gr, a, tiles);
        return;
    }
    StreamP p{};
    p.m_total = gr.m;
    p.k = gr.k;
    p.k_tiles = (int)(((gr.k + 31) / 32 + 3) / 4);
    p.n_seg = gr.n_seg;
    p.geglu = gr.geglu;
    int rt = 0;
    for (int i = 0; i < gr.n_seg; i++) {
        p.seg_n[i] = gr.seg_n[i];
        p.seg_rt0[i] = rt;
        rt += (int)((gr.seg_n[i] + 15) / 16);
    }
    p.seg_rt0[gr.n_seg] = rt;
    p.row_tiles = rt;  // GeGLU: gate and up row tiles interleaved, the same count
    if (gr.geglu && (gr.n_seg != 2 || gr.seg_n[0] != gr.seg_n[1])) throw std::runtime_error("GeGLU epilogue needs two equal segments");
    const int tile_bytes = kTileW + kTileS + (gr.has_zp ? kTileZ : 0);
    p.node = em.node;
    p.eps1 = to_f16(gr.eps1);
    p.eps2 = to_f16(gr.eps2);
    p.c_half = to_f16(0.5);
    p.c_one = to_f16(1.0);
    p.c_coef = to_f16(0.044715);
    p.c_k = to_f16(std::sqrt(2.0 / 3.14159265358979323846));
    p.c_inv_sqrt2 = to_f16(0.70710678118654752440);

    // tuning knob: resident CTAs per SM the grid should fill
    static const int ctas_per_sm = env_int("ONYXIA_GEMV_CTAS_PER_SM", 2, 1, 8);
    auto split = [&](int per_sm, int* rts, long long* grid, long long* load) {
        const long long sms = sm_count();
        *rts = (int)((p.row_tiles + sms * per_sm - 1) / (sms * per_sm));
        if (gr.geglu) *rts = (*rts + 1) & ~1;  // a CTA holds whole gate/up pairs
        *grid = (p.row_tiles + *rts - 1) / *rts;
        *load = ((*grid + sms - 1) / sms) * *rts;  // row tiles the busiest SM streams
    };
    long long grid, load;
    split(ctas_per_sm, &p.rts_per_cta, &grid, &load);
    // With a long K a CTA's fixed costs (staging K activations, the fold) are large: if one CTA per SM
    // balances as well, take that.
    if (p.k_tiles >= 64 && ctas_per_sm > 1) {
        int rts1;
        long long grid1, load1;
        split(1, &rts1, &grid1, &load1);
        if (load1 <= load) {
            p.rts_per_cta = rts1;
            grid = grid1;
        }
    }

    // Two CTAs per SM and more row tiles than CTA slots: deal the row tiles as evenly as whole tiles allow — every CTA
    // ⌊tiles / slots⌋ of them, the first ones one more (a gate/up pair more) — instead of ⌈tiles / slots⌉ to as many
    // CTAs as that takes, which leaves SMs with one CTA beside SMs with two full ones.
    p.rts_extra = 1 << 30;
    p.rts_step = 0;
    {
        const long long slots = (long long)sm_count() * ctas_per_sm;
        const int step = gr.geglu ? 2 : 1;
        long long base = p.row_tiles / slots;
        if (gr.geglu) base &= ~1LL;
        if (grid < slots && base >= step && p.rts_per_cta == base + step && ctas_per_sm > 1) {
            const long long extra = (p.row_tiles - base * slots + step - 1) / step;  // CTAs with the larger share
            if (extra > 0 && extra < slots) {
                p.rts_extra = (int)extra;
                p.rts_step = step;
                grid = slots;
            }
        }
    }

    const bool prologue = gr.w1 || gr.res || gr.w2;
    const size_t fixed = (size_t)kWarps * kStages * kStageTiles * tile_bytes + (size_t)kWarps * kStages * 8 +
                         (size_t)kWarps * 2 * 128 * sizeof(double);
    auto aux_bytes = [&](int mr) {
        size_t stage = (size_t)p.rts_per_cta * 16 * mr * 4;
        size_t pro = prologue ? (((size_t)mr * gr.k + 1) & ~(size_t)1) * 4 + (size_t)(2 * mr * kWarps + mr) * 8 : 0;
        return (std::max(stage, pro) + 127) / 128 * 128;
    };
    // activation rows per pass: as many (≤ 8) as fit beside the rings
    int rows_per_pass = 8;
    while (rows_per_pass > 1 && (size_t)p.k_tiles * 256 * rows_per_pass + aux_bytes(rows_per_pass) + fixed > kSmemBudget) rows_per_pass /= 2;
    if ((size_t)p.k_tiles * 256 + aux_bytes(1) + fixed > kSmemBudget) throw std::runtime_error("MatMulNBits: K too large for the streaming kernel");

    const Buf null{kSlotNull, 0};
    for (long long m0 = 0; m0 < gr.m; m0 += rows_per_pass) {
        const long long rows = std::min<long long>(rows_per_pass, gr.m - m0);
        const int mr = rows <= 1 ? 1 : rows <= 2 ? 2 : rows <= 4 ? 4 : 8;
        p.m0 = m0;
        p.act_bytes = (p.k_tiles * 256 * mr + 127) / 128 * 128;
        p.aux_bytes = (int)aux_bytes(mr);
        size_t smem = (size_t)p.act_bytes + p.aux_bytes + fixed;
        // several activation rows: if the full rings leave room for one CTA per SM only and a third of them for two,
        // take the small rings (the kernel is bound by the instructions of the widening, not by bytes in flight)
        const size_t fixed_small = (size_t)kWarps * kSmallStages * kSmallStageTiles * tile_bytes + (size_t)kWarps * kSmallStages * 8 +
                                   (size_t)kWarps * 2 * 128 * sizeof(double);
        const size_t two_per_sm = 112 * 1024;
        static const bool small_off = env_int("ONYXIA_GEMV_SMALL_RING", 1, 0, 1) == 0;  // diagnostics
        const bool small_ring = mr > 1 && !small_off && grid > sm_count() /* CTAs do share SMs */ && smem > two_per_sm &&
                                (size_t)p.act_bytes + p.aux_bytes + fixed_small <= two_per_sm;
        if (small_ring) smem = (size_t)p.act_bytes + p.aux_bytes + fixed_small;
        StreamFn fn = gr.has_zp ? stream_fn<true>(mr, small_ring) : stream_fn<false>(mr, small_ring);
        if (smem > 48 * 1024) ensure_max_dynamic_smem((const void*)fn, (int)kSmemBudget);
        em.launch(fn, dim3((unsigned)grid), dim3(kWarps * 32), (unsigned)smem, p,
                  {{&p.a, a.buf}, {&p.tiles, tiles.buf}, {&p.err, Buf{kSlotErr, 0}}, {&p.y[0], gr.y[0].buf},
                   {&p.y[1], gr.n_seg > 1 && !gr.geglu ? gr.y[1].buf : null}, {&p.y[2], gr.n_seg > 2 ? gr.y[2].buf : null},
                   {&p.w1, gr.w1 ? gr.w1->buf : null}, {&p.res, gr.res ? gr.res->buf : null},
                   {&p.sum_out, gr.sum_out ? gr.sum_out->buf : null}, {&p.w2, gr.w2 ? gr.w2->buf : null}},
                  "nbits_stream", /*pdl=*/true);
    }
    // One activation row, default zero points: the launch can also run as an operation of the persistent step kernel.
    if (gr.m == 1 && !gr.has_zp && (!gr.res || gr.sum_out)) {
        auto op = std::make_shared<PersistOp>();
        op->kind = POP_GEMV;
        op->node = em.node;
        op->a = a.buf;
        op->tiles = tiles.buf;
        op->n_seg = gr.n_seg;
        op->geglu = gr.geglu;
        op->k = gr.k;
        for (int i = 0; i < gr.n_seg; i++) {
            op->seg_n[i] = gr.seg_n[i];
            if (!gr.geglu || i == 0) op->y[i] = gr.y[i].buf;
        }
        op->has_w1 = gr.w1 != nullptr;
        op->has_w2 = gr.w2 != nullptr;
        op->has_res = gr.res != nullptr;
        if (gr.w1) op->w1 = gr.w1->buf;
        if (gr.w2) op->w2 = gr.w2->buf;
        if (gr.res) op->res = gr.res->buf;
        if (gr.sum_out) op->sum_out = gr.sum_out->buf;
        op->eps1 = gr.eps1;
        op->eps2 = gr.eps2;
        em.recs.back().pop = std::move(op);
    }
}

void emit_matmul_nbits_stream(Emitter& em, const NBitsDesc& d, const TRef& a, const TRef& tiles, const TRef& y) {
    NBitsGroup gr{};
    gr.m = d.m;
    gr.k = d.k;
    gr.has_zp = d.has_zp;
    gr.n_seg = 1;
    gr.seg_n[0] = d.n;
    gr.y[0] = y;
    emit_nbits_group(em, gr, a, tiles);
}

}  // namespace oxk
