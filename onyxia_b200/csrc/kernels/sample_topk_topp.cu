// Temperature / top-k / top-p (nucleus) sampling of one token per row of logits, on the device.
// Semantics: crates/onyxia-cli/src/sampling.rs:36-195 — logits divided by the temperature; top-k keeps
// the k largest (k ≥ vocabulary: everything), else top-p with 0 < p < 1 keeps the shortest prefix of
// the descending order whose cumulative softmax probability reaches p, else everything is kept; the
// token is the first index, in index order, at which the running sum of exp(l − max) over the kept
// entries reaches u · Σ, u being the caller's uniform number in [0, 1] (the reference draws it as
// next_u32 / u32::MAX from its own generator; the generator stays with the caller).
//
// Differences from the reference, both confined to ties of the arithmetic, not of the distribution:
// where it breaks ties among equal logits by an unstable selection, equal logits are kept in index
// order here; where it accumulates f32 sums one element after the other, the sums here are exact —
// exp(l − max) ∈ [0, 1] is taken as an integer multiple of 2⁻⁴⁰ and added as integers, so the result
// does not depend on how the entries are spread over threads and is the same on every run. A draw
// whose u · Σ falls within f32 rounding of a boundary between two tokens may therefore pick the
// neighbour of the reference's token.
//
// One CTA of 1024 threads per row. The cut-off value of top-k / top-p is found by a radix selection
// over the order-preserving integer image of the scaled logit (four passes of 8 bits; per pass a
// 256-bin histogram of counts and of probability mass in shared memory), then one pass forms the
// running sum: thread t owns the contiguous indices [t·chunk, (t+1)·chunk), the chunk sums are scanned
// across the CTA and the owner of the target walks its chunk.
#include "common.cuh"
#include "kernels.hpp"

namespace oxk {

namespace {

constexpr int kST = 1024;
constexpr double kUnit = 1099511627776.0;  // 2⁴⁰

struct SampleP {
    const void* x;       // [rows, cols] logits
    long long* y;        // [rows] token ids
    const float* u;      // [rows] uniform numbers in [0, 1]
    ErrWord* err;
    long long rows, cols;
    float temperature;
    long long top_k;     // 0 = off
    float top_p;         // outside (0, 1) = off
    int node;
};

// Descending order of floats as ascending order of unsigned keys: key(a) < key(b) ⇔ a > b.
__device__ __forceinline__ unsigned desc_key(float v) {
    const unsigned b = __float_as_uint(v);
    const unsigned asc = (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // ascending image
    return ~asc;
}

__device__ __forceinline__ unsigned long long mass_of(float scaled, float mx) {
    return (unsigned long long)((double)expf(scaled - mx) * kUnit);
}

// Exclusive scan of one value per thread over the CTA; `total` gets the sum. `tmp` holds kST / 32 values.
__device__ __forceinline__ unsigned long long block_scan(unsigned long long v, unsigned long long* tmp, unsigned long long* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    if (lane == 31) tmp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        unsigned long long w = tmp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long n = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += n;
        }
        tmp[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const unsigned long long before = warp ? tmp[warp - 1] : 0ull;
    *total = tmp[kST / 32 - 1];
    __syncthreads();
    return before + inc - v;
}

template <int DT> __global__ void __launch_bounds__(kST) sample_row(const SampleP p) {
    __shared__ unsigned long long hist_mass[256];
    __shared__ unsigned hist_cnt[256];
    __shared__ unsigned long long scan_tmp[kST / 32];
    __shared__ float red_f[kST / 32];
    __shared__ unsigned sel_prefix, sel_bucket;
    __shared__ unsigned long long sel_rem_mass;
    __shared__ long long sel_rem_cnt;
    const long long row = blockIdx.x, base = row * p.cols;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float temp = p.temperature;
    auto scaled_at = [&](long long c) { return ld<DT>(p.x, base + c) / temp; };

    // ── the largest finite scaled logit ──
    float mx = -INFINITY;
    for (long long c = tid; c < p.cols; c += kST) {
        const float v = scaled_at(c);
        if (isfinite(v)) mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    if (lane == 0) red_f[warp] = mx;
    __syncthreads();
    mx = red_f[0];
#pragma unroll
    for (int w = 1; w < kST / 32; w++) mx = fmaxf(mx, red_f[w]);
    __syncthreads();
    if (!(mx > -INFINITY)) {  // "All logits are NaN or Inf, cannot sample" (sampling.rs:41-44)
        if (tid == 0) {
            report(p.err, ERR_SAMPLE_NO_FINITE, p.node, row, p.cols);
            p.y[row] = 0;
        }
        return;
    }

    // ── the cut: entries with key < cut_key are kept, and the first `cut_ties` entries (in index order) whose
    //    key equals cut_key ──
    const bool use_k = p.top_k > 0 && p.top_k < p.cols;
    const bool use_p = !(p.top_k > 0) && p.top_p > 0.f && p.top_p < 1.f;
    unsigned cut_key = 0xFFFFFFFFu;      // keep everything finite
    long long cut_ties = p.cols;
    if (use_k || use_p) {
        // top-p works on probability mass: the target is p · Σ over all finite entries
        unsigned long long target_mass = 0ull;
        if (use_p) {
            unsigned long long mine = 0ull, total;
            for (long long c = tid; c < p.cols; c += kST) {
                const float v = scaled_at(c);
                if (isfinite(v)) mine += mass_of(v, mx);
            }
            block_scan(mine, scan_tmp, &total);
            target_mass = (unsigned long long)((double)p.top_p * (double)total);
            if (target_mass < 1ull) target_mass = 1ull;
        }
        if (tid == 0) {
            sel_prefix = 0u;
            sel_rem_mass = target_mass;
            sel_rem_cnt = p.top_k;
        }
        __syncthreads();
        for (int pass = 0; pass < 4; pass++) {
            const int shift = 24 - 8 * pass;
            for (int i = tid; i < 256; i += kST) {
                hist_mass[i] = 0ull;
                hist_cnt[i] = 0u;
            }
            __syncthreads();
            const unsigned prefix = sel_prefix, high_mask = pass ? 0xFFFFFFFFu << (shift + 8) : 0u;
            for (long long c = tid; c < p.cols; c += kST) {
                const float v = scaled_at(c);
                if (!isfinite(v)) continue;
                const unsigned key = desc_key(v);
                if ((key & high_mask) != prefix) continue;
                const unsigned b = (key >> shift) & 0xFFu;
                atomicAdd(&hist_cnt[b], 1u);
                if (use_p) atomicAdd(&hist_mass[b], mass_of(v, mx));
            }
            __syncthreads();
            if (tid == 0) {
                // walk the buckets in descending-logit order until the remaining target falls inside one
                unsigned b = 0;
                if (use_k) {
                    long long rem = sel_rem_cnt;
                    for (; b < 255u && (long long)hist_cnt[b] < rem; b++) rem -= hist_cnt[b];
                    sel_rem_cnt = rem;
                } else {
                    unsigned long long rem = sel_rem_mass;
                    for (; b < 255u && hist_mass[b] < rem; b++) rem -= hist_mass[b];
                    sel_rem_mass = rem;
                }
                sel_bucket = b;
                sel_prefix = prefix | (b << shift);
            }
            __syncthreads();
        }
        cut_key = sel_prefix;
        if (use_k) cut_ties = sel_rem_cnt;  // how many of the entries equal to the k-th largest are still needed
        // top-p: resolved below, once the ties have been counted
    }

    // ── index-order pass: which entries are kept, their mass, the draw ──
    const long long chunk = (p.cols + kST - 1) / kST;
    const long long c0 = (long long)tid * chunk, c1 = c0 + chunk < p.cols ? c0 + chunk : p.cols;
    // ties at the cut, counted per chunk so that they can be ranked in index order
    unsigned long long my_ties = 0ull, tie_mass = 0ull;
    for (long long c = c0; c < c1; c++) {
        const float v = scaled_at(c);
        if (isfinite(v) && desc_key(v) == cut_key) {
            my_ties++;
            tie_mass = mass_of(v, mx);
        }
    }
    unsigned long long ties_total;
    const unsigned long long ties_before = block_scan(my_ties, scan_tmp, &ties_total);
    if (use_p) {
        // every tie has the same mass; the number needed is ⌈remaining / mass⌉ (at least one: the bucket walk stopped here)
        unsigned long long m_each = tie_mass;
        // a thread without ties does not know the mass: take it from any thread that has some
        __shared__ unsigned long long tie_mass_sh;
        if (tid == 0) tie_mass_sh = 0ull;
        __syncthreads();
        if (my_ties) atomicMax(&tie_mass_sh, m_each);
        __syncthreads();
        m_each = tie_mass_sh;
        const unsigned long long rem = sel_rem_mass;
        long long need = m_each ? (long long)((rem + m_each - 1) / m_each) : (long long)ties_total;
        if (need < 1) need = 1;
        cut_ties = need;
    }
    auto kept = [&](float v, unsigned long long tie_rank) {
        if (!isfinite(v)) return false;
        const unsigned key = desc_key(v);
        return key < cut_key || (key == cut_key && (long long)tie_rank < cut_ties);
    };
    unsigned long long my_mass = 0ull;
    {
        unsigned long long rank = ties_before;
        for (long long c = c0; c < c1; c++) {
            const float v = scaled_at(c);
            const bool tie = isfinite(v) && desc_key(v) == cut_key;
            if (kept(v, rank)) my_mass += mass_of(v, mx);
            if (tie) rank++;
        }
    }
    unsigned long long kept_total;
    const unsigned long long mass_before = block_scan(my_mass, scan_tmp, &kept_total);
    // first index whose running sum reaches u · Σ (sampling.rs:176-186); the fallback is the last entry
    float u = p.u[row];
    u = u < 0.f ? 0.f : (u > 1.f ? 1.f : u);
    unsigned long long target = (unsigned long long)((double)u * (double)kept_total);
    if (target > kept_total) target = kept_total;
    // u = 0: the reference's walk stops at index 0 whatever its weight (0 ≥ 0)
    if (tid == 0) p.y[row] = target == 0ull ? 0 : p.cols - 1;
    __syncthreads();
    if (target > 0ull && mass_before < target && target <= mass_before + my_mass) {
        // the target lies in this chunk: (mass_before, mass_before + my_mass]
        unsigned long long run = mass_before, rank = ties_before;
        for (long long c = c0; c < c1; c++) {
            const float v = scaled_at(c);
            const bool tie = isfinite(v) && desc_key(v) == cut_key;
            if (kept(v, rank)) {
                run += mass_of(v, mx);
                if (run >= target) {
                    p.y[row] = c;
                    break;
                }
            }
            if (tie) rank++;
        }
    }
}

}  // namespace

void emit_sample_rows(Emitter& em, const TRef& logits, const TRef& out, Buf u, float temperature, long long top_k, float top_p) {
    SampleP p{};
    p.cols = logits.shape.back();
    p.rows = p.cols ? logits.numel() / p.cols : 0;
    if (p.rows == 0) return;
    p.temperature = temperature;
    p.top_k = top_k;
    p.top_p = top_p;
    p.node = em.node;
    dim3 g((unsigned)p.rows), b(kST);
    if (logits.dtype == DT_F32)
        em.launch(sample_row<DT_F32>, g, b, 0, p, {{&p.x, logits.buf}, {&p.y, out.buf}, {&p.u, u}, {&p.err, Buf{kSlotErr, 0}}}, "sample_row");
    else
        em.launch(sample_row<DT_F16>, g, b, 0, p, {{&p.x, logits.buf}, {&p.y, out.buf}, {&p.u, u}, {&p.err, Buf{kSlotErr, 0}}}, "sample_row");
}

}  // namespace oxk
