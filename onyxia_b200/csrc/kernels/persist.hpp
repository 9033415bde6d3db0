// The persistent decode-step kernel: host-side description of the operations
// it can execute and the builder that turns a run of them into one launch.
//
// A batch-1 decode step is a chain of ~130 small dependent operations whose
// weights stream in a few hundred nanoseconds each; launched one by one, every
// link pays a launch hand-over, a cold pipeline and a store → load round trip.
// `persist_step` runs the whole chain in ONE launch of one CTA per SM:
//   * a producer warp per CTA walks the chain ahead of the arithmetic and keeps
//     the CTA's share of every weight matrix flowing from HBM into a ring in
//     shared memory (bulk asynchronous copies, one mbarrier pair per stage), so
//     the HBM stream does not stop at operation boundaries;
//   * results travel between CTAs as tagged words — an f16 pair and the step's
//     epoch in one 64-bit store — so a consumer polls the data itself instead
//     of waiting at a grid barrier and then loading (one L2 round trip per
//     link instead of three);
//   * every wait is bounded; an expired wait records ERR_WAIT_TIMEOUT, marks the
//     CTA dead (later waits return at once) and the kernel drains and exits.
// Arithmetic and rounding points are those of the separate kernels
// (nbits_stream.cu, gqa_decode.cu), i.e. of the interpreter's primitive sequence.
#pragma once
#include <memory>

#include "kernels.hpp"

namespace oxk {

// Reserved slot: the plan's exchange area (tagged words), offset = byte position.
constexpr uint32_t kSlotXbuf = 0xFFFFFFF5u;

enum : int { POP_GEMV = 1, POP_ATTN = 2 };

// One operation of a persistent run as the lowering describes it (addresses still symbolic).
struct PersistOp {
    int kind = 0;
    int node = -1;
    // ── POP_GEMV: y_i = prologue(a) · W_iᵀ over one tile stream (see NBitsGroup) ──
    Buf a, tiles, w1, w2, res, sum_out;
    Buf y[3];
    long long seg_n[3] = {0, 0, 0};
    int n_seg = 0, geglu = 0;
    long long k = 0;
    double eps1 = 0, eps2 = 0;
    bool has_w1 = false, has_w2 = false, has_res = false;
    // ── POP_ATTN: one new token over an in-place f16 cache, batch 1 ──
    Buf q, kx, vx, cache_k, cache_v, seqlens, cos, sin, out, dyn_t;
    long long H = 0, KV = 0, D = 0, cap = 0, window = -1, half = 0, cache_rows = 0, span = 0;
    float scale = 0.f;
};

inline bool same_buf(const Buf& x, const Buf& y) { return x.slot == y.slot && x.off == y.off; }
inline bool same_op(const PersistOp& x, const PersistOp& y) {
    if (x.kind != y.kind || x.node != y.node) return false;
    const Buf* bx[] = {&x.a, &x.tiles, &x.w1, &x.w2, &x.res, &x.sum_out, &x.y[0], &x.y[1], &x.y[2], &x.q, &x.kx, &x.vx,
                       &x.cache_k, &x.cache_v, &x.seqlens, &x.cos, &x.sin, &x.out, &x.dyn_t};
    const Buf* by[] = {&y.a, &y.tiles, &y.w1, &y.w2, &y.res, &y.sum_out, &y.y[0], &y.y[1], &y.y[2], &y.q, &y.kx, &y.vx,
                       &y.cache_k, &y.cache_v, &y.seqlens, &y.cos, &y.sin, &y.out, &y.dyn_t};
    for (size_t i = 0; i < sizeof(bx) / sizeof(bx[0]); i++)
        if (!same_buf(*bx[i], *by[i])) return false;
    for (int i = 0; i < 3; i++)
        if (x.seg_n[i] != y.seg_n[i]) return false;
    return x.n_seg == y.n_seg && x.geglu == y.geglu && x.k == y.k && x.eps1 == y.eps1 && x.eps2 == y.eps2 &&
           x.has_w1 == y.has_w1 && x.has_w2 == y.has_w2 && x.has_res == y.has_res && x.H == y.H && x.KV == y.KV && x.D == y.D &&
           x.cap == y.cap && x.window == y.window && x.half == y.half && x.cache_rows == y.cache_rows && x.span == y.span &&
           x.scale == y.scale;
}

// The result of fusing a run of operations.
struct PersistLaunch {
    LaunchRec rec;          // the launch (cooperative; parameters carry the operation table)
    size_t xbuf_bytes = 0;  // exchange area the launch needs (zeroed once, then reused with growing epochs)
};

// Number of operations one launch can hold.
int persist_max_ops();
// Builds the launch for ops[0..n). `epoch` addresses the 64-bit step counter the kernel tags its words with.
// Returns false (and leaves `out` alone) when the run cannot execute persistently: too few operations,
// shared memory does not fit, an operand layout the kernel does not handle.
bool build_persist_launch(const std::vector<const PersistOp*>& ops, Buf epoch, PersistLaunch* out, std::string* why);

}  // namespace oxk
