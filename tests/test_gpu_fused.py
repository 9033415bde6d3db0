"""Fused composite kernels against the CPU oracle and against their own
decompositions running on the same device (prepare with and without the fused
registry) — the pattern of crates/onyxia-backend-wgpu/tests/gpu_test.rs:376-547.
"""
import math

import numpy as np
import pytest

from onyxia_b200 import ir, models
from onyxia_b200 import backend as be
from onyxia_b200.ir import HostTensor

from gpu_util import cuda_backend, differential
from util import assert_close, assert_tensors_match, composite_module, ht

pytestmark = pytest.mark.gpu

f32, f16 = np.float32, np.float16
RNG = np.random.default_rng(99)
GQA = "com.microsoft.GroupQueryAttention"
NBITS = "com.microsoft.MatMulNBits"
ROPE = "com.microsoft.RotaryEmbedding"


def tol(dt):
    return dict(atol=2e-3, rtol=4e-3) if dt == f16 else dict(atol=1e-4, rtol=1e-3)


def adt(dt):
    return ir.F16 if dt == f16 else ir.F32


def test_backend_supports_registry_names():
    b = cuda_backend()
    for name in ("Softmax", "SimplifiedLayerNormalization", "Gelu", ROPE, "com.microsoft.GemmaRotaryEmbedding", GQA, NBITS):
        assert b.supports(name)
    assert not b.supports("Trilu")
    assert not cuda_backend(False).supports("Softmax")


@pytest.mark.parametrize("dt", [f32, f16])
@pytest.mark.parametrize("shape", [(2, 3), (5, 257), (3, 4, 1025), (1, 1, 33), (70, 31)])
def test_softmax(dt, shape):
    x = (RNG.standard_normal(shape) * 3).astype(dt)
    m, feed = composite_module("Softmax", {"axis": len(shape) - 1}, [("x", ht(x))], [(adt(dt), list(shape))])
    differential(m, feed, also_unfused=True, **tol(dt))


def test_softmax_with_masked_entries_and_other_axis():
    x = RNG.standard_normal((4, 64)).astype(f32)
    x[:, 40:] = -np.inf
    m, feed = composite_module("Softmax", {"axis": 1}, [("x", ht(x))], [(ir.F32, [4, 64])])
    differential(m, feed, also_unfused=True)
    # not the last axis: legalised through the decomposition
    m, feed = composite_module("Softmax", {"axis": 0}, [("x", ht(x[:, :8].copy()))], [(ir.F32, [4, 8])])
    differential(m, feed)


@pytest.mark.parametrize("dt", [f32, f16])
@pytest.mark.parametrize("shape", [(1, 4), (3, 5, 640), (2, 1152), (1, 1, 5376), (7, 33)])
def test_rmsnorm(dt, shape):
    x = (RNG.standard_normal(shape) * 4).astype(dt)
    w = (1 + 0.1 * RNG.standard_normal(shape[-1])).astype(dt)
    m, feed = composite_module("SimplifiedLayerNormalization", {"epsilon": 1e-6}, [("x", ht(x)), ("w", ht(w))],
                               [(adt(dt), list(shape))])
    differential(m, feed, also_unfused=True, **tol(dt))


@pytest.mark.parametrize("dt", [f32, f16])
@pytest.mark.parametrize("approx", ["tanh", "none"])
def test_gelu(dt, approx):
    x = np.concatenate([np.array([-2, -0.5, 0, 0.5, 2], dt), (RNG.standard_normal(1000) * 3).astype(dt)])
    m, feed = composite_module("Gelu", {"approximate": approx}, [("x", ht(x))], [(adt(dt), [x.size])])
    got, _ = differential(m, feed, also_unfused=True, **tol(dt))
    if approx == "none":
        assert_close(got[0][1].numpy()[:5], [-0.0455, -0.1543, 0.0, 0.3457, 1.9545], 1e-3)


@pytest.mark.parametrize("dt", [f32, f16])
def test_geglu_and_add_norm_pattern_fusions(dt):
    """Gelu→Mul and Add→RMSNorm become single launches; results equal the unfused graph."""
    b = ir.GraphBuilder()
    s = b.sym("S")
    h = 96
    x = b.input("x", adt(dt), [s, h])
    r = b.input("r", adt(dt), [s, h])
    up = b.input("up", adt(dt), [s, h])
    w = b.constant(ht((1 + 0.1 * RNG.standard_normal(h)).astype(dt)))
    summed = b.add(x, r)
    normed = b.composite("SimplifiedLayerNormalization", {"epsilon": 1e-6}, [summed, w], [(adt(dt), [s, h])])[0]
    act = b.composite("Gelu", {"approximate": "tanh"}, [normed], [(adt(dt), [s, h])])[0]
    b.output("y", b.mul(act, up))
    b.output("resid", summed)
    m = b.finish()
    feed = {k: ht((RNG.standard_normal((5, h)) * 2).astype(dt)) for k in ("x", "r", "up")}
    differential(m, feed, also_unfused=True, **tol(dt))
    sess = cuda_backend().prepare(m.clone())
    before = sess.launch_count()
    sess.run({k: sess.upload(v) for k, v in feed.items()})
    assert sess.launch_count() - before == 2  # add+norm, gelu+mul


@pytest.mark.parametrize("dt", [f32, f16])
@pytest.mark.parametrize("heads,d,half", [(1, 4, 2), (2, 4, 2), (4, 64, 32), (2, 64, 16)])
def test_rotary(dt, heads, d, half):
    bsz, seq, maxpos = 2, 5, 16
    x = RNG.standard_normal((bsz, seq, heads * d)).astype(dt)
    pos = RNG.integers(0, maxpos, (bsz, seq)).astype(np.int64)
    ang = RNG.uniform(0, 6, (maxpos, half))
    cos, sin = np.cos(ang).astype(dt), np.sin(ang).astype(dt)
    m, feed = composite_module(ROPE, {"num_heads": heads, "interleaved": 0},
                               [("x", ht(x)), ("pos", ht(pos)), ("cos", ht(cos)), ("sin", ht(sin))],
                               [(adt(dt), [bsz, seq, heads * d])])
    differential(m, feed, also_unfused=True, **tol(dt))


def test_rotary_golden_vectors_on_device():
    # decomp.rs:802-857
    x = ht(np.arange(1, 9, dtype=f32).reshape(1, 1, 8))
    cos, sin = ht(np.array([[1, 1], [0, 0]], f32)), ht(np.array([[0, 0], [1, 1]], f32))
    m, feed = composite_module(ROPE, {"num_heads": 0}, [("x", x), ("pos", ht(np.array([[1]], np.int64))), ("cos", cos), ("sin", sin)],
                               [(ir.F32, [1, 1, 8])])
    got, _ = differential(m, feed, also_unfused=True)
    assert_close(got[0][1].numpy(), [-3, -4, 1, 2, -7, -8, 5, 6], 1e-6)


# ── MatMulNBits ──────────────────────────────────────────────────────────
def test_matmul_nbits_reference_kat_on_device():
    # decomp.rs:1098-1139; block_size 4 has no fused kernel and runs through the decomposition
    k_dim, n_dim, bs = 8, 2, 4
    q = np.array([i % 16 for i in range(n_dim * k_dim)])
    scales = np.array([0.5, 0.25, 1.0, 2.0], f32)
    a = np.array([i * 0.1 for i in range(k_dim)], f32)
    m, feed = composite_module(NBITS, {"K": k_dim, "N": n_dim, "bits": 4, "block_size": bs},
                               [("a", ht(a.reshape(1, k_dim))), ("b", HostTensor.packed_u4(q, [n_dim, 2, bs])), ("s", ht(scales))],
                               [(ir.F32, [1, n_dim])])
    got, _ = differential(m, feed)
    expect = [(a * ((q[n * 8:(n + 1) * 8] - 8) * np.repeat(scales[n * 2:(n + 1) * 2], 4))).sum() for n in range(n_dim)]
    assert_close(got[0][1].numpy(), expect, 1e-4)


@pytest.mark.parametrize("dt", [f16, f32])
@pytest.mark.parametrize("m_,k,n,zp", [(1, 64, 8, False), (1, 1152, 256, True), (3, 96, 40, False), (8, 2048, 64, True),
                                        (1, 50, 7, False), (17, 128, 33, False),
                                        # few row tiles and a long K (the shape of a down projection)
                                        (1, 6912, 1152, False), (3, 4096, 48, True), (8, 3200, 272, False), (1, 3100, 20, True)])
def test_matmul_nbits_fused_vs_oracle(dt, m_, k, n, zp):
    mod, act = models.build_matmul_nbits(m_, k, n, adt(dt), seed=5, with_zp=zp)
    t = dict(atol=2e-2, rtol=4e-3) if dt == f16 else dict(atol=1e-3, rtol=1e-3)
    differential(mod, {"a": act}, also_unfused=True, **t)


def test_matmul_nbits_mixed_scale_and_activation_dtypes():
    for a_dt, s_dt in ((ir.F32, np.float16), (ir.F16, np.float32)):
        k, n, nb = 256, 24, 8
        b = ir.GraphBuilder()
        a = b.input("a", a_dt, [2, k])
        w = b.constant(HostTensor(ir.U4, [n, nb, 32], RNG.integers(0, 256, n * nb * 16, dtype=np.uint8)))
        s = b.constant(ht(RNG.uniform(0.005, 0.02, n * nb).astype(s_dt)))
        b.output("y", b.composite(NBITS, {"K": k, "N": n, "bits": 4, "block_size": 32}, [a, w, s], [(a_dt, [2, n])])[0])
        act = RNG.standard_normal((2, k)).astype(np.float16 if a_dt == ir.F16 else np.float32)
        differential(b.finish(), {"a": ht(act)}, also_unfused=True, atol=1e-2, rtol=4e-3)


def test_matmul_nbits_linearity_at_full_size():
    """Size-independent property at a benchmark shape: y(a1 + a2) = y(a1) + y(a2) for exactly representable inputs."""
    k, n = 4096, 11008
    mod, _ = models.build_matmul_nbits(1, k, n, ir.F16, seed=2)
    sess = cuda_backend().prepare(mod)
    a1 = RNG.integers(-2, 3, (1, k)).astype(f16)
    a2 = RNG.integers(-2, 3, (1, k)).astype(f16)

    def run(a):
        (_, y), = sess.run({"a": sess.upload(ht(a))})
        return sess.download(y).numpy().astype(np.float64)

    y1, y2, y12 = run(a1), run(a2), run((a1 + a2).astype(f16))
    assert np.abs(y12 - (y1 + y2)).max() <= 2e-2 + 4e-3 * np.abs(y12).max()


# ── GroupQueryAttention ──────────────────────────────────────────────────
@pytest.mark.parametrize("dt", [f32, f16])
@pytest.mark.parametrize("batch,heads,kv,d,past,seq,window,rotary", [
    (1, 4, 1, 64, 0, 5, -1, True),      # prefill from an empty cache
    (1, 4, 1, 64, 7, 1, -1, True),      # decode
    (2, 8, 2, 64, 40, 1, 16, True),     # sliding window
    (2, 4, 4, 32, 9, 3, 4, False),      # group of 1, chunked prefill with window
    (1, 32, 8, 128, 130, 1, -1, True),  # the decode-op benchmark's head geometry
    (1, 4, 1, 256, 70, 1, 32, True),    # 1B-architecture geometry
    (3, 6, 3, 64, 5, 2, -1, True),
])
def test_gqa_fused_vs_oracle(dt, batch, heads, kv, d, past, seq, window, rotary):
    mod, feed = models.build_gqa(batch, heads, kv, d, past, seq, adt(dt), window, rotary, seed=3)
    t = dict(atol=4e-3, rtol=4e-3) if dt == f16 else dict(atol=2e-4, rtol=1e-3)
    differential(mod, feed, also_unfused=True, **t)


def test_gqa_reference_golden_vectors_on_device():
    # decomp.rs:978-1014 (window) — head dim 1 has no fused kernel: decomposition path on the device
    m, feed = composite_module(
        GQA, {"num_heads": 1, "kv_num_heads": 1, "local_window_size": 2},
        [("q", ht(np.ones((1, 1, 1), f32))), ("k", ht(np.zeros((1, 1, 1), f32))), ("v", ht(np.full((1, 1, 1), 100, f32))),
         ("pk", ht(np.zeros((1, 1, 3, 1), f32))), ("pv", ht(np.array([7, 11, 13], f32).reshape(1, 1, 3, 1))),
         ("seqlens", ht(np.array([3], np.int64))), ("total", ht(np.array([4], np.int64)))],
        [(ir.F32, [1, 1, 1]), (ir.F32, [1, 1, 4, 1]), (ir.F32, [1, 1, 4, 1])])
    got, _ = differential(m, feed)
    assert_close(got[0][1].numpy(), [124.0 / 3.0], 1e-4)


@pytest.mark.parametrize("dt", [f32, f16])
def test_gqa_ragged_seqlens_with_garbage_tail(dt):
    """Rows with fewer valid past tokens than the buffer holds: the tail must not be attended, new keys land right
    after the valid past and the rest of `present` is zero (decomp.rs:1016-1096, gpu_test.rs:817-932)."""
    batch, heads, kv, d, past, seq = 3, 4, 2, 64, 6, 1
    mod, feed = models.build_gqa(batch, heads, kv, d, past, seq, adt(dt), -1, True, seed=8, max_positions=16)
    pk, pv = feed["past_key"].numpy().copy(), feed["past_value"].numpy().copy()
    valid = [6, 2, 0]
    for b_, v in enumerate(valid):
        pk[b_, :, v:, :] = 99
        pv[b_, :, v:, :] = -99
    feed["past_key"], feed["past_value"] = ht(pk), ht(pv)
    feed["seqlens_k"] = ht(np.array([v + seq - 1 for v in valid], np.int32))
    t = dict(atol=4e-3, rtol=4e-3) if dt == f16 else dict(atol=2e-4, rtol=1e-3)
    got, _ = differential(mod, feed, also_unfused=True, **t)
    present = dict(got)["present_key"].numpy()
    assert np.all(present[1, :, 3:, :] == 0) and np.all(present[2, :, 1:, :] == 0)


def test_gqa_attention_bias():
    batch, heads, kv, d, past, seq = 2, 4, 2, 32, 5, 2
    total = past + seq
    b = ir.GraphBuilder()
    names = [("q", [batch, seq, heads * d]), ("k", [batch, seq, kv * d]), ("v", [batch, seq, kv * d]),
             ("pk", [batch, kv, past, d]), ("pv", [batch, kv, past, d])]
    ids = [b.input(n, ir.F32, s) for n, s in names]
    sl = b.input("seqlens", ir.I32, [batch])
    bias = b.input("bias", ir.F32, [1, heads, seq, total])
    outs = b.composite(GQA, {"num_heads": heads, "kv_num_heads": kv, "has_attention_bias": 1}, ids + [sl, bias],
                       [(ir.F32, [batch, seq, heads * d]), (ir.F32, [batch, kv, total, d]), (ir.F32, [batch, kv, total, d])])
    for i, o in enumerate(outs):
        b.output(f"o{i}", o)
    feed = {n: ht(RNG.standard_normal(s).astype(f32)) for n, s in names}
    feed["seqlens"] = ht(np.full(batch, total - 1, np.int32))
    feed["bias"] = ht(RNG.standard_normal((1, heads, seq, total)).astype(f32))
    differential(b.finish(), feed, also_unfused=True, atol=2e-4, rtol=1e-3)


@pytest.mark.parametrize("dt", [f32, f16])
def test_gqa_kv_feedback_appends_in_place(dt):
    """present → past over several decode steps: the device cache is appended to in place (no new
    allocations once warm), every step equals the oracle, and an older handle still reads its own rows."""
    from oracle import ref
    batch, heads, kv, d, window = 2, 4, 2, 64, 5
    np_dt = dt
    b = ir.GraphBuilder()
    P, S = b.sym("P"), b.sym("S")
    q = b.input("q", adt(dt), [batch, S, heads * d])
    k = b.input("k", adt(dt), [batch, S, kv * d])
    v = b.input("v", adt(dt), [batch, S, kv * d])
    pk = b.input("past_key", adt(dt), [batch, kv, P, d])
    pv = b.input("past_value", adt(dt), [batch, kv, P, d])
    sl = b.input("seqlens_k", ir.I32, [batch])
    cfg = models.DecoderConfig("t", 0, 0, heads, kv, d, 0, 0, act_dtype=adt(dt), max_positions=64)
    c, s = models.rope_caches(cfg)
    outs = b.composite(GQA, {"num_heads": heads, "kv_num_heads": kv, "local_window_size": window, "do_rotary": 1},
                       [q, k, v, pk, pv, sl, b.constant(ht(c)), b.constant(ht(s))],
                       [(adt(dt), [batch, S, heads * d]), (adt(dt), [batch, kv, P + S, d]), (adt(dt), [batch, kv, P + S, d])])
    b.output("out", outs[0])
    b.output("present_key", outs[1])
    b.output("present_value", outs[2])
    mod = b.finish()
    dev = cuda_backend().prepare(mod.clone())
    cpu = ref.RefBackend().prepare(mod)
    t = dict(atol=4e-3, rtol=4e-3) if dt == f16 else dict(atol=2e-4, rtol=1e-3)

    d_pk = dev.upload(ht(np.zeros((batch, kv, 0, d), np_dt)))
    d_pv = dev.upload(ht(np.zeros((batch, kv, 0, d), np_dt)))
    h_pk, h_pv = ht(np.zeros((batch, kv, 0, d), np_dt)), ht(np.zeros((batch, kv, 0, d), np_dt))
    past, old_handle, old_host, fresh_after_warm = 0, None, None, None
    for step, seq in enumerate([4, 1, 1, 1, 1, 1]):
        feed = {"q": ht(RNG.standard_normal((batch, seq, heads * d)).astype(np_dt)),
                "k": ht(RNG.standard_normal((batch, seq, kv * d)).astype(np_dt)),
                "v": ht(RNG.standard_normal((batch, seq, kv * d)).astype(np_dt)),
                "seqlens_k": ht(np.full(batch, past + seq - 1, np.int32))}
        want = dict(cpu.run({**feed, "past_key": h_pk, "past_value": h_pv}))
        got = dict(dev.run({**{n: dev.upload(x) for n, x in feed.items()}, "past_key": d_pk, "past_value": d_pv}))
        for name in ("out", "present_key", "present_value"):
            assert_tensors_match(dev.download(got[name]), want[name], **t)
        if step == 2:
            old_handle, old_host = got["present_key"], want["present_key"]
            fresh_after_warm = dev.pool_stats()[0]
        d_pk, d_pv, h_pk, h_pv = got["present_key"], got["present_value"], want["present_key"], want["present_value"]
        past += seq
    # later appends did not disturb what the older handle views, and did not allocate
    assert_tensors_match(dev.download(old_handle), old_host, **t)
    assert dev.pool_stats()[0] <= fresh_after_warm + 2  # no per-step cache reallocation
    # feeding the OLD handle again must not clobber the newer rows: it is copied, not appended to
    feed = {"q": ht(RNG.standard_normal((batch, 1, heads * d)).astype(np_dt)),
            "k": ht(RNG.standard_normal((batch, 1, kv * d)).astype(np_dt)),
            "v": ht(RNG.standard_normal((batch, 1, kv * d)).astype(np_dt)),
            "seqlens_k": ht(np.full(batch, old_host.shape[2], np.int32))}
    newest_before = dev.download(d_pk)
    dev.run({**{n: dev.upload(x) for n, x in feed.items()}, "past_key": old_handle, "past_value": old_handle})
    assert np.array_equal(dev.download(d_pk).data, newest_before.data)


def test_gqa_batched_decode_crosses_the_cluster_size_bucket_under_graph_replay():
    """Many (batch row, KV head) pairs and no window: the number of CTAs per cluster follows the length
    bucket, so it changes when the cache grows past 1024 rows — inside one plan, while the plan is being
    replayed as a CUDA graph. The captured launch must then be recorded again with the new cluster shape
    (a patched grid alone would leave keys out of the softmax). Every step is compared with the oracle."""
    from oracle import ref
    batch, heads, kv, d = 40, 4, 4, 32

    def make(nb):
        b = ir.GraphBuilder()
        P = b.sym("P")
        q = b.input("q", ir.F16, [nb, 1, heads * d])
        k = b.input("k", ir.F16, [nb, 1, kv * d])
        v = b.input("v", ir.F16, [nb, 1, kv * d])
        pk = b.input("past_key", ir.F16, [nb, kv, P, d])
        pv = b.input("past_value", ir.F16, [nb, kv, P, d])
        sl = b.input("seqlens_k", ir.I32, [nb])
        cfg = models.DecoderConfig("t", 0, 0, heads, kv, d, 0, 0, act_dtype=ir.F16, max_positions=1100)
        c, s = models.rope_caches(cfg)
        outs = b.composite(GQA, {"num_heads": heads, "kv_num_heads": kv, "local_window_size": -1, "do_rotary": 1},
                           [q, k, v, pk, pv, sl, b.constant(ht(c)), b.constant(ht(s))],
                           [(ir.F16, [nb, 1, heads * d]), (ir.F16, [nb, kv, P + 1, d]), (ir.F16, [nb, kv, P + 1, d])])
        b.output("out", outs[0])
        b.output("present_key", outs[1])
        b.output("present_value", outs[2])
        b.output("twice", b.add(outs[0], outs[0]))  # a second launch: single-launch plans are not recorded as graphs
        return b.finish()

    mod, mod_rows = make(batch), make(3)
    dev = cuda_backend().prepare(mod.clone())
    ref.set_threads(8)
    rows = np.array([0, 17, 39])
    past = 1016
    hk = RNG.standard_normal((batch, kv, past, d)).astype(f16)
    hv = RNG.standard_normal((batch, kv, past, d)).astype(f16)
    d_pk, d_pv = dev.upload(ht(hk)), dev.upload(ht(hv))
    o_pk, o_pv = ht(np.ascontiguousarray(hk[rows])), ht(np.ascontiguousarray(hv[rows]))
    worst = 0.0
    for step in range(14):  # lengths 1017 … 1030: the 1024-row bucket is left at the eighth step
        feed = {"q": RNG.standard_normal((batch, 1, heads * d)).astype(f16), "k": RNG.standard_normal((batch, 1, kv * d)).astype(f16),
                "v": RNG.standard_normal((batch, 1, kv * d)).astype(f16), "seqlens_k": np.full(batch, past, np.int32)}
        got = dict(dev.run({**{n: dev.upload(ht(x)) for n, x in feed.items()}, "past_key": d_pk, "past_value": d_pv}))
        cpu = ref.RefBackend().prepare(mod_rows.clone())
        want = dict(cpu.run({**{n: ht(np.ascontiguousarray(x[rows])) for n, x in feed.items()}, "past_key": o_pk, "past_value": o_pv}))
        diff = float(np.abs(dev.download(got["out"]).numpy()[rows].astype(f32) - want["out"].numpy().astype(f32)).max())
        worst = max(worst, diff)
        assert diff <= 4e-3, f"length {past + 1}: attention output differs by {diff}"
        d_pk, d_pv, o_pk, o_pv = got["present_key"], got["present_value"], want["present_key"], want["present_value"]
        past += 1
    assert dev.plan_stats()["graph_launches"] >= 8  # the steps did run as graph replays


@pytest.mark.parametrize("batch,heads,kv,d,past,window", [
    (1, 8, 2, 128, 700, -1),      # few pairs: clusters of 8 CTAs split the keys; 4 heads per KV head
    (3, 12, 2, 128, 333, 100),    # 6 heads per KV head: two head groups, the second only half full; window; ragged
    (40, 8, 8, 64, 300, -1),      # many pairs: one CTA each; head size 64; one head per KV head
    (5, 8, 4, 128, 1500, 600),    # two heads per KV head; window inside a long cache; ragged
    (2, 4, 1, 64, 37, -1),        # a key range shorter than three tiles
])
def test_gqa_f16_decode_steps_ragged_rows_windows_and_cluster_sizes(batch, heads, kv, d, past, window):
    """Two consecutive decode steps of the f16 kernel for head sizes up to 128 (the second one appends in place), rows of
    different lengths with garbage behind their last valid key, against the oracle: output and the whole present cache."""
    from oracle import ref
    ref.set_threads(8)
    rng = np.random.default_rng([batch, heads, kv, d, past])
    b = ir.GraphBuilder()
    P = b.sym("P")
    q = b.input("q", ir.F16, [batch, 1, heads * d])
    k = b.input("k", ir.F16, [batch, 1, kv * d])
    v = b.input("v", ir.F16, [batch, 1, kv * d])
    pk = b.input("past_key", ir.F16, [batch, kv, P, d])
    pv = b.input("past_value", ir.F16, [batch, kv, P, d])
    sl = b.input("seqlens_k", ir.I32, [batch])
    cfg = models.DecoderConfig("t", 0, 0, heads, kv, d, 0, 0, act_dtype=ir.F16, max_positions=past + 8)
    c, s = models.rope_caches(cfg)
    outs = b.composite(GQA, {"num_heads": heads, "kv_num_heads": kv, "local_window_size": window, "do_rotary": 1},
                       [q, k, v, pk, pv, sl, b.constant(ht(c)), b.constant(ht(s))],
                       [(ir.F16, [batch, 1, heads * d]), (ir.F16, [batch, kv, P + 1, d]), (ir.F16, [batch, kv, P + 1, d])])
    b.output("out", outs[0])
    b.output("present_key", outs[1])
    b.output("present_value", outs[2])
    mod = b.finish()
    dev = cuda_backend().prepare(mod.clone())
    cpu = ref.RefBackend().prepare(mod)
    # row 0 is full; the others stop earlier (what lies behind their last key is garbage the kernels must not read into the result)
    lens = np.array([past] + [int(x) for x in rng.integers(max(1, past // 3), past, batch - 1)], np.int32)
    h_pk = ht(rng.standard_normal((batch, kv, past, d)).astype(f16))
    h_pv = ht(rng.standard_normal((batch, kv, past, d)).astype(f16))
    d_pk, d_pv = dev.upload(h_pk), dev.upload(h_pv)
    for step in range(2):
        feed = {"q": ht(rng.standard_normal((batch, 1, heads * d)).astype(f16)), "k": ht(rng.standard_normal((batch, 1, kv * d)).astype(f16)),
                "v": ht(rng.standard_normal((batch, 1, kv * d)).astype(f16)), "seqlens_k": ht(lens + step)}
        want = dict(cpu.run({**feed, "past_key": h_pk, "past_value": h_pv}))
        got = dict(dev.run({**{n: dev.upload(x) for n, x in feed.items()}, "past_key": d_pk, "past_value": d_pv}))
        assert_tensors_match(dev.download(got["out"]), want["out"], atol=1e-2, rtol=4e-3)
        for name in ("present_key", "present_value"):
            assert_tensors_match(dev.download(got[name]), want[name], atol=4e-3, rtol=4e-3)
        d_pk, d_pv, h_pk, h_pv = got["present_key"], got["present_value"], want["present_key"], want["present_value"]
