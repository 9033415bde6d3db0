"""Pins the CPU oracle against the golden vectors of the reference's own unit
tests, re-expressed here:

* primitives          crates/onyxia-ir/src/interp.rs:1202-1508
* decompositions      crates/onyxia-ir/src/decomp.rs:728-1202
* MatMulNBits blob    crates/onyxia-lower/tests/lower_test.rs:246-305
* storage sizes       crates/onyxia-ir/src/types.rs:149-156
"""
import math

import numpy as np
import pytest

from onyxia_b200 import OnyxiaError, ir
from onyxia_b200.ir import HostTensor
from oracle import ref

from util import assert_close, composite_module, ht, single_prim_module

f32 = np.float32


def run1(kind, inputs, **params):
    m, feed = single_prim_module(kind, inputs, **params)
    return ref.run_once(m, feed)[0][1]


def run_composite(name, attrs, inputs, out_types):
    m, feed = composite_module(name, attrs, inputs, out_types)
    return [t for _, t in ref.run_once(m, feed)]


# ── primitives (interp.rs tests) ─────────────────────────────────────────
def test_binary_broadcast_golden():
    out = run1(ir.P_BINARY, [ht([[1, 2, 3], [4, 5, 6]], f32), ht([10, 20, 30], f32)], op=ir.ADD)
    assert out.shape == (2, 3)
    assert out.numpy().reshape(-1).tolist() == [11, 22, 33, 14, 25, 36]


def test_int_division_semantics():
    a = ht([7, -7, 1], np.int64)
    out = run1(ir.P_BINARY, [a, ht([2, 2, 1], np.int64)], op=ir.DIV)
    assert out.numpy().tolist() == [3, -3, 1]  # trunc toward zero
    with pytest.raises(OnyxiaError, match="integer division by zero"):
        run1(ir.P_BINARY, [a, ht([0, 1, 1], np.int64)], op=ir.DIV)


def test_compare_nan_semantics():
    a = ht([np.nan, 1.0], f32)
    assert run1(ir.P_COMPARE, [a, a], op=ir.EQ).numpy().tolist() == [False, True]
    assert run1(ir.P_COMPARE, [a, a], op=ir.NE).numpy().tolist() == [True, False]


def test_select_broadcasts():
    out = run1(ir.P_SELECT, [ht([[True], [False]]), ht([1, 2], f32), ht([9, 8], f32)])
    assert out.shape == (2, 2)
    assert out.numpy().reshape(-1).tolist() == [1, 2, 9, 8]


def test_matmul_golden():
    a = ht([[1, 2, 3], [4, 5, 6]], f32)
    out = run1(ir.P_MATMUL, [a, ht([[7, 8], [9, 10], [11, 12]], f32)])
    assert out.numpy().reshape(-1).tolist() == [58, 64, 139, 154]
    out2 = run1(ir.P_MATMUL, [a, ht([[7, 9, 11], [8, 10, 12]], f32)], trans_b=True)
    assert out2.numpy().reshape(-1).tolist() == [58, 64, 139, 154]


def test_matmul_batch_broadcast():
    a = ht(np.array([1, 0, 0, 1, 2, 0, 0, 2], f32).reshape(2, 1, 2, 2))
    out = run1(ir.P_MATMUL, [a, ht([[1, 2], [3, 4]], f32)])
    assert out.shape == (2, 1, 2, 2)
    assert out.numpy().reshape(-1).tolist() == [1, 2, 3, 4, 2, 4, 6, 8]


def test_reduce_golden():
    x = ht([[1, 2, 3], [4, 5, 6]], f32)
    assert run1(ir.P_REDUCE, [x], op=ir.SUM, axes=[1], keepdims=False).numpy().tolist() == [6, 15]
    mean = run1(ir.P_REDUCE, [x], op=ir.MEAN, axes=[0], keepdims=True)
    assert mean.shape == (1, 3) and mean.numpy().reshape(-1).tolist() == [2.5, 3.5, 4.5]
    mx = run1(ir.P_REDUCE, [x], op=ir.RMAX, axes=[0, 1], keepdims=False)
    assert mx.shape == () and mx.numpy().reshape(-1).tolist() == [6]


def test_transpose_round_trip():
    x = ht([[1, 2, 3], [4, 5, 6]], f32)
    t = run1(ir.P_TRANSPOSE, [x], axes=[1, 0])
    assert t.shape == (3, 2) and t.numpy().reshape(-1).tolist() == [1, 4, 2, 5, 3, 6]
    back = run1(ir.P_TRANSPOSE, [t], axes=[1, 0])
    assert np.array_equal(back.numpy(), x.numpy())


def test_concat_and_slice():
    cat = run1(ir.P_CONCAT, [ht([[1, 2]], f32), ht([[3, 4], [5, 6]], f32)], axis=0)
    assert cat.shape == (3, 2) and cat.numpy().reshape(-1).tolist() == [1, 2, 3, 4, 5, 6]
    sl = run1(ir.P_SLICE, [cat], specs=[(0, 1, 3, 1)])
    assert sl.numpy().reshape(-1).tolist() == [3, 4, 5, 6]
    rev = run1(ir.P_SLICE, [cat], specs=[(0, 2, 0, -1)])  # rows 2, 1
    assert rev.numpy().reshape(-1).tolist() == [5, 6, 3, 4]


def test_gather_embedding_and_negative_index():
    table = ht(np.array([0, 0, 1, 1, 2, 2, 3, 3], f32).reshape(4, 2))
    out = run1(ir.P_GATHER, [table, ht([3, 0, -1], np.int64)], axis=0)
    assert out.shape == (3, 2) and out.numpy().reshape(-1).tolist() == [3, 3, 0, 0, 3, 3]
    with pytest.raises(OnyxiaError, match="gather index 4 out of range for dim 4"):
        run1(ir.P_GATHER, [table, ht([4], np.int64)], axis=0)


def test_scatter_last_write_wins():
    out = run1(ir.P_SCATTER, [ht([0, 0, 0, 0], f32), ht([[1], [1]], np.int64), ht([5, 7], f32)])
    assert out.numpy().tolist() == [0, 7, 0, 0]


def test_cast_semantics():
    out = run1(ir.P_CAST, [ht([1.9, -1.9, 3.0e9], f32)], dtype=ir.I32)
    v = out.numpy().tolist()
    assert v[0] == 1 and v[1] == -1
    assert v[2] == np.int64(3000000000).astype(np.int32)  # saturates i64, wraps to i32
    b = run1(ir.P_CAST, [ht([0, 2], np.int64)], dtype=ir.BOOL)
    assert b.numpy().tolist() == [False, True]


def test_f16_round_trip():
    h = run1(ir.P_CAST, [ht([1.5, -2.25], f32)], dtype=ir.F16)
    assert h.dtype == ir.F16
    back = run1(ir.P_CAST, [h], dtype=ir.F32)
    assert back.numpy().tolist() == [1.5, -2.25]


def test_iota_and_dequantize():
    b = ir.GraphBuilder()
    b.output("out", b.iota(4, ir.I64))
    assert ref.run_once(b.finish(), {})[0][1].numpy().tolist() == [0, 1, 2, 3]
    # u4 block of 4, scale 0.5, default zero point 8: elements 8,9,10,15
    data = HostTensor(ir.U4, [1, 4], np.array([0x98, 0xFA], np.uint8))
    out = run1(ir.P_DEQUANTIZE, [data, ht([0.5], f32)], block_size=4, shape=[4])
    assert out.numpy().tolist() == [0.0, 0.5, 1.0, 3.5]


def test_dequantize_type_rule_and_storage_sizes():
    # infer.rs:780-794 — output takes the scales' dtype; types.rs:149-156 — packed sizes round up
    data = HostTensor(ir.U4, [1, 4], np.array([0x98, 0xFA], np.uint8))
    out = run1(ir.P_DEQUANTIZE, [data, ht([0.5], np.float16)], block_size=4, shape=[4])
    assert out.dtype == ir.F16
    assert [ir.storage_bytes(ir.U4, n) for n in (0, 1, 2, 3)] == [0, 1, 1, 2]
    assert ir.storage_bytes(ir.I4, 32) == 16
    assert ir.storage_bytes(ir.F32, 262144 * 640) == 671_088_640
    with pytest.raises(ValueError):
        HostTensor(ir.U4, [5], np.zeros(2, np.uint8))
    HostTensor(ir.U4, [5], np.zeros(3, np.uint8))


def test_end_to_end_rms_norm_with_symbols():
    b = ir.GraphBuilder()
    s = b.sym("S")
    x = b.input("x", ir.F32, [s, 4])
    ms = b.reduce(ir.MEAN, b.mul(x, x), [1], True)
    inv = b.unary(ir.RSQRT, b.add(ms, b.const_f32([1e-6], [1])))
    b.output("out", b.mul(x, inv))
    m = b.finish()
    (name, t), = ref.run_once(m, {"x": ht([[1, 1, 1, 1], [2, 2, 2, 2]], f32)})
    assert name == "out" and t.shape == (2, 4)
    assert np.all(np.abs(t.numpy() - 1.0) < 1e-4)


def test_binding_validation():
    b = ir.GraphBuilder()
    s = b.sym("S")
    x = b.input("x", ir.F32, [s])
    y = b.input("y", ir.F32, [s])
    b.output("sum", b.add(x, y))
    m = b.finish()
    sess = ref.RefBackend().prepare(m)
    t3, t4 = ht([1, 2, 3], f32), ht([1, 2, 3, 4], f32)
    sess.run({"x": t3, "y": t3})
    with pytest.raises(OnyxiaError, match="conflicting values") as e:
        sess.run({"x": t3, "y": t4})
    assert e.value.kind == "Binding"
    with pytest.raises(OnyxiaError, match="missing input 'y'"):
        sess.run({"x": t3})


def test_late_bound_reshape_infers_dim():
    b = ir.GraphBuilder()
    x = b.input("x", ir.F32, [2, 6])
    b.output("out", b.reshape(x, [b.sym("L"), 3]))
    out = ref.run_once(b.finish(), {"x": ht(np.arange(12, dtype=f32).reshape(2, 6))})
    assert out[0][1].shape == (4, 3)


# ── decompositions (decomp.rs tests) ─────────────────────────────────────
def test_softmax_matches_manual():
    x = ht([[1, 2, 3], [1, 1, 1]], f32)
    got = run_composite("Softmax", {"axis": 1}, [("x", x)], [(ir.F32, [2, 3])])[0].numpy().reshape(-1)
    e = np.exp(np.array([1, 2, 3], f32))
    assert_close(got[:3], e / e.sum(), 1e-6)
    assert_close(got[3:], [1 / 3] * 3, 1e-6)


def test_gelu_matches_reference():
    x = ht([-2.0, -0.5, 0.0, 0.5, 2.0], f32)
    got = run_composite("Gelu", {}, [("x", x)], [(ir.F32, [5])])[0].numpy()
    assert_close(got, [-0.0455, -0.1543, 0.0, 0.3457, 1.9545], 1e-3)


def test_trilu_upper_and_lower():
    x = ht(np.arange(1, 10, dtype=f32).reshape(3, 3))
    up = run_composite("Trilu", {"upper": 1}, [("x", x)], [(ir.F32, [3, 3])])[0]
    assert up.numpy().reshape(-1).tolist() == [1, 2, 3, 0, 5, 6, 0, 0, 9]
    lo = run_composite("Trilu", {"upper": 0, "k": 1}, [("x", x)], [(ir.F32, [3, 3])])[0]
    assert lo.numpy().reshape(-1).tolist() == [1, 2, 0, 4, 5, 6, 7, 8, 9]


def test_rms_norm_matches_manual():
    got = run_composite("SimplifiedLayerNormalization", {"epsilon": 1e-6},
                        [("x", ht([[1, 2, 3, 4]], f32)), ("w", ht([2, 2, 2, 2], f32))], [(ir.F32, [1, 4])])[0]
    ms = (1 + 4 + 9 + 16) / 4
    inv = 1 / math.sqrt(ms + 1e-6)
    assert_close(got.numpy(), [v * inv * 2 for v in (1, 2, 3, 4)], 1e-5)


ROPE = "com.microsoft.RotaryEmbedding"


def test_rotary_rotates_first_pair():
    x = ht(np.array([1, 2, 3, 4], f32).reshape(1, 1, 4))
    cos, sin = ht([[1, 1], [0, 0]], f32), ht([[0, 0], [1, 1]], f32)
    ident = run_composite(ROPE, {"num_heads": 1}, [("x", x), ("pos", ht([[0]], np.int64)), ("cos", cos), ("sin", sin)],
                          [(ir.F32, [1, 1, 4])])[0]
    assert_close(ident.numpy(), [1, 2, 3, 4], 1e-6)
    rot = run_composite(ROPE, {"num_heads": 1}, [("x", x), ("pos", ht([[1]], np.int64)), ("cos", cos), ("sin", sin)],
                        [(ir.F32, [1, 1, 4])])[0]
    assert_close(rot.numpy(), [-3, -4, 1, 2], 1e-6)


def test_rotary_infers_heads_from_cache_width():
    x = ht(np.arange(1, 9, dtype=f32).reshape(1, 1, 8))
    cos, sin = ht([[1, 1], [0, 0]], f32), ht([[0, 0], [1, 1]], f32)
    rot = run_composite(ROPE, {"num_heads": 0}, [("x", x), ("pos", ht([[1]], np.int64)), ("cos", cos), ("sin", sin)],
                        [(ir.F32, [1, 1, 8])])[0]
    assert_close(rot.numpy(), [-3, -4, 1, 2, -7, -8, 5, 6], 1e-6)


def naive_attention(q, keys, vals, past, scale, window):
    """Plain-numpy single-head causal attention; q [S,D], keys/vals [T,D]."""
    out = []
    for i, qi in enumerate(q):
        row = past + i
        logits = np.full(len(keys), -np.inf, dtype=f32)
        for j, kj in enumerate(keys):
            if j <= row and (window < 0 or j >= row - window):
                logits[j] = f32(np.dot(qi, kj)) * f32(scale)
        p = np.exp(logits - logits.max())
        p = p / p.sum()
        out.append(p @ np.asarray(vals, dtype=f32))
    return np.array(out, dtype=f32)


GQA = "com.microsoft.GroupQueryAttention"


def test_gqa_matches_naive_attention():
    h, kv, d, s, t = 2, 1, 2, 2, 1
    q = np.array([i * 0.1 - 0.3 for i in range(s * h * d)], f32)
    k_new = np.array([i * 0.2 - 0.1 for i in range(s * kv * d)], f32)
    v_new = np.array([i * 0.3 + 0.2 for i in range(s * kv * d)], f32)
    past_k = np.array([i * 0.5 for i in range(t * kv * d)], f32)
    past_v = np.array([1.0 - i * 0.4 for i in range(t * kv * d)], f32)
    outs = run_composite(
        GQA, {"num_heads": h, "kv_num_heads": kv},
        [("q", ht(q.reshape(1, s, h * d))), ("k", ht(k_new.reshape(1, s, kv * d))), ("v", ht(v_new.reshape(1, s, kv * d))),
         ("pk", ht(past_k.reshape(1, kv, t, d))), ("pv", ht(past_v.reshape(1, kv, t, d))),
         ("seqlens", ht([t + s - 1], np.int64)), ("total", ht([t + s], np.int64))],
        [(ir.F32, [1, s, h * d]), (ir.F32, [1, kv, t + s, d]), (ir.F32, [1, kv, t + s, d])])
    keys = np.concatenate([past_k.reshape(t, d), k_new.reshape(s, kv * d)[:, :d]])
    vals = np.concatenate([past_v.reshape(t, d), v_new.reshape(s, kv * d)[:, :d]])
    got = outs[0].numpy().reshape(s, h * d)
    for head in range(h):
        qh = q.reshape(s, h * d)[:, head * d:(head + 1) * d]
        expect = naive_attention(qh, keys, vals, t, 1 / math.sqrt(d), -1)
        assert_close(got[:, head * d:(head + 1) * d], expect, 1e-4)
    assert_close(outs[1].numpy().reshape(-1)[: t * d], past_k, 1e-6)
    assert_close(outs[2].numpy().reshape(-1)[t * d:], v_new, 1e-6)


def test_gqa_sliding_window_masks_old_tokens():
    outs = run_composite(
        GQA, {"num_heads": 1, "kv_num_heads": 1, "local_window_size": 2},
        [("q", ht(np.ones((1, 1, 1), f32))), ("k", ht(np.zeros((1, 1, 1), f32))), ("v", ht(np.full((1, 1, 1), 100, f32))),
         ("pk", ht(np.zeros((1, 1, 3, 1), f32))), ("pv", ht(np.array([7, 11, 13], f32).reshape(1, 1, 3, 1))),
         ("seqlens", ht([3], np.int64)), ("total", ht([4], np.int64))],
        [(ir.F32, [1, 1, 1]), (ir.F32, [1, 1, 4, 1]), (ir.F32, [1, 1, 4, 1])])
    assert_close(outs[0].numpy(), [124.0 / 3.0], 1e-4)


def test_gqa_ragged_batch_honors_seqlens():
    kv, d, s, p = 1, 2, 1, 3
    q = np.array([[0.1, -0.2], [0.3, 0.05]], f32)
    k_new = np.array([[0.5, 0.1], [-0.2, 0.4]], f32)
    v_new = np.array([[10, 20], [30, 40]], f32)
    past_k = np.array([[[0.2, 0.3], [-0.1, 0.6], [0.4, -0.5]], [[0.7, -0.3], [99, 99], [99, 99]]], f32)
    past_v = np.array([[[1, 2], [3, 4], [5, 6]], [[7, 8], [-99, -99], [-99, -99]]], f32)
    seqlens = np.array([3, 1], np.int32)
    outs = run_composite(
        GQA, {"num_heads": 1, "kv_num_heads": 1},
        [("q", ht(q.reshape(2, s, d))), ("k", ht(k_new.reshape(2, s, d))), ("v", ht(v_new.reshape(2, s, d))),
         ("pk", ht(past_k.reshape(2, kv, p, d))), ("pv", ht(past_v.reshape(2, kv, p, d))), ("seqlens", ht(seqlens))],
        [(ir.F32, [2, s, d]), (ir.F32, [2, kv, p + s, d]), (ir.F32, [2, kv, p + s, d])])
    got = outs[0].numpy().reshape(2, d)
    for row in range(2):
        valid = int(seqlens[row]) + 1 - s
        keys = np.concatenate([past_k[row][:valid], k_new[row:row + 1]])
        vals = np.concatenate([past_v[row][:valid], v_new[row:row + 1]])
        expect = naive_attention(q[row:row + 1], keys, vals, valid, 1 / math.sqrt(d), -1)
        assert_close(got[row], expect[0], 1e-4)
    row1 = outs[1].numpy().reshape(2, (p + s) * d)[1]
    assert_close(row1[:2], [0.7, -0.3], 1e-6)
    assert_close(row1[2:4], [-0.2, 0.4], 1e-6)
    assert_close(row1[4:], [0, 0, 0, 0], 1e-6)


def _nbits_case():
    k_dim, n_dim, bs = 8, 2, 4
    q_vals = np.array([i % 16 for i in range(n_dim * k_dim)], np.uint8)
    scales = np.array([0.5, 0.25, 1.0, 2.0], f32)
    a_vals = np.array([i * 0.1 for i in range(k_dim)], f32)
    n_blocks = k_dim // bs
    expect = np.zeros(n_dim, f32)
    for n in range(n_dim):
        for kk in range(k_dim):
            w = (f32(q_vals[n * k_dim + kk]) - f32(8)) * scales[n * n_blocks + kk // bs]
            expect[n] += a_vals[kk] * w
    return k_dim, n_dim, bs, n_blocks, q_vals, scales, a_vals, expect


def test_matmul_nbits_matches_float_matmul():
    k_dim, n_dim, bs, n_blocks, q_vals, scales, a_vals, expect = _nbits_case()
    bq = HostTensor.packed_u4(q_vals, [n_dim, n_blocks, bs])
    got = run_composite("com.microsoft.MatMulNBits", {"K": k_dim, "N": n_dim, "bits": 4, "block_size": bs},
                        [("a", ht(a_vals.reshape(1, k_dim))), ("b", bq), ("s", ht(scales))], [(ir.F32, [1, n_dim])])[0]
    assert_close(got.numpy(), expect, 1e-4)


def test_matmul_nbits_from_byte_blob_as_constant():
    # lower_test.rs:246-305: the weight arrives as a u8 blob [N, n_blocks, bs/2]
    # whose bytes are reinterpreted as U4 [N, n_blocks, bs]; weights are constants.
    k_dim, n_dim, bs, n_blocks, q_vals, scales, a_vals, expect = _nbits_case()
    blob = np.zeros(n_dim * n_blocks * bs // 2, np.uint8)
    for i, v in enumerate(q_vals):
        blob[i // 2] |= (v & 0xF) << ((i % 2) * 4)
    b = ir.GraphBuilder()
    a = b.input("a", ir.F32, [1, k_dim])
    w = b.constant(HostTensor(ir.U4, [n_dim, n_blocks, bs], blob))
    s = b.constant(ht(scales))
    out = b.composite("com.microsoft.MatMulNBits", {"K": k_dim, "N": n_dim, "bits": 4, "block_size": bs}, [a, w, s],
                      [(ir.F32, [1, n_dim])])[0]
    b.output("y", out)
    got = ref.run_once(b.finish(), {"a": ht(a_vals.reshape(1, k_dim))})[0][1]
    assert_close(got.numpy(), expect, 1e-4)


def test_gqa_types_check_symbolically():
    b = ir.GraphBuilder()
    s, t = b.sym("S"), b.sym("T")
    q = b.input("q", ir.F32, [1, s, 8])
    k = b.input("k", ir.F32, [1, s, 4])
    v = b.input("v", ir.F32, [1, s, 4])
    pk = b.input("pk", ir.F32, [1, 1, t, 4])
    pv = b.input("pv", ir.F32, [1, 1, t, 4])
    sl = b.input("seqlens", ir.I32, [1])
    outs = b.composite(GQA, {"num_heads": 2, "kv_num_heads": 1}, [q, k, v, pk, pv, sl],
                       [(ir.F32, [1, s, 8]), (ir.F32, [1, 1, t + s, 4]), (ir.F32, [1, 1, t + s, 4])])
    for i, o in enumerate(outs):
        b.output(f"o{i}", o)
    m = b.finish()
    m.inline_composites([])
    m.validate()
    assert all("." not in op and op[0].islower() for op in m.node_ops()), "composites remain after inlining"


def test_gqa_through_lowering_shape_past_zero():
    # lower_test.rs:442-543 in miniature: empty past, one new token → out = v per head
    h, kv, d = 2, 1, 2
    v = np.array([[[0.5, -1.5]]], f32)
    outs = run_composite(
        GQA, {"num_heads": h, "kv_num_heads": kv},
        [("q", ht(np.ones((1, 1, h * d), f32))), ("k", ht(np.ones((1, 1, kv * d), f32))), ("v", ht(v)),
         ("pk", ht(np.zeros((1, kv, 0, d), f32))), ("pv", ht(np.zeros((1, kv, 0, d), f32))), ("seqlens", ht([0], np.int32))],
        [(ir.F32, [1, 1, h * d]), (ir.F32, [1, kv, 1, d]), (ir.F32, [1, kv, 1, d])])
    assert_close(outs[0].numpy(), [0.5, -1.5, 0.5, -1.5], 1e-6)


# ── f64→f16 rounding and the lazy/fast dequantisation paths ──────────────
def test_f16_rounding_is_nearest_even_from_f64():
    l = ref.lib()
    rng = np.random.default_rng(7)
    vals = np.concatenate([rng.standard_normal(4000) * 10.0 ** rng.integers(-9, 6, 4000),
                           [0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 2.0 ** -25, 2.0 ** -25 * 1.0001, 6.1e-5, np.inf, -np.inf]])
    for v in vals:
        got = l.oxref_f64_to_f16(float(v))
        # numpy rounds f64→f16 directly (nearest even)
        want = int(np.array(v, dtype=np.float64).astype(np.float16).view(np.uint16))
        assert got == want, (v, hex(got), hex(want))
    # a value whose f64→f32→f16 double rounding differs from the direct rounding
    v = 1.0 + 2.0 ** -11 + 2.0 ** -30
    assert l.oxref_f64_to_f16(v) == int(np.float16(1.0 + 2.0 ** -10).view(np.uint16))
    assert math.isnan(l.oxref_f16_to_f64(0x7E00))


@pytest.mark.parametrize("sdt", [np.float16, np.float32])
@pytest.mark.parametrize("with_zp", [False, True])
def test_lazy_dequant_matmul_equals_materialised(sdt, with_zp):
    """The streaming Dequantize→MatMul path must give the same bits as writing
    the dequantised weight out first (forced here by a no-op Slice)."""
    rng = np.random.default_rng(3)
    n, k, bs, m = 96, 1024, 32, 3
    nb = k // bs
    q = rng.integers(0, 16, n * k)
    scales = rng.uniform(0.005, 0.02, n * nb).astype(sdt)
    zp = rng.integers(0, 16, n * nb)
    a = rng.standard_normal((m, k)).astype(sdt)
    adt = ir.F16 if sdt == np.float16 else ir.F32

    def build(force_materialise):
        b = ir.GraphBuilder()
        av = b.input("a", adt, [m, k])
        qv = b.constant(HostTensor.packed_u4(q, [n, nb, bs]))
        sv = b.constant(ht(scales.reshape(n, nb)))
        zv = b.constant(HostTensor.packed_u4(zp, [n, nb])) if with_zp else None
        w = b.dequantize(qv, sv, zv, block_size=bs, out_shape=[n, k])
        if force_materialise:
            w = b.slice(w, [(1, 0, k, 1)])
        b.output("y", b.matmul(av, w, trans_b=True))
        return b.finish()

    lazy = ref.run_once(build(False), {"a": ht(a)})[0][1]
    full = ref.run_once(build(True), {"a": ht(a)})[0][1]
    assert np.array_equal(lazy.data, full.data)
    # and against plain numpy in f64 with the same rounding points
    zpv = zp.reshape(n, nb, 1) if with_zp else 8
    w = ((q.reshape(n, nb, bs) - zpv) * scales.reshape(n, nb, 1).astype(np.float64)).astype(sdt).astype(np.float64)
    want = (a.astype(np.float64) @ w.reshape(n, k).T)
    assert_close(lazy.numpy(), want.astype(sdt), 2e-3 if sdt == np.float16 else 1e-5)


def test_threads_do_not_change_results():
    rng = np.random.default_rng(11)
    x = ht(rng.standard_normal((64, 300)).astype(np.float16))
    m1, feed = composite_module("Softmax", {"axis": 1}, [("x", x)], [(ir.F16, [64, 300])])
    m2 = m1.clone()
    ref.set_threads(1)
    a = ref.run_once(m1, feed)[0][1]
    ref.set_threads(4)
    try:
        b = ref.run_once(m2, feed)[0][1]
    finally:
        ref.set_threads(1)
    assert np.array_equal(a.data, b.data)
