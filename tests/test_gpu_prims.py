"""Every IR primitive on the device against the CPU oracle, through the C ABI.

Bit-exact for integer, bool and index work; atol 1e-4 + rtol 1e-3 for f32
(the reference's own device-vs-interpreter tolerance,
crates/onyxia-backend-wgpu/tests/gpu_test.rs:15-16); f16 results within one
f16 ulp-scale tolerance (atol 1e-3 + rtol 2e-3).
"""
import numpy as np
import pytest

from onyxia_b200 import OnyxiaError, ir
from onyxia_b200 import backend as be
from onyxia_b200.ir import HostTensor

from gpu_util import cuda_backend, differential
from util import ht, single_prim_module

pytestmark = pytest.mark.gpu

f32, f16, i64, i32 = np.float32, np.float16, np.int64, np.int32
RNG = np.random.default_rng(1234)


def tol(dtype):
    return dict(atol=1e-3, rtol=2e-3) if dtype == f16 else dict(atol=1e-4, rtol=1e-3)


def rand(shape, dtype):
    if dtype in (f32, f16):
        return (RNG.standard_normal(shape) * 2).astype(dtype)
    if dtype == np.bool_:
        return RNG.integers(0, 2, shape).astype(np.bool_)
    info = np.iinfo(dtype)
    return RNG.integers(max(info.min, -1000), min(info.max, 1000), shape, endpoint=True).astype(dtype)


def check_prim(kind, inputs, tdtype=f32, **params):
    m, feed = single_prim_module(kind, [ht(x) for x in inputs], **params)
    return differential(m, feed, **tol(tdtype))


# ── Unary ────────────────────────────────────────────────────────────────
@pytest.mark.parametrize("dtype", [f32, f16])
@pytest.mark.parametrize("op", [ir.NEG, ir.ABS, ir.SQRT, ir.RSQRT, ir.EXP, ir.LOG, ir.SIN, ir.COS, ir.TANH, ir.ERF,
                                ir.FLOOR, ir.CEIL])
def test_unary_float(op, dtype):
    x = rand((3, 257), dtype)
    if op in (ir.SQRT, ir.RSQRT, ir.LOG):
        x = np.abs(x) + dtype(0.01)
    check_prim(ir.P_UNARY, [x], dtype, op=op)


@pytest.mark.parametrize("dtype", [i64, i32, np.int8])
def test_unary_int_neg_abs_wrap(dtype):
    info = np.iinfo(dtype)
    x = np.array([0, 1, -1, info.min, info.max, 77, -77], dtype)
    check_prim(ir.P_UNARY, [x], op=ir.NEG)
    check_prim(ir.P_UNARY, [x], op=ir.ABS)
    check_prim(ir.P_UNARY, [np.array([3, 200, 0], np.uint8)], op=ir.ABS)


def test_unary_not():
    check_prim(ir.P_UNARY, [rand((33,), np.bool_)], op=ir.NOT)


# ── Binary / Compare / Select ────────────────────────────────────────────
@pytest.mark.parametrize("dtype", [f32, f16])
@pytest.mark.parametrize("op", [ir.ADD, ir.SUB, ir.MUL, ir.DIV, ir.POW, ir.MAX, ir.MIN])
def test_binary_float_broadcast(op, dtype):
    a, b = rand((2, 31, 5), dtype), rand((31, 1), dtype)
    if op == ir.POW:
        a = np.abs(a) + dtype(0.1)
    check_prim(ir.P_BINARY, [a, b], dtype, op=op)
    check_prim(ir.P_BINARY, [b, a], dtype, op=op) if op != ir.POW else None
    check_prim(ir.P_BINARY, [a, a[::-1].copy()], dtype, op=op)  # same shape, contiguous path


def test_binary_nan_and_inf():
    a = np.array([np.nan, 1.0, np.inf, -np.inf, 0.0, -0.0], f32)
    b = np.array([1.0, np.nan, 1.0, np.inf, 0.0, 5.0], f32)
    for op in (ir.MAX, ir.MIN, ir.ADD, ir.MUL, ir.DIV):
        check_prim(ir.P_BINARY, [a, b], op=op)


@pytest.mark.parametrize("dtype", [i64, i32, np.uint32, np.uint8, np.int8])
@pytest.mark.parametrize("op", [ir.ADD, ir.SUB, ir.MUL, ir.DIV, ir.MAX, ir.MIN])
def test_binary_int_exact(op, dtype):
    info = np.iinfo(dtype)
    a = np.concatenate([rand((40,), dtype), np.array([info.min, info.max, info.max], dtype)])
    b = np.concatenate([rand((40,), dtype), np.array([info.max, info.max, 2], dtype)])
    if op == ir.DIV:
        b = np.where(b == 0, 1, b).astype(dtype)
    check_prim(ir.P_BINARY, [a, b], op=op)


def test_int_division_semantics_and_error():
    check_prim(ir.P_BINARY, [np.array([7, -7, 1, np.iinfo(i64).min], i64), np.array([2, 2, 1, -1], i64)], op=ir.DIV)
    m, feed = single_prim_module(ir.P_BINARY, [ht(np.array([7, -7, 1], i64)), ht(np.array([0, 1, 1], i64))], op=ir.DIV)
    with pytest.raises(OnyxiaError, match="integer division by zero") as e:
        be.run_once(cuda_backend(), m, feed)
    assert e.value.kind == "Runtime"


def test_int_pow():
    check_prim(ir.P_BINARY, [np.array([2, -3, 7, 10, 0], i64), np.array([10, 3, 0, 30, 0], i64)], op=ir.POW)
    m, feed = single_prim_module(ir.P_BINARY, [ht(np.array([2], i64)), ht(np.array([-1], i64))], op=ir.POW)
    with pytest.raises(OnyxiaError, match="negative exponent"):
        be.run_once(cuda_backend(), m, feed)


def test_bool_logic():
    a, b = rand((5, 7), np.bool_), rand((7,), np.bool_)
    for op in (ir.AND, ir.OR, ir.XOR):
        check_prim(ir.P_BINARY, [a, b], op=op)


@pytest.mark.parametrize("dtype", [f32, f16, i64, i32, np.uint8, np.bool_])
@pytest.mark.parametrize("op", [ir.EQ, ir.NE, ir.LT, ir.LE, ir.GT, ir.GE])
def test_compare(op, dtype):
    a = rand((4, 33), dtype)
    b = a.copy()
    b[::2] = rand((2, 33), dtype)
    check_prim(ir.P_COMPARE, [a, b[:1].copy()], op=op)
    check_prim(ir.P_COMPARE, [a, b], op=op)


def test_compare_nan():
    a = np.array([np.nan, 1.0, np.nan], f32)
    b = np.array([np.nan, 1.0, 2.0], f32)
    for op in (ir.EQ, ir.NE, ir.LT, ir.GE):
        check_prim(ir.P_COMPARE, [a, b], op=op)


@pytest.mark.parametrize("dtype", [f32, f16, i64, np.uint8, np.bool_])
def test_select_three_way_broadcast(dtype):
    check_prim(ir.P_SELECT, [rand((2, 1, 5), np.bool_), rand((3, 5), dtype), rand((2, 3, 1), dtype)])


# ── Cast ─────────────────────────────────────────────────────────────────
ALL_NP = {ir.F32: f32, ir.F16: f16, ir.I64: i64, ir.I32: i32, ir.U32: np.uint32, ir.U8: np.uint8, ir.I8: np.int8,
          ir.BOOL: np.bool_}


@pytest.mark.parametrize("src", list(ALL_NP))
@pytest.mark.parametrize("dst", list(ALL_NP) + [ir.U4, ir.I4])
def test_cast_matrix(src, dst):
    x = rand((67,), ALL_NP[src])
    if src in (ir.F32, ir.F16):
        x[:6] = np.array([1.9, -1.9, 300.7, -300.7, 0.0, 65504.0], ALL_NP[src])
    check_prim(ir.P_CAST, [x], f16 if dst == ir.F16 else f32, dtype=dst)


def test_cast_float_edge_cases():
    x = np.array([3.0e9, -3.0e9, 1e30, -1e30, np.nan, np.inf, -np.inf, 0.5, -0.5], f32)
    for dst in (ir.I32, ir.I64, ir.U8, ir.I8, ir.U32, ir.BOOL):
        check_prim(ir.P_CAST, [x], dtype=dst)
    big = np.array([2 ** 53 + 1, -(2 ** 62) - 12345, 2 ** 24 + 1, 16777217, 123456789012], i64)
    check_prim(ir.P_CAST, [big], dtype=ir.F32)
    check_prim(ir.P_CAST, [np.array([2049, 2051, 65519, 65520, -70000], i64)], f16, dtype=ir.F16)


@pytest.mark.parametrize("qdt", [ir.U4, ir.I4])
@pytest.mark.parametrize("dst", [ir.I64, ir.I32, ir.U8, ir.I8, ir.F32, ir.F16, ir.BOOL, ir.U4, ir.I4])
def test_cast_unpacks_nibbles_bit_exact(qdt, dst):
    vals = RNG.integers(0, 16, 77)
    m, feed = single_prim_module(ir.P_CAST, [HostTensor.packed_u4(vals, [7, 11], qdt)], dtype=dst)
    differential(m, feed)


# ── MatMul ───────────────────────────────────────────────────────────────
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("dtype", [f32, f16])
def test_matmul_four_layouts(ta, tb, dtype):
    m_, k_, n_ = 33, 70, 45  # the reference's tiled-matmul case (gpu_test.rs:166-207)
    a = (rand((k_, m_) if ta else (m_, k_), dtype) * dtype(0.25)).astype(dtype)
    b = (rand((n_, k_) if tb else (k_, n_), dtype) * dtype(0.25)).astype(dtype)
    t = dict(atol=2e-2, rtol=4e-3) if dtype == f16 else dict(atol=1e-4, rtol=1e-3)
    m, feed = single_prim_module(ir.P_MATMUL, [ht(a), ht(b)], trans_a=ta, trans_b=tb)
    differential(m, feed, **t)


@pytest.mark.parametrize("shape", [(1, 2, 1), (1, 31, 33), (1, 257, 1), (1, 640, 64), (2, 3, 1), (64, 1, 64)])
def test_matmul_small_shapes(shape):
    m_, k_, n_ = shape
    check_prim(ir.P_MATMUL, [rand((m_, k_), f32), rand((k_, n_), f32)])


def test_matmul_batch_broadcast():
    check_prim(ir.P_MATMUL, [rand((2, 1, 5, 7), f32), rand((3, 7, 4), f32)])
    check_prim(ir.P_MATMUL, [rand((2, 3, 5, 7), f32), rand((7, 4), f32)])


def test_matmul_int_wraps():
    a = RNG.integers(-2 ** 40, 2 ** 40, (5, 9)).astype(i64)
    b = RNG.integers(-2 ** 40, 2 ** 40, (9, 4)).astype(i64)
    check_prim(ir.P_MATMUL, [a, b])
    check_prim(ir.P_MATMUL, [rand((5, 9), i32), rand((9, 4), i32)])


# ── Reduce ───────────────────────────────────────────────────────────────
@pytest.mark.parametrize("op", [ir.SUM, ir.MEAN, ir.RMAX, ir.RMIN, ir.PROD])
@pytest.mark.parametrize("axes,keep", [([1], False), ([0], True), ([0, 2], False), ([0, 1, 2], False), ([2], True)])
def test_reduce_float(op, axes, keep):
    x = rand((3, 37, 5), f32)
    if op == ir.PROD:
        x = (x * f32(0.4) + f32(1.0)).astype(f32)
    check_prim(ir.P_REDUCE, [x], op=op, axes=axes, keepdims=keep)


@pytest.mark.parametrize("op", [ir.SUM, ir.MEAN, ir.RMAX, ir.RMIN, ir.PROD])
def test_reduce_int_exact(op):
    check_prim(ir.P_REDUCE, [rand((4, 65), i64)], op=op, axes=[1], keepdims=False)
    check_prim(ir.P_REDUCE, [rand((4, 65), i32)], op=op, axes=[0], keepdims=True)


def test_reduce_f16_row():
    check_prim(ir.P_REDUCE, [rand((6, 1152), f16)], f16, op=ir.MEAN, axes=[1], keepdims=True)


@pytest.mark.parametrize("op", [ir.SUM, ir.MEAN, ir.RMAX, ir.RMIN, ir.PROD])
def test_reduce_few_outputs_over_many_elements(op):
    """Few outputs over at least 256 elements each run one CTA per output (the attention mask's row sum)."""
    check_prim(ir.P_REDUCE, [rand((1, 777), i64)], op=op, axes=[1], keepdims=False)
    check_prim(ir.P_REDUCE, [rand((3, 1300), i32)], op=op, axes=[1], keepdims=True)
    check_prim(ir.P_REDUCE, [rand((2, 300, 5), i64)], op=op, axes=[1], keepdims=False)  # strided reduced axis
    x = rand((2, 2049), f32)
    if op == ir.PROD:
        x = (x * f32(0.01) + f32(1.0)).astype(f32)
    check_prim(ir.P_REDUCE, [x], op=op, axes=[1], keepdims=False)
    check_prim(ir.P_REDUCE, [rand((5, 256), f16)], f16, op=ir.RMAX if op == ir.PROD else op, axes=[1], keepdims=True)


# ── Data movement ────────────────────────────────────────────────────────
@pytest.mark.parametrize("dtype", [f32, f16, i64, np.uint8, np.bool_])
def test_reshape_transpose_broadcast(dtype):
    x = rand((2, 3, 4), dtype)
    check_prim(ir.P_RESHAPE, [x], shape=[6, 4])
    check_prim(ir.P_TRANSPOSE, [x], axes=[2, 0, 1])
    check_prim(ir.P_TRANSPOSE, [rand((2, 5, 3, 7), dtype)], axes=[0, 2, 1, 3])
    check_prim(ir.P_BROADCAST, [rand((3, 1), dtype)], shape=[2, 3, 5])
    check_prim(ir.P_BROADCAST, [rand((), dtype)], shape=[4, 3])


def test_reshape_late_bound_and_chain():
    b = ir.GraphBuilder()
    x = b.input("x", ir.F32, [2, 6])
    r = b.reshape(x, [b.sym("L"), 3])
    b.output("out", b.unary(ir.NEG, b.reshape(r, [12])))
    b.output("view", r)
    differential(b.finish(), {"x": ht(np.arange(12, dtype=f32).reshape(2, 6))})


@pytest.mark.parametrize("dtype", [f32, i64, f16])
def test_concat_and_slice(dtype):
    a, b_, c = rand((2, 1, 3), dtype), rand((2, 4, 3), dtype), rand((2, 2, 3), dtype)
    check_prim(ir.P_CONCAT, [a, b_, c], axis=1)
    check_prim(ir.P_CONCAT, [a, a], axis=0)
    check_prim(ir.P_CONCAT, [a, a, a], axis=2)
    x = rand((5, 6, 7), dtype)
    check_prim(ir.P_SLICE, [x], specs=[(0, 1, 3, 1)])
    check_prim(ir.P_SLICE, [x], specs=[(0, 4, 0, -1), (2, 1, 7, 2)])
    check_prim(ir.P_SLICE, [x], specs=[(1, 5, 0, -2)])
    check_prim(ir.P_SLICE, [x], specs=[(1, 3, 3, 1)])  # empty result


def test_slice_symbolic_bounds():
    b = ir.GraphBuilder()
    s = b.sym("S")
    x = b.input("x", ir.F32, [s, 4])
    b.output("last", b.slice(x, [(0, s - 1, s, 1)]))
    differential(b.finish(), {"x": ht(rand((5, 4), f32))})


@pytest.mark.parametrize("dtype", [f32, f16, i64])
def test_gather(dtype):
    table = rand((7, 3, 2), dtype)
    check_prim(ir.P_GATHER, [table, np.array([[3, 0], [-1, 6]], i64)], axis=0)
    check_prim(ir.P_GATHER, [table, np.array([2, -3], i64)], axis=1)
    check_prim(ir.P_GATHER, [table, np.array(1, i64)], axis=2)


def test_gather_out_of_range_is_an_error_not_a_fault():
    m, feed = single_prim_module(ir.P_GATHER, [ht(rand((4, 2), f32)), ht(np.array([4], i64))], axis=0)
    sess = cuda_backend().prepare(m)
    outs = sess.run({k: sess.upload(v) for k, v in feed.items()})
    with pytest.raises(OnyxiaError, match="gather index 4 out of range for dim 4"):
        sess.download(outs[0][1])
    # the session stays usable
    ok = sess.run({"in0": sess.upload(feed["in0"]), "in1": sess.upload(ht(np.array([1], i64)))})
    assert np.array_equal(sess.download(ok[0][1]).numpy()[0], feed["in0"].numpy()[1])


def test_scatter_last_write_wins():
    check_prim(ir.P_SCATTER, [np.zeros(4, f32), np.array([[1], [1]], i64), np.array([5, 7], f32)])
    data = rand((4, 3, 2), f32)
    idx = np.array([[0, 1], [3, 2], [0, 1], [-1, 0]], i64)
    check_prim(ir.P_SCATTER, [data, idx, rand((4, 2), f32)])
    check_prim(ir.P_SCATTER, [data, np.array([[2], [0]], i64), rand((2, 3, 2), f32)])
    m, feed = single_prim_module(ir.P_SCATTER, [ht(np.zeros(4, f32)), ht(np.array([[9]], i64)), ht(np.array([1], f32))])
    with pytest.raises(OnyxiaError, match="scatter index 9 out of range"):
        be.run_once(cuda_backend(), m, feed)


@pytest.mark.parametrize("dtype", [ir.I64, ir.I32, ir.F32, ir.F16, ir.U8])
def test_iota_and_dim_values(dtype):
    b = ir.GraphBuilder()
    s = b.sym("S")
    x = b.input("x", ir.F32, [s, 3])
    b.output("ramp", b.iota(s * 3, dtype))
    b.output("dims", b.dim_values([s, s * s - 7, DimConst(3)]))
    b.output("x2", b.add(x, x))
    differential(b.finish(), {"x": ht(rand((5, 3), f32))})


def DimConst(v):
    return ir.DimExpr.of(v)


# ── Dequantize ───────────────────────────────────────────────────────────
@pytest.mark.parametrize("qdt", [ir.U4, ir.I4, ir.U8])
@pytest.mark.parametrize("sdt", [f32, f16])
@pytest.mark.parametrize("with_zp", [False, True])
def test_dequantize_bit_exact(qdt, sdt, with_zp):
    n, nb, bs = 5, 3, 32
    if qdt == ir.U8:
        q = HostTensor.from_numpy(RNG.integers(0, 256, (n, nb, bs)).astype(np.uint8))
        zp = HostTensor.from_numpy(RNG.integers(0, 256, (n, nb)).astype(np.uint8))
    else:
        q = HostTensor.packed_u4(RNG.integers(0, 16, n * nb * bs), [n, nb, bs], qdt)
        zp = HostTensor.packed_u4(RNG.integers(0, 16, n * nb), [n, nb], qdt)
    scales = ht(RNG.uniform(0.005, 0.02, (n, nb)).astype(sdt))
    ins = [q, scales] + ([zp] if with_zp else [])
    m, feed = single_prim_module(ir.P_DEQUANTIZE, ins, block_size=bs, shape=[n, nb * bs])
    got, want = differential(m, feed, atol=0, rtol=0)
    assert np.array_equal(got[0][1].data, want[0][1].data)


def test_dequantize_kat():
    data = HostTensor(ir.U4, [1, 4], np.array([0x98, 0xFA], np.uint8))
    m, feed = single_prim_module(ir.P_DEQUANTIZE, [data, ht(np.array([0.5], f32))], block_size=4, shape=[4])
    got, _ = differential(m, feed)
    assert got[0][1].numpy().tolist() == [0.0, 0.5, 1.0, 3.5]


# ── Session behaviour ────────────────────────────────────────────────────
def test_binding_errors_and_handle_chaining():
    b = ir.GraphBuilder()
    s = b.sym("S")
    x = b.input("x", ir.F32, [s])
    y = b.input("y", ir.F32, [s])
    b.output("sum", b.add(x, y))
    sess = cuda_backend().prepare(b.finish())
    t3, t4 = sess.upload(ht(np.array([1, 2, 3], f32))), sess.upload(ht(np.array([1, 2, 3, 4], f32)))
    (_, out), = sess.run({"x": t3, "y": t3})
    # an output handle of one run feeds a later run (crates/onyxia-backend-ref/src/lib.rs:160-185)
    (_, out2), = sess.run({"x": out, "y": t3})
    assert sess.download(out2).numpy().tolist() == [3, 6, 9]
    with pytest.raises(OnyxiaError, match="conflicting values") as e:
        sess.run({"x": t3, "y": t4})
    assert e.value.kind == "Binding"
    with pytest.raises(OnyxiaError, match="missing input 'y'"):
        sess.run({"x": t3})
    with pytest.raises(OnyxiaError, match="dtype"):
        sess.run({"x": t3, "y": sess.upload(ht(np.array([1, 2, 3], i64)))})
    fresh, reuses = sess.pool_stats()
    assert fresh > 0 and sess.resident_bytes() > 0 and sess.peak_resident_bytes() >= sess.resident_bytes()


def test_pool_reuses_buffers_across_runs():
    b = ir.GraphBuilder()
    x = b.input("x", ir.F32, [1024])
    y = b.unary(ir.EXP, b.unary(ir.NEG, b.mul(x, x)))
    b.output("y", y)
    sess = cuda_backend().prepare(b.finish())
    xin = sess.upload(ht(rand((1024,), f32)))
    for _ in range(4):
        sess.run({"x": xin})
    sess.wait_idle()
    fresh, reuses = sess.pool_stats()
    assert reuses >= 3, (fresh, reuses)


# ── movement primitives on packed nibbles ────────────────────────────────
@pytest.mark.parametrize("qdt", [ir.U4, ir.I4])
def test_movement_primitives_move_packed_nibbles_bit_exact(qdt):
    """The interpreter moves U4 / I4 elements through its integer domain (interp.rs:579-748, types.rs:7-11); the device
    widens to bytes, moves, packs again. Odd element counts exercise the half-filled last byte."""
    def q(shape):
        return HostTensor.packed_u4(RNG.integers(0, 16, int(np.prod(shape))), list(shape), qdt)

    m, feed = single_prim_module(ir.P_TRANSPOSE, [q((3, 5, 7))], axes=[2, 0, 1])
    differential(m, feed)
    m, feed = single_prim_module(ir.P_SLICE, [q((6, 9))], specs=[(0, 1, 6, 2), (1, 8, 1, -3)])
    differential(m, feed)
    m, feed = single_prim_module(ir.P_CONCAT, [q((2, 3)), q((5, 3)), q((1, 3))], axis=0)
    differential(m, feed)
    m, feed = single_prim_module(ir.P_BROADCAST, [q((1, 5))], shape=[3, 5])
    differential(m, feed)
    idx = ht(np.array([[2, 0], [-1, 3]], i64))
    m, feed = single_prim_module(ir.P_GATHER, [q((4, 5)), idx], axis=0)
    differential(m, feed)
    upd_idx = ht(np.array([[1], [3], [1]], i64))
    m, feed = single_prim_module(ir.P_SCATTER, [q((4, 5)), upd_idx, q((3, 5))])
    differential(m, feed)
    # Select is not among them: type inference rejects packed operands there (infer.rs:447-461)
    with pytest.raises(OnyxiaError, match="packed dtype"):
        single_prim_module(ir.P_SELECT, [ht(np.ones((3, 5), np.bool_)), q((3, 5)), q((3, 5))])
