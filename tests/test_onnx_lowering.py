"""ONNX bytes → module: the hand-written protobuf codec and the lowering rules of the decoder path, pinned to the
cases of the reference's own lowering tests (crates/onyxia-lower/tests/lower_test.rs: softmax :228-244,
matmul_nbits_end_to_end :246-305, unknown operator :425-440, gqa_through_lowering_runs :442-543) and to the
decoder the benchmarks use, which must lower to the same module the graph builder makes directly."""
import numpy as np
import pytest

from onyxia_b200 import ir, llm, models, onnx
from onyxia_b200.ir import HostTensor


def _run(module, feed):
    from oracle import ref
    ref.set_threads(4)
    return dict(ref.run_once(module, feed))


def test_wire_format_round_trip():
    w = onnx.OnnxWriter("g")
    w.input("x", ir.F32, ["batch", 3])
    w.initializer("w", np.arange(6, dtype=np.float32).reshape(2, 3))
    w.initializer("big", np.array([-1, (1 << 63) - 1], np.int64))
    w.node("Foo", ["x", "", "w"], ["y"], name="n0", domain="com.example", alpha=0.5, k=-3, mode="tanh", axes=[0, -1], flag=True)
    w.output("y", ir.F32, ["batch", 3])
    nodes, inits, inputs, outputs = onnx.parse_model(w.tobytes())
    assert len(nodes) == 1
    n = nodes[0]
    assert (n.op, n.domain, n.name, n.inputs, n.outputs) == ("Foo", "com.example", "n0", ["x", "", "w"], ["y"])
    assert n.attrs == {"alpha": 0.5, "k": -3, "mode": "tanh", "axes": [0, -1], "flag": 1}
    assert inputs == [("x", 1, ["batch", 3])] and outputs == ["y"]
    dtype, dims, raw = inits["w"]
    assert dtype == ir.F32 and dims == [2, 3] and np.array_equal(raw.view(np.float32), np.arange(6, dtype=np.float32))
    assert list(inits["big"][2].view(np.int64)) == [-1, (1 << 63) - 1]


def test_typed_data_fields_and_packed_dims_are_read():
    # an initializer written by another producer: packed dims, float_data / int64_data instead of raw_data
    from onyxia_b200.onnx import _enc_varint, _f_bytes, _f_int, _f_str
    import struct
    t_f = _f_bytes(1, _enc_varint(2) + _enc_varint(2)) + _f_int(2, 1) + _f_bytes(4, struct.pack("<4f", 1, 2, 3, 4)) + _f_str(8, "f")
    t_i = _f_int(1, 3) + _f_int(2, 7) + b"".join(_f_int(7, v) for v in (5, -2, 0)) + _f_str(8, "i")
    graph = _f_bytes(5, t_f) + _f_bytes(5, t_i)
    _, inits, _, _ = onnx.parse_model(_f_bytes(7, graph))
    assert inits["f"][1] == [2, 2] and list(inits["f"][2].view(np.float32)) == [1, 2, 3, 4]
    assert list(inits["i"][2].view(np.int64)) == [5, -2, 0]


def test_softmax_rule():
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, [1, 3])
    w.node("Softmax", ["x"], ["out"], axis=-1)
    w.output("out", ir.F32, [1, 3])
    out = _run(onnx.load_onnx_bytes(w.tobytes()), {"x": HostTensor.from_numpy(np.array([[0, 1, 2]], np.float32))})["out"].numpy()
    e = np.exp(np.array([0, 1, 2], np.float32))
    assert np.abs(out.reshape(-1) - e / e.sum()).max() < 1e-6


def test_matmul_nbits_u8_blob_is_read_as_nibbles():
    k, n, bs = 8, 2, 4
    q = np.array([i % 16 for i in range(n * k)], np.uint8)
    scales = np.array([0.5, 0.25, 1.0, 2.0], np.float32)
    packed = np.zeros(n * k // 2, np.uint8)
    for i, v in enumerate(q):
        packed[i // 2] |= (v & 0xF) << ((i % 2) * 4)
    w = onnx.OnnxWriter()
    w.input("a", ir.F32, [1, k])
    w.initializer("b_q", packed.reshape(n, k // bs, bs // 2))
    w.initializer("scales", scales)
    w.node("MatMulNBits", ["a", "b_q", "scales"], ["out"], domain="com.microsoft", K=k, N=n, bits=4, block_size=bs)
    w.output("out", ir.F32, [1, n])
    module = onnx.load_onnx_bytes(w.tobytes())
    assert module.node_ops() == ["com.microsoft.MatMulNBits"]
    a = (np.arange(k) * 0.1).astype(np.float32)
    got = _run(module.clone(), {"a": HostTensor.from_numpy(a.reshape(1, k))})["out"].numpy().reshape(-1)
    want = [(a * (q[r * k:(r + 1) * k].astype(np.float32) - 8.0) * np.repeat(scales[r * 2:(r + 1) * 2], bs)).sum() for r in range(n)]
    assert np.abs(got - np.array(want)).max() < 1e-4
    # and with every composite decomposed into primitives first
    got2 = _run(module.inline_composites(), {"a": HostTensor.from_numpy(a.reshape(1, k))})["out"].numpy().reshape(-1)
    assert np.abs(got2 - np.array(want)).max() < 1e-4


def test_matmul_nbits_rejects_other_widths_and_missing_attributes():
    for attrs, word in (({"K": 8, "N": 2, "bits": 8, "block_size": 4}, "bits=8"), ({"K": 8, "bits": 4, "block_size": 4}, "'N'")):
        w = onnx.OnnxWriter()
        w.input("a", ir.F32, [1, 8])
        w.initializer("b_q", np.zeros((2, 2, 2), np.uint8))
        w.initializer("scales", np.ones(4, np.float32))
        w.node("MatMulNBits", ["a", "b_q", "scales"], ["out"], domain="com.microsoft", **attrs)
        w.output("out", ir.F32, [1, 2])
        with pytest.raises(onnx.OnnxError, match=word):
            onnx.load_onnx_bytes(w.tobytes())


def test_unknown_operator_is_named():
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, [1])
    w.node("TotallyMadeUpOp", ["x"], ["out"])
    w.output("out", ir.F32, [1])
    with pytest.raises(onnx.OnnxError) as e:
        onnx.load_onnx_bytes(w.tobytes())
    assert "TotallyMadeUpOp" in str(e.value) and "no lowering rule" in str(e.value)


def _gqa_graph(extra_attrs=None, extra_inputs=()):
    h, kv, d = 2, 1, 2
    w = onnx.OnnxWriter()
    w.input("q", ir.F32, [1, "S", h * d])
    w.input("k", ir.F32, [1, "S", kv * d])
    w.input("v", ir.F32, [1, "S", kv * d])
    w.input("past_k", ir.F32, [1, kv, "T", d])
    w.input("past_v", ir.F32, [1, kv, "T", d])
    w.input("seqlens_k", ir.I32, [1])
    w.input("total_len", ir.I32, [1])
    w.node("GroupQueryAttention", ["q", "k", "v", "past_k", "past_v", "seqlens_k", "total_len", *extra_inputs],
           ["out", "present_k", "present_v"], domain="com.microsoft", num_heads=h, kv_num_heads=kv, **(extra_attrs or {}))
    w.output("out", ir.F32, [1, "S", h * d])
    w.output("present_k", ir.F32, [1, kv, "T2", d])
    w.output("present_v", ir.F32, [1, kv, "T2", d])
    return w


def test_gqa_with_symbolic_lengths_runs_from_an_empty_past():
    module = onnx.load_onnx_bytes(_gqa_graph().tobytes())
    f = lambda vals, shape: HostTensor.from_numpy(np.array(vals, np.float32).reshape(shape))
    feed = {"q": f([0.3, -0.1, 0.5, 0.2], (1, 1, 4)), "k": f([0.7, 0.7], (1, 1, 2)), "v": f([42.0, 7.0], (1, 1, 2)),
            "past_k": f([], (1, 1, 0, 2)), "past_v": f([], (1, 1, 0, 2)),
            "seqlens_k": HostTensor.from_numpy(np.array([0], np.int32)), "total_len": HostTensor.from_numpy(np.array([1], np.int32))}
    for mod in (module.clone(), module.inline_composites()):
        out = _run(mod, feed)
        assert out["out"].numpy().reshape(-1).tolist() == [42.0, 7.0, 42.0, 7.0]  # both heads attend to the one position: v
        assert np.allclose(out["present_k"].numpy().reshape(-1), [0.7, 0.7])
        assert out["present_v"].numpy().reshape(-1).tolist() == [42.0, 7.0]


def test_gqa_rejections():
    with pytest.raises(onnx.OnnxError, match="softcap"):
        onnx.load_onnx_bytes(_gqa_graph({"softcap": 30.0}).tobytes())
    with pytest.raises(onnx.OnnxError, match="cos/sin"):
        onnx.load_onnx_bytes(_gqa_graph({"do_rotary": 1}).tobytes())
    w = onnx.OnnxWriter()
    w.input("q", ir.F32, [1, "S", 4])
    w.node("GroupQueryAttention", ["q", "q", "q"], ["out"], domain="com.microsoft", num_heads=2, kv_num_heads=1)
    w.output("out", ir.F32, [1, "S", 4])
    with pytest.raises(onnx.OnnxError, match="requires q/k/v"):
        onnx.load_onnx_bytes(w.tobytes())


def test_shape_arithmetic_becomes_dimension_expressions_and_a_constraint():
    cfg = models.config_c1()
    cfg.vocab, cfg.layers = 512, 1
    module = onnx.load_onnx_bytes(onnx.export_decoder(cfg, seed=2))
    ops = module.node_ops()
    assert "shape" not in " ".join(ops).lower()           # Shape → Gather → Cast folded away
    assert ops.count("com.microsoft.GroupQueryAttention") == 1
    # the folded total_sequence_length became the bind-time check total = past + new
    from oracle import ref
    feed = {"input_ids": HostTensor.from_numpy(np.zeros((1, 2), np.int64)), "attention_mask": HostTensor.from_numpy(np.ones((1, 7), np.int64)),
            "past_key_values.0.key": HostTensor.from_numpy(np.zeros((1, cfg.kv_heads, 3, cfg.head_dim), np.float32)),
            "past_key_values.0.value": HostTensor.from_numpy(np.zeros((1, cfg.kv_heads, 3, cfg.head_dim), np.float32))}
    with pytest.raises(Exception, match="total_sequence_length"):
        ref.run_once(module, feed)


@pytest.mark.parametrize("which", ["c1", "gemma"])
def test_exported_decoder_lowers_to_the_builder_module(which):
    from oracle import ref
    ref.set_threads(8)
    if which == "c1":
        cfg = models.config_c1()
        cfg.vocab = 2048
    else:  # the 1B architecture's features at toy widths: windows, post-norms, last-token slice, f16
        cfg = models.DecoderConfig("toy", layers=3, hidden=128, heads=4, kv_heads=1, head_dim=32, ffn=256, vocab=512, act_dtype=ir.F16,
                                   max_positions=64, window=4, global_every=3, sandwich_norms=True, last_logits_only=True)
    from_onnx = onnx.load_onnx_bytes(onnx.export_decoder(cfg, seed=1))
    built = models.build_decoder(cfg, seed=1)
    assert from_onnx.node_ops() == built.node_ops()
    assert from_onnx.input_names() == built.input_names() and from_onnx.output_names() == built.output_names()
    prompt = np.random.default_rng(0).integers(0, cfg.vocab, 9).tolist()

    def loop(mod):
        s = llm.LlmSession(ref.RefBackend(), mod, 64)
        out = [s.prefill(prompt)]
        for _ in range(4):
            out.append(s.decode(llm.sample_greedy(out[-1])))
        return out

    for a, b in zip(loop(from_onnx), loop(built)):
        assert np.array_equal(a, b)


@pytest.mark.gpu
def test_decoder_from_an_onnx_file_on_the_device(tmp_path):
    from onyxia_b200 import backend as be
    cfg = models.config_c1()
    path = tmp_path / "decoder.onnx"
    path.write_bytes(onnx.export_decoder(cfg, seed=1))
    prompt = np.random.default_rng(0).integers(0, cfg.vocab, 16).tolist()

    def loop(mod):
        s = llm.LlmSession(be.CudaBackend((0,)), mod, 256)
        out = [s.prefill(prompt)]
        for _ in range(8):
            out.append(s.decode(llm.sample_greedy(out[-1])))
        return out

    for a, b in zip(loop(onnx.load_onnx(str(path))), loop(models.build_decoder(cfg, seed=1))):
        assert np.array_equal(a, b)


def test_transpose_of_a_matmul_operand_is_folded_into_the_flag():
    """MatMul(h, Transpose(W)) of a tied-embedding lm_head: the Transpose disappears (fold.rs:129-178), the value stays."""
    rng = np.random.default_rng(0)
    wt = rng.standard_normal((7, 5)).astype(np.float32)   # [vocab, hidden]
    w = onnx.OnnxWriter()
    w.input("h", ir.F32, ["batch", "seq", 5])
    w.initializer("embed", wt)
    w.node("Transpose", ["embed"], ["embed_t"], perm=[1, 0])
    w.node("MatMul", ["h", "embed_t"], ["logits"])
    w.output("logits", ir.F32, ["batch", "seq", 7])
    module = onnx.load_onnx_bytes(w.tobytes())
    assert module.node_ops() == ["matmul"]
    h = rng.standard_normal((2, 3, 5)).astype(np.float32)
    got = _run(module, {"h": HostTensor.from_numpy(h)})["logits"].numpy()
    assert np.abs(got - h @ wt.T).max() < 1e-5


def test_transpose_of_batch_axes_is_not_folded():
    b = ir.GraphBuilder()
    x = b.input("x", ir.F32, [2, 3, 4])
    y = b.input("y", ir.F32, [4, 3, 2])
    b.output("o", b.matmul(x, b.transpose(y, [2, 0, 1])))   # not a swap of the last two axes
    m = b.finish()
    assert m.fold_transposes() is False and m.node_ops() == ["transpose", "matmul"]
    # both operands, flags toggle
    b = ir.GraphBuilder()
    x = b.input("x", ir.F32, [4, 3])
    y = b.input("y", ir.F32, [5, 4])
    b.output("o", b.matmul(b.transpose(x, [1, 0]), b.transpose(y, [1, 0])))
    m = b.finish()
    assert m.fold_transposes() is True and m.node_ops() == ["matmul"]
    rng = np.random.default_rng(1)
    xv, yv = rng.standard_normal((4, 3)).astype(np.float32), rng.standard_normal((5, 4)).astype(np.float32)
    got = _run(m, {"x": HostTensor.from_numpy(xv), "y": HostTensor.from_numpy(yv)})["o"].numpy()
    assert np.abs(got - xv.T @ yv.T).max() < 1e-5


def test_reshape_with_shape_arithmetic_and_rank_one_matmul():
    # Reshape whose target is Concat(Shape(x)[0:1], [-1 → constant]) style arithmetic, and a vector · matrix product
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, ["n", 6])
    w.initializer("idx0", np.array(0, np.int64))
    w.initializer("axes0", np.array([0], np.int64))
    w.initializer("tail", np.array([2, 3], np.int64))
    w.node("Shape", ["x"], ["xs"])
    w.node("Gather", ["xs", "idx0"], ["n_scalar"], axis=0)
    w.node("Unsqueeze", ["n_scalar", "axes0"], ["n_vec"])
    w.node("Concat", ["n_vec", "tail"], ["target"], axis=0)
    w.node("Reshape", ["x", "target"], ["y"])
    w.output("y", ir.F32, ["n", 2, 3])
    module = onnx.load_onnx_bytes(w.tobytes())
    assert module.node_ops() == ["reshape"]
    xv = np.arange(24, dtype=np.float32).reshape(4, 6)
    assert np.array_equal(_run(module, {"x": HostTensor.from_numpy(xv)})["y"].numpy(), xv.reshape(4, 2, 3))

    w = onnx.OnnxWriter()
    w.input("v", ir.F32, [3])
    w.initializer("m", np.arange(12, dtype=np.float32).reshape(3, 4))
    w.node("MatMul", ["v", "m"], ["o"])
    w.output("o", ir.F32, [4])
    vv = np.array([1, 2, 3], np.float32)
    got = _run(onnx.load_onnx_bytes(w.tobytes()), {"v": HostTensor.from_numpy(vv)})["o"].numpy()
    assert got.shape == (4,) and np.array_equal(got, vv @ np.arange(12, dtype=np.float32).reshape(3, 4))


# ── the remaining rules of the reference's registry (crates/onyxia-lower/src/rules.rs:18-96) ──────────────────
def _lower_and_run(w, feed):
    module = onnx.load_onnx_bytes(w.tobytes())
    return module, {k: v.numpy() for k, v in _run(module.clone(), {k: HostTensor.from_numpy(np.ascontiguousarray(v)) for k, v in feed.items()}).items()}


def test_simple_graph_evaluates():
    # out = (x + w) * x — lower_test.rs:113-129
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, [2, 2])
    w.initializer("w", np.array([[10, 20], [30, 40]], np.float32))
    w.node("Add", ["x", "w"], ["sum"])
    w.node("Mul", ["sum", "x"], ["out"])
    w.output("out", ir.F32, [2, 2])
    module, out = _lower_and_run(w, {"x": np.array([[1, 2], [3, 4]], np.float32)})
    assert module.num_nodes == 2
    assert out["out"].reshape(-1).tolist() == [11.0, 44.0, 99.0, 176.0]


_UNARY = {"Neg": np.negative, "Abs": np.abs, "Sqrt": lambda x: np.sqrt(np.abs(x)), "Exp": np.exp, "Log": lambda x: np.log(np.abs(x) + 1),
          "Sin": np.sin, "Cos": np.cos, "Tanh": np.tanh, "Floor": np.floor, "Ceil": np.ceil}


@pytest.mark.parametrize("op", sorted(_UNARY) + ["Erf", "Not"])
def test_unary_rules(op):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((3, 5)) * 2).astype(np.float32)
    w = onnx.OnnxWriter()
    if op == "Not":
        xb = rng.random((3, 5)) > 0.5
        w.input("x", ir.BOOL, [3, 5])
        w.node("Not", ["x"], ["out"])
        w.output("out", ir.BOOL, [3, 5])
        _, out = _lower_and_run(w, {"x": xb})
        assert np.array_equal(out["out"].astype(bool), ~xb)
        return
    if op == "Sqrt":
        x = np.abs(x)
    if op == "Log":
        x = np.abs(x) + 1
    w.input("x", ir.F32, [3, 5])
    w.node(op, ["x"], ["out"])
    w.output("out", ir.F32, [3, 5])
    _, out = _lower_and_run(w, {"x": x})
    if op == "Erf":
        import math
        want = np.vectorize(math.erf)(x.astype(np.float64))
    else:
        want = {"Sqrt": np.sqrt, "Log": np.log}.get(op, _UNARY[op])(x.astype(np.float64))
    assert (np.abs(out["out"] - want) / np.maximum(1.0, np.abs(want))).max() < 2e-6  # one f32 rounding, relative above 1


def test_binary_variadic_compare_and_where_rules():
    rng = np.random.default_rng(4)
    a = rng.standard_normal((2, 4)).astype(np.float32)
    b = rng.standard_normal((4,)).astype(np.float32)
    c = rng.standard_normal((2, 1)).astype(np.float32)
    w = onnx.OnnxWriter()
    w.input("a", ir.F32, [2, 4])
    w.input("b", ir.F32, [4])
    w.input("c", ir.F32, [2, 1])
    w.initializer("two", np.array(2, np.int64))
    w.node("Max", ["a", "b", "c"], ["mx"])
    w.node("Min", ["a", "b", "c"], ["mn"])
    w.node("Max", ["a"], ["same"])
    w.node("Pow", ["a", "two"], ["sq"])          # integer exponent beside a float base
    for op in ("Equal", "Greater", "GreaterOrEqual", "Less", "LessOrEqual"):
        w.node(op, ["a", "b"], [op])
    w.node("And", ["Greater", "Less"], ["and"])
    w.node("Or", ["Greater", "Equal"], ["or"])
    w.node("Xor", ["GreaterOrEqual", "LessOrEqual"], ["xor"])
    w.node("Where", ["Greater", "a", "c"], ["pick"])
    for name, dt in (("mx", ir.F32), ("mn", ir.F32), ("same", ir.F32), ("sq", ir.F32), ("and", ir.BOOL), ("or", ir.BOOL), ("xor", ir.BOOL),
                     ("pick", ir.F32), ("Equal", ir.BOOL), ("LessOrEqual", ir.BOOL)):
        w.output(name, dt, [2, 4])
    b[1] = a[0, 1]  # one exact tie
    _, out = _lower_and_run(w, {"a": a, "b": b, "c": c})
    assert np.array_equal(out["mx"], np.maximum(np.maximum(a, b), c))
    assert np.array_equal(out["mn"], np.minimum(np.minimum(a, b), c))
    assert np.array_equal(out["same"], a)
    assert np.abs(out["sq"] - a * a).max() < 1e-6
    assert np.array_equal(out["Equal"].astype(bool), a == b) and (a == b).any()
    assert np.array_equal(out["LessOrEqual"].astype(bool), a <= b)
    assert np.array_equal(out["and"].astype(bool), (a > b) & (a < b))
    assert np.array_equal(out["or"].astype(bool), (a > b) | (a == b))
    assert np.array_equal(out["xor"].astype(bool), (a >= b) ^ (a <= b))
    assert np.array_equal(out["pick"], np.where(a > b, a, np.broadcast_to(c, a.shape)))


def test_reduce_axes_as_attribute_and_as_operand():
    # lower_test.rs:180-216
    x = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, [2, 3])
    w.node("ReduceMean", ["x"], ["out"], axes=[-1], keepdims=0)
    w.output("out", ir.F32, [2])
    assert _lower_and_run(w, {"x": x})[1]["out"].tolist() == [2.0, 5.0]
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, [2, 3])
    w.initializer("axes", np.array([0], np.int64))
    w.node("ReduceSum", ["x", "axes"], ["out"], keepdims=1)
    w.output("out", ir.F32, [1, 3])
    out = _lower_and_run(w, {"x": x})[1]["out"]
    assert out.shape == (1, 3) and out.reshape(-1).tolist() == [5.0, 7.0, 9.0]
    # the other three reductions; no axes = every axis; noop_with_empty_axes leaves the operand alone
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, [2, 3])
    w.node("ReduceMax", ["x"], ["mx"], axes=[1], keepdims=0)
    w.node("ReduceMin", ["x"], ["mn"], keepdims=0)
    w.node("ReduceProd", ["x"], ["pr"], axes=[0, -2], keepdims=1)
    w.node("ReduceSum", ["x"], ["noop"], noop_with_empty_axes=1)
    w.node("Add", ["noop", "pr"], ["sum"])
    for name, shape in (("mx", [2]), ("mn", []), ("pr", [1, 3]), ("sum", [2, 3])):
        w.output(name, ir.F32, shape)
    out = _lower_and_run(w, {"x": x})[1]
    assert out["mx"].tolist() == [3.0, 6.0] and float(out["mn"]) == 1.0
    assert out["pr"].reshape(-1).tolist() == [4.0, 10.0, 18.0]
    assert np.array_equal(out["sum"], x + np.array([[4, 10, 18]], np.float32))


def test_constant_of_shape_and_expand_over_a_symbolic_shape():
    # lower_test.rs:308-327
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, ["S", 4])
    w.initializer("bias", np.array([1, 2, 3, 4], np.float32))
    w.node("Shape", ["x"], ["shp"])
    w.node("ConstantOfShape", ["shp"], ["zeros"])
    w.node("Expand", ["bias", "shp"], ["bias_full"])
    w.node("Add", ["zeros", "bias_full"], ["out"])
    w.output("out", ir.F32, ["S", 4])
    out = _lower_and_run(w, {"x": np.zeros((2, 4), np.float32)})[1]["out"]
    assert out.shape == (2, 4) and out.reshape(-1).tolist() == [1, 2, 3, 4, 1, 2, 3, 4]


def test_constant_of_shape_keeps_the_value_tensors_type():
    # lower_test.rs:330-358: an i64 ones-fill must survive with its type
    w = onnx.OnnxWriter()
    w.input("x", ir.I64, [3])
    w.node("Shape", ["x"], ["shp"])
    w.node("ConstantOfShape", ["shp"], ["ones"], value=np.array([1], np.int64))
    w.node("Add", ["ones", "x"], ["out"])
    w.output("out", ir.I64, [3])
    out = _lower_and_run(w, {"x": np.array([10, 20, 30], np.int64)})[1]["out"]
    assert out.dtype == np.int64 and out.tolist() == [11, 21, 31]


def test_shape_value_consumed_by_a_tensor_operation_is_evaluated_at_run_time():
    # lower_test.rs:361-415: seqlens = Shape(mask)[1] - 1 expanded to [batch, 1]
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, ["B", "T"])
    w.initializer("idx0", np.array(0, np.int64))
    w.initializer("idx1", np.array(1, np.int64))
    w.initializer("c1", np.array(1, np.int64))
    w.initializer("ax0", np.array([0], np.int64))
    w.initializer("one_vec", np.array([1], np.int64))
    w.node("Shape", ["x"], ["shp"])
    w.node("Gather", ["shp", "idx1"], ["t"], axis=0)
    w.node("Sub", ["t", "c1"], ["tm1"])
    w.node("Unsqueeze", ["tm1", "ax0"], ["u"])
    w.node("Gather", ["shp", "idx0"], ["b"], axis=0)
    w.node("Unsqueeze", ["b", "ax0"], ["bu"])
    w.node("Concat", ["bu", "one_vec"], ["tgt"], axis=0)
    w.node("Expand", ["u", "tgt"], ["out"])
    w.output("out", ir.I64, ["B", 1])
    module, out = _lower_and_run(w, {"x": np.zeros((2, 5), np.float32)})
    assert "dim_values" in " ".join(module.node_ops()).lower().replace("dimvalues", "dim_values")
    assert out["out"].shape == (2, 1) and out["out"].reshape(-1).tolist() == [4, 4]


def test_slice_sentinel_negative_symbolic_and_stepped_bounds():
    # lower_test.rs:418-429
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, [5])
    w.initializer("starts", np.array([1], np.int64))
    w.initializer("ends", np.array([np.iinfo(np.int64).max], np.int64))
    w.node("Slice", ["x", "starts", "ends"], ["out"])
    w.output("out", ir.F32, [4])
    x = np.array([10, 11, 12, 13, 14], np.float32)
    assert _lower_and_run(w, {"x": x})[1]["out"].tolist() == [11, 12, 13, 14]
    # negative bounds on a named axis, a stride, an end past the extent, and an end that is shape arithmetic
    w = onnx.OnnxWriter()
    w.input("m", ir.F32, ["R", 6])
    w.input("probe", ir.F32, ["K"])
    w.initializer("s", np.array([-4], np.int64))
    w.initializer("e", np.array([-1], np.int64))
    w.initializer("ax", np.array([-1], np.int64))
    w.node("Slice", ["m", "s", "e", "ax"], ["mid"])
    w.initializer("s0", np.array([0], np.int64))
    w.initializer("e9", np.array([9], np.int64))
    w.initializer("ax1", np.array([1], np.int64))
    w.initializer("st2", np.array([2], np.int64))
    w.node("Slice", ["m", "s0", "e9", "ax1", "st2"], ["even"])
    w.node("Shape", ["probe"], ["k"])
    w.initializer("ax0", np.array([0], np.int64))
    w.node("Slice", ["m", "s0", "k", "ax0"], ["head"])
    w.output("mid", ir.F32, ["R", 3])
    w.output("even", ir.F32, ["R", 3])
    w.output("head", ir.F32, ["K", 6])
    m = np.arange(24, dtype=np.float32).reshape(4, 6)
    out = _lower_and_run(w, {"m": m, "probe": np.zeros(3, np.float32)})[1]
    assert np.array_equal(out["mid"], m[:, -4:-1]) and np.array_equal(out["even"], m[:, 0:9:2]) and np.array_equal(out["head"], m[:3])


def test_squeeze_scatter_range_trilu_and_constant_nodes():
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, [1, 3, 1, 4])
    w.input("len_probe", ir.F32, ["L"])
    w.initializer("ax", np.array([0, -2], np.int64))
    w.node("Squeeze", ["x", "ax"], ["sq"])        # [3, 4]
    w.node("Squeeze", ["x"], ["sq_all"])          # every extent-1 axis
    w.node("Constant", [], ["idx"], value=np.array([[2], [0]], np.int64))
    w.node("Constant", [], ["upd"], value=np.array([[9, 9, 9, 9], [7, 7, 7, 7]], np.float32))
    w.node("ScatterND", ["sq", "idx", "upd"], ["sc"])
    w.node("Trilu", ["sq"], ["up"])
    w.node("Constant", [], ["km1"], value_int=-1)
    w.node("Trilu", ["sq", "km1"], ["low"], upper=0)
    # Range(2, 2 + 3·L, 3): symbolic limit, constant start and delta
    w.node("Shape", ["len_probe"], ["l"])
    w.initializer("three", np.array([3], np.int64))
    w.initializer("two", np.array([2], np.int64))
    w.node("Mul", ["l", "three"], ["l3"])
    w.node("Add", ["l3", "two"], ["lim"])
    w.initializer("zero_ax", np.array([0], np.int64))
    w.node("Squeeze", ["lim", "zero_ax"], ["lim_s"])
    w.node("Constant", [], ["start"], value_int=2)
    w.node("Constant", [], ["delta"], value_int=3)
    w.node("Range", ["start", "lim_s", "delta"], ["rng"])
    for name, dt, shape in (("sq_all", ir.F32, [3, 4]), ("sc", ir.F32, [3, 4]), ("up", ir.F32, [3, 4]), ("low", ir.F32, [3, 4]), ("rng", ir.I64, ["L"])):
        w.output(name, dt, shape)
    x = np.arange(12, dtype=np.float32).reshape(1, 3, 1, 4) + 1
    module, out = _lower_and_run(w, {"x": x, "len_probe": np.zeros(4, np.float32)})
    m = x.reshape(3, 4)
    assert np.array_equal(out["sq_all"], m)
    want = m.copy()
    want[2], want[0] = 9, 7
    assert np.array_equal(out["sc"], want)
    assert np.array_equal(out["up"], np.triu(m)) and np.array_equal(out["low"], np.tril(m, -1))
    assert out["rng"].tolist() == [2, 5, 8, 11]
    assert "Trilu" in module.node_ops()
    with pytest.raises(onnx.OnnxError, match="reduction"):
        w2 = onnx.OnnxWriter()
        w2.input("d", ir.F32, [3])
        w2.input("i", ir.I64, [1, 1])
        w2.input("u", ir.F32, [1])
        w2.node("ScatterND", ["d", "i", "u"], ["o"], reduction="add")
        w2.output("o", ir.F32, [3])
        onnx.load_onnx_bytes(w2.tobytes())


@pytest.mark.parametrize("op", ["RotaryEmbedding", "GemmaRotaryEmbedding"])
def test_rotary_embedding_rule(op):
    heads, d, seq, maxpos = 2, 8, 3, 16
    rng = np.random.default_rng(9)
    x = rng.standard_normal((1, seq, heads * d)).astype(np.float32)
    ang = np.outer(np.arange(maxpos), 1.0 / 10000 ** (np.arange(d // 2) / (d // 2))).astype(np.float32)
    pos = np.array([[5, 6, 7]], np.int64)
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, [1, "S", heads * d])
    w.input("pos", ir.I64, [1, "S"])
    w.initializer("cos", np.cos(ang))
    w.initializer("sin", np.sin(ang))
    w.node(op, ["x", "pos", "cos", "sin"], ["out"], domain="com.microsoft", num_heads=heads, interleaved=0)
    w.output("out", ir.F32, [1, "S", heads * d])
    module, out = _lower_and_run(w, {"x": x, "pos": pos})
    assert module.node_ops() == ["com.microsoft." + op]
    x4 = x.reshape(1, seq, heads, d)
    c, s = np.cos(ang)[pos[0]][None, :, None, :], np.sin(ang)[pos[0]][None, :, None, :]
    x1, x2 = x4[..., :d // 2], x4[..., d // 2:]
    want = np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], -1).reshape(1, seq, heads * d)
    assert np.abs(out["out"] - want).max() < 1e-5


@pytest.mark.gpu
def test_graph_of_plain_operators_on_the_device():
    """A graph mixing the plain rules (mask building, reductions, rotary, a stepped slice) gives on the device what
    the CPU interpreter gives: integers and booleans bit-exact, f32 within 1e-5."""
    from onyxia_b200 import backend as be
    heads, d = 2, 8
    rng = np.random.default_rng(12)
    ang = np.outer(np.arange(32), 1.0 / 10000 ** (np.arange(d // 2) / (d // 2))).astype(np.float32)
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, [1, "S", heads * d])
    w.input("pos", ir.I64, [1, "S"])
    w.initializer("cos", np.cos(ang))
    w.initializer("sin", np.sin(ang))
    w.node("RotaryEmbedding", ["x", "pos", "cos", "sin"], ["rot"], domain="com.microsoft", num_heads=heads)
    # causal mask from Range / Unsqueeze / LessOrEqual, applied with Where
    w.node("Shape", ["pos"], ["shp"])
    w.initializer("i1", np.array(1, np.int64))
    w.node("Gather", ["shp", "i1"], ["s"], axis=0)
    w.node("Constant", [], ["zero"], value_int=0)
    w.node("Constant", [], ["one"], value_int=1)
    w.node("Range", ["zero", "s", "one"], ["r"])
    w.initializer("ax0", np.array([0], np.int64))
    w.initializer("ax1", np.array([1], np.int64))
    w.node("Unsqueeze", ["r", "ax0"], ["cols"])
    w.node("Unsqueeze", ["r", "ax1"], ["rows"])
    w.node("LessOrEqual", ["cols", "rows"], ["causal"])
    w.node("Transpose", ["rot"], ["rot_t"], perm=[0, 2, 1])
    w.node("MatMul", ["rot", "rot_t"], ["scores"])                      # [1, S, S]
    w.node("Constant", [], ["neg"], value=np.array(-1e9, np.float32))
    w.node("Where", ["causal", "scores", "neg"], ["masked"])
    w.node("Softmax", ["masked"], ["p"], axis=-1)
    w.node("ReduceMax", ["p"], ["pmax"], axes=[-1], keepdims=0)
    w.node("ReduceMean", ["rot"], ["mean"], axes=[1], keepdims=1)
    w.node("Trilu", ["scores"], ["lower"], upper=0)
    w.initializer("s0", np.array([1], np.int64))
    w.initializer("e0", np.array([1 << 40], np.int64))
    w.initializer("ax2", np.array([2], np.int64))
    w.initializer("st", np.array([3], np.int64))
    w.node("Slice", ["rot", "s0", "e0", "ax2", "st"], ["strided"])
    w.node("Tanh", ["strided"], ["act"])
    for name, dt, shape in (("causal", ir.BOOL, ["S", "S"]), ("p", ir.F32, [1, "S", "S"]), ("pmax", ir.F32, [1, "S"]),
                            ("mean", ir.F32, [1, 1, heads * d]), ("lower", ir.F32, [1, "S", "S"]), ("act", ir.F32, [1, "S", 5]), ("r", ir.I64, ["S"])):
        w.output(name, dt, shape)
    module = onnx.load_onnx_bytes(w.tobytes())
    for seq in (1, 7, 33):
        feed = {"x": HostTensor.from_numpy(rng.standard_normal((1, seq, heads * d)).astype(np.float32)),
                "pos": HostTensor.from_numpy(np.arange(seq, dtype=np.int64).reshape(1, seq) % 32)}
        want = _run(module.clone(), feed)
        got = dict(be.run_once(be.CudaBackend((0,)), module.clone(), feed))
        for name, t in want.items():
            a, b = got[name].numpy(), t.numpy()
            assert a.shape == b.shape, name
            if b.dtype.kind == "f":
                assert np.abs(a - b).max() <= 1e-5, name
            else:
                assert np.array_equal(a, b), name


def test_reshape_infers_the_free_dimension_beside_symbolic_extents():
    """-1 in a Reshape target: the element count divided by the known extents when that is exact (a monomial
    division, dim.rs:254-280), otherwise a symbol bound from the element count when the graph runs (rules.rs:247-259)."""
    assert (ir.DimExpr.sym(0) * ir.DimExpr.sym(1) * 6).div_exact(ir.DimExpr.sym(1) * 3) == ir.DimExpr.sym(0) * 2
    assert (ir.DimExpr.sym(0) * 4 + 4).div_exact(2) == ir.DimExpr.sym(0) * 2 + 2
    assert (ir.DimExpr.sym(0) * 3).div_exact(2) is None and ir.DimExpr.of(8).div_exact(ir.DimExpr.sym(0) + 1) is None
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, ["B", "S", 256])
    w.input("y", ir.F32, ["R", 3])
    w.initializer("heads", np.array([0, 0, 4, -1], np.int64))
    w.initializer("pairs", np.array([-1, 2], np.int64))
    w.initializer("halves", np.array([2, -1], np.int64))
    w.node("Reshape", ["x", "heads"], ["h"])       # 256 / 4 = 64, constant
    w.node("Reshape", ["x", "pairs"], ["p"])       # B·S·256 / 2 = 128·B·S, symbolic and exact
    w.node("Reshape", ["y", "halves"], ["q"])      # 3·R / 2: only known when R is
    w.output("h", ir.F32, ["B", "S", 4, 64])
    w.output("p", ir.F32, ["N", 2])
    w.output("q", ir.F32, [2, "M"])
    module = onnx.load_onnx_bytes(w.tobytes())
    x = np.arange(2 * 3 * 256, dtype=np.float32).reshape(2, 3, 256)
    y = np.arange(12, dtype=np.float32).reshape(4, 3)
    out = _run(module, {"x": HostTensor.from_numpy(x), "y": HostTensor.from_numpy(y)})
    assert np.array_equal(out["h"].numpy(), x.reshape(2, 3, 4, 64))
    assert np.array_equal(out["p"].numpy(), x.reshape(-1, 2))
    assert np.array_equal(out["q"].numpy(), y.reshape(2, 6))
    with pytest.raises(onnx.OnnxError, match="at most one -1"):
        w2 = onnx.OnnxWriter()
        w2.input("x", ir.F32, [4, 4])
        w2.initializer("t", np.array([-1, -1], np.int64))
        w2.node("Reshape", ["x", "t"], ["o"])
        w2.output("o", ir.F32, [4, 4])
        onnx.load_onnx_bytes(w2.tobytes())


def test_external_tensor_data_from_files_and_from_buffers(tmp_path):
    """Initializers whose bytes live outside the model (data_location = EXTERNAL, parser.rs:297-380): read from the file
    beside the model, or from buffers handed over with the bytes; a missing file or range is named."""
    rng = np.random.default_rng(3)
    wgt = rng.standard_normal((4, 3)).astype(np.float32)
    bias = rng.standard_normal(3).astype(np.float32)
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, ["B", 4])
    w.initializer("w", wgt, external="weights.bin")
    w.initializer("b", bias, external="weights.bin")
    w.node("MatMul", ["x", "w"], ["xw"])
    w.node("Add", ["xw", "b"], ["y"])
    w.output("y", ir.F32, ["B", 3])
    model = w.tobytes()
    assert set(w.external) == {"weights.bin"} and len(w.external["weights.bin"]) == 64 + 12
    (tmp_path / "m.onnx").write_bytes(model)
    (tmp_path / "weights.bin").write_bytes(bytes(w.external["weights.bin"]))
    x = rng.standard_normal((2, 4)).astype(np.float32)
    want = x @ wgt + bias
    for module in (onnx.load_onnx(str(tmp_path / "m.onnx")), onnx.load_onnx_bytes(model, {"weights.bin": bytes(w.external["weights.bin"])})):
        got = _run(module, {"x": HostTensor.from_numpy(x)})["y"].numpy()
        assert np.abs(got - want).max() < 1e-5
    with pytest.raises(onnx.OnnxError, match="external file"):
        onnx.load_onnx_bytes(model)
    with pytest.raises(onnx.OnnxError, match="not provided"):
        onnx.load_onnx_bytes(model, {})
    with pytest.raises(onnx.OnnxError, match="outside the buffer"):
        onnx.load_onnx_bytes(model, {"weights.bin": b"\0" * 16})
    (tmp_path / "weights.bin").unlink()
    with pytest.raises(onnx.OnnxError, match="not found"):
        onnx.load_onnx(str(tmp_path / "m.onnx"))


def _tensor_bytes(dt, dims, **typed):
    """A TensorProto written field by field: dims (1), data_type (2), float_data (4, packed), int32_data (5), int64_data (7), name (8)."""
    import struct
    from onyxia_b200.onnx import _f_bytes, _f_int, _f_str
    t = b"".join(_f_int(1, d) for d in dims) + _f_int(2, dt) + _f_str(8, "w")
    if "f" in typed:
        t += _f_bytes(4, struct.pack(f"<{len(typed['f'])}f", *typed["f"]))
    t += b"".join(_f_int(5, v) for v in typed.get("i32", ()))
    t += b"".join(_f_int(7, v) for v in typed.get("i64", ()))
    t += b"".join(_f_int(11, v) for v in typed.get("u64", ()))
    return t


def test_typed_data_fields_follow_the_declared_type():
    # parser.rs:662-711: every case gives the bytes raw_data would hold
    import struct
    from onyxia_b200.onnx import _parse_tensor
    cases = [((1, [2], dict(f=[1.5, -2.0])), struct.pack("<2f", 1.5, -2.0)),
             ((7, [2], dict(i64=[-1, 7])), struct.pack("<2q", -1, 7)),
             ((2, [3], dict(i32=[0, 128, 255])), bytes([0, 128, 255])),          # uint8 in int32_data
             ((9, [2], dict(i32=[1, 0])), bytes([1, 0])),                        # bool in int32_data
             ((10, [2], dict(i32=[0x3C00, 0xC000])), struct.pack("<2H", 0x3C00, 0xC000)),  # float16 bit patterns: 1.0, −2.0
             ((6, [2], dict(i32=[-5, 9])), struct.pack("<2i", -5, 9)),
             ((12, [1], dict(u64=[4000000000])), struct.pack("<I", 4000000000))]
    for (dt, dims, typed), want in cases:
        _, _, got_dims, raw = _parse_tensor(_tensor_bytes(dt, dims, **typed))
        assert got_dims == dims and raw.tobytes() == want, (dt, typed)
    assert _parse_tensor(_tensor_bytes(1, [0]))[3].size == 0                      # a zero-element tensor may be empty


def test_initializer_without_data_or_with_the_wrong_typed_field_is_an_error():
    # parser.rs:713-735: never a silently empty weight
    from onyxia_b200.onnx import _parse_tensor
    with pytest.raises(onnx.OnnxError, match="carries no data"):
        _parse_tensor(_tensor_bytes(1, [4]))
    with pytest.raises(onnx.OnnxError, match="float_data is populated"):
        _parse_tensor(_tensor_bytes(7, [1], f=[1.0]))
    with pytest.raises(onnx.OnnxError, match="int64_data is populated"):
        _parse_tensor(_tensor_bytes(1, [1], i64=[3]))
    with pytest.raises(onnx.OnnxError, match="int32_data with data type"):
        _parse_tensor(_tensor_bytes(1, [1], i32=[3]))


def test_input_dimension_without_value_or_name_is_the_symbol_unknown():
    # parser.rs:611-623
    from onyxia_b200.onnx import _f_bytes, _f_int, _f_str
    dims = _f_bytes(1, b"") + _f_bytes(1, _f_int(1, 3))           # one empty Dimension, then dim_value 3
    vi = lambda name: _f_str(1, name) + _f_bytes(2, _f_bytes(1, _f_int(1, 1) + _f_bytes(2, dims)))
    node = _f_str(1, "x") + _f_str(2, "y") + _f_str(4, "Neg")
    graph = _f_bytes(1, node) + _f_str(2, "g") + _f_bytes(11, vi("x")) + _f_bytes(12, vi("y"))
    module = onnx.load_onnx_bytes(_f_bytes(7, graph))
    x = np.arange(6, dtype=np.float32).reshape(2, 3)
    assert module.eval_input_shape(0, {"unknown": 2}) == (2, 3)
    assert np.array_equal(_run(module, {"x": HostTensor.from_numpy(x)})["y"].numpy(), -x)


def test_graph_outputs_that_are_shape_values():
    # lib.rs:506-529: constant shape values leave as i64 constants, symbolic ones are refused, unknown names are named
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, ["B", 3, 5])
    w.node("Shape", ["x"], ["shp"], start=1)
    w.node("Neg", ["x"], ["y"])
    w.output("shp", ir.I64, [2])
    w.output("y", ir.F32, ["B", 3, 5])
    out = _run(onnx.load_onnx_bytes(w.tobytes()), {"x": HostTensor.from_numpy(np.zeros((2, 3, 5), np.float32))})
    assert out["shp"].numpy().tolist() == [3, 5] and out["shp"].numpy().dtype == np.int64
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, ["B", 3])
    w.node("Shape", ["x"], ["shp"])
    w.output("shp", ir.I64, [2])
    with pytest.raises(onnx.OnnxError, match="symbolic shape value"):
        onnx.load_onnx_bytes(w.tobytes())
    w = onnx.OnnxWriter()
    w.input("x", ir.F32, [1])
    w.node("Neg", ["x"], ["y"])
    w.output("z", ir.F32, [1])
    with pytest.raises(onnx.OnnxError, match="never produced"):
        onnx.load_onnx_bytes(w.tobytes())
