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
