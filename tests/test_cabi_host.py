"""CPU-side checks of the C ABI and the host logic: the libraries load, export
every symbol ``include/onyxia_cuda.h`` declares, and the module builder behaves
like the reference's (dim algebra crates/onyxia-ir/src/dim.rs:485-625, inference
errors infer.rs:514-795, validation, legalisation). No compute call is made.
"""
import ctypes as C
import os
import re

import numpy as np
import pytest

from onyxia_b200 import OnyxiaError, _ffi, ir, models
from onyxia_b200.ir import DimExpr, HostTensor

from util import ht

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "onyxia_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ox_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    lib = C.CDLL(_ffi.cuda_path(), mode=C.RTLD_GLOBAL) if os.path.exists(_ffi.ir_path()) and _ffi.ir_lib() else None
    names = header_functions()
    assert len(names) >= 45
    for n in names:
        assert hasattr(lib, n), f"libonyxia_cuda.so does not export {n}"
    assert set(names) == set(_ffi.SIGNATURES), set(names) ^ set(_ffi.SIGNATURES)


def test_backend_fails_loudly_without_a_gpu_or_works_with_one():
    import torch
    from onyxia_b200 import backend as be
    if torch.cuda.is_available():
        assert be.CudaBackend((0,)).supports("Softmax")
    else:
        with pytest.raises(OnyxiaError, match="no CUDA device available") as e:
            be.CudaBackend((0,))
        assert e.value.kind == "Runtime"


def test_dim_algebra_is_canonical():
    b = ir.GraphBuilder()
    s, t = b.sym("S"), b.sym("T")
    assert s * 4 + s == s * 5
    assert (s + t) * (s - t) == s * s - t * t
    assert (s + 3) - s == 3 and ((s + 3) - s).as_const() == 3
    assert (s * 0).as_const() == 0
    assert (s - s + 7).as_const() == 7
    assert (DimExpr.of(2) - 5).as_const() is None  # negative constants are not dims
    assert s + t == t + s and s * t == t * s
    assert b.sym("S") == s  # interning


def test_inference_errors_surface_at_the_call_site():
    b = ir.GraphBuilder()
    x = b.input("x", ir.F32, [2])
    y = b.input("y", ir.I64, [2])
    with pytest.raises(OnyxiaError, match="dtype mismatch") as e:
        b.add(x, y)
    assert e.value.kind == "Shape"  # wrapped by the builder like builder.rs:155-166
    s, t = b.sym("S"), b.sym("T")
    a = b.input("a", ir.F32, [s, 3])
    c = b.input("c", ir.F32, [t, 3])
    with pytest.raises(OnyxiaError, match="cannot broadcast dim"):
        b.add(a, c)
    with pytest.raises(OnyxiaError, match="contraction mismatch"):
        b.matmul(a, a)
    assert b.module().value_type_str(b.matmul(a, c, trans_b=True)) == "f32[S, T]"
    with pytest.raises(OnyxiaError, match="element count mismatch"):
        b.reshape(x, [3])
    with pytest.raises(OnyxiaError, match="not a permutation"):
        b.transpose(a, [0, 0])
    with pytest.raises(OnyxiaError, match="requires constant bounds"):
        b.slice(a, [(0, 0, s, 2)])
    with pytest.raises(OnyxiaError, match="axes must be sorted and unique"):
        b.reduce(ir.SUM, a, [1, 0], False)
    with pytest.raises(OnyxiaError, match="gather indices must be i64"):
        b.gather(a, x, 0)
    with pytest.raises(OnyxiaError, match="expected bool"):
        b.select(x, x, x)
    with pytest.raises(OnyxiaError, match="packed dtype"):
        q = b.constant(HostTensor(ir.U4, [4], np.zeros(2, np.uint8)))
        b.cmp(ir.EQ, q, q)
    with pytest.raises(OnyxiaError, match="expects 2 inputs, got 1"):
        b.prim(ir.P_BINARY, [x], op=ir.ADD)
    # symbolic shapes flow through concat / slice / gather
    cat = b.concat([a, a], 0)
    assert b.module().value_type_str(cat) == "f32[2*S, 3]"
    assert b.module().value_type_str(b.slice(cat, [(0, s, s * 2, 1)])) == "f32[S, 3]"
    idx = b.input("idx", ir.I64, [t])
    assert b.module().value_type_str(b.gather(a, idx, 1)) == "f32[S, T]"


def test_dequantize_type_rule():
    b = ir.GraphBuilder()
    q = b.constant(HostTensor(ir.U4, [2, 3, 32], np.zeros(96, np.uint8)))
    s = b.constant(ht(np.ones((2, 3), np.float16)))
    out = b.dequantize(q, s, block_size=32, out_shape=[2, 96])
    assert b.module().value_type_str(out) == "f16[2, 96]"
    with pytest.raises(OnyxiaError, match="last dim 32 != block_size 16"):
        b.dequantize(q, s, block_size=16, out_shape=[2, 96])
    with pytest.raises(OnyxiaError, match="element count mismatch"):
        b.dequantize(q, s, block_size=32, out_shape=[2, 95])
    with pytest.raises(OnyxiaError, match="data must be u4/i4/u8"):
        b.dequantize(s, s, block_size=32, out_shape=[2, 96])


def test_constants_are_size_checked_and_attribute_errors_are_precise():
    b = ir.GraphBuilder()
    with pytest.raises(OnyxiaError, match="constant data size mismatch") as e:
        dims = (C.c_uint64 * 1)(3)
        out = C.c_int32()
        buf = (C.c_uint8 * 11)()
        _ffi.check(_ffi.ir_lib().ox_module_add_const(b.module().handle, ir.F32, dims, 1, buf, 11, 0, C.byref(out)))
    assert e.value.kind == "InvalidGraph"
    x = b.input("x", ir.F32, [2, 4])
    out = b.composite("Softmax", {"axis": "oops"}, [x], [(ir.F32, [2, 4])])
    b.output("y", out[0])
    m = b.finish()
    with pytest.raises(OnyxiaError, match="expected int, found str") as e:
        m.inline_composites([])
    assert e.value.kind == "Attribute"
    with pytest.raises(OnyxiaError, match="must declare at least one output"):
        ir.GraphBuilder().composite("Softmax", {}, [], [])


def test_legalisation_keeps_supported_composites_and_checks_declared_types():
    cfg = models.config_c1()
    cfg.vocab, cfg.layers = 64, 1
    m = models.build_decoder(cfg, seed=0)
    assert m.node_ops().count("com.microsoft.MatMulNBits") == 8
    kept = m.clone().inline_composites(["com.microsoft.MatMulNBits", "Softmax"])
    ops = kept.node_ops()
    assert "com.microsoft.GroupQueryAttention" not in ops and "Softmax" in ops and "com.microsoft.MatMulNBits" in ops
    assert "com.microsoft.RotaryEmbedding" not in ops  # emitted by the GQA decomposition, inlined recursively
    full = m.clone().inline_composites([])
    assert all(op[0].islower() and "." not in op for op in full.node_ops())
    full.validate()
    # a composite whose declared output type disagrees with its decomposition is rejected
    b = ir.GraphBuilder()
    x = b.input("x", ir.F32, [2, 4])
    b.output("y", b.composite("Softmax", {"axis": 1}, [x], [(ir.F32, [2, 5])])[0])
    with pytest.raises(OnyxiaError, match="declared output type"):
        b.finish().inline_composites([])
    b = ir.GraphBuilder()
    x = b.input("x", ir.F32, [2])
    b.output("y", b.composite("com.example.Unknown", {}, [x], [(ir.F32, [2])])[0])
    with pytest.raises(OnyxiaError, match="no kernel and no decomposition") as e:
        b.finish().inline_composites([])
    assert e.value.kind == "Unsupported"


def test_module_io_introspection_matches_llm_session_needs():
    from onyxia_b200 import llm
    cfg = models.config_c1()
    cfg.vocab, cfg.layers = 64, 2
    m = models.build_decoder(cfg, seed=0)
    names = m.input_names()
    assert names[:2] == ["input_ids", "attention_mask"] and "past_key_values.1.value" in names
    assert m.output_names()[0] == "logits"
    assert llm.discover_kv_pairs(m) == [(f"present.{l}.{kv}", f"past_key_values.{l}.{kv}") for l in range(2) for kv in ("key", "value")]
    i = names.index("past_key_values.0.key")
    assert m.input_desc(i) == (ir.F32, 4)
    bind = {"batch_size": 1, "sequence_length": 3, "past_sequence_length": 5, "total_sequence_length": 8}
    assert m.eval_input_shape(i, bind) == (1, cfg.kv_heads, 5, cfg.head_dim)
    assert m.eval_input_shape(1, bind) == (1, 8)


def test_greedy_sampler_keeps_the_last_maximum():
    from onyxia_b200 import llm
    assert llm.sample_greedy(np.array([1.0, 3.0, 3.0, 2.0], np.float32)) == 2
    assert llm.sample_greedy(np.array([5.0], np.float32)) == 0
    with pytest.raises(ValueError):
        llm.sample_greedy(np.array([], np.float32))


def test_byte_accounting_matches_the_roofline_figures():
    cfg = models.config_gemma3_1b()
    assert cfg.weight_bytes_per_token() == 562_360_320  # 26 × 15 095 808 + 169 869 312
    assert [cfg.layer_window(l) for l in range(6)] == [512, 512, 512, 512, 512, -1]
    c27 = models.config_gemma3_27b()
    assert c27.weight_bytes_per_token() == 15_191_801_856
