"""Shared helpers for the tests: single-node modules and dtype-aware comparison."""
from __future__ import annotations

import numpy as np

from onyxia_b200 import ir
from onyxia_b200.ir import HostTensor


def ht(a, dtype=None) -> HostTensor:
    a = np.asarray(a)
    if dtype is not None:
        a = a.astype(dtype)
    return HostTensor.from_numpy(a)


def single_prim_module(kind, inputs, **params):
    """Module with one primitive over static-shaped inputs named in0, in1, ….

    `inputs` is a list of HostTensor; returns (module, feed dict).
    """
    b = ir.GraphBuilder()
    ids, feed = [], {}
    for i, t in enumerate(inputs):
        ids.append(b.input(f"in{i}", t.dtype, list(t.shape)))
        feed[f"in{i}"] = t
    out = b.prim(kind, ids, **params)
    b.output("out", out)
    return b.finish(), feed


def composite_module(name, attrs, inputs, out_types):
    """Module with one composite ≙ `run_composite` (crates/onyxia-ir/src/decomp.rs:674-716).

    `inputs` is a list of (name, HostTensor); out_types a list of (dtype, shape).
    """
    b = ir.GraphBuilder()
    ids, feed = [], {}
    for n, t in inputs:
        ids.append(b.input(n, t.dtype, list(t.shape)))
        feed[n] = t
    outs = b.composite(name, attrs, ids, out_types)
    for i, o in enumerate(outs):
        b.output(f"out{i}", o)
    return b.finish(), feed


def assert_close(actual, expect, tol):
    """|a − e| ≤ tol + |e|·tol, the reference's own closeness test (decomp.rs:718-726)."""
    actual = np.asarray(actual, dtype=np.float64).reshape(-1)
    expect = np.asarray(expect, dtype=np.float64).reshape(-1)
    assert actual.shape == expect.shape, (actual.shape, expect.shape)
    bad = np.abs(actual - expect) > tol + np.abs(expect) * tol
    assert not bad.any(), f"element {np.argmax(bad)}: {actual[np.argmax(bad)]} vs {expect[np.argmax(bad)]}"


def assert_tensors_match(got: HostTensor, want: HostTensor, atol=1e-4, rtol=1e-3):
    """Device-vs-interpreter comparison ≙ crates/onyxia-backend-wgpu/tests/gpu_test.rs:22-74:
    exact for integer and bool tensors, atol + rtol·|want| for floats."""
    assert got.dtype == want.dtype, (ir.DTYPE_NAMES[got.dtype], ir.DTYPE_NAMES[want.dtype])
    assert tuple(got.shape) == tuple(want.shape), (got.shape, want.shape)
    if got.dtype in (ir.F32, ir.F16):
        g = got.numpy().astype(np.float64).reshape(-1)
        w = want.numpy().astype(np.float64).reshape(-1)
        both_nan = np.isnan(g) & np.isnan(w)
        same_inf = np.isinf(w) & (g == w)
        ok = both_nan | same_inf | (np.abs(g - w) <= atol + rtol * np.abs(w))
        assert ok.all(), (f"{(~ok).sum()} of {ok.size} elements differ; first at {np.argmax(~ok)}: "
                          f"{g[np.argmax(~ok)]} vs {w[np.argmax(~ok)]}; max abs {np.nanmax(np.abs(g - w))}")
    else:
        assert np.array_equal(got.data, want.data), "integer/bool tensors must be bit-exact"
