"""Differential harness for the GPU tests: the same module and the same inputs
run on the CUDA backend (through the C ABI) and on the CPU oracle, compared
dtype-aware — the shape of crates/onyxia-backend-wgpu/tests/gpu_test.rs:22-74.
"""
from __future__ import annotations

import functools

from onyxia_b200 import backend as be
from oracle import ref

from util import assert_tensors_match


@functools.lru_cache(maxsize=None)
def cuda_backend(fused: bool = True):
    return be.CudaBackend((0,)) if fused else be.CudaBackend.without_fused_kernels((0,))


def differential(module, feed, *, atol=1e-4, rtol=1e-3, fused=True, also_unfused=False, threads=8):
    """Run `module` on the oracle and on the device; compare every output.

    Returns (device outputs, oracle outputs) as lists of (name, HostTensor).
    """
    ref.set_threads(threads)
    want = ref.run_once(module.clone(), feed)
    variants = [fused] + ([False] if also_unfused and fused else [])
    got = None
    for f in variants:
        got = be.run_once(cuda_backend(f), module.clone(), feed)
        assert [n for n, _ in got] == [n for n, _ in want]
        for (name, g), (_, w) in zip(got, want):
            try:
                assert_tensors_match(g, w, atol=atol, rtol=rtol)
            except AssertionError as e:
                raise AssertionError(f"output '{name}' (fused={f}): {e}") from None
    return got, want
