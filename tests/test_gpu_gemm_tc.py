"""MatMulNBits with more than 8 activation rows runs as a tcgen05 GEMM (accumulator in tensor memory):
the sweep shapes of the MatMulNBits op benchmark at reduced sizes, against the CPU oracle, which
evaluates the Dequantize + MatMul decomposition (crates/onyxia-ir/src/decomp.rs:615-663)."""
import numpy as np
import pytest

from onyxia_b200 import backend as be
from onyxia_b200 import ir, models
from oracle import ref

from gpu_util import cuda_backend

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,k,n,zp", [(16, 128, 128, False), (9, 256, 48, False), (64, 512, 256, False), (24, 1152, 1024, True),
                                      (100, 1152, 1024, False), (300, 2048, 2048, False), (512, 1024, 272, False),
                                      (64, 96, 40, True),
                                      # K not a multiple of 8: rows are not 16-byte aligned, the activations go by plain loads
                                      (20, 100, 48, False), (130, 1004, 272, True),
                                      # a few row blocks more than a whole wave of CTAs: only those are cut along K
                                      (130, 1024, 19200, False), (16, 1024, 38400, False)])
def test_matmul_nbits_many_rows_matches_oracle(m, k, n, zp):
    module, act = models.build_matmul_nbits(m, k, n, act_dtype=ir.F16, seed=m + k, with_zp=zp)
    ref.set_threads(8)
    want = ref.run_once(module.clone(), {"a": act})[0][1].numpy().astype(np.float32)
    got = be.run_once(cuda_backend(), module.clone(), {"a": act})[0][1].numpy().astype(np.float32)
    # f32 accumulation against the oracle's f64, both rounded to f16 once: one f16 ulp of the largest output
    bound = 2e-3 + 2.0 ** -10 * np.abs(want).max()
    assert np.abs(got - want).max() <= bound, (float(np.abs(got - want).max()), float(bound))


def test_rows_do_not_depend_on_the_pass_they_ran_in():
    """The same activation row gives the same result whether it runs in the GEMV (≤ 8 rows) or the GEMM."""
    k, n = 1152, 1024
    module, act = models.build_matmul_nbits(40, k, n, act_dtype=ir.F16, seed=3)
    big = be.run_once(cuda_backend(), module.clone(), {"a": act})[0][1].numpy().astype(np.float32)
    small_mod, _ = models.build_matmul_nbits(4, k, n, act_dtype=ir.F16, seed=3)
    a4 = ir.HostTensor.from_numpy(act.numpy()[:4].copy())
    small = be.run_once(cuda_backend(), small_mod, {"a": a4})[0][1].numpy().astype(np.float32)
    # f32 (tensor memory) vs f64 (GEMV) accumulation: at most one f16 ulp apart
    assert np.abs(big[:4] - small).max() <= 2.0 ** -10 * np.abs(small).max() + 1e-3


def test_long_k_stays_close_to_the_f64_accumulation():
    """K = 6912 (54 steps of 128): the tensor core's f32 accumulator drifts along a chain of MMAs, so the
    kernel rotates over several accumulators and may cut K into pieces. After the single rounding to f16
    all but a small share of the outputs must equal the oracle's (f64 accumulation) bit for bit, and none
    may be further than one f16 ulp of the largest output away."""
    m, k, n = 24, 6912, 1152
    module, act = models.build_matmul_nbits(m, k, n, act_dtype=ir.F16, seed=5)
    ref.set_threads(8)
    want = ref.run_once(module.clone(), {"a": act})[0][1].numpy()
    got = be.run_once(cuda_backend(), module.clone(), {"a": act})[0][1].numpy()
    differing = float((got != want).mean())
    assert differing <= 0.01, differing  # measured 0.15 %; a single accumulator chain gives 2.6 %
    assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= 2.0 ** -10 * np.abs(want.astype(np.float32)).max()
