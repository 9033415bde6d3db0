"""The allocation-free argmax entry point (`ox_session_argmax_last_into`) against
the pooled one (`ox_session_argmax_last`) and against numpy, through the C ABI.

Collected last on purpose: the scratch it uses is a fixed array shared by every
call on the device, so the test must also pass after everything else has run.
"""
import numpy as np
import pytest

from onyxia_b200 import ir
from onyxia_b200 import backend as be
from onyxia_b200._ffi import OnyxiaError
from onyxia_b200.ir import HostTensor

pytestmark = pytest.mark.gpu


def _session():
    g = ir.GraphBuilder()
    x = g.input("x", ir.F32, [4])
    g.output("y", g.unary(ir.NEG, x))
    return be.CudaBackend((0,)).prepare(g.finish())


def _last_max(a):
    """Index of the maximum over the last axis, the highest index among equal maxima."""
    return (a.shape[-1] - 1 - np.argmax(a[..., ::-1], axis=-1)).astype(np.int64)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("rows,cols", [(1, 262144), (3, 5000), (64, 4096), (2, 7)])
def test_argmax_into_matches_pooled_entry_point_twice(dtype, rows, cols):
    s = _session()
    rng = np.random.default_rng(rows * 1000 + cols)
    out = s.upload(HostTensor.from_numpy(np.full(rows, -7, dtype=np.int64)))
    for call in range(2):  # two calls in a row share the scratch: the counters must be back at zero
        a = rng.standard_normal((rows, cols)).astype(dtype)
        # plant equal maxima, one pair straddling the split between CTAs
        a[:, cols // 3] = 9.0
        a[:, (2 * cols) // 3] = 9.0
        if call == 1:
            a[0, cols - 1] = 9.0
        logits = s.upload(HostTensor.from_numpy(a))
        want = s.download(s.argmax_last(logits)).numpy().reshape(rows)
        before = s.pool_stats()
        resident = s.resident_bytes()
        s.argmax_last_into(logits, out)
        assert s.pool_stats() == before and s.resident_bytes() == resident  # nothing came from the pool
        got = s.download(out).numpy().reshape(rows)
        assert np.array_equal(got, want)
        assert np.array_equal(got, _last_max(a))


def test_argmax_into_rejects_what_the_fixed_scratch_cannot_hold():
    s = _session()
    logits = s.upload(HostTensor.from_numpy(np.zeros((65, 8), dtype=np.float32)))
    out = s.upload(HostTensor.from_numpy(np.zeros(65, dtype=np.int64)))
    with pytest.raises(OnyxiaError, match="64 rows"):
        s.argmax_last_into(logits, out)
    small = s.upload(HostTensor.from_numpy(np.zeros((2, 8), dtype=np.float32)))
    with pytest.raises(OnyxiaError, match="one element per row"):
        s.argmax_last_into(small, out)
    ints = s.upload(HostTensor.from_numpy(np.zeros((2, 8), dtype=np.int32)))
    out2 = s.upload(HostTensor.from_numpy(np.zeros(2, dtype=np.int64)))
    with pytest.raises(OnyxiaError, match="f32 or f16"):
        s.argmax_last_into(ints, out2)
    # a failed call leaves the scratch usable
    ok = s.upload(HostTensor.from_numpy(np.arange(16, dtype=np.float32).reshape(2, 8)))
    s.argmax_last_into(ok, out2)
    assert s.download(out2).numpy().tolist() == [7, 7]
