"""Device top-k / top-p / temperature sampling against a restatement of the reference's sampler
(crates/onyxia-cli/src/sampling.rs:36-195) in numpy: same f32 arithmetic, sums accumulated one element after the
other, the uniform number supplied by the test instead of the reference's generator.

The device adds exactly where the reference adds in f32, so the two can only disagree when u·Σ lies within the
reference's own rounding error of a boundary between two tokens; the tests assert identical tokens wherever the
restatement's margin to the nearest boundary exceeds that error, and in every case that the device's token is the
one whose exact (f64) cumulative interval contains u·Σ."""
import numpy as np
import pytest

from onyxia_b200 import backend as be
from onyxia_b200.ir import HostTensor

pytestmark = pytest.mark.gpu
f32 = np.float32


def _from_distribution(l, u):
    """sample_from_distribution (sampling.rs:156-195); also returns the margin of u·Σ to the nearest boundary, relative to Σ."""
    finite = np.isfinite(l)
    mx = f32(np.max(l[finite]))
    e = np.where(finite, np.exp((l - mx).astype(f32)).astype(f32), f32(0)).astype(f32)
    cum = np.cumsum(e, dtype=f32)  # one element after the other, in f32
    total = cum[-1]
    rand_val = f32(u) * total
    hit = np.nonzero(cum >= rand_val)[0]
    idx = int(hit[0]) if hit.size else len(l) - 1
    lo = cum[idx - 1] if idx > 0 else f32(0)
    margin = min(abs(float(cum[idx]) - float(rand_val)), abs(float(rand_val) - float(lo))) / float(total)
    return idx, margin


def _kept_mask(l, top_k, top_p):
    n = len(l)
    order = np.argsort(-l, kind="stable")  # descending, equal values in index order
    if top_k > 0:
        if top_k >= n:
            return np.ones(n, bool), 1.0
        keep = np.zeros(n, bool)
        keep[order[:top_k]] = True
        return keep, 1.0
    if 0.0 < top_p < 1.0:
        s = l[order]
        e = np.exp((s - s[0]).astype(f32)).astype(f32)
        total = np.cumsum(e, dtype=f32)[-1]
        probs = (e / total).astype(f32)
        cum = np.cumsum(probs, dtype=f32)
        hit = np.nonzero(cum >= f32(top_p))[0]
        cutoff = int(hit[0]) + 1 if hit.size else n
        keep = np.zeros(n, bool)
        keep[order[:cutoff]] = True
        edge = abs(float(cum[cutoff - 1]) - top_p)
        if cutoff >= 2:
            edge = min(edge, abs(float(cum[cutoff - 2]) - top_p))
        return keep, edge
    return np.ones(n, bool), 1.0


def ref_sample(logits, temperature, top_k, top_p, u):
    """sample (sampling.rs:36-65) with the generator's output `u` given. Returns (token, margin, cut-off edge, kept mask)."""
    x = (logits.astype(f32) / f32(temperature)).astype(f32)
    keep, edge = _kept_mask(x, top_k, top_p)
    filt = np.where(keep, x, f32(-np.inf)).astype(f32)
    tok, margin = _from_distribution(filt, u)
    return tok, margin, edge, keep


def _device_sample(sess, logits, temperature, top_k, top_p, us):
    t = sess.upload(HostTensor.from_numpy(np.ascontiguousarray(logits)))
    return sess.download(sess.sample_last(t, temperature, top_k, top_p, us)).numpy().reshape(-1)


def _session():
    from onyxia_b200 import ir
    b = ir.GraphBuilder()
    x = b.input("x", ir.F32, [1])
    b.output("y", b.add(x, x))
    return be.CudaBackend((0,)).prepare(b.finish())


def _check(logits_rows, temperature, top_k, top_p, us, err_scale, own_tol=1e-6):
    sess = _session()
    got = _device_sample(sess, logits_rows, temperature, top_k, top_p, us)
    same = 0
    for r in range(logits_rows.shape[0]):
        tok, margin, edge, keep = ref_sample(logits_rows[r], temperature, top_k, top_p, us[r])
        d = int(got[r])
        # the device's token must own u·Σ in exact arithmetic over the same kept set (skipped when the cut-off itself is a rounding call)
        if edge > 1e-4:
            x = logits_rows[r].astype(np.float64) / np.float64(f32(temperature))
            e = np.where(keep, np.exp(x - x[keep].max()), 0.0)
            cum = np.cumsum(e)
            target = float(f32(us[r])) * cum[-1]
            lo = cum[d - 1] if d > 0 else 0.0
            tol = own_tol * cum[-1]
            assert keep[d] or us[r] == 0.0 or own_tol > 1e-6, f"row {r}: token {d} is outside the kept set"
            assert lo - tol <= target <= cum[d] + tol, f"row {r}: token {d} does not own u·Σ"
        # and equal the reference's wherever the reference's own f32 sums leave no doubt
        if margin > err_scale and edge > 1e-4:
            assert d == tok, f"row {r}: device {d}, reference {tok} (margin {margin:.2e})"
            same += 1
    return same


@pytest.mark.parametrize("mode", ["plain", "top_k", "top_p", "k_over_vocab", "p_off"])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_sampling_small_vocabulary(mode, dtype):
    rng = np.random.default_rng(7)
    rows, vocab = 48, 1000
    logits = (rng.standard_normal((rows, vocab)) * 2.5).astype(dtype)
    us = rng.random(rows).astype(f32)
    top_k, top_p = {"plain": (0, 0.0), "top_k": (17, 0.0), "top_p": (0, 0.8), "k_over_vocab": (5000, 0.3), "p_off": (0, 1.0)}[mode]
    same = _check(logits, 0.7, top_k, top_p, us, err_scale=2e-5)
    assert same >= rows * 3 // 4  # nearly every draw is far from a boundary


def test_sampling_full_vocabulary():
    rng = np.random.default_rng(11)
    rows, vocab = 6, 262144
    logits = (rng.standard_normal((rows, vocab)) * 4.0).astype(np.float16)
    us = rng.random(rows).astype(f32)
    assert _check(logits, 1.0, 50, 0.0, us, err_scale=1e-5) >= rows - 1        # few kept entries: the f32 sums are nearly exact
    # thousands of kept entries: the reference's f32 running sum of the sorted probabilities is itself off by ~1e-4, so its
    # cut-off (and with it Σ) can sit a few tail entries beside the exact one
    _check(logits, 0.8, 0, 0.9, us, err_scale=1e-3, own_tol=5e-4)
    _check(logits, 1.3, 0, 0.0, us, err_scale=1e-2)                            # everything kept


def test_sampling_ties_edges_and_greedy():
    sess = _session()
    # equal logits are kept in index order; u = 1 takes the last kept entry, u = 0 index 0 (the reference's walk stops there)
    flat = np.zeros((1, 64), f32)
    assert int(_device_sample(sess, flat, 1.0, 4, 0.0, [1.0])[0]) == 3
    assert int(_device_sample(sess, flat, 1.0, 4, 0.0, [0.0])[0]) == 0
    assert int(_device_sample(sess, flat, 1.0, 4, 0.0, [0.30])[0]) == 1   # four equal masses: (0.25, 0.5] belongs to index 1
    peaked = np.full((1, 64), -5.0, f32)
    peaked[0, 40], peaked[0, 9] = 3.0, 3.0
    assert int(_device_sample(sess, peaked, 1.0, 1, 0.0, [0.999])[0]) == 9   # top-1 among equals: the lower index
    assert int(_device_sample(sess, peaked, 1.0, 0, 0.4, [0.999])[0]) == 9   # p = 0.4 is reached by the first of the two (0.495)
    assert int(_device_sample(sess, peaked, 1.0, 0, 0.5, [0.999])[0]) == 40  # p = 0.5 needs both
    # non-finite entries carry no weight
    holes = np.array([[-np.inf, 1.0, np.nan, 1.0, -np.inf]], f32)
    assert int(_device_sample(sess, holes, 1.0, 0, 0.0, [0.75])[0]) == 3
    # temperature ≤ 1e-6: greedy, the last of equal maxima
    assert int(_device_sample(sess, peaked, 0.0, 5, 0.5, [0.1])[0]) == 40
    # a row without any finite value is an error at the next synchronising call
    bad = np.full((1, 8), np.nan, f32)
    with pytest.raises(Exception, match="cannot sample"):
        _device_sample(sess, bad, 1.0, 0, 0.0, [0.5])
        sess.wait_idle()


def test_native_loop_draws_the_next_token_on_the_device():
    """ox_llm_step_sampled: the token is the one the sampler picks from the step's own last-position logits."""
    from onyxia_b200 import ir, llm, models
    cfg = models.DecoderConfig("sampled-loop", layers=2, hidden=256, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1024,
                               act_dtype=ir.F16, max_positions=64, last_logits_only=True)
    prompt = np.random.default_rng(3).integers(0, cfg.vocab, 12).tolist()
    backend = be.CudaBackend((0,))
    a = llm.NativeLlmSession(backend, models.build_decoder(cfg, seed=2), 64)
    b = llm.NativeLlmSession(backend, models.build_decoder(cfg, seed=2), 64)
    rng = np.random.default_rng(5)
    ids = prompt
    for step in range(6):
        u = float(rng.random())
        logits = b.step_logits(ids)          # same model, same history: the logits the sampled step sees
        tok = a.step_sampled(ids, 0.9, 20, 0.0, u)
        want, margin, _, keep = ref_sample(logits.astype(f32), 0.9, 20, 0.0, u)
        assert keep[tok]
        if margin > 1e-5:
            assert tok == want, (step, tok, want)
        ids = [tok]
