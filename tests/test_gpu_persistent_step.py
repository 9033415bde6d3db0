"""The one-launch decode step against the oracle and against the launch-per-operator path, over the shapes the
fused kernel specialises on: head dimension 64 / 128 / 256, query heads per KV head 1 / 2 / 4 / 8, local windows,
both GELU forms, with and without the post-norms. The device runs every shape twice — persistent kernel on and
off — and both must agree with the interpreter (exec.rs:21-110 driving interp.rs) on the greedy ids and within
the f16 logit tolerance of the benchmark definition (2e-2)."""
import numpy as np
import pytest

from onyxia_b200 import backend as be
from onyxia_b200 import ir, llm, models

pytestmark = pytest.mark.gpu


def _cfg(head_dim, heads, kv_heads, *, window=-1, sandwich=False, tanh=True, layers=3, ffn=1024):
    return models.DecoderConfig(name=f"persist-d{head_dim}-h{heads}-kv{kv_heads}", layers=layers, hidden=512, heads=heads,
                                kv_heads=kv_heads, head_dim=head_dim, ffn=ffn, vocab=2048, act_dtype=ir.F16, max_positions=256,
                                window=window, global_every=2 if window >= 0 else 0, sandwich_norms=sandwich,
                                last_logits_only=True, gelu_tanh=tanh)


def _loop(backend, module, prompt, forced):
    s = llm.LlmSession(backend, module, 256)
    logits = [s.prefill(prompt)]
    for tok in forced:
        logits.append(s.decode(tok))
    return logits, s


SHAPES = [
    # head_dim, heads, kv_heads, window, sandwich, tanh
    (64, 8, 4, -1, False, True),
    (64, 8, 1, 12, True, True),
    (64, 4, 4, -1, False, False),
    (128, 4, 2, -1, True, True),
    (128, 8, 2, 12, False, False),
    (256, 4, 1, 12, True, True),
    (256, 2, 2, -1, False, True),
]


@pytest.mark.parametrize("head_dim,heads,kv_heads,window,sandwich,tanh", SHAPES)
def test_persistent_step_matches_oracle_and_separate_launches(head_dim, heads, kv_heads, window, sandwich, tanh):
    from oracle import ref
    ref.set_threads(8)
    cfg = _cfg(head_dim, heads, kv_heads, window=window, sandwich=sandwich, tanh=tanh)
    module = models.build_decoder(cfg, seed=head_dim + heads)
    rng = np.random.default_rng(heads * 7 + kv_heads)
    prompt = rng.integers(0, cfg.vocab, 20).tolist()
    steps = 10
    # oracle free-runs; the device paths are fed the oracle's tokens so one flipped argmax cannot hide the rest
    s = llm.LlmSession(ref.RefBackend(), module.clone(), 256)
    want, toks = [s.prefill(prompt)], []
    for _ in range(steps):
        toks.append(llm.sample_greedy(want[-1]))
        want.append(s.decode(toks[-1]))

    fused, sf = _loop(be.CudaBackend((0,)), module.clone(), prompt, toks)
    plain, sp = _loop(be.CudaBackend((0,), disable_persistent_step=True), module.clone(), prompt, toks)
    lf, lp = sf.session.launch_count(), sp.session.launch_count()
    assert lf < lp, f"the persistent kernel did not take the decode step ({lf} launches against {lp})"
    for name, got in (("persistent", fused), ("separate", plain)):
        for i, (g, w) in enumerate(zip(got, want)):
            assert llm.sample_greedy(g) == llm.sample_greedy(w), f"{name}: greedy id differs at step {i}"
            d = float(np.abs(g.astype(np.float64) - w.astype(np.float64)).max())
            assert d <= 2e-2, f"{name}: logits differ by {d} at step {i}"


def test_persistent_step_when_rows_are_shorter_than_the_cache():
    """The attention mask can name fewer tokens than the cache holds rows (left context dropped by the caller):
    the new row is appended at the row's own length, later rows are cleared — same as the separate kernels."""
    from oracle import ref
    ref.set_threads(8)
    cfg = _cfg(64, 8, 4, layers=2)
    module = models.build_decoder(cfg, seed=11)
    rng = np.random.default_rng(2)
    past, valid = 24, 17
    feed = {"input_ids": ir.HostTensor.from_numpy(rng.integers(0, cfg.vocab, (1, 1)).astype(np.int64))}
    mask = np.zeros((1, past + 1), np.int64)
    mask[0, :valid] = 1
    feed["attention_mask"] = ir.HostTensor.from_numpy(mask)
    for l in range(cfg.layers):
        for part in ("key", "value"):
            feed[f"past_key_values.{l}.{part}"] = ir.HostTensor.from_numpy(
                rng.standard_normal((1, cfg.kv_heads, past, cfg.head_dim)).astype(np.float16))
    want = dict(ref.run_once(module.clone(), feed))
    for opts in ({}, {"disable_persistent_step": True}):
        got = dict(be.run_once(be.CudaBackend((0,), **opts), module.clone(), feed))
        assert np.abs(got["logits"].numpy().astype(np.float64) - want["logits"].numpy().astype(np.float64)).max() <= 2e-2
        for l in range(cfg.layers):
            for part in ("key", "value"):
                g, w = got[f"present.{l}.{part}"].numpy(), want[f"present.{l}.{part}"].numpy()
                assert g.shape == w.shape
                assert np.abs(g.astype(np.float32) - w.astype(np.float32)).max() <= 2e-3, (l, part)


@pytest.mark.parametrize("batch,seq,past", [(1, 7, 0), (2, 5, 3), (3, 1, 6), (1, 1, 9)])
def test_last_token_slice_inside_the_lm_head_group(batch, seq, past):
    """The last-token Slice sits between the final norm chain and the lm_head. One row of one sequence is a contiguous
    row range (the group's prologue starts there); the last rows of several sequences are not (the chain then runs as
    separate launches in front of the slice). Both must give the interpreter's logits."""
    from oracle import ref
    ref.set_threads(8)
    cfg = _cfg(64, 4, 2, sandwich=True, layers=2)
    module = models.build_decoder(cfg, seed=21)
    rng = np.random.default_rng(batch * 10 + seq)
    feed = {"input_ids": ir.HostTensor.from_numpy(rng.integers(0, cfg.vocab, (batch, seq)).astype(np.int64)),
            "attention_mask": ir.HostTensor.from_numpy(np.ones((batch, past + seq), np.int64))}
    for l in range(cfg.layers):
        for part in ("key", "value"):
            feed[f"past_key_values.{l}.{part}"] = ir.HostTensor.from_numpy(
                rng.standard_normal((batch, cfg.kv_heads, past, cfg.head_dim)).astype(np.float16))
    want = dict(ref.run_once(module.clone(), feed))["logits"].numpy().astype(np.float64)
    got = dict(be.run_once(be.CudaBackend((0,)), module, feed))["logits"].numpy().astype(np.float64)
    assert got.shape == want.shape == (batch, 1, cfg.vocab)
    assert np.abs(got - want).max() <= 2e-2
    assert np.array_equal(got.argmax(-1), want.argmax(-1))
