"""GroupQueryAttention over many new positions (prefill) on the tensor-core kernel, against the interpreter's
decomposition (decomp.rs:357-613) on the same seeded inputs: causal mask, sliding windows, a non-empty past, ragged
rows, query blocks that end inside a tile, every head dimension the kernel specialises on.

Bounds: the present caches (rotary + placement, no sums) must match to an f16 spacing; the attention output is
an f32 tensor-core sum where the interpreter adds in f64, so single elements may sit one or two f16 spacings
beside it (values are averages of N(0,1) rows: spacing ≤ 4.9e-4 below 1, 9.8e-4 below 2)."""
import numpy as np
import pytest

from onyxia_b200 import backend as be
from onyxia_b200 import ir, models
from onyxia_b200.ir import HostTensor

pytestmark = pytest.mark.gpu

CASES = [
    # batch, heads, kv, head_dim, past, seq, window
    (1, 4, 1, 256, 0, 512, -1),     # the 1B configuration's global layers
    (1, 4, 1, 256, 0, 512, 100),    # a window shorter than the prompt
    (1, 4, 1, 256, 300, 200, 511),  # chunked prefill behind a past, the 1B window
    (2, 8, 2, 128, 37, 70, 64),     # 27B-style heads, blocks that end inside a tile
    (3, 4, 4, 64, 5, 17, -1),       # one query head per KV head, the smallest block count
    (1, 32, 16, 128, 0, 96, 1024),  # the 27B configuration's head counts
]


def _run_both(mod, feed):
    from oracle import ref
    ref.set_threads(16)
    want = dict(ref.run_once(mod.clone(), feed))
    got = dict(be.run_once(be.CudaBackend((0,)), mod, feed))
    return got, want


def _check(got, want):
    o, w = got["out"].numpy().astype(np.float64), want["out"].numpy().astype(np.float64)
    d = np.abs(o - w)
    assert np.isfinite(o).all()
    assert d.max() <= 4e-3, f"attention output differs by {d.max()}"
    assert (d > 0).mean() <= 0.15, f"{(d > 0).mean():.3f} of the outputs differ from the interpreter's f16 value"
    for name in ("present_key", "present_value"):
        g, x = got[name].numpy().astype(np.float32), want[name].numpy().astype(np.float32)
        assert g.shape == x.shape and np.abs(g - x).max() <= 2e-3, name


@pytest.mark.parametrize("batch,heads,kv,d,past,seq,window", CASES)
def test_prefill_attention_matches_the_decomposition(batch, heads, kv, d, past, seq, window):
    mod, feed = models.build_gqa(batch, heads, kv, d, past, seq, ir.F16, window, True, seed=d + seq, max_positions=past + seq)
    got, want = _run_both(mod, feed)
    _check(got, want)


def test_prefill_attention_with_ragged_rows():
    """Rows whose valid past is shorter than the past tensor: the new keys land right after the valid rows, the tail of the
    past is never attended and the rest of `present` is zero (decomp.rs:1016-1096)."""
    batch, heads, kv, d, past, seq = 3, 4, 2, 64, 40, 33
    mod, feed = models.build_gqa(batch, heads, kv, d, past, seq, ir.F16, 24, True, seed=5, max_positions=past + seq)
    pk, pv = feed["past_key"].numpy().copy(), feed["past_value"].numpy().copy()
    valid = [40, 11, 0]
    for b_, v in enumerate(valid):
        pk[b_, :, v:, :] = 99
        pv[b_, :, v:, :] = -99
    feed["past_key"], feed["past_value"] = HostTensor.from_numpy(pk), HostTensor.from_numpy(pv)
    feed["seqlens_k"] = HostTensor.from_numpy(np.array([v + seq - 1 for v in valid], np.int32))
    got, want = _run_both(mod, feed)
    _check(got, want)
    present = got["present_key"].numpy()
    assert np.all(present[1, :, 11 + seq:, :] == 0) and np.all(present[2, :, seq:, :] == 0)


def test_prefill_then_decode_share_one_cache():
    """A 64-token prefill through the tensor-core kernel, then decode steps appended in place: the decode steps read the
    rows the prefill wrote."""
    from oracle import ref
    from onyxia_b200 import llm
    ref.set_threads(16)
    cfg = models.DecoderConfig("prefill-then-decode", layers=2, hidden=256, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1024,
                               act_dtype=ir.F16, max_positions=128, window=40, global_every=2, last_logits_only=True)
    module = models.build_decoder(cfg, seed=4)
    prompt = np.random.default_rng(1).integers(0, cfg.vocab, 64).tolist()

    def loop(backend, mod):
        s = llm.LlmSession(backend, mod, 128)
        out = [s.prefill(prompt)]
        for _ in range(6):
            out.append(s.decode(llm.sample_greedy(out[-1])))
        return out

    want = loop(ref.RefBackend(), module.clone())
    got = loop(be.CudaBackend((0,)), module)
    for i, (g, w) in enumerate(zip(got, want)):
        assert llm.sample_greedy(g) == llm.sample_greedy(w), i
        assert np.abs(g.astype(np.float64) - w.astype(np.float64)).max() <= 2e-2, i
