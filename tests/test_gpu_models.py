"""Whole-decoder parity on the device: the KV-cache loop of ``LlmSession`` over
the CUDA backend against the same loop over the CPU oracle, on seeded synthetic
decoders with the benchmark configurations' shapes.

Tolerances (from the benchmark definition): fp32 logits within 1e-3 max-abs
with identical greedy token ids; fp16-activation logits within 2e-2.
"""
import numpy as np
import pytest

from onyxia_b200 import backend as be
from onyxia_b200 import ir, llm, models

from gpu_util import cuda_backend

pytestmark = pytest.mark.gpu


def _loop(backend, module, prompt, steps, forced=None, max_len=4096):
    s = llm.LlmSession(backend, module, max_len)
    logits = [s.prefill(prompt)]
    toks = []
    for i in range(steps):
        tok = llm.sample_greedy(logits[-1])
        toks.append(tok)
        logits.append(s.decode(forced[i] if forced is not None else tok))
    return logits, toks, s


def test_c1_two_layer_decoder_fp32_prefill_and_16_greedy_steps():
    from oracle import ref
    ref.set_threads(8)
    cfg = models.config_c1()
    module = models.build_decoder(cfg, seed=1)
    prompt = np.random.default_rng(0).integers(0, cfg.vocab, 16).tolist()
    want, want_toks, _ = _loop(ref.RefBackend(), module.clone(), prompt, 16)
    got, got_toks, s = _loop(cuda_backend(), module.clone(), prompt, 16)
    assert got_toks == want_toks, "greedy token ids must be identical"
    worst = max(float(np.abs(g - w).max()) for g, w in zip(got, want))
    assert worst <= 1e-3, f"fp32 logits differ by {worst}"
    # the same module with every composite decomposed on the device
    unf, unf_toks, _ = _loop(cuda_backend(False), module.clone(), prompt, 4)
    assert unf_toks == want_toks[:4]
    assert max(float(np.abs(g - w).max()) for g, w in zip(unf, want)) <= 1e-3


def test_c1_full_sequence_logits_match_per_position():
    """Every position of the prefill logits, not only the last (cf. examples/debug-prefill.rs:72-92)."""
    from oracle import ref
    ref.set_threads(8)
    cfg = models.config_c1()
    module = models.build_decoder(cfg, seed=3)
    prompt = np.random.default_rng(5).integers(0, cfg.vocab, 9)
    feed = {"input_ids": ir.HostTensor.from_numpy(prompt.reshape(1, -1).astype(np.int64)),
            "attention_mask": ir.HostTensor.from_numpy(np.ones((1, 9), np.int64))}
    for l in range(cfg.layers):
        z = ir.HostTensor.from_numpy(np.zeros((1, cfg.kv_heads, 0, cfg.head_dim), np.float32))
        feed[f"past_key_values.{l}.key"] = z
        feed[f"past_key_values.{l}.value"] = z
    want = dict(ref.run_once(module.clone(), feed))
    got = dict(be.run_once(cuda_backend(), module, feed))
    assert np.abs(got["logits"].numpy() - want["logits"].numpy()).max() <= 1e-3
    assert np.array_equal(got["logits"].numpy().argmax(-1), want["logits"].numpy().argmax(-1))
    for l in range(cfg.layers):
        for kv in ("key", "value"):
            assert np.abs(got[f"present.{l}.{kv}"].numpy() - want[f"present.{l}.{kv}"].numpy()).max() <= 1e-4


def _reduced_1b(layers=6):
    cfg = models.config_gemma3_1b()
    cfg.layers = layers  # layer 5 is the global one; widths, vocab and windows are the full model's
    cfg.window = 16      # short window so the short test prompt crosses it
    cfg.max_positions = 128
    return cfg


def test_gemma3_1b_arch_reduced_depth_fp16_parity():
    from oracle import ref
    ref.set_threads(8)
    cfg = _reduced_1b()
    module = models.build_decoder(cfg, seed=7)
    prompt = np.random.default_rng(1).integers(0, cfg.vocab, 24).tolist()
    steps = 6
    want, want_toks, _ = _loop(ref.RefBackend(), module.clone(), prompt, steps)
    # teacher-forced with the oracle's tokens so one near-tie cannot derail later steps
    got, got_toks, s = _loop(cuda_backend(), module.clone(), prompt, steps, forced=want_toks)
    worst = max(float(np.abs(g - w).max()) for g, w in zip(got, want))
    assert worst <= 2e-2, f"fp16 logits differ by {worst}"
    for g_tok, w_tok, w in zip(got_toks, want_toks, want):
        top2 = np.sort(w)[-2:]
        if top2[1] - top2[0] > 4e-2:  # outside the tolerance band the greedy id must agree
            assert g_tok == w_tok
    assert sum(g == w for g, w in zip(got_toks, want_toks)) >= steps - 1


def test_gemma3_1b_arch_full_depth_prefill_decode_consistency():
    """Full 26-layer model, no oracle: logits after prefill(n+1) equal logits after prefill(n) + decode(1),
    a size-independent property tying the prefill path, the decode path and the in-place KV append together."""
    cfg = models.config_gemma3_1b()
    module = models.build_decoder(cfg, seed=11)
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, cfg.vocab, 600).tolist()  # crosses the 512-token window of the local layers
    a = llm.LlmSession(cuda_backend(), module.clone(), 2048)
    full = a.prefill(prompt)
    b = llm.LlmSession(cuda_backend(), module.clone(), 2048)
    b.prefill(prompt[:-3])
    for t in prompt[-3:-1]:
        b.decode(t)
    inc = b.decode(prompt[-1])
    assert np.isfinite(full).all()
    assert np.abs(full - inc).max() <= 2e-2, float(np.abs(full - inc).max())
    # the device-side argmax picks the same token as the host-side greedy sampler
    nxt = llm.sample_greedy(inc)
    logits_host = a.decode(nxt)
    tok_dev = b.step_greedy([nxt], [b.sequence_length()])
    top2 = np.sort(logits_host)[-2:]
    assert tok_dev == llm.sample_greedy(logits_host) or top2[1] - top2[0] < 4e-2


def test_tensor_parallel_two_gpus_match_one():
    """Two ranks (torchrun, one GPU each, NCCL all-reduce) reproduce the single-GPU logits within the f16 bound."""
    import os
    import subprocess
    import sys

    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.path.join(root, "tests"), NCCL_NVLS_ENABLE="0",
               GLOO_SOCKET_IFNAME="lo", PYTHONUNBUFFERED="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29541", os.path.join(root, "tests", "tp_gpu_worker.py")],
                       env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-4000:]
    assert "max abs diff vs one GPU" in r.stdout


def test_native_generation_loop_matches_the_python_loop():
    """`ox_llm_step` (the loop inside the library) and `LlmSession` produce the same greedy tokens and logits."""
    cfg = models.config_c1()
    cfg.vocab = 4096
    module = models.build_decoder(cfg, seed=9)
    prompt = np.random.default_rng(4).integers(0, cfg.vocab, 12).tolist()
    py = llm.LlmSession(cuda_backend(), module.clone(), 128)
    nat = llm.NativeLlmSession(cuda_backend(), module.clone(), 128)
    t_py, t_nat = py.step_greedy(prompt, list(range(len(prompt)))), nat.step_greedy(prompt)
    assert t_py == t_nat
    for _ in range(6):
        t_py, t_nat = py.step_greedy([t_py], [py.sequence_length()]), nat.step_greedy([t_nat])
        assert t_py == t_nat
    assert nat.sequence_length() == py.sequence_length()
    a, b = py.decode(t_py), nat.step_logits([t_nat])
    assert np.array_equal(a, b)
    with pytest.raises(Exception):
        llm.NativeLlmSession(cuda_backend(), module.clone(), 4).step_greedy(prompt)


def test_long_decode_crosses_length_buckets_and_cache_growth(monkeypatch):
    """300 greedy steps after a 500-token prompt on a 2-layer 1B-architecture model: the attention launches are
    re-sized when the length leaves its 256-row bucket, the caches outgrow their capacity and move (the spare
    room is cut to 256 rows here so that this happens within the test), the plan is patched every step and
    replayed as a CUDA graph — and the last logits still equal those of one prefill over the whole sequence."""
    monkeypatch.setenv("ONYXIA_KV_ROOM", "256")
    cfg = models.config_gemma3_1b()
    cfg.layers, cfg.vocab = 2, 8192
    module = models.build_decoder(cfg, seed=21)
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, cfg.vocab, 500).tolist()
    nat = llm.NativeLlmSession(cuda_backend(), module.clone(), 2048)
    toks = [nat.step_greedy(prompt)]
    for _ in range(299):
        toks.append(nat.step_greedy([toks[-1]]))
    inc = nat.step_logits([toks[-1]])
    assert nat.sequence_length() == 800
    whole = llm.LlmSession(cuda_backend(), module.clone(), 2048)
    full = whole.prefill(prompt + toks)
    assert np.isfinite(inc).all()
    assert np.abs(full - inc).max() <= 2e-2, float(np.abs(full - inc).max())


def test_generate_hands_the_token_over_on_the_device():
    """ox_llm_generate (ids never leave the device between steps) gives the tokens of the one-call-per-step loop."""
    cfg = models.DecoderConfig("generate", layers=2, hidden=256, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1024,
                               act_dtype=ir.F16, max_positions=128, last_logits_only=True)
    prompt = np.random.default_rng(8).integers(0, cfg.vocab, 10).tolist()
    backend = be.CudaBackend((0,))
    a = llm.NativeLlmSession(backend, models.build_decoder(cfg, seed=6), 128)
    b = llm.NativeLlmSession(backend, models.build_decoder(cfg, seed=6), 128)
    want = [a.step_greedy(prompt)]
    for _ in range(19):
        want.append(a.step_greedy([want[-1]]))
    got = b.generate(prompt, 12)
    got += b.generate([got[-1]], 8)      # continues from where the first call stopped
    assert got == want
    assert a.sequence_length() == b.sequence_length()
    with pytest.raises(Exception, match="max_seq_len"):
        b.generate([got[-1]], 200)
