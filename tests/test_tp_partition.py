"""Tensor-parallel partition pass, on the CPU: the ranks' modules run on the oracle (one interpreter per
rank, as threads of this process or as `gloo` processes) with the all-reduce supplied by the test, and must
reproduce the unpartitioned module."""
import os
import subprocess
import sys
import threading

import numpy as np
import pytest

from onyxia_b200 import ir, llm, models
from onyxia_b200.ir import HostTensor
from oracle import ref

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def small_cfg(act=ir.F32, zp=True):
    cfg = models.config_c1()
    cfg.layers, cfg.vocab = 2, 512
    cfg.act_dtype = act
    cfg.explicit_zero_points = zp
    return cfg


def test_partition_picks_the_megatron_pairs():
    cfg = small_cfg()
    m = models.build_decoder(cfg, seed=3)
    col, row, attn = m.tp_stats(2)
    # per layer: q, k, v, gate, up split along N; o, down along K; lm_head stays whole
    assert (col, row, attn) == (5 * cfg.layers, 2 * cfg.layers, cfg.layers)
    assert m.tp_stats(3) == (0, 0, 0) or m.tp_stats(3)[2] == 0  # 8 heads / 2 KV heads do not divide by 3
    part = m.tp_partition(2, 1)
    i = part.input_names().index("past_key_values.0.key")
    shape = part.eval_input_shape(i, {"batch_size": 1, "sequence_length": 1, "past_sequence_length": 5, "total_sequence_length": 6})
    assert tuple(shape) == (1, cfg.kv_heads // 2, 5, cfg.head_dim)


class ThreadRanks:
    """All-reduce among interpreter threads of one process: every rank adds its buffer into a shared sum."""

    def __init__(self, world):
        self.world = world
        self.barrier = threading.Barrier(world)
        self.lock = threading.Lock()
        self.acc = None

    def __call__(self, view):
        with self.lock:
            self.acc = view.astype(np.float64) if self.acc is None else self.acc + view.astype(np.float64)
        self.barrier.wait()
        total = self.acc
        self.barrier.wait()
        view[...] = total.astype(view.dtype)
        if self.barrier.wait() == 0:
            self.acc = None
        self.barrier.wait()


def run_ranks_as_threads(module, world, prompt, steps):
    """Prefill + greedy decode on `world` interpreters; returns rank 0's logits per step."""
    hook = ThreadRanks(world)
    ref.set_allreduce_hook(hook)
    ref.set_threads(1)
    out = [None] * world
    errs = []

    def work(rank):
        try:
            lm = llm.LlmSession(ref.RefBackend(), module.tp_partition(world, rank), 64)
            logits = [lm.prefill(prompt)]
            for _ in range(steps):
                logits.append(lm.decode(llm.sample_greedy(logits[-1])))
            out[rank] = logits
        except Exception as e:  # noqa: BLE001 - surface it in the main thread
            errs.append(e)
            hook.barrier.abort()

    ts = [threading.Thread(target=work, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    ref.set_allreduce_hook(None)
    if errs:
        raise errs[0]
    return out


@pytest.mark.parametrize("world", [2])
@pytest.mark.parametrize("act", [ir.F32, ir.F16])
def test_partitioned_decoder_matches_the_whole_one(world, act):
    cfg = small_cfg(act)
    module = models.build_decoder(cfg, seed=5)
    prompt = np.random.default_rng(1).integers(0, cfg.vocab, 6).tolist()
    whole = llm.LlmSession(ref.RefBackend(), module.clone(), 64)
    want = [whole.prefill(prompt)]
    for _ in range(3):
        want.append(whole.decode(llm.sample_greedy(want[-1])))
    got = run_ranks_as_threads(module, world, prompt, 3)
    tol = 1e-4 if act == ir.F32 else 2e-2
    for r in range(world):
        for w, g in zip(want, got[r]):
            assert np.abs(w - g).max() <= tol, float(np.abs(w - g).max())
    # all ranks hold identical logits
    for w0, w1 in zip(got[0], got[1]):
        assert np.array_equal(w0, w1)


def test_two_gloo_processes_agree_with_one():
    """The same check with the ranks as two processes and torch.distributed (gloo) as the all-reduce."""
    script = os.path.join(ROOT, "tests", "tp_gloo_worker.py")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29531", PYTHONPATH=ROOT + os.pathsep + os.path.join(ROOT, "tests"))
    procs = [subprocess.Popen([sys.executable, script, str(r), "2"], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
    assert "max abs diff" in outs[0]
