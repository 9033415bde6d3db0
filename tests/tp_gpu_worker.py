"""One tensor-parallel rank on its own GPU (launched by torchrun, one process per GPU). Every rank
prepares its partition of a small f16 decoder, runs prefill + greedy decode, and rank 0 compares the
logits with the unpartitioned model on its GPU. torch.distributed (gloo) only passes the group id."""
import os
import sys

import numpy as np
import torch.distributed as dist

from onyxia_b200 import backend as be
from onyxia_b200 import ir, llm, models


def main():
    import faulthandler
    faulthandler.dump_traceback_later(int(os.environ.get("ONYXIA_TP_TEST_WATCHDOG_S", "240")), exit=True)  # a hang ends with a stack dump
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo")
    print(f"rank {rank}: process group up", flush=True)
    cfg = models.config_c1()
    cfg.act_dtype = ir.F16
    cfg.layers, cfg.vocab = 2, 4096
    cfg.explicit_zero_points = False
    module = models.build_decoder(cfg, seed=7)
    col, row, attn = module.tp_stats(world)
    assert col == 5 * cfg.layers and row == 2 * cfg.layers and attn == cfg.layers, (col, row, attn)
    prompt = np.random.default_rng(3).integers(0, cfg.vocab, 24).tolist()

    backend = be.CudaBackend((local,))
    backend.join_tp_torch()
    print(f"rank {rank}: joined the tensor-parallel group, peer all-reduce {'on' if backend.peer_allreduce() else 'off'}", flush=True)
    if os.environ.get("ONYXIA_DISABLE_PEER_ALLREDUCE", "0") in ("", "0"):
        assert backend.peer_allreduce(), "the peer-memory all-reduce did not come up (CUDA IPC between the ranks' GPUs)"
    # the all-reduce by itself on integer-valued data (sums are exact in f16): messages that take the peer-memory
    # kernel (16 B … 1 MB), one beyond its staging slot (NCCL), repeated so that the staging slots rotate and a
    # CUDA graph replays the launch
    from onyxia_b200.ir import HostTensor
    for n_elem in (8, 1000 * 8, 64 * 5376, 524288 + 64):
        b = ir.GraphBuilder()
        x = b.input("x", ir.F16, [n_elem])
        y = b.composite("onyxia.AllReduce", {}, [x], [(ir.F16, [n_elem])])[0]
        b.output("y", b.add(y, y))  # a second launch, so that the plan is replayed as a graph
        sess = backend.prepare(b.finish())
        base = (np.arange(n_elem) % 7).astype(np.float16)
        want = 2.0 * base * sum(r + 1 for r in range(world))
        for it in range(9):
            feed = {"x": sess.upload(HostTensor.from_numpy((base * (rank + 1) + it).astype(np.float16)))}
            out = sess.download(dict(sess.run(feed))["y"]).numpy().astype(np.float32)
            assert np.array_equal(out, want + 2.0 * it * world), (n_elem, it, np.abs(out - want - 2.0 * it * world).max())
    print(f"rank {rank}: all-reduce sizes ok", flush=True)

    lm = llm.LlmSession(backend, module.tp_partition(world, rank), 256)
    got = [lm.prefill(prompt)]
    print(f"rank {rank}: prefill done", flush=True)
    toks = []
    for _ in range(12):
        toks.append(llm.sample_greedy(got[-1]))
        got.append(lm.decode(toks[-1]))

    print(f"rank {rank}: decode done", flush=True)
    # all ranks hold the same logits
    mine = np.stack(got)
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    for other in gathered:
        assert np.array_equal(other, mine)

    if rank == 0:
        whole = llm.LlmSession(be.CudaBackend((local,)), module, 256)
        want = [whole.prefill(prompt)]
        for t in toks:  # teacher-forced with the partitioned run's tokens
            want.append(whole.decode(t))
        diff = max(float(np.abs(w - g).max()) for w, g in zip(want, got))
        print(f"tp={world} max abs diff vs one GPU: {diff:.5f}", flush=True)
        assert diff <= 2e-2, diff
    dist.barrier()

    # the 27B-architecture block at full width (hidden 5376, 32Q/16KV heads of 128, FFN 21504), two layers, one
    # batched decode step over a short synthetic past: partitioned vs whole
    from onyxia_b200.ir import HostTensor
    cfg = models.config_gemma3_27b()
    cfg.layers, cfg.vocab, cfg.max_positions = 2, 8192, 64
    cfg.scale_range = (0.001, 0.004)  # keeps this width inside the f16 range (the benchmark's range overflows in the interpreter too)
    module = models.build_decoder(cfg, seed=3)
    B, past = 16, 24
    rng = np.random.default_rng(9)
    ids = rng.integers(0, cfg.vocab, (B, 1)).astype(np.int64)
    kv_full = {f"past_key_values.{l}.{part}": rng.standard_normal((B, cfg.kv_heads, past, cfg.head_dim)).astype(np.float16)
               for l in range(cfg.layers) for part in ("key", "value")}

    def run(bk, mod, kv_heads):
        sess = bk.prepare(mod)
        feed = {"input_ids": sess.upload(HostTensor.from_numpy(ids)),
                "attention_mask": sess.upload(HostTensor.from_numpy(np.ones((B, past + 1), np.int64)))}
        for name, arr in kv_full.items():
            feed[name] = sess.upload(HostTensor.from_numpy(np.ascontiguousarray(arr[:, kv_heads])))
        out = dict(sess.run(feed))
        return sess.download(out["logits"]).numpy().astype(np.float32)

    per = cfg.kv_heads // world
    mine = run(backend, module.tp_partition(world, rank), slice(rank * per, (rank + 1) * per))
    if rank == 0:
        whole = run(be.CudaBackend((local,)), module, slice(0, cfg.kv_heads))
        d = np.abs(whole - mine)
        diff, mean = float(d.max()), float(d.mean())
        print(f"tp={world} 27B-architecture width, 2 layers, batch {B}: vs one GPU max abs diff {diff:.5f}, mean {mean:.6f}", flush=True)
        # Same bounds as the single-GPU check of this width against the interpreter: the two runs add their f32
        # tensor-core partial sums in different orders (K is cut between the ranks), which moves single logits by a
        # few f16 spacings; the greedy ids must not move.
        assert np.array_equal(whole.argmax(-1), mine.argmax(-1)), "greedy ids differ between the partitioned and the whole model"
        assert mean <= 1e-2 and diff <= 0.125, (mean, diff)
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} ok", flush=True)


if __name__ == "__main__":
    main()
