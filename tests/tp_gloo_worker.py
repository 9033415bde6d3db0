"""One tensor-parallel rank on the CPU oracle; the all-reduce is torch.distributed over gloo.
Usage: tp_gloo_worker.py <rank> <world>. Rank 0 also runs the unpartitioned module and compares."""
import sys

import numpy as np
import torch
import torch.distributed as dist

from onyxia_b200 import ir, llm, models
from oracle import ref


def main():
    rank, world = int(sys.argv[1]), int(sys.argv[2])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = models.config_c1()
    cfg.layers, cfg.vocab = 2, 512
    module = models.build_decoder(cfg, seed=5)
    prompt = np.random.default_rng(1).integers(0, cfg.vocab, 6).tolist()

    def allreduce(view):
        t = torch.from_numpy(view.astype(np.float64))
        dist.all_reduce(t)
        view[...] = t.numpy().astype(view.dtype)

    ref.set_allreduce_hook(allreduce)
    ref.set_threads(1)
    lm = llm.LlmSession(ref.RefBackend(), module.tp_partition(world, rank), 64)
    got = [lm.prefill(prompt)]
    for _ in range(2):
        got.append(lm.decode(llm.sample_greedy(got[-1])))
    ref.set_allreduce_hook(None)
    if rank == 0:
        whole = llm.LlmSession(ref.RefBackend(), module, 64)
        want = [whole.prefill(prompt)]
        for _ in range(2):
            want.append(whole.decode(llm.sample_greedy(want[-1])))
        diff = max(float(np.abs(w - g).max()) for w, g in zip(want, got))
        print("max abs diff", diff)
        assert diff <= 1e-4, diff
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
