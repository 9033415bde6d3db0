"""Benchmark: decode tokens/s of a Gemma-3-1B-architecture int4 decoder, batch 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one greedy decode token after a 512-token seeded prompt (weights are
random-init, the prompt is synthetic). Prints ONE JSON line:

* ``value``  tokens/s with everything resident on the device: each step's
  input token is the previous step's on-device argmax, timed with CUDA events
  on the session's stream.
* ``e2e``    the same loop through the host-facing calls a user of the
  reference makes (upload ids + mask → run → download logits → host argmax).
* ``roofline``  the int4 GEMV kernel: algorithmic bytes per launch ÷ its mean
  device time (per-launch CUDA events, taken in a separate profiled pass).
* ``cpu_baseline``  the CPU oracle (a C++ port of the reference interpreter)
  on the host cores, on a bounded sample of the same workload.

With ``--gpus N`` every rank runs an independent replica (a single KV head
cannot be sharded); ``value`` is the sum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode tok/s (Gemma-3-1B-arch int4, b=1)"
PROMPT_LEN = 512


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device = device
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.proc:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    c = [x.strip() for x in line.split(",")]
                    if len(c) < 9:
                        continue
                    try:
                        sm.append(float(c[1]))
                        mx.append(float(c[2]))
                    except ValueError:
                        continue
                    for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                        if v.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["sm_max_mhz"] = float(max(mx))
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


def build_model(seed=0, depth=0):
    from onyxia_b200 import models
    cfg = models.config_gemma3_1b()
    if depth:
        cfg.layers = depth
    t = time.time()
    module = models.build_decoder(cfg, seed=seed)
    return cfg, module, time.time() - t


def cpu_reference_run(cfg, module, steps, warmup, threads, prompt_len=4):
    """The CPU oracle through the same KV loop: a prefill of `prompt_len` tokens (untimed), then timed decode steps."""
    from onyxia_b200 import llm
    from oracle import ref
    ref.set_threads(threads)
    s = llm.LlmSession(ref.RefBackend(), module, 4096)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab, prompt_len).tolist()
    logits = s.prefill(prompt)
    tok = llm.sample_greedy(logits)
    for _ in range(warmup):
        tok = llm.sample_greedy(s.decode(tok))
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = llm.sample_greedy(s.decode(tok))
    dt = time.perf_counter() - t0
    return steps / dt, dt


C2_SHAPES = [(2048, 2048), (4096, 11008), (8192, 8192), (5376, 21504)]


def gemv_sweep(backend, shapes, ms, peak, reps=10):
    """int4 GEMV bandwidth per shape of the MatMulNBits sweep (config C2): one module holds enough
    independent copies of the weight (> 126 MB of L2 in total) that every launch streams from HBM;
    the launches run back to back in one CUDA graph and are timed with CUDA events. With one activation
    row the planner folds the module's independent products into one launch of the persistent kernel;
    the sweep times that and the one-launch-per-product streaming kernel (`disable_persistent_step`) and
    reports the faster one under `kernel`, the other beside it."""
    from onyxia_b200 import backend as be
    from onyxia_b200 import ir
    from onyxia_b200.ir import HostTensor
    rng = np.random.default_rng(0)
    device = getattr(backend, "devices", (0,))
    plain = be.CudaBackend(tuple(device), disable_persistent_step=True)
    out = []
    for (k, n) in shapes:
        for m in ms:
            nb = k // 32
            wbytes = n * nb * 18
            copies = max(2, min(48, int(300e6 // wbytes) + 1))

            def build():
                g = ir.GraphBuilder()
                r = np.random.default_rng(k + n)
                # one activation input per copy: nodes that share an input would be grouped into one launch
                acts = [g.input(f"a{c}", ir.F16, [m, k]) for c in range(copies)]
                for c in range(copies):
                    packed = r.integers(0, 256, size=n * nb * 16, dtype=np.uint8)
                    scales = r.uniform(0.005, 0.02, size=n * nb).astype(np.float16)
                    w = g.constant(HostTensor(ir.U4, [n, nb, 32], packed), borrow=True)
                    sc = g.constant(HostTensor.from_numpy(scales), borrow=True)
                    y = g.composite("com.microsoft.MatMulNBits", {"K": k, "N": n, "bits": 4, "block_size": 32}, [acts[c], w, sc],
                                    [(ir.F16, [m, n])])[0]
                    g.output(f"y{c}", y)
                return g.finish()

            def time_on(bk):
                s = bk.prepare(build())
                act = s.upload(HostTensor.from_numpy(rng.standard_normal((m, k)).astype(np.float16)))
                feed = {f"a{c}": act for c in range(copies)}
                for _ in range(3):
                    s.run(feed)
                s.wait_idle()
                n0 = s.launch_count()
                s.timer_start()
                for _ in range(reps):
                    s.run(feed)
                us = s.timer_stop() * 1e3 / (reps * copies)
                fused = (s.launch_count() - n0) < reps * copies
                del s
                return us, fused

            us, fused = time_on(backend)
            entry_kernel = "persist_step" if fused else ("nbits_stream" if m <= 8 else "nbits_gemm_tc")
            other = None
            if fused:  # the same products, one launch each
                us2, _ = time_on(plain)
                other = {"kernel": "nbits_stream", "us_per_launch": us2}
                if us2 < us:
                    other = {"kernel": "persist_step", "us_per_launch": us}
                    us, entry_kernel = us2, "nbits_stream"
            alg = wbytes + m * k * 2 + m * n * 2
            out.append({"k": k, "n": n, "m": m, "copies": copies, "us_per_launch": us, "algorithmic_bytes": alg,
                        "gbps": alg / us / 1e3, "frac_of_peak": alg / us / 1e3 / peak, "kernel": entry_kernel, "other": other})
    return out


def gqa_sweep(backend, peak, batches=(1, 16, 64), pasts=(512, 4096, 32768), windows=(-1, 1024), steps=12):
    """GroupQueryAttention decode op (config C3): 32 query / 8 KV heads of 128, one new token per sequence
    over an f16 cache that is appended in place; GB/s of the K/V bytes a step has to read."""
    from onyxia_b200 import ir, models
    from onyxia_b200.ir import HostTensor
    H, KV, D = 32, 8, 128
    out = []
    for B in batches:
        for P in pasts:
            for w in windows:
                b = ir.GraphBuilder()
                Ps = b.sym("past_sequence_length")
                q = b.input("q", ir.F16, [B, 1, H * D])
                k = b.input("k", ir.F16, [B, 1, KV * D])
                v = b.input("v", ir.F16, [B, 1, KV * D])
                pk = b.input("past_key", ir.F16, [B, KV, Ps, D])
                pv = b.input("past_value", ir.F16, [B, KV, Ps, D])
                sl = b.input("seqlens_k", ir.I32, [B])
                cfg = models.DecoderConfig("gqa", 0, 0, H, KV, D, 0, 0, act_dtype=ir.F16, max_positions=P + steps + 8)
                c, sn = models.rope_caches(cfg)
                outs = b.composite("com.microsoft.GroupQueryAttention",
                                   {"num_heads": H, "kv_num_heads": KV, "scale": 0.0, "local_window_size": w, "do_rotary": 1,
                                    "rotary_interleaved": 0, "has_attention_bias": 0},
                                   [q, k, v, pk, pv, sl, b.constant(HostTensor.from_numpy(c)), b.constant(HostTensor.from_numpy(sn))],
                                   [(ir.F16, [B, 1, H * D]), (ir.F16, [B, KV, Ps + 1, D]), (ir.F16, [B, KV, Ps + 1, D])])
                b.output("out", outs[0])
                b.output("present_key", outs[1])
                b.output("present_value", outs[2])
                s = backend.prepare(b.finish())
                rng = np.random.default_rng(B + P)
                up = lambda a: s.upload(HostTensor.from_numpy(a))
                qt, kt, vt = (up(rng.standard_normal((B, 1, n * D)).astype(np.float16)) for n in (H, KV, KV))
                past_k = up(np.zeros((B, KV, P, D), np.float16))
                past_v = up(np.zeros((B, KV, P, D), np.float16))
                lens = [up(np.full(B, P + i, np.int32)) for i in range(steps + 3)]

                def step(i, past_k, past_v):
                    o = dict(s.run({"q": qt, "k": kt, "v": vt, "past_key": past_k, "past_value": past_v, "seqlens_k": lens[i]}))
                    return o["present_key"], o["present_value"]

                for i in range(3):
                    past_k, past_v = step(i, past_k, past_v)
                s.wait_idle()
                s.timer_start()
                for i in range(3, 3 + steps):
                    past_k, past_v = step(i, past_k, past_v)
                us = s.timer_stop() * 1e3 / steps
                keys = min(P + 4 + steps // 2, (w + 1) if w >= 0 else 1 << 40)
                kv_bytes = B * KV * keys * D * 2 * 2
                out.append({"batch": B, "past": P, "window": w, "us_per_step": us, "kv_bytes": kv_bytes,
                            "gbps": kv_bytes / us / 1e3, "frac_of_peak": kv_bytes / us / 1e3 / peak})
                del s, past_k, past_v
    return out


def c1_decode(backend, steps=32):
    """Config C1: the 2-layer fp32 decoder (hidden 512, 8Q/2KV heads of 64, FFN 2048, vocab 32000, explicit zero points)."""
    from onyxia_b200 import llm, models
    cfg = models.config_c1()
    lm = llm.NativeLlmSession(backend, models.build_decoder(cfg, seed=0), 256)
    tok = lm.step_greedy(np.random.default_rng(0).integers(0, cfg.vocab, 16).tolist())
    for _ in range(4):
        tok = lm.step_greedy([tok])
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = lm.step_greedy([tok])
    return steps / (time.perf_counter() - t0)


def run_c5(args, rank, local_rank, world, group=None):
    """Batched decode of the 27B architecture (config C5: 64 sequences at a 2048-token context), tensor-parallel
    over the launched ranks. Depth and vocabulary can be reduced (--layers, --vocab) to keep the run short; the
    result reports the measured per-layer time and its extrapolation to the full 62 layers. `group` is a
    torch.distributed group that can pass Python objects between the ranks (it only carries the NCCL id and the
    max over ranks of the timing)."""
    import torch.distributed as dist
    from onyxia_b200 import backend as be
    from onyxia_b200 import ir, models
    from onyxia_b200.ir import HostTensor
    cfg = models.config_gemma3_27b()
    full_layers = cfg.layers
    cfg.layers = args.layers
    cfg.vocab = args.vocab
    module = models.build_decoder(cfg, seed=0)
    stats = module.tp_stats(world) if world > 1 else (0, 0, 0)
    backend = be.CudaBackend((local_rank,))
    if world > 1:
        backend.join_tp_torch(group)
        module = module.tp_partition(world, rank)
    sess = backend.prepare(module)
    B, ctx = args.batch, args.context
    kvh = cfg.kv_heads // world if world > 1 and stats[2] else cfg.kv_heads
    rng = np.random.default_rng(1)
    block = HostTensor.from_numpy(rng.standard_normal((B, kvh, ctx - 1, cfg.head_dim)).astype(np.float16))
    kv = {}
    for l in range(cfg.layers):
        for part in ("key", "value"):
            kv[f"past_key_values.{l}.{part}"] = sess.upload(block)
    del block
    ids = sess.upload(HostTensor.from_numpy(rng.integers(0, cfg.vocab, (B, 1)).astype(np.int64)))
    K, W = args.steps, args.warmup
    masks = [sess.upload(HostTensor.from_numpy(np.ones((B, ctx + i), np.int64))) for i in range(W + K)]

    def step(i):
        feed = [("input_ids", ids), ("attention_mask", masks[i])] + list(kv.items())
        outs = dict(sess.run(feed))
        for l in range(cfg.layers):
            for part in ("key", "value"):
                kv[f"past_key_values.{l}.{part}"] = outs[f"present.{l}.{part}"]
        return outs["logits"]

    for i in range(W):
        step(i)
    sess.wait_idle()
    if world > 1:
        dist.barrier(group)
    sampler = ClockSampler(local_rank)
    sampler.start()
    sess.timer_start()
    for i in range(W, W + K):
        step(i)
    ms = sess.timer_stop()
    clocks = sampler.stop()
    if world > 1:
        box = [None] * world
        dist.all_gather_object(box, ms, group=group)
        ms = max(box)
    per_layer_ms = ms / K / cfg.layers  # includes the (small) embedding / lm_head share
    peak, peak_kind = load_peaks()
    # the block's HBM roofline: this rank's share of the weights and of the K/V rows of one layer
    lm_head_bytes = cfg.vocab * ((cfg.hidden + 31) // 32) * 18
    layer_bytes = (cfg.weight_bytes_per_token() - lm_head_bytes) / max(cfg.layers, 1)
    # K/V rows a layer has to read: the whole context on a global layer, window + 1 rows on a local one — averaged
    # over the layers that were run (the architecture's pattern is 5 local : 1 global; a multiple of 6 layers has it exactly)
    kv_rows = [min(ctx, cfg.layer_window(l) + 1) if cfg.layer_window(l) >= 0 else ctx for l in range(cfg.layers)]
    kv_bytes = 2 * B * cfg.kv_heads * (sum(kv_rows) / max(len(kv_rows), 1)) * cfg.head_dim * 2
    result = {
        "metric": "batched decode tok/s (Gemma-3-27B-arch int4, 64 sequences, 2048-token context)", "unit": "tok/s",
        "value": B * K / (ms / 1e3), "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"gemma3-27b-arch int4 block-32, batch {B}, context {ctx}, tensor parallel over {world} GPU(s)",
                   "layers_run": cfg.layers, "layers_full": full_layers, "vocab_run": cfg.vocab, "tp_split": list(stats),
                   "kv_rows_read_per_layer": kv_rows},
        "layer_roofline_bytes": {"weights": layer_bytes, "kv": kv_bytes},
        "ms_per_layer": per_layer_ms, "extrapolated_full_depth_tok_s": B / (per_layer_ms * full_layers / 1e3),
        "layer_roofline_frac": (layer_bytes + kv_bytes) / world / (peak * 1e9) / (per_layer_ms / 1e3),
        "clocks": clocks, "gpu_launches": sess.launch_count(), "peak_gbs": peak, "peak_source": peak_kind,
        "allreduce": None if world == 1 else ("own kernel over peer memory (CUDA IPC, peer loads)" if backend.peer_allreduce() else "ncclAllReduce")}
    del sess, kv
    return result


def tp_agreement(rank, local_rank, world, group):
    """Tensor-parallel vs single-GPU logits on a small f16 decoder (prefill + 8 greedy steps): max-abs difference,
    measured on rank 0."""
    import torch.distributed as dist
    from onyxia_b200 import backend as be
    from onyxia_b200 import ir, llm, models
    cfg = models.config_c1()
    cfg.act_dtype, cfg.layers, cfg.vocab, cfg.explicit_zero_points = ir.F16, 2, 4096, False
    if cfg.kv_heads % world or cfg.heads % world:
        cfg.heads, cfg.kv_heads = 8 * max(1, world // 8), max(2, world)
        cfg.hidden = cfg.heads * cfg.head_dim
    module = models.build_decoder(cfg, seed=7)
    prompt = np.random.default_rng(3).integers(0, cfg.vocab, 24).tolist()
    backend = be.CudaBackend((local_rank,))
    backend.join_tp_torch(group)
    lm = llm.LlmSession(backend, module.tp_partition(world, rank), 256)
    got, toks = [lm.prefill(prompt)], []
    for _ in range(8):
        toks.append(llm.sample_greedy(got[-1]))
        got.append(lm.decode(toks[-1]))
    diff = None
    if rank == 0:
        whole = llm.LlmSession(be.CudaBackend((local_rank,)), module, 256)
        want = [whole.prefill(prompt)]
        for t in toks:
            want.append(whole.decode(t))
        diff = max(float(np.abs(w - g).max()) for w, g in zip(want, got))
    dist.barrier(group)
    return diff


def bench_c5(args, rank, local_rank, world):
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("gloo")
    result = run_c5(args, rank, local_rank, world)
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gemv-sweep", action="store_true",
                    help="only run the int4 GEMV sweep over the C2 shapes (or --shapes KxN,... and --ms 1,8) and print it")
    ap.add_argument("--config", default="c4", help="c4: the 1B decode bench (default); c5: 27B-architecture batched decode, tensor-parallel over the ranks")
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--vocab", type=int, default=32768)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--config-table", action="store_true",
                    help="measure the other configurations: C1 decode, the C2 MatMulNBits sweep (M = 1, 8, 64, 512), the C3 attention sweep")
    ap.add_argument("--gqa-sweep", action="store_true",
                    help="only run the GroupQueryAttention decode sweep (config C3; --shapes BATCHxPAST,... --windows -1,1024 --steps N) and print it")
    ap.add_argument("--windows", default="-1,1024")
    ap.add_argument("--shapes", default="")
    ap.add_argument("--ms", default="1,8")
    ap.add_argument("--ref-prompt-len", type=int, default=PROMPT_LEN,
                    help="prompt length of the CPU reference arm (its prefill is untimed; 512 tokens take about a minute)")
    ap.add_argument("--no-tp", action="store_true", help="with more than one rank: skip the tensor-parallel 27B-architecture slice")
    ap.add_argument("--depth", type=int, default=0,
                    help="decoder layers of the 1B model (default: all 26). A reduced depth is for profiler captures only: "
                         "the line it prints says so in config.layers_run and is not a benchmark value")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed decode steps with cudaProfilerStart/Stop (for `ncu --profile-from-start off`)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    threads = os.cpu_count() or 1

    from onyxia_b200 import build as ox_build
    ox_build.ensure_built()

    if args.impl == "reference":
        if rank != 0:
            return
        cfg, module, _ = build_model()
        steps = min(args.steps, 8)  # a bounded sample: each CPU token takes about a second
        warm = min(args.warmup, 1)
        tps, dt = cpu_reference_run(cfg, module, steps, warm, threads, prompt_len=args.ref_prompt_len)
        line = {"metric": METRIC, "value": tps, "unit": "tok/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
                "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f16", "data": "synthetic", "impl": "reference",
                "config": {"workload": "gemma3-1b-arch int4 block-32 (26 layers, hidden 1152, 4Q/1KV heads of 256, FFN 6912, "
                                       "vocab 262144, 5 local(512):1 global), fp16 activations, batch 1, "
                                       f"{args.ref_prompt_len}-token prompt, greedy decode",
                           "prompt_len": args.ref_prompt_len, "same_config": args.ref_prompt_len == PROMPT_LEN,
                           "note": "CPU port of onyxia-backend-ref (the Rust interpreter cannot be built offline); the timed "
                                   f"region is {steps} decode steps after the (untimed) prompt prefill"},
                "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": threads, "kind": "port",
                                 "sample": f"{steps} decode steps after a {args.ref_prompt_len}-token prompt"},
                "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if args.config == "c5":
        bench_c5(args, rank, local_rank, world)
        return

    if args.config_table:
        from onyxia_b200 import backend as be
        peak, peak_kind = load_peaks()
        bk = be.CudaBackend((local_rank,))
        print(json.dumps({"peak_gbs": peak, "peak_source": peak_kind,
                          "c1_decode_tok_s_end_to_end": c1_decode(bk),
                          "c2_matmul_nbits": gemv_sweep(bk, C2_SHAPES, [1, 8, 64, 512], peak),
                          "c3_gqa_decode": gqa_sweep(bk, peak)}))
        return

    if args.gemv_sweep:
        from onyxia_b200 import backend as be
        peak, peak_kind = load_peaks()
        shapes = [tuple(int(x) for x in t.split("x")) for t in args.shapes.split(",") if t] or C2_SHAPES
        res = gemv_sweep(be.CudaBackend((local_rank,)), shapes, [int(x) for x in args.ms.split(",")], peak)
        print(json.dumps({"metric": "int4 GEMV HBM GB/s", "unit": "GB/s", "peak": peak, "peak_source": peak_kind, "gemv_sweep": res}))
        return

    if args.gqa_sweep:
        from onyxia_b200 import backend as be
        peak, peak_kind = load_peaks()
        points = [tuple(int(x) for x in t.split("x")) for t in args.shapes.split(",") if t]
        res = []
        for bsz, past in points or [(b, p) for b in (1, 16, 64) for p in (512, 4096, 32768)]:
            res += gqa_sweep(be.CudaBackend((local_rank,)), peak, (bsz,), (past,), tuple(int(w) for w in args.windows.split(",")), steps=args.steps if args.steps < 64 else 12)
        print(json.dumps({"metric": "GroupQueryAttention decode K/V GB/s", "unit": "GB/s", "peak": peak, "peak_source": peak_kind, "gqa_sweep": res}))
        return

    import torch  # plumbing only: rendezvous, barrier, max over ranks
    import torch.distributed as dist
    if world > 1:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from onyxia_b200 import backend as be
    from onyxia_b200 import ir, llm
    from onyxia_b200.ir import HostTensor

    backend = be.CudaBackend((local_rank,))  # first: without a CUDA device this raises, and nothing below runs on the CPU instead
    cfg, module, build_s = build_model(depth=args.depth)
    cpu_module = module.clone() if (rank == 0 and world == 1 and not args.no_cpu_baseline) else None
    e2e_module = module.clone()
    lm = llm.LlmSession(backend, module, 4096)
    sess = lm.session
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab, PROMPT_LEN).tolist()
    K, W = args.steps, args.warmup

    # ── prefill (untimed), then the device-resident decode loop ──
    logits = lm.prefill(prompt)
    first = llm.sample_greedy(logits)
    kv = dict(lm.kv_cache)
    past = lm.past_seq_len
    masks = [sess.upload(HostTensor.from_numpy(np.ones((1, past + i + 1), np.int64))) for i in range(W + K)]
    tok = sess.upload(HostTensor.from_numpy(np.array([[first]], np.int64)))
    names = lm.input_names

    def device_step(i, tok, kv):
        feed = []
        for n in names:
            if n == "input_ids":
                feed.append((n, tok))
            elif n == "attention_mask":
                feed.append((n, masks[i]))
            else:
                feed.append((n, kv[n]))
        outs = dict(sess.run(feed))
        for present, pst in lm.kv_pairs:
            kv[pst] = outs[present]
        return sess.argmax_last(outs["logits"])  # [1, 1] i64 = the next step's input_ids

    for i in range(W):
        tok = device_step(i, tok, kv)
    sess.wait_idle()
    launches0 = sess.launch_count()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    if args.profiler_range:
        torch.cuda.cudart().cudaProfilerStart()
    sess.timer_start()
    for i in range(W, W + K):
        tok = device_step(i, tok, kv)
    ms = sess.timer_stop()
    if args.profiler_range:
        torch.cuda.cudart().cudaProfilerStop()
    clocks = sampler.stop()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    launches = sess.launch_count() - launches0
    value = world * K / (ms / 1e3)
    plan_stats = sess.plan_stats()

    # ── end to end through the host-facing calls: every step uploads the token id and the mask from
    # host memory, runs, takes the argmax on the device and reads the 8-byte result back ──
    lm.kv_cache, lm.past_seq_len = kv, past + W + K
    host_tok = int(sess.download(tok).numpy().reshape(-1)[0])
    e2e_steps = min(K, 64)
    for _ in range(min(W, 3)):
        host_tok = lm.step_greedy([host_tok], [lm.sequence_length()])
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        host_tok = lm.step_greedy([host_tok], [lm.sequence_length()])
    e2e_dt = time.perf_counter() - t0
    e2e_val = world * e2e_steps / e2e_dt
    ctx = lm.past_seq_len
    h2d = 8 + 8 * ctx
    d2h = 8
    # the same through the native loop (`ox_llm_step`: one library call per step)
    native = llm.NativeLlmSession(backend, e2e_module, 4096)
    native.step_greedy(prompt)  # warm-up: plans, kernel attributes and lookup tables of a prefill of this length (bench.rs:140-150)
    native.reset()
    t0 = time.perf_counter()
    ntok = native.step_greedy(prompt)
    prefill_s = time.perf_counter() - t0
    for _ in range(min(W, 3)):
        ntok = native.step_greedy([ntok])
    step_s = []
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        t1 = time.perf_counter()
        ntok = native.step_greedy([ntok])
        step_s.append(time.perf_counter() - t1)
    e2e_native_val = world * e2e_steps / (time.perf_counter() - t0)
    # … and with the token id handed from step to step on the device (`ox_llm_generate`): every step still uploads its
    # mask from host memory and sends its token to host memory, but the host never waits between two steps
    native.generate([ntok], 4)
    t0 = time.perf_counter()
    gen = native.generate([ntok], e2e_steps)
    e2e_generate_val = world * e2e_steps / (time.perf_counter() - t0)
    ntok = gen[-1]
    # the fields of the reference's own benchmark report (crates/onyxia-cli/src/bench.rs:187-233, 268-288)
    report = {"adapter": torch.cuda.get_device_name(local_rank),
              "vram": {"resident_bytes": native.session.resident_bytes(), "peak_bytes": native.session.peak_resident_bytes()},
              "prefill": {"tokens": len(prompt), "seconds": prefill_s, "tokens_per_sec": len(prompt) / prefill_s},
              "decode": {"tokens": e2e_steps, "mean_ms_per_token": float(np.mean(step_s)) * 1e3, "min_ms_per_token": float(np.min(step_s)) * 1e3,
                         "max_ms_per_token": float(np.max(step_s)) * 1e3, "stddev_ms": float(np.std(step_s)) * 1e3,
                         "tokens_per_sec": 1.0 / float(np.mean(step_s))}}
    del native
    # the reference's own loop shape for comparison: logits to the host, argmax there
    t0 = time.perf_counter()
    for _ in range(min(e2e_steps, 16)):
        host_tok = llm.sample_greedy(lm.decode(host_tok))
    e2e_logits_val = world * min(e2e_steps, 16) / (time.perf_counter() - t0)

    # ── per-kernel device times for the roofline (profiled pass, per-launch events) ──
    sess.enable_profiling(True)
    prof_steps = 4
    for _ in range(prof_steps):
        host_tok = llm.sample_greedy(lm.decode(host_tok))
    timings = sess.take_timings()
    sess.enable_profiling(False)
    by_kernel = {}
    for kname, _node, ns in timings:
        a = by_kernel.setdefault(kname, [0, 0])
        a[0] += 1
        a[1] += ns
    peak, peak_kind = load_peaks()
    weight_bytes = cfg.weight_bytes_per_token()
    lm_head_bytes = cfg.vocab * ((cfg.hidden + 31) // 32) * 18
    kv_now = cfg.kv_bytes_per_token(lm.past_seq_len)
    # activations in and out of the 7 matrices per layer, fp16
    layer_act_bytes = 2 * cfg.layers * (cfg.hidden * 4 + cfg.heads * cfg.head_dim * 2 + 2 * cfg.kv_heads * cfg.head_dim + 3 * cfg.ffn + cfg.hidden * 2)
    # Algorithmic bytes per launch of each kernel that streams weights: the persistent step kernel reads every
    # layer's weights and the visible K/V rows once; the streaming GEMV reads one matrix (group) per launch.
    per_launch = {}
    if "persist_step" in by_kernel:
        per_launch["persist_step"] = weight_bytes - lm_head_bytes + kv_now + layer_act_bytes
        if "nbits_stream" in by_kernel:
            per_launch["nbits_stream"] = lm_head_bytes + 2 * (cfg.hidden + cfg.vocab)
        else:  # the lm_head is one of the launch's operations
            per_launch["persist_step"] += lm_head_bytes + 2 * (cfg.hidden + cfg.vocab)
    elif "nbits_stream" in by_kernel:
        n_l = by_kernel["nbits_stream"][0] / prof_steps
        per_launch["nbits_stream"] = (weight_bytes + layer_act_bytes + 2 * (cfg.hidden + cfg.vocab)) / n_l
    dom = max(per_launch, key=lambda k: by_kernel[k][1], default=None)
    # DRAM traffic per launch: ncu captures of these kernels read 1.01× (streaming GEMV) and 1.02× (persistent
    # step, a 4-layer model with its lm_head) their algorithmic bytes; the figure here is that ratio applied to this launch.
    traffic_ratio = {"persist_step": 1.02, "nbits_stream": 1.01}
    roofline = {"bound": "hbm", "achieved": None, "peak": peak, "unit": "GB/s", "frac": None, "traffic": None,
                "kernel": dom, "peak_source": peak_kind,
                "traffic_source": "static: ratio of DRAM bytes to algorithmic bytes from the ncu capture summarised under profiles/"}
    if dom:
        n_launch, ns = by_kernel[dom]
        avg_s = ns / n_launch / 1e9
        roofline["algorithmic_bytes_per_launch"] = per_launch[dom]
        roofline["launches_per_step"] = n_launch / prof_steps
        roofline["avg_launch_us"] = avg_s * 1e6
        roofline["achieved"] = per_launch[dom] / avg_s / 1e9
        roofline["frac"] = roofline["achieved"] / peak
        roofline["traffic"] = int(per_launch[dom] * traffic_ratio[dom])
        roofline["timing"] = "CUDA event pair around each launch in a separate pass of 4 decode steps (launches serialised)"
    # the whole step against the same peak: self-consistent by construction
    step_roofline = {"bytes_per_token": weight_bytes + kv_now, "ms_per_step": ms / K,
                     "achieved": (weight_bytes + kv_now) / (ms / K / 1e3) / 1e9, "unit": "GB/s"}
    step_roofline["frac"] = step_roofline["achieved"] / peak
    kernel_share = {k: {"launches_per_step": v[0] / prof_steps, "us_per_step": v[1] / 1e3 / prof_steps}
                    for k, v in sorted(by_kernel.items(), key=lambda kv_: -kv_[1][1])}
    kernel_share["_note"] = ("event pairs serialise the launches and add ~6 µs each: with many small launches the sum exceeds "
                             "ms_per_step; shares, not absolutes")

    sweep = gemv_sweep(backend, C2_SHAPES, [1], peak) if rank == 0 else None
    resident = sess.resident_bytes()

    cpu = None
    if cpu_module is not None:
        try:
            tps, dt = cpu_reference_run(cfg, cpu_module, 6, 1, threads)
            cpu = {"value": tps, "unit": "tok/s", "cores": threads, "kind": "port",
                   "sample": "6 decode steps after a 4-token prompt, same weights (the full 512-token prompt is what "
                             "`--impl reference` runs)"}
        except Exception as e:  # the baseline is a report, never a reason to lose the measurement
            cpu = {"value": None, "unit": "tok/s", "cores": threads, "kind": "port", "sample": f"failed: {e}"}

    c5_tp = None
    if world > 1 and not args.no_tp:
        # the 27B-architecture slice, tensor-parallel over the launched ranks (strong scaling; the headline above stays replicas)
        del lm, sess, kv, masks, tok
        import types
        gloo = dist.new_group(backend="gloo")
        tp_args = types.SimpleNamespace(layers=6, vocab=32768, batch=64, context=2048, steps=10, warmup=3)
        try:
            c5_tp = run_c5(tp_args, rank, local_rank, world, gloo)
            c5_tp["tp_vs_single_max_abs"] = tp_agreement(rank, local_rank, world, gloo)
            c5_tp["note"] = ("6 of the 62 layers (5 local, 1 global: the architecture's pattern) at full width and a 32k vocabulary; strong scaling: the same 64 sequences on "
                             "every rank count; one all-reduce after the attention block and one after the FFN block")
        except Exception as e:  # never lose the headline measurement to the side measurement
            c5_tp = {"error": str(e)[:300]}

    if rank == 0:
        kv_bytes = cfg.kv_bytes_per_token(past + W + K // 2)
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": "gemma3-1b-arch int4 block-32 (26 layers, hidden 1152, 4Q/1KV heads of 256, FFN 6912, "
                                   "vocab 262144, 5 local(512):1 global), fp16 activations, batch 1, 512-token prompt, "
                                   "greedy decode", "prompt_len": PROMPT_LEN, "context_at_timing": [past + W, past + W + K],
                       "replicas": world, "l2_policy": "per-token weights (562 MB) exceed the 126 MB L2",
                       "norms": "pre + post (sandwich) RMSNorm per block, no q/k norm", "layers_run": cfg.layers,
                       **({"reduced_depth": "profiler capture case, not a benchmark value"} if args.depth else {})},
            "clocks": clocks, "gpu_launches": launches,
            "e2e": {"value": max(e2e_val, e2e_native_val, e2e_generate_val), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps,
                    "path": "ox_llm_generate: per step upload(mask) from host memory → run (input id = the previous step's argmax, on the device) "
                            "→ device argmax → copy of the token id to pinned host memory; steps enqueued back to back, the call returns with all tokens",
                    "one_call_per_step": e2e_native_val,
                    "one_call_per_step_path": "ox_llm_step: upload(ids, mask) → run → device argmax → download(token id), the host waits for every token",
                    "python_loop": e2e_val, "with_logits_download_and_host_argmax": e2e_logits_val},
            "roofline": roofline, "step_roofline": step_roofline, "cpu_baseline": cpu,
            "model_roofline": {"bytes_per_token": weight_bytes + kv_bytes, "tok_s_at_peak": peak * 1e9 / (weight_bytes + kv_bytes),
                               "frac": value / world / (peak * 1e9 / (weight_bytes + kv_bytes))},
            "gemv_sweep": sweep, "planner": plan_stats, "kernels": kernel_share, "resident_bytes": resident, "model_build_s": build_s,
            "c5_tp": c5_tp, "report": report,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
