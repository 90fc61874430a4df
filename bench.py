#!/usr/bin/env python
"""Headline benchmark: decode tok/s (and cold prefill seconds) of the dense 27B-class NVFP4 GQA
decoder, 64 layers / hidden 5120 / 40 q + 8 kv heads x 128 / FFN 17408 / vocab 151936, FP8 KV cache,
random-init N(0, 0.02) weights quantised to NVFP4, synthetic uniform-random prompts.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--concurrency C] [--prompt-len L]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...   (N > 1, tensor parallel)

A step is one decode pass of C concurrent sequences (C tokens).  K steps are timed on the device
with CUDA events between barrier + synchronize, max over ranks; rank 0 prints one JSON line.
`--impl reference` reports why the reference engine cannot run on this machine.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

# Reference numbers (tok/s, high end of the published range) for the closest published model:
# Qwen3.8-27B NVFP4 on 1 / 2 / 4 GB10 nodes, C1 and C8 decode, cold prefill seconds at 2K/8K/32K.
PUBLISHED = {
    "c8": {1: 244.0, 2: 368.9, 4: 430.5, 8: 430.5},
    "c1": {1: 59.8, 2: 105.4, 4: 165.5, 8: 165.5},
    "prefill_s": {1: (1.198, 3.943, 16.634), 2: (1.198, 4.232, 17.285), 4: (1.058, 3.897, 15.646),
                  8: (1.058, 3.897, 15.646)},
}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        super().__init__(daemon=True)
        self.gpu, self.rows, self.stop_flag = gpu_index, [], False

    def run(self):
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.gpu)], capture_output=True, text=True, timeout=5).stdout
                for line in out.strip().splitlines():
                    self.rows.append([c.strip() for c in line.split(",")])
            except Exception:
                pass
            time.sleep(0.2)

    def summary(self):
        sm = sorted(int(float(r[1])) for r in self.rows if len(r) > 2 and r[1].replace(".", "").isdigit())
        mx = [int(float(r[2])) for r in self.rows if len(r) > 2 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for i, nm in enumerate(names):
                if len(r) > 5 + i and r[5 + i].lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.rows)}


def reference_arm(args):
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference is a CMake C++/CUDA 13 project for sm_121a + libibverbs with no Python package "
                      "(pip install: 'neither setup.py nor pyproject.toml found'); it has no sm_100 build"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=64, help="debug only: a run with fewer layers is not a valid number")
    ap.add_argument("--reducer", default="peer", choices=["peer", "nccl"])
    ap.add_argument("--prefill-lens", default="", help="comma list of cold-prefill lengths to time as extras")
    ap.add_argument("--also-c1", action="store_true", help="also time C=1 decode as an extra")
    ap.add_argument("--bf12-head", action="store_true",
                    help="keep the bf16 lm head in its lossless 12-bit resident form (same logits bit for bit)")
    ap.add_argument("--layer-kernel", action="store_true",
                    help="decode through the persistent decode-layer kernel instead of the per-operator launch sequence")
    ap.add_argument("--no-fuse-ar", action="store_true",
                    help="tensor parallel: separate all-reduce kernels instead of the GEMM-epilogue push + fold")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL only bootstraps (handle exchange, barriers, the final max over ranks): no need for NVLS multicast set-up
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"

    from dgpp_b200.engine.llm_engine import LLMEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel
    from dgpp_b200.ops import core as ops

    cfg = DenseConfig.dense_27b(layers=args.layers)
    t_init = time.time()
    model = DenseModel.random_init(cfg, device=dev, seed=0, tp_rank=rank, tp_size=world)
    if args.bf12_head:
        model.pack_bf12()
    torch.cuda.synchronize()
    t_init = time.time() - t_init

    reducer = None
    if world > 1:
        if args.reducer == "peer":
            from dgpp_b200.parallel.peer import PeerReducer
            reducer = PeerReducer(cfg.hidden, max_rows=max(args.concurrency, 2048), device=dev)
        else:
            from dgpp_b200.parallel.tp import NcclReducer
            reducer = NcclReducer()

    C, L, K, W = args.concurrency, args.prompt_len, args.steps, args.warmup
    prefill_lens = [int(x) for x in args.prefill_lens.split(",") if x]
    max_len = max([L + K + W + 8] + [p + 8 for p in prefill_lens])
    eng = LLMEngine(model, max_batch=C, max_seq_len=max_len, prefill_chunk=2048, reducer=reducer,
                    fuse_ar=not args.no_fuse_ar, fused_decode=args.layer_kernel)

    g = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, cfg.vocab, (L,), generator=g).tolist() for _ in range(C)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- prefill all sequences (cold), then arm decode
    firsts = torch.zeros(C, dtype=torch.int32, device=dev)
    barrier()
    t0 = time.perf_counter()
    for s, p in enumerate(prompts):
        assert eng.kv.reserve(s, L + K + W + 8)
        firsts[s:s + 1].copy_(eng.prefill(s, p))
    barrier()
    prefill_all_s = time.perf_counter() - t0
    eng.start_decode(list(range(C)), firsts)

    # ---- device-timed decode steps
    for _ in range(max(W, 3)):
        eng.decode_step(C)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(K):
        eng.decode_step(C)
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    ops.check_status()

    # ---- end-to-end: the public generate() API, host tokens in pinned memory, per-step readback
    barrier()
    e2e_t = {}
    t0 = time.perf_counter()
    eng.generate(prompts, max_tokens=K + 1, stream_tokens=True, timings=e2e_t)
    barrier()
    e2e_decode_s = e2e_t["decode_s"]
    sampler.stop_flag = True
    sampler.join(timeout=2)

    extras = {"prefill_all_s": prefill_all_s, "init_s": t_init, "e2e_prefill_s": e2e_t.get("prefill_s")}
    if args.also_c1:
        eng.start_decode([0], firsts[:1])
        for _ in range(3):
            eng.decode_step(1)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(K):
            eng.decode_step(1)
        b.record()
        barrier()
        extras["c1_decode_tok_s"] = 1000.0 * K / a.elapsed_time(b)
    for pl in prefill_lens:
        p = torch.randint(0, cfg.vocab, (pl,), generator=g).tolist()
        eng.kv.release(0)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.prefill(0, p)
        b.record()
        barrier()
        extras[f"prefill_s_{pl}"] = a.elapsed_time(b) / 1000.0

    vals = torch.tensor([ms, e2e_decode_s * 1000.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms, e2e_ms = vals.tolist()
    if rank == 0:
        tok_s = 1000.0 * C * K / ms
        e2e_tok_s = 1000.0 * C * K / e2e_ms
        key = "c8" if C >= 8 else "c1"
        base = PUBLISHED[key].get(world)
        line = {
            "metric": f"decode_tok_s_c{C}", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": K,
            "warmup": max(W, 3), "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (tok_s / base) if base else None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours",
            "config": {"model": "dense-27B-class GQA decoder, NVFP4 weights (e2m1 + e4m3/16 + fp32), bf16 "
                                "activations, FP8 e4m3 KV, 64L/5120h/40q8kv/128d/17408ffn/151936v",
                       "global_batch": C, "seq_len": L, "parallelism": f"tp{world}", "decode": "greedy, no spec",
                       "layers": cfg.layers,
                       "l2": "inputs larger than L2: every step streams all weights (>14 GB) from HBM"},
            "clocks": sampler.summary(),
            "e2e": {"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": C * 4, "d2h_bytes_per_step": C * 4,
                    "note": "generate(stream_tokens=True): prompt ids H2D from pinned memory at prefill; every decode "
                            "step copies its input ids H2D from pinned memory and reads the picked ids back D2H "
                            "before the next launch"},
            "gpu_launches": eng.launches_per_step() * K,
            "extras": extras,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
