"""CPU plumbing run (no GPU): a seeded synthetic request trace through the native tokenizer, chat-template
renderer, continuous-batching scheduler and block-hash prefix cache, with the fp32 2-layer reference decoder as
the engine.  With --world 2 the model is tensor-parallel over gloo on 127.0.0.1 and every rank must produce the
same tokens and the same scheduler digests.

    python -m dgpp_b200.engine.plumbing [--requests 64] [--max-tokens 32] [--world 1]

Trace: prompts of 16..512 ids drawn uniformly from a 4096-entry vocabulary, half of them starting with one shared
256-token prefix, greedy decoding.  Prints one JSON line per rank.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import random
import sys
import time

import torch


def build_trace(n: int, seed: int = 0, vocab: int = 4096, shared_len: int = 256):
    rng = random.Random(seed)
    shared = [rng.randrange(vocab) for _ in range(shared_len)]
    reqs = []
    for i in range(n):
        ln = rng.randint(16, 512)
        if i % 2 == 0:
            p = shared + [rng.randrange(vocab) for _ in range(max(1, ln - shared_len))]
        else:
            p = [rng.randrange(vocab) for _ in range(ln)]
        reqs.append((f"req-{i}", p))
    return reqs


def text_stack_pass(reqs):
    """Exercise tokenizer + chat template on the trace: ids -> text -> template -> ids (byte-level, lossless)."""
    from ..runtime import rt

    tok = rt.Tokenizer.byte_level([(b"a", b"b"), (b"ab", b"c")], [("<|im_start|>", 300, True), ("<|im_end|>", 301, True)],
                                  rt.SplitPattern.Qwen2)
    tpl = rt.ChatTemplate("{% for m in messages %}<|im_start|>{{ m.role }}\n{{ m.content }}<|im_end|>\n{% endfor %}"
                          "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}")
    total = 0
    for rid, p in reqs:
        text = " ".join(str(t) for t in p[:32])
        rendered = tpl.render_json(json.dumps({"messages": [{"role": "user", "content": text}],
                                               "add_generation_prompt": True}))
        ids = tok.encode(rendered)
        assert tok.decode(ids).decode() == rendered
        total += len(ids)
    return total


def run(args) -> dict:
    from ..models.dense import DenseConfig, DenseModel
    from ..ops import reference as ref
    from ..runtime import rt
    from .adapters import ReferenceEngine

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    all_reduce = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo")

        def all_reduce(t):
            # fixed ascending-rank fp32 fold: every rank computes the same bits
            parts = [torch.empty_like(t, dtype=torch.float32) for _ in range(world)]
            dist.all_gather(parts, t.float().contiguous())
            acc = parts[0].clone()
            for p in parts[1:]:
                acc += p
            return acc.to(t.dtype)

    torch.manual_seed(0)
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // max(world, 1)))
    cfg = DenseConfig.plumbing_fp32()
    model = DenseModel.random_init(cfg, device="cpu", seed=0, std=0.02, tp_rank=rank, tp_size=world)
    reqs = build_trace(args.requests, seed=args.seed)
    t_text = time.time()
    text_tokens = text_stack_pass(reqs)
    t_text = time.time() - t_text
    with ref.activation_dtype(torch.float32):
        eng = ReferenceEngine(model, slots=args.slots, num_blocks=args.blocks, block_tokens=16, max_context=1024,
                              all_reduce=all_reduce)
        sc = rt.SchedulerConfig()
        sc.prefill_chunk = 256
        sc.prefill_budget_idle = 512
        sc.prefill_budget_busy = 256
        sched = rt.Scheduler(eng, sc)
        for rid, p in reqs:
            sched.submit(rid, p, args.max_tokens)
        t0 = time.time()
        sched.run(1 << 24)
        dt = time.time() - t0
    out = {}
    for kind, rid, a, b in sched.events():
        if kind == "token":
            out.setdefault(rid, []).append(a)
    h = hashlib.sha256(json.dumps(out, sort_keys=True).encode()).hexdigest()
    m = sched.meters()
    res = {"rank": rank, "world": world, "requests": len(reqs), "tokens_sha256": h, "op_digest": sched.op_digest(),
           "prefix_digest": sched.prefix_digest(), "prefix_hit_tokens": m["prefix_hit_tokens"],
           "decode_tokens": m["decode_tokens"], "prefill_tokens": m["prefill_tokens"], "seconds": round(dt, 3),
           "tok_per_s": round(sum(len(v) for v in out.values()) / max(dt, 1e-9), 1), "text_stack_tokens": text_tokens,
           "text_stack_seconds": round(t_text, 4), "first": out[reqs[0][0]][:8]}
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return res


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--max-tokens", type=int, default=32)
    ap.add_argument("--slots", type=int, default=8)
    ap.add_argument("--blocks", type=int, default=1024)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--world", type=int, default=1, help="spawn this many gloo ranks on 127.0.0.1")
    args = ap.parse_args(argv)
    if args.world > 1 and "RANK" not in os.environ:
        import subprocess

        port = 29500 + (os.getpid() % 1000)
        procs = []
        for r in range(args.world):
            env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(args.world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
            cmd = [sys.executable, "-m", "dgpp_b200.engine.plumbing", "--requests", str(args.requests), "--max-tokens",
                   str(args.max_tokens), "--slots", str(args.slots), "--blocks", str(args.blocks), "--seed", str(args.seed)]
            procs.append(subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, text=True))
        rc = 0
        for p in procs:
            o, _ = p.communicate(timeout=1800)
            sys.stdout.write(o)
            rc |= p.returncode
        return rc
    print(json.dumps(run(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
