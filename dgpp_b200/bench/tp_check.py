"""Multi-GPU collective check and timing (run under torchrun, one rank per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m dgpp_b200.bench.tp_check

Checks, on N ranks: the peer-memory one-shot all-reduce against a fixed-order fp32 fold and NCCL (values and time), the
vocab-sharded pick merge, the fused GEMM -> reduce-scatter -> all-gather path against GEMM + fold, and a tensor-parallel
engine run (separate collectives, the GEMM-epilogue push + fold, and the persistent decode-layer kernel with its
in-kernel cross-rank fold; twice each) for bit-identical tokens across ranks and runs.  All times are CUDA-event times,
maximum over ranks.  TP_HEADS sets the tiny model's head count (default 8).  Every check that prints False makes
the process exit 1; `--out FILE` also appends rank 0's result lines to FILE.
(reference counterparts: apps/bus_check.cpp, apps/nic_regress.cpp.)
"""

import os
import sys
import time

import torch
import torch.distributed as dist


FAILS = []
OUT = None


def say(*parts, ok=True) -> None:
    """Print a result line on rank 0 (and append it to the --out file); ok=False records a failed check."""
    line = " ".join(str(p) for p in parts)
    if not ok:
        FAILS.append(line)
    if int(os.environ.get("RANK", "0")) == 0:
        print(line, flush=True)
        if OUT:
            with open(OUT, "a") as f:
                f.write(line + "\n")


def main() -> int:
    global OUT
    if "--out" in sys.argv:
        OUT = sys.argv[sys.argv.index("--out") + 1]
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"]); local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local); dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from dgpp_b200.parallel.peer import PeerReducer
    from dgpp_b200.parallel.tp import NcclReducer
    from dgpp_b200.ops import core as ops
    BF = torch.bfloat16
    red = PeerReducer(5120, 2048, dev)
    torch.manual_seed(rank)
    for rows in (1, 8, 64, 2048, 3000):
        x = torch.randn(rows, 5120, device=dev).to(BF)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        want = sum(p.float() for p in parts).to(BF)   # ascending-rank fp32 fold
        y = x.clone(); red.all_reduce(y); torch.cuda.synchronize(); ops.check_status()
        same = torch.equal(y, want)
        ys = [torch.empty_like(y) for _ in range(world)]; dist.all_gather(ys, y)
        ident = all(torch.equal(ys[0], q) for q in ys)
        say(f"all_reduce rows={rows}: matches fixed-order fold={same} identical across ranks={ident}", ok=same and ident)
    # timing vs NCCL (graph-captured, 50 calls)
    for rows in (1, 8, 64):
        x = torch.randn(rows, 5120, device=dev).to(BF)
        for name, fn in (("peer", lambda: red.all_reduce(x)), ("nccl", lambda: dist.all_reduce(x))):
            for _ in range(5): fn()
            torch.cuda.synchronize(); dist.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(50): fn()
            g.replay(); torch.cuda.synchronize(); dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); g.replay(); g.replay(); b.record(); torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b) / 100 * 1000], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX)
            say(f"  {name} all_reduce rows={rows} (x5120 bf16): {t.item():.1f} us (max over ranks)")
    ops.check_status()
    # pick merge
    ids = torch.arange(8, device=dev, dtype=torch.int32) + 1000 * rank
    vals = torch.tensor([float((i * 7 + rank * 3) % 5) for i in range(8)], device=dev)
    gv = [torch.empty_like(vals) for _ in range(world)]; gi = [torch.empty_like(ids) for _ in range(world)]
    dist.all_gather(gv, vals); dist.all_gather(gi, ids)
    red.merge_picks(ids, vals); torch.cuda.synchronize(); ops.check_status()
    GV = torch.stack(gv); GI = torch.stack(gi); best = torch.argmax(GV, 0)
    ok = torch.equal(ids, GI.gather(0, best[None])[0])
    say("pick merge ok:", ok, ok=ok)
    # fused GEMM -> reduce-scatter -> all-gather vs GEMM + fixed-order fold
    from dgpp_b200.quant.formats import random_quant_linear
    for T in (100, 128, 300, 2048):
        torch.manual_seed(100 + rank)
        w = random_quant_linear(5120, 1024, "nvfp4", dev)
        a = torch.randn(T, 1024, device=dev).to(BF)
        torch.manual_seed(7)
        x0 = torch.randn(T, 5120, device=dev).to(BF)
        part = ops.gemm_tc(a, w, splits=1)            # the push epilogue runs without split K: same accumulation order
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        want = (x0.float() + sum(p.float() for p in parts).to(BF).float()).to(BF)
        for rep in range(3):
            x = x0.clone()
            bn = ops.gemm_tc_push(a, w, red.comm)
            red.rs_ag(x, bn)
            torch.cuda.synchronize(); ops.check_status()
            ok = torch.equal(x, want)
            xs = [torch.empty_like(x) for _ in range(world)]; dist.all_gather(xs, x)
            ident = all(torch.equal(xs[0], q) for q in xs)
            say(f"rs_ag T={T} rep={rep}: matches fold={ok} identical across ranks={ident} maxdiff={(x.float()-want.float()).abs().max().item():.4f}", ok=ok and ident)
        # sequence-parallel boundary: fold + residual + RMSNorm at the owner, normed rows all-gathered INTO the next GEMM
        nw = (1 + 0.1 * torch.randn(5120, device=dev, generator=torch.Generator(device=dev).manual_seed(3))).to(BF)
        torch.manual_seed(300)
        w2 = random_quant_linear(1024, 5120, "nvfp4", dev)
        bn0 = ops.pick_bn(T)
        y_want = ops.gemm_tc(ops.rmsnorm(want, nw, 1e-6), w2, bn=bn0, splits=1)
        tiles = (T + bn0 - 1) // bn0
        tpr = (tiles + world - 1) // world
        r0, r1 = min(rank * tpr, tiles) * bn0, min(min((rank + 1) * tpr, tiles) * bn0, T)
        for rep in range(2):
            x = x0.clone()
            bn = ops.gemm_tc_push(a, w, red.comm)
            red.rs_norm_push(x, nw, 1e-6, bn)
            y = ops.gemm_tc_ag(w2, red.comm, T, bn=bn)
            torch.cuda.synchronize(); ops.check_status()
            ok_y = torch.equal(y, y_want)
            ok_x = torch.equal(x[r0:r1], want[r0:r1])
            say(f"rs_norm_push + ag GEMM T={T} rep={rep}: GEMM output == unfused={ok_y} own residual rows == fold={ok_x} "
                f"maxdiff={(y.float() - y_want.float()).abs().max().item():.4f}", ok=ok_y and ok_x)
        # mixed with the one-shot all-reduce (shared epoch / slots)
        y = part.clone(); red.all_reduce(y); torch.cuda.synchronize(); ops.check_status()
    # timing: GEMM + all_reduce vs GEMM-push + rs_ag at a prefill chunk
    T = 2048
    w = random_quant_linear(5120, 5120 // world // 256 * 256 or 256, "nvfp4", dev)
    a = torch.randn(T, w.k, device=dev).to(BF)
    x = torch.randn(T, 5120, device=dev).to(BF)
    d = torch.empty(T, 5120, device=dev, dtype=BF)
    def unfused():
        ops.gemm_tc(a, w, out=d); red.all_reduce(d)
    nw = torch.ones(5120, device=dev, dtype=BF)
    w2 = random_quant_linear(2048, 5120, "nvfp4", dev)
    d2 = torch.empty(T, 2048, device=dev, dtype=BF)
    xn = torch.empty(T, 5120, device=dev, dtype=BF)
    def fused():
        red.rs_ag(x, ops.gemm_tc_push(a, w, red.comm))
    def fused_next():
        red.rs_ag(x, ops.gemm_tc_push(a, w, red.comm)); ops.rmsnorm(x, nw, 1e-6, out=xn); ops.gemm_tc(xn, w2, out=d2)
    def seqpar_next():
        bn = ops.gemm_tc_push(a, w, red.comm); red.rs_norm_push(x, nw, 1e-6, bn); ops.gemm_tc_ag(w2, red.comm, T, out=d2, bn=bn)
    def gemm_only():
        ops.gemm_tc(a, w, out=d)
    def ar_only():
        red.all_reduce(d)
    for name, fn in (("gemm alone", gemm_only), ("all_reduce alone", ar_only), ("gemm + all_reduce", unfused),
                     ("gemm_push + rs_ag", fused), ("gemm_push + rs_ag + norm + next GEMM (N=2048)", fused_next),
                     ("gemm_push + rs_norm_push + all-gather GEMM (N=2048)", seqpar_next)):
        for _ in range(3): fn()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10): fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 10 * 1000], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX)
        say(f"  {name} T={T} N=5120 K={w.k}: {t.item():.1f} us (max over ranks)")
    ops.check_status()
    # TP engine vs reference tokens; fused GEMM->all-reduce vs separate all-reduce kernel, each run twice
    from dgpp_b200.engine.llm_engine import LLMEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel
    heads = int(os.environ.get("TP_HEADS", "8"))
    cfg = DenseConfig.tiny(hidden=512, q_heads=heads, kv_heads=heads, head_dim=128, ffn=2048, vocab=4096, layers=3)
    model = DenseModel.random_init(cfg, device=dev, seed=0, std=0.05, tp_rank=rank, tp_size=world)
    say("local q heads (padded):", model.hq_local, "o.k", model.layers[0].o.k, "down.k", model.layers[0].down.k)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (150, 33)]
    # (GEMM-epilogue push + fold, persistent decode-layer kernel): separate collectives, push + fold, layer kernel
    from dgpp_b200.engine.options import EngineOptions
    modes = [("separate", False, False), ("push+fold", True, False), ("layer kernel", True, True),
             ("push+fold, residual rows gathered (no sequence-parallel boundary)", True, None)]
    runs = []
    for name, fuse, fused in modes + modes:
        opts = EngineOptions(seq_parallel=fused is not None)
        eng = LLMEngine(model, max_batch=2, max_seq_len=512, prefill_chunk=128, reducer=red, fuse_ar=fuse,
                        fused_decode=bool(fused), options=opts)
        if fused and not eng.runner._fused_ok(2):
            say("layer kernel does not apply to this shard shape (skipped)")
        runs.append(eng.generate(prompts, max_tokens=12))
        ops.check_status()
        del eng
    objs = [None] * world; dist.all_gather_object(objs, runs)
    k = len(modes)
    same_ranks = all(o == objs[0] for o in objs)
    say("tokens identical across ranks:", same_ranks, ok=same_ranks)
    for i, (name, _, _) in enumerate(modes):
        rep = runs[i] == runs[i + k]
        agree = runs[i] == runs[0]
        say(f"{name}: run1 == run2: {rep}  == separate collectives: {agree}", ok=rep and agree)
    for i, r in enumerate(runs[:k]): say("  ", modes[i][0], r[0])
    # vocabulary-sharded sampling: candidate tables instead of a logits gather; same tokens on every rank and the tokens of
    # the unsharded sampler on the gathered rows
    from dgpp_b200.sampling.device import DeviceSampler, SamplingParams
    vocab_l, rows_s = 4096, 6
    smp = DeviceSampler(vocab_l * world, rows_s, slots=2, device=dev)
    torch.manual_seed(900 + rank)
    sl = (torch.randn(rows_s, vocab_l, device=dev) * 3).contiguous()
    sp = [SamplingParams(), SamplingParams(top_logprobs=4), SamplingParams(temperature=0.8, top_k=40, seed=1),
          SamplingParams(temperature=1.0, top_p=0.9, seed=2), SamplingParams(temperature=0.7, min_p=0.05, seed=3, top_logprobs=5),
          SamplingParams(temperature=0.5, top_k=10, seed=4, logit_bias={7: 3.0, vocab_l * world - 2: 5.0})]
    picks = smp.sample_sharded(sl, rank * vocab_l, sp, [-1] * rows_s, list(range(rows_s)), count_picks=False)
    allsl = [torch.empty_like(sl) for _ in range(world)]; dist.all_gather(allsl, sl)
    ref = smp.sample(torch.cat(allsl, 1).contiguous(), sp, [-1] * rows_s, list(range(rows_s)), count_picks=False)
    toks = [p.token for p in picks]
    allt = [None] * world; dist.all_gather_object(allt, toks)
    same = all(t == allt[0] for t in allt)
    eq = all(a.token == b.token for a, b in zip(picks, ref) if a.on_device and b.on_device)
    say(f"sharded sampling: identical across ranks={same} == unsharded sampler on the gathered rows={eq} tokens={toks}",
        ok=same and eq)
    # scheduler + kernel engine on every rank: the same prompt three times (prefix cache off, then on) must give the
    # same tokens every time on every rank (the cached runs attach shared KV blocks and prefill only the tail)
    from dgpp_b200.engine.adapters import KernelEngine
    from dgpp_b200.runtime import rt
    for prefix in (False, True):
        keng = KernelEngine(LLMEngine(model, max_batch=4, max_seq_len=1024, prefill_chunk=256, reducer=red))
        sc = rt.SchedulerConfig(); sc.prefix_cache = prefix; sc.prefix_min_tokens = 16
        sched = rt.Scheduler(keng, sc)
        outs = []
        for rid in ("a", "b", "c"):
            sched.submit(rid, list(range(100, 400)), 12)
            sched.run(100000)
            outs.append([a for kind, r, a, b in sched.events() if kind == "token"])
        ops.check_status()
        allo = [None] * world; dist.all_gather_object(allo, outs)
        eq, req = outs[0] == outs[1] == outs[2], all(o == allo[0] for o in allo)
        say(f"scheduler prefix_cache={prefix}: runs equal={eq} ranks equal={req} "
            f"hit tokens={sched.meters()['prefix_hit_tokens']}", ok=eq and req)
        if not eq:
            for o in outs: say("   ", o)
        del sched, keng
    dist.barrier(); red.close(); dist.destroy_process_group()
    if FAILS:
        print(f"rank {rank}: {len(FAILS)} check(s) failed", file=sys.stderr, flush=True)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
