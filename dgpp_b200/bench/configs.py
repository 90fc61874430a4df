"""End-to-end timings of the MoE model families at their named shapes (random-init weights, synthetic prompts).

    python bench.py --config 4 [--steps K] [--warmup W] [--layers L]     hybrid GDN + gated attention + MoE (Qwen-Next style)
    python bench.py --config 2 [--steps K] [--warmup W] [--layers L]     MLA + MoE (DeepSeek-V3-style Flash)
    python bench.py --config 3 ...                                       config 2 + lightning indexer, sparse MLA

Each run builds the model at the named shape, prefills C sequences, times `K` decode steps at C = 1 and C = 8 (CUDA
events around the whole step loop, host work of the runner included; a decode pass is one captured CUDA graph per batch
width) and cold prefills at the named lengths.  One JSON line per run.  `--layers` below the named depth is a debugging
aid; its numbers are marked `"valid": false`.
(reference counterparts: docs/benchmarks.md method section; the per-family forward checks under apps/.)
"""
from __future__ import annotations

import json
import time
from typing import List

import torch


def _time_decode(runner, vocab: int, slots: List[int], steps: int, warmup: int, gen) -> float:
    """ms per decode step for the listed request slots (greedy: feeds back argmax ids)."""
    toks = torch.randint(0, vocab, (len(slots),), generator=gen).tolist()
    for _ in range(max(warmup, 3)):
        logits = runner.decode(slots, toks)
        toks = torch.argmax(logits[:len(slots)], -1).tolist()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        logits = runner.decode(slots, toks)
        toks = torch.argmax(logits[:len(slots)], -1).tolist()      # the step's result is read back every step
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _time_spec(runner, vocab: int, slots: List[int], steps: int, warmup: int, gen):
    """(ms per speculative step, tokens emitted per step over all listed requests)."""
    pend = torch.randint(0, vocab, (len(slots),), generator=gen).tolist()
    for _ in range(max(warmup, 3)):
        pend = [o[-1] for o in runner.spec_step(slots, pend)]
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    emitted = 0
    e0.record()
    for _ in range(steps):
        outs = runner.spec_step(slots, pend)                      # reads the verdict back every step
        pend = [o[-1] for o in outs]
        emitted += sum(len(o) for o in outs)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps, emitted / steps


def _time_prefill(runner, vocab: int, slot: int, n: int, gen, chunk: int) -> float:
    runner.reset(slot)
    toks = torch.randint(0, vocab, (n,), generator=gen).tolist()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    runner.prefill(slot, toks, chunk=chunk)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1000.0


def _lean_experts(args) -> int:
    """The grouped kernels read the stacked expert tensors; the per-expert copies (oracle inputs) are not kept.
    Returns the activation terms used by the expert GEMMs at prefill sizes (--moe-prefill-terms, default 1 = W4A4)."""
    from ..models.moe import MoEBlock, MoEWeights
    MoEWeights.KEEP_EXPERT_LISTS = False
    MoEBlock.PREFILL_TERMS = int(getattr(args, "moe_prefill_terms", 1) or 1)
    return MoEBlock.PREFILL_TERMS


def run_config4(args, dev) -> dict:
    from ..models.hybrid import HybridConfig, HybridModel, HybridRunner
    from ..models.moe import MoEConfig

    layers = args.layers if args.layers < 48 else 48
    depth = int(getattr(args, "mtp", 0) or 0)
    cfg = HybridConfig(layers=layers, hidden=2048, full_every=4, q_heads=16, kv_heads=2, head_dim=256, gdn_k_heads=16,
                       gdn_v_heads=16, gdn_dk=128, gdn_dv=128, vocab=151936, mtp=depth > 0,
                       moe=MoEConfig(hidden=2048, experts=512, top_k=10, moe_ffn=512, shared_ffn=512, router="softmax"))
    t0 = time.time()
    terms = _lean_experts(args)
    model = HybridModel.random_init(cfg, dev, seed=0, std=0.02, fmt="nvfp4")
    torch.cuda.synchronize()
    init_s = time.time() - t0
    C, chunk = 8, 2048
    prefix, suffix = 16384, 512
    runner = HybridRunner(model, max_rows=chunk, slots=C, max_seq_len=prefix + suffix + 4096, device=dev)
    if depth:
        runner.enable_spec(depth)
    g = torch.Generator().manual_seed(4)
    out = {"config": 4, "model": "hybrid GDN(16v/16qk x128, chunked scan) 3:1 gated GQA(16q/2kv x256) + MoE 512e top-10 + shared, "
                                 f"hidden 2048, {layers} layers, NVFP4 weights, FP8 KV", "layers": layers,
           "valid": layers == 48, "init_s": round(init_s, 1),
           "mtp": f"depth {depth}: MTP head drafts, 1 + {depth} rows verified per step, device commit / rollback" if depth else "off",
           "moe_prefill_act_terms": terms}
    out["prefill_s_2048"] = _time_prefill(runner, cfg.vocab, 0, 2048, g, chunk)
    # the trace's shape: a 16K shared prefix, then a unique suffix.  A prefix hit restores the prefix's KV blocks and
    # recurrent-state snapshot, so its prefill cost is the suffix run on top of the resident prefix.
    out["prefill_s_16384"] = _time_prefill(runner, cfg.vocab, 0, prefix, g, chunk)
    toks = torch.randint(0, cfg.vocab, (suffix,), generator=g).tolist()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    runner.prefill(0, toks, chunk=chunk)
    e1.record()
    torch.cuda.synchronize()
    out["prefix_hit_prefill_s_16k_plus_512"] = e0.elapsed_time(e1) / 1000.0
    for s in range(1, C):
        runner.reset(s)
        runner.prefill(s, torch.randint(0, cfg.vocab, (2048,), generator=g).tolist(), chunk=chunk)
    if depth:
        ms1, tps1 = _time_spec(runner, cfg.vocab, [0], args.steps, args.warmup, g)
        ms8, tps8 = _time_spec(runner, cfg.vocab, list(range(C)), args.steps, args.warmup, g)
        out.update(c1_decode_tok_s=1000.0 * tps1 / ms1, c1_ms_per_step=ms1, c1_tokens_per_step=tps1,
                   c8_decode_tok_s=1000.0 * tps8 / ms8, c8_ms_per_step=ms8, c8_tokens_per_step=tps8 / C,
                   acceptance="random-init weights: the head's drafts are almost never the model's pick, so a step emits "
                              "~1 token and pays for the drafts and the extra verify rows; tokens per step is measured",
                   steps=args.steps, context="slot 0 at ~17K, slots 1-7 at 2K")
        return out
    ms1 = _time_decode(runner, cfg.vocab, [0], args.steps, args.warmup, g)
    ms8 = _time_decode(runner, cfg.vocab, list(range(C)), args.steps, args.warmup, g)
    out.update(c1_decode_tok_s=1000.0 / ms1, c1_ms_per_step=ms1, c8_decode_tok_s=1000.0 * C / ms8, c8_ms_per_step=ms8,
               steps=args.steps, context="slot 0 at ~17K, slots 1-7 at 2K")
    return out


def run_config2(args, dev, indexer: bool = False) -> dict:
    from ..models.mla_moe import MlaMoeConfig, MlaMoeModel, MlaMoeRunner
    from ..models.moe import MoEConfig

    layers = args.layers if args.layers < 48 else 48
    cfg = MlaMoeConfig(layers=layers, hidden=4096, heads=32, q_lora=1024, kv_lora=512, nope=128, rope=64, v_dim=128,
                       ffn=12288, dense_layers=min(2, layers), vocab=129280,
                       moe=MoEConfig(hidden=4096, experts=256, top_k=8, moe_ffn=1536, shared_ffn=1536, n_group=8,
                                     topk_group=4, router="sigmoid", routed_scaling=2.5),
                       index_heads=64 if indexer else 0, index_dim=128, index_topk=2048,
                       yarn_factor=4.0 if indexer else 1.0, yarn_orig_ctx=32768,
                       index_key_fp8=indexer and not getattr(args, "index_bf16", False))
    t0 = time.time()
    terms = _lean_experts(args)
    model = MlaMoeModel.random_init(cfg, dev, seed=0, std=0.02, fmt="nvfp4")
    torch.cuda.synchronize()
    init_s = time.time() - t0
    C = 8
    lens = [int(x) for x in str(getattr(args, "prompt_lens", "") or args.prompt_len).split(",")]
    max_len = max(lens) + 512
    # the indexer keeps a [chunk, context] fp32 score matrix (1 GB at 2048 x 131072)
    chunk = int(getattr(args, "prefill_chunk", 0) or 0) or 2048
    # cache bytes of C independent requests at the longest prompt; when they do not fit beside the weights, the other
    # slots continue slot 0's prefix (shared blocks, private tails)
    per_slot = max_len * ((cfg.kv_lora + cfg.rope) + (cfg.index_dim if indexer else 0)) * 2 * layers
    shared = C * per_slot > 0.7 * torch.cuda.mem_get_info()[0]
    runner = MlaMoeRunner(model, max_rows=chunk, slots=C, max_seq_len=max_len, device=dev,
                          shared_tail_blocks=(512 // cfg.page + 1) if shared else 0)
    g = torch.Generator().manual_seed(2)
    out = {"config": 3 if indexer else 2,
           "model": "MLA (q_lora 1024, kv_lora 512, nope 128 + rope 64, v 128, 32 heads) + MoE 256e top-8 (8 groups, top-4) + shared, "
                    f"hidden 4096, {layers} layers ({cfg.dense_layers} dense FFN 12288), NVFP4 weights, bf16 latent cache"
                    + (f", lightning indexer 64 x 128 ({'e4m3 keys with per-token scales' if cfg.index_key_fp8 else 'bf16 keys'}), "
                       "top-2048 sparse attention, YaRN factor 4 over 32768" if indexer else ""),
           "layers": layers, "valid": layers == 48, "init_s": round(init_s, 1), "moe_prefill_act_terms": terms,
           "note": "weights NVFP4 throughout (the family's MXFP4 experts and FP8 128x128 attention weights map onto the same "
                   "block-scaled / converter kernels); attention through the absorbed-latent decode kernel for prefill rows too"}
    if len(lens) == 1 and lens[0] <= 8192:
        L = lens[0]
        out[f"prefill_s_{L}"] = _time_prefill(runner, cfg.vocab, 0, L, g, chunk)
        for s in range(1, C):
            runner.reset(s)
            runner.prefill(s, torch.randint(0, cfg.vocab, (L,), generator=g).tolist(), chunk=chunk)
        ms1 = _time_decode(runner, cfg.vocab, [0], args.steps, args.warmup, g)
        ms8 = _time_decode(runner, cfg.vocab, list(range(C)), args.steps, args.warmup, g)
        out.update(c1_decode_tok_s=1000.0 / ms1, c1_ms_per_step=ms1, c8_decode_tok_s=1000.0 * C / ms8, c8_ms_per_step=ms8,
                   steps=args.steps, context=L)
        return out
    # long prompts: slot 0 is prefilled (timed); the other seven contexts are copies of its cache (or, when eight
    # full-length caches do not fit, readers of its blocks), which costs a decode step what eight prompts would
    out["contexts"] = ("slot 0 prefilled; slots 1-7 read its prefix blocks and append to private tails (8 full-length caches "
                       "do not fit beside the weights on one GPU)" if shared else
                       "slot 0 prefilled; its cache rows copied into the blocks of slots 1-7")
    for L in lens:
        for s in range(C):
            runner.reset(s)
        out[f"prefill_s_{L}"] = _time_prefill(runner, cfg.vocab, 0, L, g, chunk)
        ms1 = _time_decode(runner, cfg.vocab, [0], args.steps, args.warmup, g)
        base = runner.lengths[0] // cfg.page * cfg.page if shared else runner.lengths[0]
        for s in range(1, C):
            if shared:
                runner.att.share_prefix(s, base)
            else:
                runner.att.clone_prefix(s, base)
            runner.lengths[s] = base
        ms8 = _time_decode(runner, cfg.vocab, list(range(C)), args.steps, args.warmup, g)
        out[f"ctx_{L}"] = {"c1_decode_tok_s": 1000.0 / ms1, "c1_ms_per_step": ms1, "c8_decode_tok_s": 1000.0 * C / ms8,
                           "c8_ms_per_step": ms8}
    out["steps"] = args.steps
    return out


def run_config2_ep(args, dev, rank: int, world: int) -> dict:
    """Config 2 under expert parallelism on `world` GPUs of one box: attention weights replicated, every MoE layer's experts
    split over the ranks, each rank serving C / world of the C = 8 requests; the rows of a layer go to their experts'
    owners and come back through the token-sharded all-to-all kernels.  All ranks step in lockstep."""
    import torch.distributed as dist

    from ..models.mla_moe import MlaMoeConfig, MlaMoeModel, MlaMoeRunner
    from ..models.moe import MoEConfig

    layers = args.layers if args.layers < 48 else 48
    cfg = MlaMoeConfig(layers=layers, hidden=4096, heads=32, q_lora=1024, kv_lora=512, nope=128, rope=64, v_dim=128,
                       ffn=12288, dense_layers=min(2, layers), vocab=129280,
                       moe=MoEConfig(hidden=4096, experts=256, top_k=8, moe_ffn=1536, shared_ffn=1536, n_group=8,
                                     topk_group=4, router="sigmoid", routed_scaling=2.5))
    _lean_experts(args)
    model = MlaMoeModel.random_init(cfg, dev, seed=0, std=0.02, fmt="nvfp4", ep_rank=rank, ep_size=world)
    C = 8
    assert C % world == 0
    mine = C // world
    L = args.prompt_len
    # the owners' tile buffers hold every rank's pairs of a pass: the chunk shrinks with the rank count
    chunk = int(getattr(args, "prefill_chunk", 0) or 0) or max(256, 4096 // world)
    runner = MlaMoeRunner(model, max_rows=chunk, slots=mine, max_seq_len=L + 512, device=dev)
    g = torch.Generator().manual_seed(2 + rank)

    def mx(v: float) -> float:
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    dist.barrier()
    out = {"config": 2, "parallelism": f"ep{world}: experts split over {world} GPUs (token-sharded all-to-all inside the captured "
                                       f"pass), attention replicated, {mine} of the {C} requests per GPU",
           "layers": layers, "valid": layers == 48}
    out[f"prefill_s_{L}"] = mx(_time_prefill(runner, cfg.vocab, 0, L, g, chunk))
    for s in range(1, mine):
        runner.reset(s)
        runner.prefill(s, torch.randint(0, cfg.vocab, (L,), generator=g).tolist(), chunk=chunk)
    dist.barrier()
    ms1 = mx(_time_decode(runner, cfg.vocab, [0], args.steps, args.warmup, g))
    dist.barrier()
    msc = mx(_time_decode(runner, cfg.vocab, list(range(mine)), args.steps, args.warmup, g))
    out.update(c1_ms_per_step=ms1, c1_decode_tok_s=1000.0 / ms1,
               c1_note=f"one request per GPU ({world} in all, the others keep the exchange in step): tok/s of one request",
               c8_ms_per_step=msc, c8_decode_tok_s=1000.0 * C / msc, steps=args.steps, context=L)
    return out


def run_config4_ep(args, dev, rank: int, world: int) -> dict:
    """Config 4 under expert parallelism: GDN / attention layers replicated, the 512 experts of every layer split over the
    ranks, each rank serving C / world of the C = 8 requests (see run_config2_ep)."""
    import torch.distributed as dist

    from ..models.hybrid import HybridConfig, HybridModel, HybridRunner
    from ..models.moe import MoEConfig

    layers = args.layers if args.layers < 48 else 48
    cfg = HybridConfig(layers=layers, hidden=2048, full_every=4, q_heads=16, kv_heads=2, head_dim=256, gdn_k_heads=16,
                       gdn_v_heads=16, gdn_dk=128, gdn_dv=128, vocab=151936,
                       moe=MoEConfig(hidden=2048, experts=512, top_k=10, moe_ffn=512, shared_ffn=512, router="softmax"))
    _lean_experts(args)
    model = HybridModel.random_init(cfg, dev, seed=0, std=0.02, fmt="nvfp4", ep_rank=rank, ep_size=world)
    C, chunk, L = 8, max(256, 4096 // world), args.prompt_len
    mine = C // world
    runner = HybridRunner(model, max_rows=chunk, slots=mine, max_seq_len=L + 1024, device=dev)
    g = torch.Generator().manual_seed(4 + rank)

    def mx(v: float) -> float:
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    dist.barrier()
    out = {"config": 4, "parallelism": f"ep{world}: experts split over {world} GPUs (token-sharded all-to-all inside the captured "
                                       f"pass), mixers replicated, {mine} of the {C} requests per GPU",
           "layers": layers, "valid": layers == 48}
    out[f"prefill_s_{L}"] = mx(_time_prefill(runner, cfg.vocab, 0, L, g, chunk))
    for s in range(1, mine):
        runner.reset(s)
        runner.prefill(s, torch.randint(0, cfg.vocab, (L,), generator=g).tolist(), chunk=chunk)
    dist.barrier()
    ms1 = mx(_time_decode(runner, cfg.vocab, [0], args.steps, args.warmup, g))
    dist.barrier()
    msc = mx(_time_decode(runner, cfg.vocab, list(range(mine)), args.steps, args.warmup, g))
    out.update(c1_ms_per_step=ms1, c1_decode_tok_s=1000.0 / ms1,
               c1_note=f"one request per GPU ({world} in all, the others keep the exchange in step): tok/s of one request",
               c8_ms_per_step=msc, c8_decode_tok_s=1000.0 * C / msc, steps=args.steps, context=L)
    return out


def run(config: int, args) -> int:
    from ..ops import core as ops

    import os
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        assert config in (2, 4), "more than one GPU: --config 2 and 4 run expert parallel; config 3 is a single-GPU arm"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        res = run_config2_ep(args, dev, rank, world) if config == 2 else run_config4_ep(args, dev, rank, world)
        ops.check_status()
        res["n_gpus"] = world
        res["data"] = "synthetic"
        if rank == 0:
            print(json.dumps(res))
        dist.barrier()
        dist.destroy_process_group()
        return 0
    if config == 4:
        res = run_config4(args, dev)
    elif config in (2, 3):
        res = run_config2(args, dev, indexer=config == 3)
    else:
        raise SystemExit(f"--config {config}: 2, 3 or 4")
    ops.check_status()
    res["n_gpus"] = 1
    res["data"] = "synthetic"
    print(json.dumps(res))
    return 0
