"""Expert parallelism check and timing, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m dgpp_b200.bench.ep_check [--out FILE] [--hidden H --experts E --top-k K --ffn F --rows R]

Every rank builds the same MoE block twice from one seed: with all experts (the single-rank prefill path, the oracle) and
with its own expert block (the all-to-all path).  Ranks hold different numbers of rows.  Checks, per rank: the all-to-all
result equals the oracle bit for bit, repeated exchanges are identical, the device status block is clean.  Prints the time
per exchange (CUDA events, max over ranks) and the NVLink bytes per row against the all-reduce form.  Exits 1 if any check
fails.  (reference counterpart: apps/bus_check.cpp style collective drills.)
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--ffn", type=int, default=512)
    ap.add_argument("--rows", type=int, default=256, help="rows of rank 0; rank r holds rows + 8 r")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    from dgpp_b200.models.moe import MoEBlock, MoEConfig, MoEWeights
    from dgpp_b200.ops import core as ops
    from dgpp_b200.parallel.ep import EpMoE

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = MoEConfig(hidden=args.hidden, experts=args.experts, top_k=args.top_k, moe_ffn=args.ffn, shared_ffn=args.ffn,
                    routed_scaling=1.5)
    full = MoEWeights.random_init(cfg, dev, seed=21, std=0.05)
    mine = MoEWeights.random_init(cfg, dev, seed=21, std=0.05, ep_rank=rank, ep_size=world, shared_everywhere=True)
    rows = args.rows + 8 * rank
    oracle = MoEBlock(full, max_rows=16, device=dev, prefill_terms=3)
    ep = EpMoE(mine, max_rows=args.rows + 8 * world, device=dev, act_terms=3)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(rows, cfg.hidden, device=dev, generator=g).to(torch.bfloat16)
    lines, ok_all = [], True

    def say(msg: str, ok: bool = True) -> None:
        nonlocal ok_all
        ok_all &= bool(ok)
        lines.append(f"[rank {rank}/{world}] {msg}" + ("" if ok else "   <-- FAILED"))

    want = oracle.forward_gathered(x)
    got = ep.forward(x)
    got2 = ep.forward(x)
    torch.cuda.synchronize()
    say(f"all-to-all == single-rank path (rows {rows}): {torch.equal(got, want)} maxdiff "
        f"{(got.float() - want.float()).abs().max().item():.3g}", torch.equal(got, want))
    say(f"repeat identical: {torch.equal(got, got2)}", torch.equal(got, got2))
    try:
        ops.check_status()
        say("device status clean")
    except RuntimeError as e:
        say(f"device status: {e}", False)
    # timing
    for _ in range(3):
        ep.forward(x)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        ep.forward(x)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ar_bytes = 2.0 * (world - 1) / world * cfg.hidden * 2
    say(f"exchange + experts: {ms.item():.3f} ms per block (max over ranks); NVLink bytes per row: all-to-all "
        f"{ep.nvlink_bytes_per_row():.0f} vs ring all-reduce of replicated rows {ar_bytes:.0f} (x {world} ranks each computing "
        f"all rows' router and shared expert)")
    ep.close()

    # ---- a whole MLA + MoE model under expert parallelism (attention replicated, every rank serving its own request):
    # logits against the same model on one rank
    from dgpp_b200.models.mla_moe import MlaMoeConfig, MlaMoeModel, MlaMoeRunner
    mcfg = MlaMoeConfig(layers=3, hidden=1024, heads=8, q_lora=256, kv_lora=128, nope=64, rope=32, v_dim=64, ffn=2048,
                        vocab=2048, dense_layers=1,
                        moe=MoEConfig(hidden=1024, experts=16, top_k=4, moe_ffn=512, shared_ffn=512))
    full = MlaMoeModel.random_init(mcfg, dev, seed=3, std=0.04, fmt="nvfp4")
    part = MlaMoeModel.random_init(mcfg, dev, seed=3, std=0.04, fmt="nvfp4", ep_rank=rank, ep_size=world)
    r_full = MlaMoeRunner(full, max_rows=64, slots=1, max_seq_len=256, device=dev)
    r_ep = MlaMoeRunner(part, max_rows=64, slots=1, max_seq_len=256, device=dev)
    if world > 1:
        say(f"model runner uses the all-to-all path in {len(r_ep.ep)} layers", len(r_ep.ep) == 2)
    g3 = torch.Generator().manual_seed(100 + rank)
    toks = torch.randint(0, mcfg.vocab, (110,), generator=g3).tolist()
    a = r_full.prefill(0, toks[:100], chunk=64)[-1].clone()
    b = r_ep.prefill(0, toks[:100], chunk=64)[-1].clone()
    cos = torch.nn.functional.cosine_similarity(a.float(), b.float(), dim=0).item()
    say(f"model prefill logits, expert parallel vs one rank: cosine {cos:.6f} argmax equal {int(a.argmax()) == int(b.argmax())}",
        cos >= 0.999)
    worst, same = 1.0, 0
    for s_ in range(6):
        a = r_full.decode([0], [toks[100 + s_]])[0]
        b = r_ep.decode([0], [toks[100 + s_]])[0]
        worst = min(worst, torch.nn.functional.cosine_similarity(a.float(), b.float(), dim=0).item())
        same += int(a.argmax()) == int(b.argmax())
    torch.cuda.synchronize()
    say(f"model decode logits over 6 graph-replayed steps: worst cosine {worst:.6f}, argmax equal in {same} of 6", worst >= 0.995)
    # the hybrid family through the same path
    from dgpp_b200.models.hybrid import HybridConfig, HybridModel, HybridRunner
    hcfg = HybridConfig(layers=4, hidden=512, full_every=4, q_heads=4, kv_heads=2, head_dim=128, gdn_k_heads=2, gdn_v_heads=4,
                        gdn_dk=128, gdn_dv=128, ffn=1024, vocab=2048,
                        moe=MoEConfig(hidden=512, experts=16, top_k=2, moe_ffn=512, shared_ffn=512))
    hfull = HybridRunner(HybridModel.random_init(hcfg, dev, seed=5, std=0.05, fmt="nvfp4"), 64, 1, 256, dev)
    hpart = HybridRunner(HybridModel.random_init(hcfg, dev, seed=5, std=0.05, fmt="nvfp4", ep_rank=rank, ep_size=world), 64, 1,
                         256, dev)
    htoks = torch.randint(0, hcfg.vocab, (70,), generator=g3).tolist()
    a = hfull.prefill(0, htoks[:64], chunk=32)[-1].clone()
    b = hpart.prefill(0, htoks[:64], chunk=32)[-1].clone()
    cos = torch.nn.functional.cosine_similarity(a.float(), b.float(), dim=0).item()
    worst = 1.0
    for s_ in range(5):
        a = hfull.decode([0], [htoks[64 + s_]])[0]
        b = hpart.decode([0], [htoks[64 + s_]])[0]
        worst = min(worst, torch.nn.functional.cosine_similarity(a.float(), b.float(), dim=0).item())
    torch.cuda.synchronize()
    say(f"hybrid model, expert parallel vs one rank: prefill cosine {cos:.6f}, worst decode cosine {worst:.6f}",
        cos >= 0.999 and worst >= 0.995)
    try:
        ops.check_status()
        say("device status clean after the model run")
    except RuntimeError as e:
        say(f"device status after the model run: {e}", False)
    text = "\n".join(lines)
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, (text, ok_all))
        if rank == 0:
            text = "\n".join(t for t, _ in gathered)
            ok_all = all(o for _, o in gathered)
        dist.destroy_process_group()
    if rank == 0:
        print(text)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                f.write(text + "\n")
    return 0 if ok_all else 1


if __name__ == "__main__":
    sys.exit(main())
