"""Kernel micro-benchmarks with roofline fractions.

    python -m dgpp_b200.bench.micro gemm_fp4 --rows 8 --n 34816 --k 5120 [--terms 3] [--splits 0]
    python -m dgpp_b200.bench.micro gemm_tc --rows 2048 --n 5120 --k 5120 [--fmt nvfp4]
    python -m dgpp_b200.bench.micro attn_decode --rows 8 --ctx 2048 [--hq 40 --hkv 8 --splits 4]
    python -m dgpp_b200.bench.micro attn_prefill --ctx 8192 [--hq 40 --hkv 8]
    python -m dgpp_b200.bench.micro act_quant --rows 8 --k 5120 [--mode rmsnorm]
    python -m dgpp_b200.bench.micro gdn --rows 8192 [--hv 32]
    python -m dgpp_b200.bench.micro moe --rows 8 [--experts 128 --top-k 8]
    python -m dgpp_b200.bench.micro decode_layer --rows 8 --ctx 2048     (phase timeline of one layer-boundary launch)

Timing: the launches are captured in a CUDA graph, replayed `--reps` times between CUDA events after a warm-up replay.
Weight-streaming kernels rotate over enough weight copies to exceed the 126 MB L2, so every launch reads its
weights from HBM.  Fractions are "of measured": the copy bandwidth / cuBLAS bf16 throughput in MEASURED_PEAKS.json
at the repository root (fallback 6650 GB/s, 1590 TFLOP/s when the file is absent).  `--once` runs a few plain
launches without graph or timing (the form used under a profiler).  Prints one JSON line.
(reference counterparts: benchmarks/micro/*.)
"""
from __future__ import annotations

import argparse
import json
import math
import os
from pathlib import Path

import torch

BF = torch.bfloat16
L2_BYTES = 126 << 20


def peaks() -> dict:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        j = json.loads(p.read_text())
        return {"hbm_gbs": j["hbm_gbs"], "tflops": j["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}


def graph_time(fns, reps: int) -> float:
    """Mean milliseconds per launch of the callables in `fns` (captured once, replayed)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for f in fns:
            f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps / len(fns)


def run(fns, args) -> float:
    if args.once:
        for f in fns[:3]:
            f()
        torch.cuda.synchronize()
        return float("nan")
    return graph_time(fns, args.reps)


def report(args, name: str, ms: float, bytes_: float = 0.0, flops: float = 0.0, **extra) -> None:
    pk = peaks()
    out = {"kernel": name, "us": round(ms * 1e3, 2), "peaks": pk["source"], **extra}
    if bytes_:
        gbs = bytes_ / ms / 1e6
        out.update(gb_s=round(gbs, 1), frac_hbm=round(gbs / pk["hbm_gbs"], 3))
    if flops:
        tf = flops / ms / 1e9
        out.update(tflops=round(tf, 1), frac_tensor=round(tf / pk["tflops"], 3))
    print(json.dumps(out), flush=True)


def bench_gemm_fp4(args, dev):
    from ..ops import core as ops
    from ..quant.formats import random_quant_linear

    n, k, rows = args.n, args.k, args.rows
    w_bytes = n * k // 2 + n * k // 16
    copies = max(2, min(16, math.ceil(2 * L2_BYTES / w_bytes))) if rows <= 64 else 2
    ws = [random_quant_linear(n, k, "nvfp4", dev) for _ in range(copies)]
    x = torch.randn(rows, k, device=dev).to(BF)
    terms = args.terms if rows <= 64 else 1
    xa = ops.act_quant_nvfp4(x, terms)
    out = torch.empty(rows, n, device=dev, dtype=BF)
    splits = args.splits or None
    fns = [(lambda w=w: ops.gemm_fp4(xa, w, out=out, splits=splits)) for w in ws]
    ms = run(fns, args)
    ops.check_status()
    if args.trace:
        # phase timestamps of CTA (0,0,0) of one cold launch (weights not in L2), ns since kernel entry
        from ..ops._lib import call, ptr
        t = torch.zeros(8, dtype=torch.int64, device=dev)
        call("dgpp_gemm_fp4_set_trace", ptr(t))
        fns[1 % len(fns)]()
        torch.cuda.synchronize()
        call("dgpp_gemm_fp4_set_trace", None)
        v = t.tolist()
        names = ["entry", "prologue_done", "prev_grid_done", "first_stage_landed", "last_mma_issued", "acc_complete",
                 "epilogue_done"]
        print(json.dumps({"kernel": "gemm_fp4_trace", "n": n, "k": k, "ns_since_entry":
                          {nm: v[i] - v[0] for i, nm in enumerate(names)}}))
    report(args, "gemm_fp4", ms, bytes_=w_bytes + rows * k * terms // 2 + rows * n * 2, flops=2.0 * rows * n * k,
           rows=rows, n=n, k=k, terms=terms, weight_copies=copies)


def bench_gemm_tc(args, dev):
    from ..ops import core as ops
    from ..quant.formats import random_quant_linear

    n, k, rows = args.n, args.k, args.rows
    ops.PAIR_GEMM = not args.no_pair
    ws = [random_quant_linear(n, k, args.fmt, dev) for _ in range(2)]
    x = torch.randn(rows, k, device=dev).to(BF)
    out = torch.empty(rows, n, device=dev, dtype=BF)
    fns = [(lambda w=w: ops.gemm_tc(x, w, out=out)) for w in ws]
    ms = run(fns, args)
    ops.check_status()
    report(args, "gemm_tc", ms, bytes_=ws[0].nbytes + rows * k * 2 + rows * n * 2, flops=2.0 * rows * n * k, rows=rows, n=n, k=k,
           fmt=args.fmt, cta_pairs=bool(ops.PAIR_GEMM and rows >= ops.PAIR_GEMM_MIN_ROWS and args.fmt in ("nvfp4", "mxfp4")
                                        and n % 256 == 0))


def bench_gemm_fp8(args, dev):
    """Native FP8 linear (activation quantiser timed separately) against the converter path on the same weights."""
    from ..ops import core as ops
    from ..quant.formats import random_quant_linear

    n, k, rows = args.n, args.k, args.rows
    copies = max(2, min(16, math.ceil(2 * L2_BYTES / (n * k)))) if rows <= 64 else 2
    ws = [random_quant_linear(n, k, "fp8", dev) for _ in range(copies)]
    x = torch.randn(rows, k, device=dev).to(BF)
    xa = ops.fp8_act_quant(x)
    out = torch.empty(rows, n, device=dev, dtype=BF)
    splits = args.splits or None
    ms = run([(lambda w=w: ops.gemm_fp8(xa, w, out=out, splits=splits)) for w in ws], args)
    ops.check_status()
    report(args, "gemm_fp8", ms, bytes_=n * k + rows * k + rows * n * 2, flops=2.0 * rows * n * k, rows=rows, n=n, k=k)
    ms = run([lambda: ops.fp8_act_quant(x, out=xa)], args)
    report(args, "fp8_act_quant", ms, bytes_=rows * k * 3, rows=rows, k=k)
    ms = run([(lambda w=w: ops.gemm_tc(x, w, out=out)) for w in ws], args)
    report(args, "gemm_tc (fp8 weights through the converter warps)", ms, bytes_=n * k + rows * k * 2 + rows * n * 2,
           flops=2.0 * rows * n * k, rows=rows, n=n, k=k)


def bench_mla(args, dev):
    """Latent attention decode: tensor-core kernel against the CUDA-core kernel (rows requests at context ctx)."""
    from ..ops import core as ops

    rows, ctx, heads, page = args.rows, args.ctx, args.hq, 64
    blocks_per = ctx // page + 2
    cache = (torch.randn(rows * blocks_per + 1, page, 576, device=dev) * 0.3).to(BF)
    table = (1 + torch.arange(rows * blocks_per, device=dev, dtype=torch.int32)).view(rows, blocks_per).contiguous()
    q = (torch.randn(rows, heads, 576, device=dev) * 0.3).to(BF)
    req = torch.arange(rows, dtype=torch.int32, device=dev)
    pos = torch.full((rows,), ctx - 1, dtype=torch.int32, device=dev)
    sp = args.splits or 4
    for tc in (True, False):
        ms = run([lambda tc=tc: ops.mla_decode(q, cache, table, req, pos, 0.07, 512, 64, splits=sp, tensor_cores=tc)], args)
        ops.check_status()
        report(args, "mla_decode_tc" if tc else "mla_decode (CUDA cores)", ms, bytes_=rows * ctx * 576 * 2.0,
               flops=2.0 * rows * heads * ctx * (576 + 512), rows=rows, ctx=ctx, heads=heads, splits=sp)


def _cache(dev, hq, hkv, ctx, page=64, slots=1, d=128):
    from ..engine.kv_cache import PagedKV
    from ..ops import core as ops, reference as ref

    per = ctx // page + 2
    kv = PagedKV(1, hkv, d, slots * per + 2, slots, per, page, True, dev)
    inv_freq, _ = ref.rope_inv_freq(d, 1e4, dev)
    for s in range(slots):
        assert kv.reserve(s, ctx)
        qkv = torch.randn(ctx, (hq + 2 * hkv) * d, device=dev).to(BF)
        pos = torch.arange(ctx, device=dev, dtype=torch.int32)
        req = torch.full((ctx,), s, device=dev, dtype=torch.int32)
        ops.rope_kv_write(qkv, pos, req, kv.block_table, inv_freq, kv.layers[0], hq, hkv, d)
    return kv, qkv


def bench_attn_decode(args, dev):
    from ..ops import core as ops

    hq, hkv, ctx, rows, d = args.hq, args.hkv, args.ctx, args.rows, args.head_dim
    kv, _ = _cache(dev, hq, hkv, ctx, slots=rows, d=d)
    q = torch.randn(rows, (hq + 2 * hkv) * d, device=dev).to(BF)
    pos = torch.full((rows,), ctx - 1, device=dev, dtype=torch.int32)
    req = torch.arange(rows, device=dev, dtype=torch.int32)
    out = torch.empty(rows, hq * d, device=dev, dtype=BF)
    sp = args.splits or 4
    scratch = (torch.empty(rows * hq * sp * 2, device=dev), torch.empty(rows * hq * sp * d, device=dev))
    fn = lambda: ops.attn_decode_tc(q, q.stride(0), kv.layers[0], kv.block_table, req, pos, hq, hkv, d, 0.088, splits=sp,
                                    scratch=scratch, out=out)
    ms = run([fn] * 4, args)
    ops.check_status()
    report(args, "attn_decode_tc", ms, bytes_=2.0 * rows * ctx * hkv * d, flops=4.0 * rows * hq * ctx * d, rows=rows, ctx=ctx,
           hq=hq, hkv=hkv, head_dim=d, splits=sp)


def bench_sparse_attn(args, dev):
    """Block-sparse decode: index scores + block selection (token-key form), then attention over the kept blocks."""
    from ..ops import core as ops, reference as ref

    hq, hkv, ctx, rows, d, blk, topk = args.hq, args.hkv, args.ctx, args.rows, args.head_dim, args.sparse_block, args.sparse_topk
    kv, _ = _cache(dev, hq, hkv, ctx, page=blk, slots=rows, d=d)
    blocks = kv.layers[0].k.shape[0]
    di = 128
    index = torch.randn(blocks, blk, di, device=dev).to(BF)
    iqk = torch.randn(rows, (hkv + 1) * di, device=dev).to(BF)
    q = torch.randn(rows, (hq + 2 * hkv) * d, device=dev).to(BF)
    pos = torch.full((rows,), ctx - 1, device=dev, dtype=torch.int32)
    req = torch.arange(rows, device=dev, dtype=torch.int32)
    max_sel = ctx // blk + 1
    sel = torch.empty(rows, hkv, topk, dtype=torch.int32, device=dev)
    out = torch.empty(rows, hq * d, device=dev, dtype=BF)
    sp = args.splits or 8
    scratch = (torch.empty(rows * hq * sp * 2, device=dev), torch.empty(rows * hq * sp * d, device=dev))
    scores = torch.empty(rows, hkv, max_sel, device=dev)
    f_sel = lambda: ops.msa_index_select(iqk, index, kv.block_table, req, pos, hkv, di, blk, topk, max_sel, out=sel, scores=scores)
    f_att = lambda: ops.attn_decode(q, q.stride(0), kv.layers[0], kv.block_table, req, pos, hq, hkv, d, 0.088, splits=sp,
                                    scratch=scratch, out=out, sel=sel, sel_block=blk)
    f_sel()
    ms_sel = run([f_sel] * 4, args)
    ms_att = run([f_att] * 4, args)
    ops.check_status()
    report(args, "msa_index_select", ms_sel, bytes_=2.0 * rows * ctx * di, rows=rows, ctx=ctx, index_heads=hkv, block=blk, topk=topk)
    kept = min(topk, ctx // blk + 1) * blk
    report(args, "attn_decode_sparse", ms_att, bytes_=2.0 * rows * kept * hkv * d, rows=rows, ctx=ctx, kept_tokens=kept, hq=hq,
           hkv=hkv, head_dim=d, splits=sp)
    for tsp in (1, 2, 4):
        f_tc = lambda: ops.attn_decode_tc(q, q.stride(0), kv.layers[0], kv.block_table, req, pos, hq, hkv, d, 0.088, splits=tsp,
                                          scratch=scratch, out=out, sel=sel, sel_block=blk)
        ms_tc = run([f_tc] * 4, args)
        ops.check_status()
        report(args, "attn_decode_tc_sparse", ms_tc, bytes_=2.0 * rows * kept * hkv * d, rows=rows, ctx=ctx, kept_tokens=kept,
               hq=hq, hkv=hkv, head_dim=d, splits=tsp)


def bench_engram(args, dev):
    """Hashed n-gram memory site: lookup (hash + gather + decode), projection, stream gate."""
    from ..models.engram import Engram, EngramConfig
    from ..ops import core as ops

    rows, H, hc = args.rows, args.k, 4
    cfg = EngramConfig(max_ngram=4, heads=4, head_dim=128, bucket=args.bucket)
    e = Engram.random_init(cfg, [0], 131072, hc, H, dev, seed=0)
    L = e.layers[0]
    toks = torch.randint(0, 131072, (rows,), device=dev, dtype=torch.int32)
    prev = torch.randint(0, 131072, (3, rows), device=dev, dtype=torch.int32)
    st = torch.randn(rows, hc, H, device=dev).to(BF)
    emb = ops.engram_embed(toks, prev, e.token_map, L.multipliers, L.primes, L.offsets, L.table, L.table_sf, e.pad_class)
    kvp = ops.linear(emb, L.wkv)
    f_emb = lambda: ops.engram_embed(toks, prev, e.token_map, L.multipliers, L.primes, L.offsets, L.table, L.table_sf,
                                     e.pad_class, out=emb)
    f_gate = lambda: ops.engram_gate(st, kvp, L.q_weight, L.k_weight, 1e-6)
    ms_e = run([f_emb] * 4, args)
    ms_g = run([f_gate] * 4, args)
    ops.check_status()
    slots = cfg.slots
    report(args, "engram_embed", ms_e, bytes_=rows * slots * (cfg.head_dim * 3 + cfg.head_dim // 32), rows=rows, slots=slots,
           table_rows=int(L.table.shape[0]))
    report(args, "engram_gate", ms_g, bytes_=rows * (2 * hc * H * 2 + (hc + 1) * H * 2), rows=rows, streams=hc, hidden=H)


def bench_attn_prefill(args, dev):
    from ..ops import core as ops

    hq, hkv, ctx, d = args.hq, args.hkv, args.ctx, args.head_dim
    kv, qkv = _cache(dev, hq, hkv, ctx, d=d)
    out = torch.empty(ctx, hq * d, device=dev, dtype=BF)
    fn = lambda: ops.attn_prefill_tc(qkv, qkv.stride(0), kv.layers[0], kv.block_table[0], 0, hq, hkv, d, 0.088, out=out)
    ms = run([fn] * 2, args)
    ops.check_status()
    report(args, "attn_prefill_tc", ms, flops=4.0 * ctx * ctx / 2 * d * hq, bytes_=2.0 * ctx * hkv * d + 4.0 * ctx * hq * d,
           ctx=ctx, hq=hq, hkv=hkv, head_dim=d, note="causal, bf16-equivalent FLOPs (two-term fp8 operands issue 4x the MMAs)")


def bench_act_quant(args, dev):
    from ..ops import core as ops

    rows, k = args.rows, args.k
    x = torch.randn(rows, k, device=dev).to(BF)
    d = torch.randn(rows, k, device=dev).to(BF)
    w = torch.ones(k, device=dev, dtype=BF)
    xa = ops.act_quant_nvfp4(x, args.terms)
    if args.mode == "rmsnorm":
        fn = lambda: ops.act_quant_nvfp4(x, out=xa, mode="rmsnorm", delta=d, norm_w=w)
    elif args.mode == "swiglu":
        gu = torch.randn(rows, 2 * k, device=dev).to(BF)
        fn = lambda: ops.act_quant_nvfp4(gu, out=xa, mode="swiglu")
    else:
        fn = lambda: ops.act_quant_nvfp4(x, out=xa)
    ms = run([fn] * 8, args)
    report(args, "act_quant_" + args.mode, ms, bytes_=rows * k * 2 * (3 if args.mode == "rmsnorm" else 1) + rows * k * args.terms * 0.5625,
           rows=rows, k=k, terms=args.terms)


def bench_gdn(args, dev):
    from ..models.gdn import GdnConfig, GdnLayer, GdnState, GdnWeights

    cfg = GdnConfig(hidden=2048, k_heads=args.hv // 2, v_heads=args.hv, dk=128, dv=128)
    w = GdnWeights.random_init(cfg, dev, seed=1)
    layer, st = GdnLayer(w, args.rows, dev), GdnState(cfg, 1, dev)
    x = torch.randn(args.rows, cfg.hidden, device=dev).to(BF)
    out = torch.empty_like(x)
    from ..ops import core as ops
    fn = lambda: layer.forward(x, st, out, slot=0)
    res = {}
    for name, chunked in (("chunked", True), ("sequential", False)):
        ops.GDN_CHUNKED = chunked
        res[name + "_layer_ms"] = run([fn], args)
        # the scan alone: preparation + recurrence on the layer's convolution output
        c = cfg
        nq = c.k_heads * c.dk
        conv = torch.randn(args.rows, 2 * nq + c.v_heads * c.dv, device=dev).to(BF)
        ab = torch.randn(args.rows, 2 * c.v_heads, device=dev).to(BF)
        o = torch.empty(args.rows, c.v_heads * c.dv, device=dev, dtype=BF)
        scan = lambda: ops.gdn_recurrent(conv[:, :nq], conv[:, nq:2 * nq], conv[:, 2 * nq:], ab[:, :c.v_heads],
                                         ab[:, c.v_heads:], w.A_log, w.dt_bias, st.ssm, o, c.k_heads, c.v_heads, c.dk,
                                         c.dv, None, 0, True)
        res[name + "_scan_ms"] = run([scan], args)
    ops.GDN_CHUNKED = True
    report(args, "gdn_layer_prefill", res["chunked_layer_ms"], rows=args.rows, v_heads=args.hv,
           note="in_proj + conv + recurrence + gated norm + out_proj of one layer; *_scan_ms: preparation + recurrence only",
           **res)


def bench_moe(args, dev):
    from ..models.moe import MoEBlock, MoEConfig, MoEWeights

    cfg = MoEConfig(hidden=args.k, experts=args.experts, top_k=args.top_k, moe_ffn=args.moe_ffn, shared_ffn=args.moe_ffn)
    w = MoEWeights.random_init(cfg, dev, seed=1)
    blk = MoEBlock(w, max_rows=16, device=dev)
    x = torch.randn(args.rows, cfg.hidden, device=dev).to(BF)
    out = torch.empty_like(x)
    fn = lambda: blk.forward(x, out)
    ms = run([fn] * 2, args)
    active = int(blk.n_active)
    per_expert = 3 * cfg.hidden * cfg.moe_ffn * 0.5625
    report(args, "moe_block_decode", ms, bytes_=(active + 1) * per_expert, rows=args.rows, experts=args.experts, top_k=args.top_k,
           active_experts=active)


def bench_decode_layer(args, dev):
    """One launch of the persistent decode-layer kernel on the 27B-class layer shapes (3-layer model, prefilled to
    --ctx): CUDA-event time and the %globaltimer phase stamps of CTA 0 and of the last CTA, weights rotated out of L2
    before every launch."""
    import ctypes as C

    from ..engine.llm_engine import LLMEngine
    from ..models.dense import DenseConfig, DenseModel
    from ..ops import _lib, core as ops

    rows, ctx = args.rows, args.ctx
    cfg = DenseConfig.dense_27b(layers=3)
    model = DenseModel.random_init(cfg, device=dev, seed=0)
    eng = LLMEngine(model, max_batch=rows, max_seq_len=ctx + 256, prefill_chunk=2048, use_graphs=False,
                    fused_decode=True)
    g = torch.Generator().manual_seed(1)
    firsts = torch.zeros(rows, dtype=torch.int32, device=dev)
    for s_ in range(rows):
        assert eng.kv.reserve(s_, ctx + 64)
        firsts[s_:s_ + 1].copy_(eng.prefill(s_, torch.randint(0, cfg.vocab, (ctx,), generator=g).tolist()))
    eng.start_decode(list(range(rows)), firsts)
    for _ in range(3):
        eng.decode_step(rows)
    torch.cuda.synchronize()
    tr = torch.zeros(64, dtype=torch.int64, device=dev)
    _lib.declare("dgpp_decode_layer_set_trace", [C.c_void_p])
    _lib.call("dgpp_decode_layer_set_trace", tr.data_ptr())
    r = eng.runner
    launch = r._fused_plan(rows, eng.d_positions[:rows], eng.d_row_req[:rows], r.decode_splits)[1]
    names = {1: "row_a", 2: "gemm", 3: "unitq", 4: "rope", 5: "row_c"}
    out = []
    for _ in range(max(2, min(args.reps, 5))):
        junk = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev)
        junk.fill_(1)
        del junk
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        launch.launch()
        e1.record()
        torch.cuda.synchronize()
        t, a = tr.cpu().tolist(), launch.a
        rec = {"event_us": e0.elapsed_time(e1) * 1000.0}
        for sel, nm in ((0, "cta0"), (1, "cta_last")):
            b = t[sel * 32 + 30]
            rec[nm] = [[f"{names[a.ph_type[ph]]}{a.ph_idx[ph]}", t[sel * 32 + 2 * ph] - b, t[sel * 32 + 2 * ph + 1] - b]
                       for ph in range(a.nphase)]
        out.append(rec)
    _lib.call("dgpp_decode_layer_set_trace", None)
    ops.check_status()
    print(json.dumps({"kernel": "decode_layer", "rows": rows, "ctx": ctx, "unit": "ns since kernel entry [phase, start, end]",
                      "launches": out}))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm_fp4", "gemm_tc", "gemm_fp8", "attn_decode", "attn_prefill", "act_quant", "gdn",
                                       "moe", "mla", "decode_layer", "sparse_attn", "engram"])
    ap.add_argument("--sparse-block", type=int, default=128)
    ap.add_argument("--sparse-topk", type=int, default=16)
    ap.add_argument("--bucket", type=int, default=200003, help="engram: rows per (n-gram size, head) range")
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--n", type=int, default=5120)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--terms", type=int, default=3)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--fmt", default="nvfp4")
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--hq", type=int, default=40)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128, choices=(128, 256))
    ap.add_argument("--hv", type=int, default=32)
    ap.add_argument("--mode", default="rmsnorm", choices=["plain", "rmsnorm", "swiglu"])
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--moe-ffn", type=int, default=1536)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--no-pair", action="store_true", help="gemm_tc: keep 4-bit prefill GEMMs on the single-CTA kernel")
    ap.add_argument("--trace", action="store_true", help="gemm_fp4: print the phase timestamps of one CTA")
    ap.add_argument("--once", action="store_true", help="a few plain launches, no graph, no timing (for profilers)")
    args = ap.parse_args(argv)
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    {"gemm_fp4": bench_gemm_fp4, "gemm_tc": bench_gemm_tc, "gemm_fp8": bench_gemm_fp8, "mla": bench_mla, "attn_decode": bench_attn_decode, "attn_prefill": bench_attn_prefill,
     "act_quant": bench_act_quant, "gdn": bench_gdn, "moe": bench_moe,
     "decode_layer": bench_decode_layer, "sparse_attn": bench_sparse_attn, "engram": bench_engram}[args.kernel](args, dev)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
