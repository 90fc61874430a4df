"""Numerics of the sm_100a kernels against the PyTorch fp32 restatements in ops/reference.py."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _close(a, b, rtol, atol):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    lim = atol + rtol * b.abs()
    bad = (err > lim).sum().item()
    assert bad == 0, f"{bad}/{a.numel()} out of tolerance, max err {err.max().item():.4g}"


def test_embed_rmsnorm_swiglu_argmax(dev):
    from dgpp_b200.ops import core as ops, reference as ref

    torch.manual_seed(0)
    table = torch.randn(1000, 512, device=dev).to(BF)
    ids = torch.randint(0, 1000, (7,), device=dev, dtype=torch.int32)
    assert torch.equal(ops.embed_gather(ids, table), ref.embed_gather(ids, table))

    for hidden in (256, 5120):
        x = torch.randn(5, hidden, device=dev).to(BF)
        d = torch.randn(5, hidden, device=dev).to(BF)
        w = (1 + 0.1 * torch.randn(hidden, device=dev)).to(BF)
        y = ops.rmsnorm(x.clone(), w, 1e-6)
        yr, _ = ref.rmsnorm(x, w, 1e-6)
        _close(y, yr, 2 ** -7, 1e-3)
        xr = x.clone()
        y2 = ops.rmsnorm(xr, w, 1e-6, delta=d)
        yr2, res = ref.rmsnorm(x, w, 1e-6, d)
        assert torch.equal(xr, res)
        _close(y2, yr2, 2 ** -7, 1e-3)

    gu = torch.randn(3, 2 * 1024, device=dev).to(BF) * 3
    _close(ops.swiglu(gu), ref.swiglu(gu), 2 ** -7, 1e-3)
    _close(ops.swiglu(gu, limit=2.0), ref.swiglu(gu, 2.0), 2 ** -7, 1e-3)

    logits = torch.randn(4, 151936, device=dev)
    logits[1, 777] = 50.0
    logits[1, 90000] = 50.0  # tie -> lowest index
    i, v = ops.argmax(logits)
    ir, vr = ref.argmax(logits)
    assert torch.equal(i, ir) and int(i[1]) == 777
    i2, _ = ops.argmax(logits.to(BF), id_base=1000)
    assert torch.equal(i2, ref.argmax(logits.to(BF), 1000)[0])


@pytest.mark.parametrize("rows,vocab", [(8, 151936), (1, 16384), (3, 18991), (64, 32000), (70, 32000), (5, 4096)])
def test_argmax_cluster_and_single_cta_agree(dev, rows, vocab):
    """Few long rows take the cluster kernel (a row spread over 8 CTAs), the rest one CTA per row; both follow
    'largest value, lowest index', also when the tie straddles two CTAs' slices or a row is constant."""
    from dgpp_b200.ops import core as ops, reference as ref

    torch.manual_seed(21)
    logits = torch.randn(rows, vocab, device=dev)
    logits[0, vocab - 1] = 60.0
    logits[0, vocab // 8 + 5] = 60.0                      # the same maximum in slice 1 and in the last slice
    if rows > 2:
        logits[1] = 0.25                                   # constant row: index 0
        logits[2] = float("-inf")                          # fully masked row: index 0
    i, v = ops.argmax(logits, id_base=7)
    ir, vr = ref.argmax(logits, 7)
    torch.cuda.synchronize()
    assert torch.equal(i, ir) and torch.equal(v, vr)
    assert int(i[0]) == vocab // 8 + 5 + 7
    ib, _ = ops.argmax(logits.to(BF))
    assert torch.equal(ib, ref.argmax(logits.to(BF))[0])


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4", "bf16"])
@pytest.mark.parametrize("rows", [1, 3, 4])
def test_gemv(dev, fmt, rows):
    from dgpp_b200.ops import core as ops, reference as ref
    from dgpp_b200.quant.formats import quantize

    torch.manual_seed(1)
    n, k = 520, 1024
    w = quantize(torch.randn(n, k, device=dev) * 0.05, fmt)
    x = torch.randn(rows, k, device=dev).to(BF)
    y = ops.gemv(x, w)
    _close(y, ref.linear(x, w), 2 ** -6, 2e-3)


@pytest.mark.parametrize("fmt,a_f16", [("bf16", 0), ("nvfp4", 0), ("fp8", 0), ("mxfp4", 0), ("mxfp8", 0), ("int8", 0),
                                       ("int4", 0)])
@pytest.mark.parametrize("rows,bn,splits", [(1, 16, 1), (8, 16, 4), (37, 64, 1), (130, 128, 2), (300, 256, 1)])
def test_gemm_tc(dev, fmt, a_f16, rows, bn, splits):
    from dgpp_b200.ops import core as ops, reference as ref
    from dgpp_b200.quant.formats import quantize

    torch.manual_seed(2)
    n, k = 384 + 64, 1024
    w = quantize(torch.randn(n, k, device=dev) * 0.05, fmt)
    x = torch.randn(rows, k, device=dev).to(BF)
    y = ops.gemm_tc(x, w, bn=bn, splits=splits, a_f16=a_f16)
    ops.check_status()
    # fp8 block weights reach the tensor core as bf16(e4m3 * scale): compare against that operand
    # (likewise int8 / int4: bf16(code * scale))
    wr = w if fmt not in ("fp8", "int8", "int4") else quantize(w.dequant().to(BF).float(), "bf16")
    yr = ref.linear(x, wr)
    _close(y, yr, 2 ** -6, 4e-3)
    # fp32 output + fused residual
    res = torch.randn(rows, n, device=dev).to(BF)
    y2 = ops.gemm_tc(x, w, resid=res, bn=bn, splits=splits, a_f16=a_f16)
    ops.check_status()
    _close(y2, ref.linear(x, wr, resid=res), 2 ** -6, 8e-3)


@pytest.mark.parametrize("rows,bn,splits", [(1, 16, 1), (8, 16, 4), (37, 64, 1), (130, 128, 2), (300, 256, 1)])
def test_gemm_tc_bf12_is_bitwise_the_bf16_kernel(dev, rows, bn, splits):
    """The 12-bit resident form feeds the tensor cores the exact bf16 bits (escaped outliers included), so the
    converter path returns what the plain bf16 kernel returns, bit for bit."""
    from dgpp_b200.ops import core as ops
    from dgpp_b200.quant.formats import QuantLinear, bf12_decode, bf12_encode

    torch.manual_seed(12)
    n, k = 384 + 64, 1024
    wb = (torch.randn(n, k, device=dev) * 0.05).to(BF)
    # outliers far outside every row's exponent window: first / last column, row tile edges, a zero, a whole zero row
    wb[0, 0], wb[0, k - 1], wb[127, 513], wb[128, 64], wb[n - 1, k - 1] = 3e20, -1e-30, 0.0, 7e15, -2e-25
    wb[200] = 0
    wb[300, ::3] = 1e-28                                  # a row with hundreds of escapes (binary search depth)
    q = bf12_encode(wb)
    assert q is not None and torch.equal(bf12_decode(q).view(torch.int16), wb.view(torch.int16))
    w16 = QuantLinear("bf16", n, k, wb)
    x = torch.randn(rows, k, device=dev).to(BF)
    y = ops.gemm_tc(x, q, bn=bn, splits=splits)
    y32 = torch.empty(rows, n, device=dev, dtype=torch.float32)
    ops.gemm_tc(x, q, out32=y32, bn=bn, splits=splits)
    want = ops.gemm_tc(x, w16, bn=bn, splits=splits)
    want32 = torch.empty(rows, n, device=dev, dtype=torch.float32)
    ops.gemm_tc(x, w16, out32=want32, bn=bn, splits=splits)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(y.view(torch.int16), want.view(torch.int16))
    assert torch.equal(y32, want32)


def test_gemm_tc_is_deterministic_and_row_independent(dev):
    from dgpp_b200.ops import core as ops
    from dgpp_b200.quant.formats import quantize

    torch.manual_seed(3)
    w = quantize(torch.randn(512, 2048, device=dev) * 0.05, "nvfp4")
    x = torch.randn(8, 2048, device=dev).to(BF)
    y1 = ops.gemm_tc(x, w, bn=16, splits=4)
    y2 = ops.gemm_tc(x, w, bn=16, splits=4)
    assert torch.equal(y1, y2)
    y3 = ops.gemm_tc(x[:1].contiguous(), w, bn=16, splits=4)
    assert torch.equal(y1[:1], y3)
    ops.check_status()


def _fill_cache(dev, kv, slot, k, v):
    """Write fp32 k/v [T, hkv, d] for request `slot` directly into the paged cache (reference codec)."""
    from dgpp_b200.ops import reference as ref

    T = k.shape[0]
    assert kv.reserve(slot, T)
    for li, layer in enumerate(kv.layers):
        for t in range(T):
            blk = kv.req_blocks[slot][t // kv.page]
            off = t % kv.page
            if kv.fp8:
                kq, ks = ref.quant_kv_fp8(k[t])
                vq, vs = ref.quant_kv_fp8(v[t])
                layer.k[blk, :, off] = kq
                layer.v[blk, :, off] = vq
                layer.k_scale[blk, :, off] = ks
                layer.v_scale[blk, :, off] = vs
            else:
                layer.k[blk, :, off] = k[t].to(BF)
                layer.v[blk, :, off] = v[t].to(BF)


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("hq,hkv,d", [(10, 2, 128), (16, 2, 256), (4, 2, 64)])
def test_rope_kv_and_decode_attention(dev, fp8, hq, hkv, d):
    from dgpp_b200.engine.kv_cache import PagedKV
    from dgpp_b200.ops import core as ops, reference as ref

    torch.manual_seed(4)
    page, ctx = 64, 333
    kv = PagedKV(1, hkv, d, 64, 4, 16, page, fp8, dev)
    inv_freq, _ = ref.rope_inv_freq(d, 1e4, dev)
    # fill the cache by running the kernel over ctx rows of one request, then decode one more row
    rows = ctx
    qkv = torch.randn(rows, (hq + 2 * hkv) * d, device=dev).to(BF)
    pos = torch.arange(rows, device=dev, dtype=torch.int32)
    req = torch.full((rows,), 2, device=dev, dtype=torch.int32)
    assert kv.reserve(2, rows)
    ref_q = ref.apply_rope(qkv[:, :hq * d].float().view(rows, hq, d), pos, inv_freq, d)
    ref_k = ref.apply_rope(qkv[:, hq * d:(hq + hkv) * d].float().view(rows, hkv, d), pos, inv_freq, d)
    ref_v = qkv[:, (hq + hkv) * d:].float().view(rows, hkv, d)
    ops.rope_kv_write(qkv, pos, req, kv.block_table, inv_freq, kv.layers[0], hq, hkv, d)
    _close(qkv[:, :hq * d].view(rows, hq, d), ref_q, 2 ** -6, 2e-2)
    if fp8:
        kq, ks = ref.quant_kv_fp8(ref_k)
        vq, vs = ref.quant_kv_fp8(ref_v)
        kd = kq.view(torch.float8_e4m3fn).float() * ks.unsqueeze(-1)
        vd = vq.view(torch.float8_e4m3fn).float() * vs.unsqueeze(-1)
    else:
        kd, vd = ref._r(ref_k), ref._r(ref_v)
    scale = 1.0 / math.sqrt(d)
    # decode attention for the last 3 rows (each sees positions <= its own), both split settings
    for splits in (1, 4):
        out = ops.attn_decode(qkv, qkv.stride(0), kv.layers[0], kv.block_table, req, pos, hq, hkv, d, scale,
                              splits=splits)
        q_all = qkv[:, :hq * d].float().view(rows, hq, d)
        want = ref.attention(q_all, kd, vd, scale, causal_offset=0).reshape(rows, hq * d)
        # an e4m3 code of K/V may differ by one step from the oracle when sincos differs in the last ulp
        _close(out, want, 3e-2, 0.1 if fp8 else 3e-2)
        assert (out.float() - want).abs().mean().item() < 5e-3


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_tiny_model_engine_matches_reference(dev, fmt):
    from dgpp_b200.engine.llm_engine import LLMEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel

    cfg = DenseConfig.tiny(weight_fmt=fmt)
    model = DenseModel.random_init(cfg, device=dev, seed=0, std=0.05)
    eng = LLMEngine(model, max_batch=2, max_seq_len=256, prefill_chunk=64)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (70, 33)]
    out = eng.generate(prompts, max_tokens=6)
    from dgpp_b200.ops import core as ops
    ops.check_status()
    # oracle: greedy decode with the reference forward, allowing a near-tie to differ
    for p, got in zip(prompts, out):
        toks = torch.tensor(p, device=dev)
        logits, kv = model.forward_reference(toks)
        seq = []
        cur = logits[-1]
        for step in range(6):
            top2 = torch.topk(cur.float(), 2)
            want = int(top2.indices[0])
            margin = float(top2.values[0] - top2.values[1])
            if got[step] != want:
                assert margin < 0.05, f"step {step}: got {got[step]} want {want} margin {margin}"
                break
            seq.append(want)
            logits, kv = model.forward_reference(torch.tensor([want], device=dev), start_pos=len(p) + step, kv=kv)
            cur = logits[-1]
    # graph replay determinism: same prompts, same tokens
    out2 = eng.generate(prompts, max_tokens=6)
    assert out == out2


@pytest.mark.parametrize("fp8", [True, False])
def test_sliding_window_and_sink_logits(dev, fp8):
    """Sliding-window decode attention with a per-head sink column against the fp32 reference."""
    from dgpp_b200.engine.kv_cache import PagedKV
    from dgpp_b200.ops import core as ops, reference as ref

    torch.manual_seed(9)
    hq, hkv, d, page, rows, window = 8, 2, 128, 64, 300, 96
    kv = PagedKV(1, hkv, d, 64, 4, 16, page, fp8, dev)
    inv_freq, _ = ref.rope_inv_freq(d, 1e4, dev)
    qkv = torch.randn(rows, (hq + 2 * hkv) * d, device=dev).to(BF)
    pos = torch.arange(rows, device=dev, dtype=torch.int32)
    req = torch.full((rows,), 1, device=dev, dtype=torch.int32)
    assert kv.reserve(1, rows)
    ref_k = ref.apply_rope(qkv[:, hq * d:(hq + hkv) * d].float().view(rows, hkv, d), pos, inv_freq, d)
    ref_v = qkv[:, (hq + hkv) * d:].float().view(rows, hkv, d)
    ops.rope_kv_write(qkv, pos, req, kv.block_table, inv_freq, kv.layers[0], hq, hkv, d)
    if fp8:
        kq, ks = ref.quant_kv_fp8(ref_k)
        vq, vs = ref.quant_kv_fp8(ref_v)
        kd = kq.view(torch.float8_e4m3fn).float() * ks.unsqueeze(-1)
        vd = vq.view(torch.float8_e4m3fn).float() * vs.unsqueeze(-1)
    else:
        kd, vd = ref._r(ref_k), ref._r(ref_v)
    scale = 1.0 / math.sqrt(d)
    sink = torch.tensor([-2.0, 0.0, 1.5, 3.0, -30.0, 0.5, 8.0, 2.0], device=dev)
    q_all = qkv[:, :hq * d].float().view(rows, hq, d)
    want = ref.attention(q_all, kd, vd, scale, causal_offset=0, window=window, sink=sink).reshape(rows, hq * d)
    plain = ref.attention(q_all, kd, vd, scale, causal_offset=0, window=window).reshape(rows, hq * d)
    assert (want - plain).abs().max() > 0.05            # the sink column takes probability mass away
    for splits in (1, 3):
        out = ops.attn_decode(qkv, qkv.stride(0), kv.layers[0], kv.block_table, req, pos, hq, hkv, d, scale,
                              splits=splits, window=window, sink=sink)
        _close(out, want, 3e-2, 0.1 if fp8 else 3e-2)
        assert (out.float() - want).abs().mean().item() < 5e-3
    ops.check_status()


@pytest.mark.parametrize("sinks", [False, True])
def test_windowed_sink_model_engine_matches_reference(dev, sinks):
    """Sliding-window layers (every second layer global), with and without sink logits, through the engine."""
    from dgpp_b200.engine.llm_engine import LLMEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel
    from dgpp_b200.ops import core as ops

    cfg = DenseConfig.tiny(hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, layers=4, sliding_window=40,
                           global_every=2, attn_sinks=sinks)
    model = DenseModel.random_init(cfg, device=dev, seed=2, std=0.05)
    assert [L.window for L in model.layers] == [40, 0, 40, 0]
    eng = LLMEngine(model, max_batch=2, max_seq_len=256, prefill_chunk=64)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (150, 47)]
    out = eng.generate(prompts, max_tokens=6)
    ops.check_status()
    for p, got in zip(prompts, out):
        logits, kv = model.forward_reference(torch.tensor(p, device=dev))
        cur = logits[-1]
        for step in range(6):
            top2 = torch.topk(cur.float(), 2)
            want = int(top2.indices[0])
            if got[step] != want:
                assert float(top2.values[0] - top2.values[1]) < 0.05, f"step {step}: got {got[step]} want {want}"
                break
            logits, kv = model.forward_reference(torch.tensor([want], device=dev), start_pos=len(p) + step, kv=kv)
            cur = logits[-1]
    # the window matters: the same weights without it decode differently somewhere
    cfg2 = DenseConfig.tiny(hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, layers=4, attn_sinks=sinks)
    model2 = DenseModel.random_init(cfg2, device=dev, seed=2, std=0.05)
    l1, _ = model.forward_reference(torch.tensor(prompts[0], device=dev))
    l2, _ = model2.forward_reference(torch.tensor(prompts[0], device=dev))
    assert (l1[-1] - l2[-1]).abs().max() > 1e-3


def test_speculative_lookup_decode_equals_plain_greedy(dev):
    """Greedy speculative decoding (context-lookup drafts verified as extra rows of the decode pass) emits exactly
    the tokens of plain greedy decoding, and on a repetitive prompt most drafts are accepted."""
    from dgpp_b200.engine.adapters import KernelEngine
    from dgpp_b200.engine.llm_engine import LLMEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel
    from dgpp_b200.ops import core as ops
    from dgpp_b200.runtime import rt

    cfg = DenseConfig.tiny(hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2048, layers=2)
    model = DenseModel.random_init(cfg, device=dev, seed=0, std=0.05)
    g = torch.Generator().manual_seed(11)
    motif = torch.randint(0, cfg.vocab, (12,), generator=g).tolist()
    prompts = {"rep": motif * 8, "rnd": torch.randint(0, cfg.vocab, (70,), generator=g).tolist()}

    def run(spec):
        eng = KernelEngine(LLMEngine(model, max_batch=4, max_seq_len=512, prefill_chunk=64), spec_drafts=spec)
        s = rt.Scheduler(eng, rt.SchedulerConfig())
        for rid, p in prompts.items():
            s.submit(rid, p, 40)
        s.run(100000)
        out = {}
        for kind, rid, a, b in s.events():
            if kind == "token":
                out.setdefault(rid, []).append(a)
        ops.check_status()
        return out, s.meters(), eng

    plain, m0, _ = run(0)
    spec, m1, eng = run(3)
    assert spec == plain and all(len(v) == 40 for v in spec.values())
    assert eng.spec_proposed > 0
    # fewer decode passes than tokens when drafts land (a random-init model repeats itself often enough after a
    # repetitive prompt; the equality above is the contract, this only checks that the path is live)
    assert m1["decode_passes"] <= m0["decode_passes"]


@pytest.mark.parametrize("plen", [300, 77])
def test_prefix_cache_hit_reproduces_the_uncached_tokens(dev, plen):
    """The same prompt twice through scheduler + kernel engine: the second run attaches the cached KV blocks, prefills
    only the tail, and emits exactly the first run's tokens."""
    from dgpp_b200.engine.adapters import KernelEngine
    from dgpp_b200.engine.llm_engine import LLMEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel
    from dgpp_b200.ops import core as ops
    from dgpp_b200.runtime import rt

    cfg = DenseConfig.tiny(hidden=512, q_heads=8, kv_heads=8, head_dim=128, ffn=2048, vocab=4096, layers=2)
    model = DenseModel.random_init(cfg, device=dev, seed=0, std=0.05)
    eng = KernelEngine(LLMEngine(model, max_batch=4, max_seq_len=1024, prefill_chunk=256))
    sc = rt.SchedulerConfig()
    sc.prefix_min_tokens = 16
    s = rt.Scheduler(eng, sc)
    prompt = list(range(100, 100 + plen))
    outs = []
    for rid in ("a", "b", "c"):
        s.submit(rid, prompt, 12)
        s.run(100000)
        outs.append([a for kind, r, a, b in s.events() if kind == "token"])
    ops.check_status()
    m = s.meters()
    assert m["prefix_hit_tokens"] >= 2 * (plen // 64) * 64
    assert outs[1] == outs[0] and outs[2] == outs[0], outs
