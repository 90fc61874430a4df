"""GPU numerics for the tcgen05 paths: block-scaled NVFP4 GEMM + residual-term activation quantiser, FP8
tensor-core decode attention, FP8 tensor-core prefill flash attention.  Every kernel is compared with a plain
PyTorch fp32 restatement of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


@pytest.mark.parametrize("terms,tol", [(1, 0.2), (2, 2.5e-2), (3, 3e-3)])
def test_act_quant_residual_terms_round_trip(dev, terms, tol):
    from dgpp_b200.ops import core as ops

    torch.manual_seed(1)
    x = torch.randn(8, 1024, device=dev).to(BF)
    xa = ops.act_quant_nvfp4(x, terms)
    rel = (xa.dequant() - x.float()).abs().max().item() / x.float().abs().max().item()
    assert rel < tol


@pytest.mark.parametrize("rows,bn,terms,splits,n,k", [(4, 16, 1, 1, 384, 1024), (4, 16, 3, 1, 384, 1024), (8, 16, 3, 2, 448, 2048),
                                                       (40, 64, 3, 1, 256, 1024), (100, 128, 1, 1, 256, 1024),
                                                       (300, 256, 1, 1, 384, 1024), (30, 32, 2, 2, 256, 2048),
                                                       (8, 16, 3, 5, 640, 5120), (1, 16, 3, 7, 256, 17408),
                                                       (13, 16, 3, 8, 128, 4096)])
def test_gemm_fp4_matches_fp32_reference(dev, rows, bn, terms, splits, n, k):
    from dgpp_b200.ops import core as ops, reference as ref
    from dgpp_b200.quant.formats import quantize

    torch.manual_seed(2)
    w = quantize(torch.randn(n, k, device=dev) * 0.05, "nvfp4")
    x = torch.randn(rows, k, device=dev).to(BF)
    xa = ops.act_quant_nvfp4(x, terms, bn=bn)
    y = ops.gemm_fp4(xa, w, splits=splits)
    torch.cuda.synchronize()
    ops.check_status()
    if splits > 1:
        # both split-K forms (cluster fold through distributed shared memory, workspace fold by the last CTA) add
        # the same partials in the same order: identical bits, and repeatable
        y_ws = ops.gemm_fp4(xa, w, splits=splits, cluster=False)
        y_cl = ops.gemm_fp4(xa, w, splits=splits, cluster=True)
        torch.cuda.synchronize()
        ops.check_status()
        assert torch.equal(y_cl, y) and torch.equal(y_ws, y_cl)
    # against the product of the operands the kernel actually saw (exact up to fp32 order + one bf16 rounding)
    yq = xa.dequant() @ w.dequant().t()
    assert (y.float() - yq).abs().max().item() <= 1e-2 * yq.abs().max().item()
    # against exact bf16 activations: three residual terms are bf16-grade
    if terms == 3:
        yx = ref.linear(x, w, out_fp32=True)
        assert (y.float() - yx).abs().max().item() <= 1.2e-2 * yx.abs().max().item()


def test_fused_producers_match_reference(dev):
    from dgpp_b200.ops import core as ops, reference as ref

    torch.manual_seed(3)
    H, I = 1024, 2048
    x = torch.randn(5, H, device=dev).to(BF)
    d = torch.randn(5, H, device=dev).to(BF)
    wn = (1 + 0.1 * torch.randn(H, device=dev)).to(BF)
    xr, xo = x.clone(), torch.empty_like(x)
    xa = ops.act_quant_nvfp4(xr, 3, mode="rmsnorm", delta=d, norm_w=wn, x_out=xo)
    yr, res = ref.rmsnorm(x, wn, 1e-6, d)
    assert torch.equal(xr, res)                                           # residual stream updated in place
    assert (xo.float() - yr.float()).abs().max().item() <= 0.04
    assert ((xa.dequant() - yr.float()).abs().max() / yr.float().abs().max()).item() < 1e-2
    gu = (torch.randn(5, 2 * I, device=dev) * 2).to(BF)
    ao = torch.empty(5, I, device=dev, dtype=BF)
    xa = ops.act_quant_nvfp4(gu, 3, mode="swiglu", x_out=ao)
    ar = ref.swiglu(gu)
    assert (ao.float() - ar.float()).abs().max().item() <= 0.07
    assert ((xa.dequant() - ar.float()).abs().max() / ar.float().abs().max()).item() < 1e-2


def _filled_cache(dev, hq, hkv, ctx, page, slot, d=128):
    from dgpp_b200.engine.kv_cache import PagedKV
    from dgpp_b200.ops import core as ops, reference as ref

    kv = PagedKV(1, hkv, d, max(64, 4 * (ctx // page + 2)), 4, ctx // page + 2, page, True, dev)
    inv_freq, _ = ref.rope_inv_freq(d, 1e4, dev)
    qkv = torch.randn(ctx, (hq + 2 * hkv) * d, device=dev).to(BF)
    pos = torch.arange(ctx, device=dev, dtype=torch.int32)
    req = torch.full((ctx,), slot, device=dev, dtype=torch.int32)
    assert kv.reserve(slot, ctx)
    ops.rope_kv_write(qkv, pos, req, kv.block_table, inv_freq, kv.layers[0], hq, hkv, d)
    return kv, qkv, pos, req


def _torch_attention(kv, qkv, slot, rows_pos, hq, hkv, scale, d=128):
    """fp32 attention over the dequantised cache contents for the query rows at positions rows_pos."""
    from dgpp_b200.ops import reference as ref

    cache = kv.layers[0]
    ctx = int(rows_pos.max().item()) + 1
    blocks = kv.block_table[slot].long()
    page = cache.page
    tok = torch.arange(ctx, device=qkv.device)
    blk, off = blocks[tok // page], tok % page
    k = cache.k[blk, :, off].view(torch.float8_e4m3fn).float() * cache.k_scale[blk, :, off].unsqueeze(-1)
    v = cache.v[blk, :, off].view(torch.float8_e4m3fn).float() * cache.v_scale[blk, :, off].unsqueeze(-1)
    outs = []
    for p in rows_pos.tolist():
        q = qkv[p, :hq * d].float().view(1, hq, d)
        outs.append(ref.attention(q, k[:p + 1], v[:p + 1], scale).reshape(1, hq * d))
    return torch.cat(outs)


@pytest.mark.parametrize("hq,hkv,ctx,page,splits", [(10, 2, 333, 64, 1), (10, 2, 333, 64, 2), (40, 8, 2048, 64, 4),
                                                    (8, 1, 700, 16, 2), (16, 2, 1000, 128, 3)])
def test_attn_decode_tc(dev, hq, hkv, ctx, page, splits):
    from dgpp_b200.ops import core as ops

    torch.manual_seed(4)
    kv, qkv, pos, req = _filled_cache(dev, hq, hkv, ctx, page, slot=2)
    scale = 1.0 / math.sqrt(128)
    sel = torch.tensor([ctx - 1, ctx // 2, 5], device=dev)
    q, p_, r_ = qkv[sel].contiguous(), pos[sel].contiguous(), req[sel].contiguous()
    out = ops.attn_decode_tc(q, q.stride(0), kv.layers[0], kv.block_table, r_, p_, hq, hkv, 128, scale, splits=splits)
    torch.cuda.synchronize()
    ops.check_status()
    want = _torch_attention(kv, qkv, 2, sel, hq, hkv, scale)
    assert (out.float() - want).abs().max().item() < 0.02


@pytest.mark.parametrize("hq,hkv,ctx,splits", [(40, 8, 2048, 4), (16, 2, 700, 3), (8, 8, 333, 2)])
def test_attn_combine_quant_matches_unfused(dev, hq, hkv, ctx, splits):
    """The quantiser that folds the split-KV partials itself writes the same bf16 rows and the same NVFP4 terms
    (payload, block scales, row scales) as the stand-alone combine kernel followed by the plain quantiser."""
    from dgpp_b200.ops import core as ops

    torch.manual_seed(14)
    kv, qkv, pos, req = _filled_cache(dev, hq, hkv, ctx, 64, slot=2)
    scale = 1.0 / math.sqrt(128)
    sel = torch.tensor([ctx - 1, ctx // 2, 5, ctx // 3, 64], device=dev)
    q, p_, r_ = qkv[sel].contiguous(), pos[sel].contiguous(), req[sel].contiguous()
    rows, k = sel.numel(), hq * 128
    scratch = (torch.empty(rows * hq * splits * 2, dtype=torch.float32, device=dev),
               torch.empty(rows * hq * splits * 128, dtype=torch.float32, device=dev))
    want_x = ops.attn_decode_tc(q, q.stride(0), kv.layers[0], kv.block_table, r_, p_, hq, hkv, 128, scale,
                                splits=splits, scratch=scratch)
    want = ops.act_quant_nvfp4(want_x, terms=3, bn=16, mode="plain")
    assert ops.attn_decode_tc(q, q.stride(0), kv.layers[0], kv.block_table, r_, p_, hq, hkv, 128, scale,
                              splits=splits, scratch=scratch, partials_only=True) is None
    got = ops.QuantAct(want.rows_pad, k, 3, 16, dev)
    got_x = torch.zeros(rows, k, dtype=torch.bfloat16, device=dev)
    ops.attn_combine_quant(scratch, rows, splits, hq, 128, out=got, x_out=got_x)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(got_x, want_x)
    assert torch.equal(got.g, want.g) and torch.equal(got.q, want.q) and torch.equal(got.sf, want.sf)


@pytest.mark.parametrize("hq,hkv,ctx,page,pos0,T", [(10, 2, 256, 64, 0, 256), (10, 2, 700, 64, 0, 700),
                                                   (40, 8, 1000, 64, 300, 513), (8, 2, 400, 16, 77, 200),
                                                   (4, 4, 130, 128, 1, 129)])
def test_attn_prefill_tc(dev, hq, hkv, ctx, page, pos0, T):
    from dgpp_b200.ops import core as ops

    torch.manual_seed(5)
    kv, qkv, pos, req = _filled_cache(dev, hq, hkv, ctx, page, slot=1)
    scale = 1.0 / math.sqrt(128)
    q = qkv[pos0:pos0 + T]
    out = ops.attn_prefill_tc(q, q.stride(0), kv.layers[0], kv.block_table[1], pos0, hq, hkv, 128, scale)
    torch.cuda.synchronize()
    ops.check_status()
    # spot-check rows spread over the chunk (first, tile edges, last) against fp32 attention
    rows = sorted({0, 1, min(T - 1, 127), min(T - 1, 128), T // 2, T - 1})
    want = _torch_attention(kv, qkv, 1, torch.tensor([pos0 + r for r in rows], device=dev), hq, hkv, scale)
    got = out[torch.tensor(rows, device=dev)].float()
    assert (got - want).abs().max().item() < 0.02
    # and every row against the CUDA-core decode kernel
    base = ops.attn_decode(q, q.stride(0), kv.layers[0], kv.block_table, req[pos0:pos0 + T].contiguous(),
                           pos[pos0:pos0 + T].contiguous(), hq, hkv, 128, scale, splits=1)
    assert (out.float() - base.float()).abs().max().item() < 0.03


@pytest.mark.parametrize("hq,hkv,ctx,page,splits", [(16, 2, 333, 64, 1), (16, 2, 1500, 64, 5), (8, 2, 700, 16, 2),
                                                    (4, 4, 130, 128, 3), (16, 2, 300, 64, 16)])
def test_attn_decode_tc_head_dim_256(dev, hq, hkv, ctx, page, splits):
    """head_dim 256: two 128-byte halves per K / V / q tile; splits past the end of a short context write empty partials."""
    from dgpp_b200.ops import core as ops

    torch.manual_seed(14)
    d = 256
    kv, qkv, pos, req = _filled_cache(dev, hq, hkv, ctx, page, slot=2, d=d)
    scale = 1.0 / math.sqrt(d)
    sel = torch.tensor([ctx - 1, ctx // 2, 5], device=dev)
    q, p_, r_ = qkv[sel].contiguous(), pos[sel].contiguous(), req[sel].contiguous()
    out = ops.attn_decode_tc(q, q.stride(0), kv.layers[0], kv.block_table, r_, p_, hq, hkv, d, scale, splits=splits)
    torch.cuda.synchronize()
    ops.check_status()
    want = _torch_attention(kv, qkv, 2, sel, hq, hkv, scale, d=d)
    assert (out.float() - want).abs().max().item() < 0.02


@pytest.mark.parametrize("hq,hkv,ctx,page,pos0,T", [(16, 2, 256, 64, 0, 256), (16, 2, 700, 64, 0, 700),
                                                   (8, 2, 1000, 64, 300, 513), (8, 2, 400, 16, 77, 200),
                                                   (4, 4, 130, 128, 1, 129)])
def test_attn_prefill_tc_head_dim_256(dev, hq, hkv, ctx, page, pos0, T):
    """head_dim 256 prefill kernel (two softmax sets, one per output half) against fp32 attention and the CUDA-core rows."""
    from dgpp_b200.ops import core as ops

    torch.manual_seed(15)
    d = 256
    kv, qkv, pos, req = _filled_cache(dev, hq, hkv, ctx, page, slot=1, d=d)
    scale = 1.0 / math.sqrt(d)
    q = qkv[pos0:pos0 + T]
    out = ops.attn_prefill_tc(q, q.stride(0), kv.layers[0], kv.block_table[1], pos0, hq, hkv, d, scale)
    torch.cuda.synchronize()
    ops.check_status()
    rows = sorted({0, 1, min(T - 1, 127), min(T - 1, 128), T // 2, T - 1})
    want = _torch_attention(kv, qkv, 1, torch.tensor([pos0 + r for r in rows], device=dev), hq, hkv, scale, d=d)
    got = out[torch.tensor(rows, device=dev)].float()
    assert (got - want).abs().max().item() < 0.02
    base = ops.attn_decode(q, q.stride(0), kv.layers[0], kv.block_table, req[pos0:pos0 + T].contiguous(),
                           pos[pos0:pos0 + T].contiguous(), hq, hkv, d, scale, splits=1)
    assert (out.float() - base.float()).abs().max().item() < 0.03


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("rows,n,k", [(512, 512, 1024), (700, 1024, 512), (300, 256, 2048), (2048, 5120, 1024)])
def test_pair_gemm_is_bit_identical_to_the_single_cta_kernel(fmt, rows, n, k):
    """4-bit prefill GEMM on CTA pairs (one 256 x 256 MMA tile per pair, each CTA converting its own weight rows and
    loading its own token half): same bits as the single-CTA kernel, with and without the residual add, for token
    counts that leave the second CTA's half partly or wholly outside the matrix."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dgpp_b200.ops import core as ops
    from dgpp_b200.quant.formats import random_quant_linear

    dev = torch.device("cuda:0")
    torch.manual_seed(rows + n)
    w = random_quant_linear(n, k, fmt, dev)
    x = torch.randn(rows, k, device=dev).to(torch.bfloat16)
    resid = torch.randn(rows, n, device=dev).to(torch.bfloat16)
    old = ops.PAIR_GEMM
    try:
        ops.PAIR_GEMM = False
        want, want_r = ops.gemm_tc(x, w, splits=1), ops.gemm_tc(x, w, resid=resid, splits=1)
    finally:
        ops.PAIR_GEMM = old
    got, got_r = ops.gemm_tc_pair(x, w), ops.gemm_tc_pair(x, w, resid=resid)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(got, want) and torch.equal(got_r, want_r)
    ref = (x.float() @ w.dequant().float().t())
    assert (got.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2
