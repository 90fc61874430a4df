"""Mixture-of-experts block on the GPU: router kernel vs the fp32 PyTorch router, grouped NVFP4 expert GEMMs +
ordered combine vs the PyTorch oracle of the expert MLPs."""
import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


@pytest.mark.parametrize("experts,k,n_group,topk_group,router", [(64, 8, 1, 1, "sigmoid"), (128, 8, 8, 4, "sigmoid"),
                                                                 (32, 4, 1, 1, "softmax"), (256, 6, 8, 3, "sigmoid")])
def test_router_matches_reference(dev, experts, k, n_group, topk_group, router):
    from dgpp_b200.models.moe import MoEConfig, MoEWeights, route_reference
    from dgpp_b200.ops import core as ops

    torch.manual_seed(1)
    cfg = MoEConfig(hidden=1024, experts=experts, top_k=k, moe_ffn=256, n_group=n_group, topk_group=topk_group,
                    router=router, routed_scaling=2.5)
    w = MoEWeights.random_init(cfg, dev, seed=2, fmt="bf16")
    x = torch.randn(9, cfg.hidden, device=dev).to(BF)
    logits = torch.empty(9, experts, dtype=torch.float32, device=dev)
    ids, wts = ops.moe_route(x, w.gate, w.bias, k, n_group, topk_group, router == "softmax", True, 2.5, logits_out=logits)
    rid, rw, rl = route_reference(x, w)
    torch.cuda.synchronize()
    assert (logits - rl).abs().max().item() < 2e-3
    # identical expert sets wherever the fp32 summation order cannot flip a near tie
    same = (ids == rid).all(-1)
    assert same.float().mean().item() >= 0.8
    assert torch.allclose(wts[same], rw[same], rtol=2e-3, atol=1e-5)
    assert (ids[:, 1:] > ids[:, :-1]).all()                     # ascending, no duplicates


@pytest.mark.parametrize("rows,shared", [(1, 0), (8, 512), (16, 0)])
def test_moe_block_matches_reference(dev, rows, shared):
    from dgpp_b200.models.moe import MoEBlock, MoEConfig, MoEWeights, moe_reference
    from dgpp_b200.ops import core as ops

    torch.manual_seed(3)
    cfg = MoEConfig(hidden=1024, experts=32, top_k=4, moe_ffn=512, shared_ffn=shared, routed_scaling=1.5)
    w = MoEWeights.random_init(cfg, dev, seed=4, std=0.05)
    blk = MoEBlock(w, max_rows=16, device=dev, prefill_terms=3)
    x = torch.randn(rows, cfg.hidden, device=dev).to(BF)
    out = torch.empty(rows, cfg.hidden, dtype=BF, device=dev)
    blk.forward(x, out)
    torch.cuda.synchronize()
    ops.check_status()
    # the oracle uses the ids / weights the device router picked (near ties may order differently in fp32)
    want = moe_reference(x, w, ids=blk.ids[:rows].long(), wts=blk.wts[:rows])
    err = (out.float() - want.float()).abs().max().item()
    assert err <= 2e-2 * want.float().abs().max().item() + 2e-3, err
    assert int(blk.n_active) == len(set(blk.ids[:rows].flatten().tolist()))
    # the gathered (prefill-sized) path agrees as well
    big = blk.forward_gathered(x)
    assert (big.float() - want.float()).abs().max().item() <= 2e-2 * want.float().abs().max().item() + 2e-3
    # second call with other rows reuses every buffer
    x2 = torch.randn(rows, cfg.hidden, device=dev).to(BF)
    blk.forward(x2, out)
    want2 = moe_reference(x2, w, ids=blk.ids[:rows].long(), wts=blk.wts[:rows])
    assert (out.float() - want2.float()).abs().max().item() <= 2e-2 * want2.float().abs().max().item() + 2e-3


@pytest.mark.parametrize("cap,rows", [(32, 24), (32, 32), (64, 40)])
def test_wide_decode_blocks_match_the_oracle_and_the_16_row_block(dev, cap, rows):
    """Token tiles of 32 / 64 rows on the decode path (more live requests, speculative verify rows), with the large
    buffers drawn from a pool shared by two blocks: the oracle's values, and row for row the bits of the 16-row block."""
    from dgpp_b200.models.moe import MoEBlock, MoEConfig, MoEWeights, moe_reference
    from dgpp_b200.ops import core as ops

    torch.manual_seed(13)
    cfg = MoEConfig(hidden=1024, experts=32, top_k=4, moe_ffn=512, shared_ffn=512, routed_scaling=1.5)
    w = MoEWeights.random_init(cfg, dev, seed=4, std=0.05)
    w2 = MoEWeights.random_init(cfg, dev, seed=5, std=0.05)
    pool = {}
    wide, other = MoEBlock(w, max_rows=cap, device=dev, pool=pool), MoEBlock(w2, max_rows=cap, device=dev, pool=pool)
    assert wide.y.data_ptr() == other.y.data_ptr() and wide.ids.data_ptr() != other.ids.data_ptr()
    narrow = MoEBlock(w, max_rows=16, device=dev)
    x = torch.randn(rows, cfg.hidden, device=dev).to(BF)
    out = torch.empty(rows, cfg.hidden, dtype=BF, device=dev)
    other.forward(x, out)                      # leaves its values in the shared buffers
    wide.forward(x, out)
    torch.cuda.synchronize()
    ops.check_status()
    want = moe_reference(x, w, ids=wide.ids[:rows].long(), wts=wide.wts[:rows])
    err = (out.float() - want.float()).abs().max().item()
    assert err <= 2e-2 * want.float().abs().max().item() + 2e-3, err
    part = torch.empty(16, cfg.hidden, dtype=BF, device=dev)
    for o in range(0, rows, 16):
        n = min(16, rows - o)
        narrow.forward(x[o:o + n], part[:n])
        assert torch.equal(part[:n], out[o:o + n]), o
    torch.cuda.synchronize()
    ops.check_status()


def test_mxfp4_experts_stream_through_the_block_scaled_grouped_gemm(dev):
    """MXFP4 expert weights (e8m0 scale per 32) are re-expressed exactly in the block-scaled layout and run on the
    same grouped tensor-core GEMM; the oracle decodes the stored MXFP4 tensors."""
    from dgpp_b200.models.moe import MoEBlock, MoEConfig, MoEWeights, moe_reference
    from dgpp_b200.ops import core as ops
    from dgpp_b200.quant.formats import mxfp4_as_nvfp4

    torch.manual_seed(5)
    cfg = MoEConfig(hidden=1024, experts=16, top_k=4, moe_ffn=512, shared_ffn=512, routed_scaling=1.0)
    w = MoEWeights.random_init(cfg, dev, seed=6, std=0.05, fmt="mxfp4")
    assert w.experts_gu[0].fmt == "mxfp4" and w.gu_q is not None
    conv = mxfp4_as_nvfp4(w.experts_down[3])
    assert torch.equal(conv.dequant(), w.experts_down[3].dequant())          # value for value
    assert conv.payload.data_ptr() == w.experts_down[3].payload.data_ptr()   # the code bytes are not copied
    blk = MoEBlock(w, max_rows=16, device=dev)
    x = torch.randn(8, cfg.hidden, device=dev).to(BF)
    out = torch.empty(8, cfg.hidden, dtype=BF, device=dev)
    blk.forward(x, out)
    torch.cuda.synchronize()
    ops.check_status()
    want = moe_reference(x, w, ids=blk.ids[:8].long(), wts=blk.wts[:8])
    err = (out.float() - want.float()).abs().max().item()
    assert err <= 2e-2 * want.float().abs().max().item() + 2e-3, err


@pytest.mark.parametrize("T,k,E,e0,e1", [(7, 4, 32, 0, 32), (300, 8, 64, 0, 64), (1000, 10, 512, 0, 512), (257, 6, 64, 16, 48)])
def test_segment_sort_is_a_stable_counting_sort_into_tiles(dev, T, k, E, e0, e1):
    from dgpp_b200.ops import core as ops

    g = torch.Generator().manual_seed(T)
    ids = torch.stack([torch.randperm(E, generator=g)[:k].sort().values for _ in range(T)]).to(torch.int32).to(dev)
    bn = 64
    max_tiles = (T * k + bn - 1) // bn + (e1 - e0)
    pair_row, tile_expert, n_tiles = ops.moe_segment_sort(ids, bn, max_tiles, e0, e1)
    torch.cuda.synchronize()
    ops.check_status()
    flat = ids.flatten().tolist()
    rows = pair_row.tolist()
    te = tile_expert.tolist()
    nt = int(n_tiles)
    # expected: experts in ascending order, each padded to whole tiles; pairs keep their order inside an expert
    want_rows, tile = {}, 0
    for e in range(e0, e1):
        ps = [p for p, x in enumerate(flat) if x == e]
        for r, p in enumerate(ps):
            want_rows[p] = (tile + r // bn) * bn + r % bn
        ntile = (len(ps) + bn - 1) // bn
        assert te[tile:tile + ntile] == [e - e0] * ntile
        tile += ntile
    assert nt == tile and all(x == -1 for x in te[tile:])
    for p, x in enumerate(flat):
        assert rows[p] == (want_rows[p] if e0 <= x < e1 else -1)


@pytest.mark.parametrize("rows,shared,terms,tol", [(100, 512, 3, 2e-2), (700, 0, 3, 2e-2), (700, 512, 1, 1.2e-1),
                                                   (300, 0, 2, 4e-2)])
def test_moe_prefill_path_matches_the_expert_loop(dev, rows, shared, terms, tol):
    """Prefill-sized rows through the sort + tile list + grouped block-scaled GEMMs against the per-expert host loop
    (exact W4A16 GEMMs) and, on a few rows, against the PyTorch oracle.  terms = residual NVFP4 terms of the activations:
    1 is plain W4A4 (4-bit activation error), 3 is the decode path's near-bf16 form."""
    from dgpp_b200.models.moe import MoEBlock, MoEConfig, MoEWeights, moe_reference
    from dgpp_b200.ops import core as ops

    torch.manual_seed(7)
    cfg = MoEConfig(hidden=1024, experts=32, top_k=4, moe_ffn=512, shared_ffn=shared, routed_scaling=1.5)
    w = MoEWeights.random_init(cfg, dev, seed=8, std=0.05)
    blk = MoEBlock(w, max_rows=16, device=dev, prefill_terms=terms)
    x = torch.randn(rows, cfg.hidden, device=dev).to(BF)
    got = blk.forward_gathered(x)
    got2 = blk.forward_gathered(x)
    loop = blk.forward_looped(x)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(got, got2)                                         # deterministic, buffers reusable
    scale = loop.float().abs().max().item()
    assert (got.float() - loop.float()).abs().max().item() <= tol * scale + 2e-3
    ids, wts = ops.moe_route(x[:9], w.gate, w.bias, cfg.top_k, cfg.n_group, cfg.topk_group, False, True, 1.5)
    want = moe_reference(x[:9], w, ids=ids.long(), wts=wts)
    assert (got[:9].float() - want.float()).abs().max().item() <= tol * want.float().abs().max().item() + 2e-3
