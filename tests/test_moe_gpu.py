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
    blk = MoEBlock(w, max_rows=16, device=dev)
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
