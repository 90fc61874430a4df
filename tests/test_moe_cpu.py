"""Router / MoE oracle properties on CPU."""
import torch

from dgpp_b200.models.moe import MoEConfig, MoEWeights, moe_reference, route_reference


def test_route_reference_contract():
    cfg = MoEConfig(hidden=64, experts=16, top_k=4, moe_ffn=32, n_group=4, topk_group=2, routed_scaling=2.0)
    w = MoEWeights.random_init(cfg, "cpu", seed=0, fmt="bf16")
    x = torch.randn(5, 64).to(torch.bfloat16)
    ids, wts, logits = route_reference(x, w)
    assert ids.shape == (5, 4) and (ids[:, 1:] > ids[:, :-1]).all()
    # at most topk_group groups are used per token
    assert all(len({int(e) // 4 for e in row}) <= 2 for row in ids.tolist())
    # weights come from the uncorrected scores, normalised, times the scaling factor
    sc = torch.sigmoid(logits).gather(1, ids.long())
    assert torch.allclose(wts, sc / sc.sum(-1, keepdim=True) * 2.0, rtol=1e-6)
    # exact ties go to the lower expert id
    w.gate[:] = 0
    w.bias[:] = 0
    ids, wts, _ = route_reference(x, w)
    assert ids.tolist() == [[0, 1, 2, 3]] * 5          # groups 0 and 1 win the tie, then the lowest expert ids


def test_moe_reference_matches_dense_formula():
    cfg = MoEConfig(hidden=64, experts=4, top_k=2, moe_ffn=32, shared_ffn=48)
    w = MoEWeights.random_init(cfg, "cpu", seed=1, std=0.1, fmt="bf16")
    x = torch.randn(3, 64).to(torch.bfloat16)
    ids, wts, _ = route_reference(x, w)
    out = moe_reference(x, w)
    t = 1
    acc = torch.zeros(64)
    for j in range(2):
        e = int(ids[t, j])
        h = (x[t].float() @ w.experts_gu[e].dequant().t()).to(torch.bfloat16).float()
        a = (torch.nn.functional.silu(h[:32]).to(torch.bfloat16).float() * h[32:]).to(torch.bfloat16).float()
        acc += wts[t, j] * (a @ w.experts_down[e].dequant().t()).to(torch.bfloat16).float()
    h = (x[t].float() @ w.shared_gu.dequant().t()).to(torch.bfloat16).float()
    a = (torch.nn.functional.silu(h[:48]).to(torch.bfloat16).float() * h[48:]).to(torch.bfloat16).float()
    acc += (a @ w.shared_down.dequant().t()).to(torch.bfloat16).float()
    assert torch.allclose(out[t].float(), acc.to(torch.bfloat16).float(), atol=2e-2)


def test_mxfp4_is_reexpressed_exactly_in_the_block_scaled_layout():
    import torch
    from dgpp_b200.quant.formats import mxfp4_as_nvfp4, quantize
    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.02
    w[3] *= 300.0
    w[7, :64] = 0.0
    q = quantize(w, "mxfp4")
    r = mxfp4_as_nvfp4(q)
    assert r is not None and r.fmt == "nvfp4" and r.scale.numel() == 64 * 256 // 16
    assert torch.equal(r.dequant(), q.dequant())
    assert r.payload.data_ptr() == q.payload.data_ptr()
    w[9] *= 1e9                                   # more than 18 octaves between block scales: refused, not rounded
    assert mxfp4_as_nvfp4(quantize(w, "mxfp4")) is None
