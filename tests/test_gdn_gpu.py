"""Gated DeltaNet layer: CUDA kernels against the token-by-token PyTorch oracle; prefill in chunks and single-token
decode carry the same state."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


@pytest.mark.parametrize("hk,hv,dk,dv", [(2, 4, 128, 128), (4, 4, 64, 64), (2, 8, 128, 64)])
def test_gdn_layer_matches_reference_and_carries_state(dev, hk, hv, dk, dv):
    from dgpp_b200.models.gdn import GdnConfig, GdnLayer, GdnState, GdnWeights, gdn_reference
    from dgpp_b200.ops import core as ops

    torch.manual_seed(7)
    cfg = GdnConfig(hidden=512, k_heads=hk, v_heads=hv, dk=dk, dv=dv)
    w = GdnWeights.random_init(cfg, dev, seed=3)
    T = 37
    x = torch.randn(T, cfg.hidden, device=dev).to(BF)
    conv_ref = torch.zeros(cfg.conv_width - 1, cfg.conv_channels, device=dev)
    ssm_ref = torch.zeros(hv, dk, dv, device=dev)
    want = gdn_reference(x, w, conv_ref, ssm_ref)
    layer = GdnLayer(w, 64, dev)
    st = GdnState(cfg, 3, dev)
    out = torch.empty(T, cfg.hidden, dtype=BF, device=dev)
    # prefill 20 tokens in two chunks into slot 1, then 17 single-token decode steps batched with another slot
    layer.forward(x[:12], st, out[:12], slot=1)
    layer.forward(x[12:20], st, out[12:20], slot=1)
    rs = torch.tensor([1, 2], dtype=torch.int32, device=dev)
    tmp = torch.empty(2, cfg.hidden, dtype=BF, device=dev)
    for t in range(20, T):
        xb = torch.stack([x[t], x[(t * 7) % T]])
        layer.forward(xb, st, tmp, row_slot=rs)
        out[t] = tmp[0]
    torch.cuda.synchronize()
    ops.check_status()
    scale = want.float().abs().max().item()
    assert (out.float() - want.float()).abs().max().item() <= 3e-2 * scale
    assert (st.ssm[1] - ssm_ref).abs().max().item() <= 2e-2 * ssm_ref.abs().max().item() + 1e-4
    assert (st.conv[1] - conv_ref).abs().max().item() <= 4e-2          # one bf16 step of the projection output
    assert st.ssm[0].abs().max().item() == 0.0            # untouched slot
