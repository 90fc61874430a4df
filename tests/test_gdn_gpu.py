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


@pytest.mark.parametrize("dk,hk,hv", [(128, 2, 4), (64, 4, 4)])
def test_kda_per_channel_decay_recurrence(dev, dk, hk, hv):
    """KDA form of the delta rule (decay per key channel): prefill run, batched decode rows and runs with per-row
    snapshots against the fp32 oracle."""
    from dgpp_b200.ops import core as ops, reference as ref

    torch.manual_seed(21)
    T, dv, slots = 37, 128, 3
    g = lambda *s: torch.randn(*s, device=dev)
    q, k, v = g(T, hk * dk).to(BF), g(T, hk * dk).to(BF), g(T, hv * dv).to(BF)
    gate, beta = g(T, hv * dk).to(BF), g(T, hv).to(BF)
    A_log, dt_bias = torch.log(torch.rand(hv, device=dev) * 2 + 0.5), g(hv * dk) * 0.5
    lb = -5.0
    state = torch.zeros(slots, hv, dk, dv, device=dev)
    state[1] = g(hv, dk, dv) * 0.1
    want_state = state[1].clone()
    want = ref.kda_recurrent(q, k, v, gate, beta, A_log, dt_bias, lb, want_state, hk, hv, dk, dv)
    out = torch.empty(T, hv * dv, dtype=BF, device=dev)
    ops.kda_recurrent(q, k, v, gate, beta, A_log, dt_bias, lb, state, out, hk, hv, dk, dv, slot=1, sequential=True)
    torch.cuda.synchronize()
    ops.check_status()
    assert (out.float() - want.float()).abs().max().item() <= 2e-2 * want.float().abs().max().item() + 1e-3
    assert (state[1] - want_state).abs().max().item() <= 1e-3 * want_state.abs().max().item() + 1e-4
    # runs of 4 rows for two requests with per-row snapshots: snapshot j equals the state after j + 1 tokens
    state2 = torch.zeros(slots, hv, dk, dv, device=dev)
    rows = torch.tensor([2, 2, 2, 2, 0, 0, 0, 0], dtype=torch.int32, device=dev)
    snap = torch.zeros(8, hv, dk, dv, device=dev)
    out2 = torch.empty(8, hv * dv, dtype=BF, device=dev)
    ops.kda_recurrent(q[:8], k[:8], v[:8], gate[:8], beta[:8], A_log, dt_bias, lb, state2, out2, hk, hv, dk, dv,
                      row_slot=rows, sequential=False, seg=4, snap=snap)
    torch.cuda.synchronize()
    s_ref = torch.zeros(hv, dk, dv, device=dev)
    w1 = ref.kda_recurrent(q[:2], k[:2], v[:2], gate[:2], beta[:2], A_log, dt_bias, lb, s_ref, hk, hv, dk, dv)
    assert (snap[1] - s_ref).abs().max().item() <= 1e-3 * s_ref.abs().max().item() + 1e-4
    assert (out2[:2].float() - w1.float()).abs().max().item() <= 2e-2 * w1.float().abs().max().item() + 1e-3
    assert torch.equal(state2[2], snap[3]) and torch.equal(state2[0], snap[7])
