"""Chunked Gated DeltaNet scan (gdn_chunk.cu) against the token-sequential kernel and an fp64 restatement of the
recurrence: same outputs and final state up to fp32 re-association, identical on a second run."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _oracle(q, k, v, alpha, beta, A_log, dt_bias, S0, hk, hv, dk, dv):
    T = q.shape[0]
    rep = hv // hk
    qf = q.double().view(T, hk, dk)
    kf = k.double().view(T, hk, dk)
    qn = (qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5).repeat_interleave(rep, 1)
    kn = (kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(rep, 1)
    g = -torch.exp(A_log.double()) * F.softplus(alpha.double() + dt_bias.double())
    b = torch.sigmoid(beta.double())
    vv = v.double().view(T, hv, dv)
    S = S0.double().clone()
    out = torch.zeros(T, hv, dv, dtype=torch.float64, device=q.device)
    for t in range(T):
        S *= torch.exp(g[t]).view(-1, 1, 1)
        u = b[t].unsqueeze(-1) * (vv[t] - torch.einsum("hkv,hk->hv", S, kn[t]))
        S += torch.einsum("hk,hv->hkv", kn[t], u)
        out[t] = torch.einsum("hkv,hk->hv", S, qn[t])
    return out.reshape(T, hv * dv), S


@pytest.mark.parametrize("T,hk,hv,dk,dv", [(64, 2, 4, 128, 128), (200, 1, 2, 128, 128), (333, 2, 2, 64, 64), (1024, 2, 4, 128, 128)])
def test_chunked_scan_matches_sequential_and_oracle(T, hk, hv, dk, dv):
    from dgpp_b200.ops import core as ops

    dev = torch.device("cuda", 0)
    torch.manual_seed(T)
    q = torch.randn(T, hk * dk, device=dev).to(BF)
    k = torch.randn(T, hk * dk, device=dev).to(BF)
    v = torch.randn(T, hv * dv, device=dev).to(BF)
    ab = torch.randn(T, 2 * hv, device=dev).to(BF)
    alpha, beta = ab[:, :hv], ab[:, hv:]
    A_log = torch.rand(hv, device=dev) * 0.5 - 1.0
    dt_bias = torch.rand(hv, device=dev) - 0.5
    S0 = (torch.randn(2, hv, dk, dv, device=dev) * 0.1).contiguous()
    want, S_want = _oracle(q, k, v, alpha, beta, A_log, dt_bias, S0[1], hk, hv, dk, dv)

    def run(chunked):
        ops.GDN_CHUNKED = chunked
        st = S0.clone()
        out = torch.empty(T, hv * dv, device=dev, dtype=BF)
        ops.gdn_recurrent(q, k, v, alpha, beta, A_log, dt_bias, st, out, hk, hv, dk, dv, slot=1, sequential=True)
        torch.cuda.synchronize()
        return out, st

    try:
        o_seq, s_seq = run(False)
        o_chk, s_chk = run(True)
        o_chk2, s_chk2 = run(True)
    finally:
        ops.GDN_CHUNKED = True
    ops.check_status()
    assert torch.equal(o_chk, o_chk2) and torch.equal(s_chk, s_chk2)            # deterministic
    assert torch.equal(s_chk[0], S0[0])                                        # other slots untouched
    scale = want.abs().max().item()
    for name, o, s in (("sequential", o_seq, s_seq), ("chunked", o_chk, s_chk)):
        assert (o.double() - want).abs().max().item() <= 1.5e-2 * scale, name     # bf16 output rounding
        assert (s[1].double() - S_want).abs().max().item() <= 2e-4 * S_want.abs().max().item() + 1e-5, name
    # the two kernels agree to fp32 re-association (well inside one bf16 step of the outputs)
    assert (o_chk.float() - o_seq.float()).abs().max().item() <= 8e-3 * scale
    assert (s_chk[1] - s_seq[1]).abs().max().item() <= 1e-4 * S_want.abs().max().item() + 1e-5
