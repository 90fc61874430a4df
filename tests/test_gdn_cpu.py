"""Gated DeltaNet oracle on CPU: chunked evaluation carries the state exactly; decay and write strength behave."""
import torch

from dgpp_b200.models.gdn import GdnConfig, GdnWeights, gdn_reference


def test_chunked_equals_whole_and_state_semantics():
    cfg = GdnConfig(hidden=64, k_heads=2, v_heads=4, dk=16, dv=8)
    w = GdnWeights.random_init(cfg, "cpu", seed=1)
    x = torch.randn(9, 64).to(torch.bfloat16)
    cs, ss = torch.zeros(3, cfg.conv_channels), torch.zeros(4, 16, 8)
    y = gdn_reference(x, w, cs, ss)
    cs2, ss2 = torch.zeros(3, cfg.conv_channels), torch.zeros(4, 16, 8)
    y2 = torch.cat([gdn_reference(x[:2], w, cs2, ss2), gdn_reference(x[2:3], w, cs2, ss2), gdn_reference(x[3:], w, cs2, ss2)])
    # (the CPU matmul may round differently for different row counts: states agree to fp32 noise)
    assert (y.float() - y2.float()).abs().max() < 1e-3 and torch.allclose(ss, ss2, atol=1e-5) and torch.allclose(cs, cs2, atol=1e-2)
    assert ss.abs().max() > 0
    # a large decay rate wipes the memory between tokens: the state then only holds the last token's write
    w.A_log.fill_(8.0)
    cs3, ss3 = torch.zeros(3, cfg.conv_channels), torch.zeros(4, 16, 8)
    gdn_reference(x, w, cs3, ss3)
    cs4, ss4 = cs3.clone(), torch.zeros(4, 16, 8)
    cs4[:] = 0
    hist = torch.zeros(3, cfg.conv_channels)
    gdn_reference(x[:-1], w, hist, torch.zeros(4, 16, 8))      # conv tail before the last token
    gdn_reference(x[-1:], w, hist, ss4)                         # last token alone on an empty memory
    assert torch.allclose(ss3, ss4, atol=1e-5)
