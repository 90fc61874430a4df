"""KDA + MLA + hyper-connection family oracle on CPU: causality per mixer kind, stream bookkeeping."""
import torch

from dgpp_b200.models.glm_flash import GlmFlashConfig, GlmFlashModel
from dgpp_b200.models.moe import MoEConfig


def _cfg(**kw):
    base = dict(layers=2, hidden=256, vocab=512, k_heads=2, v_heads=2, dk=64, dv=64, heads=4, q_lora=128, kv_lora=64,
                nope=32, rope=16, v_dim=32, ffn=512)
    base.update(kw)
    return GlmFlashConfig(**base)


def test_oracle_is_causal_for_recurrent_and_latent_layers():
    toks = torch.randint(0, 512, (14,), generator=torch.Generator().manual_seed(0))
    for kw in (dict(mla_every=100), dict(mla_every=1), dict(mla_every=2, moe=MoEConfig(hidden=256, experts=8, top_k=2,
                                                                                        moe_ffn=128, shared_ffn=128))):
        m = GlmFlashModel.random_init(_cfg(**kw), "cpu", seed=1)
        full, part = m.forward_reference(toks), m.forward_reference(toks[:9])
        assert torch.isfinite(full).all() and full.shape == (14, 512)
        assert (full[:9] - part).abs().max().item() < 0.02 * full.abs().max().item(), kw     # bf16 rounding flips only


def test_layer_pattern_and_projection_widths():
    c = _cfg(layers=8, mla_every=4)
    assert [c.is_mla(i) for i in range(8)] == [False, False, False, True] * 2
    assert c.conv_channels == 2 * 2 * 64 + 2 * 64 and c.kda_cols == c.conv_channels + 2 * 64 + 2 + 2 * 64
    m = GlmFlashModel.random_init(c, "cpu", seed=2)
    assert sum(L.kda is not None for L in m.layers) == 6 and sum(L.mla is not None for L in m.layers) == 2
    assert m.layers[0].att_hc.fn.shape == ((2 + c.streams) * c.streams, c.streams * c.hidden)
