"""Sliding-window / global hybrid family oracle on CPU: causality, the window really limiting sliding layers, the
sink column, the draft layer's pairing."""
import torch

from dgpp_b200.models.mimo import MimoConfig, MimoModel


def _cfg(**kw):
    base = dict(layers=4, hidden=256, q_heads=4, kv_heads=1, swa_kv_heads=2, head_dim=64, rotary_dim=32, window=8,
                ffn=512, vocab=512)
    base.update(kw)
    return MimoConfig(**base)


def test_oracle_is_causal_and_kinds_follow_the_pattern():
    cfg = _cfg()
    m = MimoModel.random_init(cfg, "cpu", seed=1)
    assert [L.swa for L in m.layers] == [True, True, True, False]
    assert m.layers[0].qkv.n == (4 + 2 * 2) * 64 and m.layers[3].qkv.n == (4 + 2 * 1) * 64
    assert m.layers[0].sink is not None and m.layers[3].sink is None and m.draft_layer.swa
    t = torch.randint(0, 512, (30,), generator=torch.Generator().manual_seed(0))
    full = m.forward_reference(t)
    t2 = t.clone()
    t2[20] = (t2[20] + 3) % 512
    diff = (m.forward_reference(t2) - full).abs().max(1).values
    assert diff[:20].max().item() == 0.0 and diff[20:].min().item() > 0.0


def test_window_limits_sliding_layers_and_sink_matters():
    # sliding layers only: a change at position 2 cannot reach position 2 + layers * (window - 1) + 1 or later
    cfg = _cfg(layers=2, swa_layers=[True, True], window=4, draft=False)
    m = MimoModel.random_init(cfg, "cpu", seed=2)
    t = torch.randint(0, 512, (24,), generator=torch.Generator().manual_seed(1))
    full = m.forward_reference(t)
    t2 = t.clone()
    t2[2] = (t2[2] + 1) % 512
    diff = (m.forward_reference(t2) - full).abs().max(1).values
    reach = 2 + 2 * (4 - 1)
    assert diff[2:reach + 1].max().item() > 0.0 and diff[reach + 1:].max().item() == 0.0
    # the sink takes softmax mass: removing it changes the result
    for L in m.layers:
        L.sink = None
    assert (m.forward_reference(t) - full).abs().max().item() > 1e-3


def test_draft_layer_pairs_hidden_with_the_next_token():
    cfg = _cfg()
    m = MimoModel.random_init(cfg, "cpu", seed=3)
    t = torch.randint(0, 512, (16,), generator=torch.Generator().manual_seed(2))
    logits, hidden = m.forward_reference(t, return_hidden=True)
    assert hidden.shape == (16, 256) and hidden.dtype == torch.bfloat16
    d = m.draft_reference(hidden[:15], t[1:])
    assert d.shape == (15, 512) and bool(torch.isfinite(d).all())
    # causal in both inputs: a later next-token does not move earlier draft rows
    t3 = t.clone()
    t3[10] = (t3[10] + 7) % 512
    d3 = m.draft_reference(hidden[:15], t3[1:])
    diff = (d3 - d).abs().max(1).values
    assert diff[:9].max().item() == 0.0 and diff[9].item() > 0.0
