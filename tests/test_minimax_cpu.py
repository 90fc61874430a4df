"""Block-sparse GQA family oracle on CPU: the block selection against a direct restatement of its rule, causality,
the sparse mask really dropping tokens, and the scaled-sigmoid activation."""
import math

import torch

from dgpp_b200.models.minimax import MinimaxConfig, MinimaxModel, select_blocks_reference
from dgpp_b200.models.moe import MoEConfig
from dgpp_b200.ops import reference as ref


def _select_direct(iq, ik, block, topk):
    """Row by row, the way the rule reads: score every visible token, block maximum, own block first, best `topk`."""
    T, ih, _ = iq.shape
    nb = (T + block - 1) // block
    keep = torch.zeros(T, ih, nb, dtype=torch.bool)
    for t in range(T):
        for h in range(ih):
            blocks = t // block + 1
            sc = [-math.inf] * blocks
            for s in range(t + 1):
                sc[s // block] = max(sc[s // block], float(iq[t, h] @ ik[s]))
            sc[-1] = math.inf
            ids = sorted(range(blocks), key=lambda b: (-sc[b], b))[:topk]
            keep[t, h, ids] = True
    return keep


def test_block_selection_matches_the_rule():
    g = torch.Generator().manual_seed(3)
    iq, ik = torch.randn(70, 2, 16, generator=g), torch.randn(70, 16, generator=g)
    got = select_blocks_reference(iq, ik, block=8, topk=3)
    assert torch.equal(got, _select_direct(iq, ik, 8, 3))
    assert got.sum(-1).max().item() == 3 and got[5].sum(-1).tolist() == [1, 1]          # one block exists at row 5
    t = torch.arange(70)
    assert bool(got[t, :, t // 8].all())                                                 # the own block is always kept
    # ties go to the lower block id
    iq1, ik1 = torch.ones(40, 1, 4), torch.ones(40, 4)
    tie = select_blocks_reference(iq1, ik1, block=8, topk=2)
    assert tie[39, 0].tolist() == [True, False, False, False, True]


def _cfg(**kw):
    base = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, rotary_dim=32, index_dim=64, sparse_block=8,
                sparse_topk=2, dense_ffn=512, vocab=512)
    base.update(kw)
    return MinimaxConfig(**base)


def test_oracle_is_causal_and_sparse():
    cfg = _cfg()
    m = MinimaxModel.random_init(cfg, "cpu", seed=1)
    t = torch.randint(0, 512, (40,), generator=torch.Generator().manual_seed(0))
    full = m.forward_reference(t)
    t2 = t.clone()
    t2[30] = (t2[30] + 3) % 512
    diff = (m.forward_reference(t2) - full).abs().max(1).values
    assert diff[:30].max().item() == 0.0 and diff[30:].min().item() > 0.0
    # with every block kept the result differs: the selection really removes tokens
    dense = MinimaxModel(_cfg(sparse_topk=64), m.embed, m.layers, m.final_norm, m.head, m.inv_freq).forward_reference(t)
    assert torch.equal(dense[:16], full[:16])                  # two blocks or fewer: nothing to drop yet
    assert (dense[24:] - full[24:]).abs().max().item() > 1e-4
    # the kept set of one layer: own block + one more, future blocks never
    xn = ref.rmsnorm(ref.embed_gather(t, m.embed), m.layers[0].in_norm, cfg.eps, one_plus_w=True)[0]
    _, keep = m.attention_reference(m.layers[0], xn, torch.arange(40), return_keep=True)
    assert keep.shape == (40, 2, 5) and keep[39].sum(-1).tolist() == [2, 2] and not bool(keep[10, :, 2:].any())


def test_scaled_sigmoid_activation_and_moe_layers():
    gu = torch.tensor([[9.0, -1.0, 0.5, 2.0, 9.0, -9.0, 0.25, -0.5]]).to(torch.bfloat16)
    out = ref.swiglu(gu, 7.0, 1.702).float()
    g, u = torch.tensor([7.0, -1.0, 0.5, 2.0]), torch.tensor([7.0, -7.0, 0.25, -0.5])
    want = g * torch.sigmoid(1.702 * g) * (u + 1)
    assert torch.allclose(out[0], want, rtol=2e-2, atol=1e-2)
    assert not torch.allclose(out, ref.swiglu(gu, 7.0).float())
    moe = MoEConfig(hidden=256, experts=8, top_k=2, moe_ffn=256, shared_ffn=256, routed_scaling=2.0, swiglu_limit=7.0,
                    swiglu_alpha=1.702)
    cfg = _cfg(moe=moe, moe_layers=[False, True])
    m = MinimaxModel.random_init(cfg, "cpu", seed=2)
    assert m.layers[0].moe is None and m.layers[0].gate_up is not None and m.layers[1].moe is not None
    t = torch.randint(0, 512, (20,), generator=torch.Generator().manual_seed(1))
    out = m.forward_reference(t)
    assert out.shape == (20, 512) and bool(torch.isfinite(out).all())
