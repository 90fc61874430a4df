"""Hybrid (GDN + full attention, dense / MoE, MTP) oracle on CPU."""
import torch

from dgpp_b200.models.hybrid import HybridConfig, HybridModel
from dgpp_b200.models.moe import MoEConfig
from dgpp_b200.runtime import rt


def _cfg(**kw):
    base = dict(layers=4, hidden=64, full_every=4, q_heads=2, kv_heads=1, head_dim=32, gdn_k_heads=1, gdn_v_heads=2,
                gdn_dk=16, gdn_dv=16, ffn=128, vocab=96)
    base.update(kw)
    return HybridConfig(**base)


def test_forward_reference_is_causal_and_deterministic():
    m = HybridModel.random_init(_cfg(), "cpu", seed=1, std=0.2)
    ids = torch.randint(0, 96, (9,))
    full = m.forward_reference(ids)
    assert full.shape == (9, 96) and torch.isfinite(full).all()
    part = m.forward_reference(ids[:5])
    assert torch.allclose(full[:5], part, atol=2e-2)           # later tokens do not change earlier logits
    assert torch.equal(full, m.forward_reference(ids))


def test_moe_variant_runs():
    m = HybridModel.random_init(_cfg(moe=MoEConfig(experts=8, top_k=2, moe_ffn=32, shared_ffn=32)), "cpu", seed=2, std=0.2)
    ids = torch.randint(0, 96, (6,))
    assert torch.isfinite(m.forward_reference(ids)).all()


def test_mtp_drafts_verified_by_target_equal_plain_greedy():
    m = HybridModel.random_init(_cfg(mtp=True), "cpu", seed=3, std=0.3)
    prompt = [5, 17, 3, 5, 17, 3, 5]

    def greedy(n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(m.forward_reference(torch.tensor(seq))[-1].argmax()))
        return seq

    plain = greedy(12)
    seq, passes, proposed, accepted = list(prompt), 0, 0, 0
    # bootstrap: one target pass gives the first token and the hidden states for the MTP head
    logits, hidden = m.forward_reference(torch.tensor(seq), return_hidden=True)
    seq.append(int(logits[-1].argmax()))
    passes += 1
    while len(seq) < len(plain):
        # draft x_{t+2} from (hidden_t, x_{t+1}) at the last position
        ml = m.mtp_reference(hidden[-1:], torch.tensor(seq[-1:]))
        draft = [int(ml[-1].argmax())]
        logits, hid = m.forward_reference(torch.tensor(seq + draft), return_hidden=True)
        passes += 1
        picks = logits[-2:].argmax(-1).tolist()                 # target picks after seq and after seq + draft
        acc, emitted, keep = rt.spec_judge(len(seq) - 1, draft, picks, budget=len(plain) - len(seq))
        proposed += 1
        accepted += acc
        seq += emitted
        hidden = hid[:len(seq) - 1]                             # hidden of the last COMMITTED input row
    assert seq == plain
    assert passes <= 12
