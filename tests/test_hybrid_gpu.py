"""Hybrid family on the GPU: kernel runner (GDN state + paged KV + MoE) against the PyTorch oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


@pytest.mark.parametrize("moe", [False, True])
def test_hybrid_runner_matches_reference(dev, moe):
    from dgpp_b200.models.hybrid import HybridConfig, HybridModel, HybridRunner
    from dgpp_b200.models.moe import MoEConfig
    from dgpp_b200.ops import core as ops

    cfg = HybridConfig(layers=4, hidden=512, full_every=4, q_heads=4, kv_heads=2, head_dim=128, gdn_k_heads=2,
                       gdn_v_heads=4, gdn_dk=128, gdn_dv=128, ffn=1024, vocab=2048,
                       moe=MoEConfig(experts=16, top_k=2, moe_ffn=512, shared_ffn=512) if moe else None)
    m = HybridModel.random_init(cfg, dev, seed=5, std=0.05)
    r = HybridRunner(m, max_rows=64, slots=3, max_seq_len=256, device=dev)
    g = torch.Generator().manual_seed(1)
    a = torch.randint(0, cfg.vocab, (50,), generator=g).tolist()
    b = torch.randint(0, cfg.vocab, (23,), generator=g).tolist()
    la = r.prefill(1, a[:40], chunk=16).clone()      # three chunks (the runner returns a view of its logits buffer)
    lb = r.prefill(2, b[:20], chunk=64).clone()
    want_a = m.forward_reference(torch.tensor(a, device=dev))
    want_b = m.forward_reference(torch.tensor(b, device=dev))
    torch.cuda.synchronize()
    ops.check_status()

    def close(got, want):
        return (got - want).abs().max().item() <= 0.06 * want.abs().max().item() + 0.02

    assert close(la[0], want_a[39]) and close(lb[0], want_b[19])
    # batched decode of both requests, three steps (teacher-forced with the reference tokens)
    for s in range(3):
        out = r.decode([1, 2], [a[40 + s], b[20 + s]])
        assert close(out[0], want_a[40 + s]) and close(out[1], want_b[20 + s]), s
    assert r.lengths[1] == 43 and r.lengths[2] == 23
    r.reset(1)
    assert r.lengths[1] == 0
