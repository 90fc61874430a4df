"""Sliding-window / global hybrid family on the GPU: kernel runner and draft layer against the oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


@pytest.mark.parametrize("moe", [False, True])
def test_mimo_runner_and_draft_layer_match_oracle(dev, moe):
    from dgpp_b200.models.mimo import MimoConfig, MimoModel, MimoRunner
    from dgpp_b200.models.moe import MoEConfig
    from dgpp_b200.ops import core as ops

    mc = MoEConfig(hidden=512, experts=16, top_k=2, moe_ffn=512, shared_ffn=0) if moe else None
    cfg = MimoConfig(layers=4, hidden=512, q_heads=8, kv_heads=2, swa_kv_heads=4, head_dim=128, rotary_dim=64, window=24,
                     ffn=1024, vocab=2048, moe=mc)
    m = MimoModel.random_init(cfg, dev, seed=8)
    r = MimoRunner(m, max_rows=64, slots=2, max_seq_len=256, device=dev)
    g = torch.Generator().manual_seed(3)
    a = torch.randint(0, cfg.vocab, (110,), generator=g).tolist()
    b = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    want_a, hid_a = m.forward_reference(torch.tensor(a, device=dev), return_hidden=True)
    want_b = m.forward_reference(torch.tensor(b, device=dev))
    cosines = []

    def close(got, want, what):
        cos = torch.nn.functional.cosine_similarity(got.float(), want.float(), dim=0).item()
        cosines.append(cos)
        if not moe:                      # (a near-tie in the router picks another expert: judged over all rows below)
            assert cos >= 0.985, (what, cos)
            err = (got - want).abs().max().item()
            assert err <= 0.08 * want.abs().max().item() + 0.03, (what, err)

    # request a in two chunks; the hidden rows of each chunk feed the draft layer with the tokens that follow them
    la = None
    draft_rows = []
    for lo, hi in ((0, 64), (64, 100)):
        la = r.prefill(1, a[lo:hi], chunk=64).clone()
        draft_rows.append(r.draft_rows(1, r.hidden[:hi - lo].clone(), a[lo + 1:hi + 1]).clone())
    lb = r.prefill(0, b[:30], chunk=16).clone()
    torch.cuda.synchronize()
    ops.check_status()
    close(la[-1], want_a[99], "prefill a")
    close(lb[-1], want_b[29], "prefill b")
    want_d = m.draft_reference(hid_a[:100], torch.tensor(a[1:101], device=dev))
    got_d = torch.cat(draft_rows)
    assert r.draft_len[1] == 100
    for p in (0, 30, 63, 64, 99):
        close(got_d[p], want_d[p], f"draft {p}")
    for s in range(6):
        out = r.decode([1, 0], [a[100 + s], b[30 + s]])
        close(out[0], want_a[100 + s], f"decode a {s}")
        close(out[1], want_b[30 + s], f"decode b {s}")
    torch.cuda.synchronize()
    ops.check_status()
    good = sum(1 for c in cosines if c >= 0.98)
    assert good >= 0.75 * len(cosines) and min(cosines) >= 0.5, cosines
    r.reset(0)
    assert torch.equal(r.prefill(0, b[:30], chunk=16), lb)
