"""Expert-parallel all-to-all path on one GPU: a single-rank communicator loops back to itself, so dispatch, receive plan,
tile sort, return and ordered combine all run; the result must equal the single-rank prefill path bit for bit."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


@pytest.mark.parametrize("shared", [512, 0])
def test_ep_all_to_all_single_rank_equals_prefill_path(dev, shared):
    from dgpp_b200.models.moe import MoEBlock, MoEConfig, MoEWeights
    from dgpp_b200.ops import core as ops
    from dgpp_b200.parallel.ep import EpMoE

    torch.manual_seed(11)
    cfg = MoEConfig(hidden=1024, experts=16, top_k=4, moe_ffn=512, shared_ffn=shared, routed_scaling=1.5)
    w = MoEWeights.random_init(cfg, dev, seed=5, std=0.05)
    blk = MoEBlock(w, max_rows=16, device=dev, prefill_terms=3)
    ep = EpMoE(w, max_rows=128, device=dev, act_terms=3)
    try:
        for rows in (100, 7, 128, 1):                      # consecutive exchanges alternate the slot parity
            x = torch.randn(rows, cfg.hidden, device=dev).to(BF)
            got = ep.forward(x)
            want = blk.forward_gathered(x)
            torch.cuda.synchronize()
            ops.check_status()
            assert torch.equal(got, want), rows
    finally:
        ep.close()
