"""Latent attention kernels: dense and sparse MLA decode, lightning-indexer scores, exact top-k selection."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def _pool(dev, reqs, ctxs, page, d, seed):
    torch.manual_seed(seed)
    max_blocks = max(ctxs) // page + 2
    blocks = reqs * max_blocks + 3
    cache = (torch.randn(blocks, page, d, device=dev) * 0.5).to(BF)
    perm = torch.randperm(blocks, device=dev)[:reqs * max_blocks].view(reqs, max_blocks).to(torch.int32)
    return cache, perm


@pytest.mark.parametrize("heads,dc,dr,page,splits", [(16, 512, 64, 64, 1), (20, 512, 64, 128, 4), (8, 128, 32, 16, 3)])
def test_mla_decode_dense_and_sparse(dev, heads, dc, dr, page, splits):
    from dgpp_b200.models.mla import gather_rows, mla_reference, topk_reference
    from dgpp_b200.ops import core as ops

    ctxs = [700, 33, 257]
    cache, table = _pool(dev, 3, ctxs, page, dc + dr, seed=1)
    q = (torch.randn(3, heads, dc + dr, device=dev) * 0.3).to(BF)
    row_req = torch.tensor([0, 1, 2], dtype=torch.int32, device=dev)
    pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device=dev)
    scale = 1.0 / math.sqrt(dc // 4 + dr)
    out = ops.mla_decode(q, cache, table, row_req, pos, scale, dc, dr, splits=splits)
    torch.cuda.synchronize()
    ops.check_status()
    for r, n in enumerate(ctxs):
        want = mla_reference(q[r], gather_rows(cache, table[r], n), scale, dc)
        assert (out[r].float() - want).abs().max().item() < 1e-2
    # sparse: 64 selected positions per row
    k = 64
    sc = torch.randn(3, max(ctxs), device=dev)
    sel = torch.stack([topk_reference(sc[r, :n], k) for r, n in enumerate(ctxs)])
    out = ops.mla_decode(q, cache, table, row_req, pos, scale, dc, dr, sel=sel.contiguous(), splits=min(splits, 2))
    torch.cuda.synchronize()
    ops.check_status()
    for r, n in enumerate(ctxs):
        want = mla_reference(q[r], gather_rows(cache, table[r], n), scale, dc, sel=sel[r])
        assert (out[r].float() - want).abs().max().item() < 1e-2


@pytest.mark.parametrize("heads,page,splits,ctxs", [(32, 64, 1, [700, 33, 257, 128]), (32, 64, 4, [2048, 129, 1, 640]),
                                                    (20, 128, 3, [700, 33, 257, 500]), (40, 16, 2, [300, 64, 65, 1000])])
def test_mla_decode_tensor_cores(dev, heads, page, splits, ctxs):
    """tcgen05 latent attention (one tile feeds both products, MN-major second operand) against the fp32 oracle and the
    CUDA-core kernel; head groups of 32, partial groups, splits that fall beyond short contexts."""
    from dgpp_b200.models.mla import gather_rows, mla_reference
    from dgpp_b200.ops import core as ops

    dc, dr = 512, 64
    cache, table = _pool(dev, len(ctxs), ctxs, page, dc + dr, seed=3)
    q = (torch.randn(len(ctxs), heads, dc + dr, device=dev) * 0.3).to(BF)
    row_req = torch.arange(len(ctxs), dtype=torch.int32, device=dev)
    pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device=dev)
    scale = 1.0 / math.sqrt(128 + dr)
    out = ops.mla_decode(q, cache, table, row_req, pos, scale, dc, dr, splits=splits, tensor_cores=True)
    base = ops.mla_decode(q, cache, table, row_req, pos, scale, dc, dr, splits=splits, tensor_cores=False)
    torch.cuda.synchronize()
    ops.check_status()
    for r, n in enumerate(ctxs):
        want = mla_reference(q[r], gather_rows(cache, table[r], n), scale, dc)
        assert (out[r].float() - want).abs().max().item() < 1.5e-2, (r, n)
    assert (out.float() - base.float()).abs().max().item() < 2e-2
    # sparse form: the softmax warps gather the listed tokens themselves
    from dgpp_b200.models.mla import topk_reference
    k = 200
    sc = torch.randn(len(ctxs), max(ctxs), device=dev)
    sel = torch.stack([topk_reference(sc[r, :n], k) for r, n in enumerate(ctxs)]).contiguous()
    out = ops.mla_decode(q, cache, table, row_req, pos, scale, dc, dr, sel=sel, splits=min(splits, 2), tensor_cores=True)
    torch.cuda.synchronize()
    ops.check_status()
    for r, n in enumerate(ctxs):
        want = mla_reference(q[r], gather_rows(cache, table[r], n), scale, dc, sel=sel[r])
        assert (out[r].float() - want).abs().max().item() < 1.5e-2, ("sparse", r, n)


def test_indexer_scores_and_topk(dev):
    from dgpp_b200.models.mla import gather_rows, index_scores_reference, topk_reference
    from dgpp_b200.ops import core as ops

    ctxs = [3000, 100, 2049]
    hi, di, page = 16, 128, 64
    kidx, table = _pool(dev, 3, ctxs, page, di, seed=2)
    q = torch.randn(3, hi, di, device=dev).to(BF)
    w = torch.rand(3, hi, device=dev)
    row_req = torch.tensor([0, 1, 2], dtype=torch.int32, device=dev)
    pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device=dev)
    for tc in (False, True):                     # CUDA-core kernel, then the tcgen05 kernel (tiles of 128 tokens)
        scores = ops.dsa_index(q, w, kidx, table, row_req, pos, max(ctxs), tensor_cores=tc)
        torch.cuda.synchronize()
        ops.check_status()
        for r, n in enumerate(ctxs):
            want = index_scores_reference(q[r], w[r], gather_rows(kidx, table[r], n))
            assert torch.allclose(scores[r, :n], want, rtol=2e-3, atol=2e-2), (tc, r)
            assert torch.isinf(scores[r, n:]).all(), (tc, r)
    # ties: quantise the scores so that equal values exist
    scores = (scores * 2).round() / 2
    k = 512
    got = ops.topk_select(scores, pos, k)
    torch.cuda.synchronize()
    ops.check_status()
    for r, n in enumerate(ctxs):
        assert torch.equal(got[r], topk_reference(scores[r, :n], k)), r
