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


def test_indexer_scores_over_fp8_keys(dev):
    """Index keys cached as e4m3 with per-token scales: the append kernel's codes and scales equal the host
    quantisation, and the tensor-core scores (two-term e4m3 queries) equal the oracle over the DEQUANTISED keys."""
    from dgpp_b200.models.mla import index_scores_reference
    from dgpp_b200.ops import core as ops

    torch.manual_seed(8)
    ctxs = [1500, 100, 513]
    hi, di, page = 64, 128, 64
    max_blocks = max(ctxs) // page + 2
    blocks = len(ctxs) * max_blocks + 3
    table = torch.randperm(blocks, device=dev)[:len(ctxs) * max_blocks].view(len(ctxs), max_blocks).to(torch.int32)
    cache = torch.zeros(blocks, page, di, dtype=torch.uint8, device=dev)
    kscale = torch.ones(blocks, page, dtype=torch.float32, device=dev)
    keys = []
    for r, n in enumerate(ctxs):
        k = (torch.randn(n, di, device=dev) * (0.2 + torch.rand(n, 1, device=dev) * 3)).to(BF)
        k[5] = 0                                                     # an all-zero key keeps scale 1
        keys.append(k)
        pos = torch.arange(n, dtype=torch.int32, device=dev)
        ops.dsa_key_append_fp8(k, pos, torch.full((n,), r, dtype=torch.int32, device=dev), table, cache, kscale)
    torch.cuda.synchronize()
    deq = []
    for r, n in enumerate(ctxs):
        k = keys[r].float()
        am = k.abs().amax(-1, keepdim=True)
        sc = torch.where(am > 0, am / 448.0, torch.ones_like(am))
        want_codes = (k / sc).to(torch.float8_e4m3fn)
        blk = table[r, torch.arange(n, device=dev) // page].long()
        got_codes = cache[blk, torch.arange(n, device=dev) % page].view(torch.float8_e4m3fn)
        # same codes but for the odd value that sits on a rounding boundary of the division (one code step at most)
        differ = got_codes.view(torch.uint8) != want_codes.view(torch.uint8)
        assert differ.float().mean().item() < 2e-3, (r, differ.float().mean().item())
        step = (got_codes.float() - want_codes.float()).abs() / want_codes.float().abs().clamp_min(2.0 ** -6)
        assert step.max().item() <= 0.13, (r, step.max().item())
        got_sc = kscale[blk, torch.arange(n, device=dev) % page]
        assert torch.allclose(got_sc, sc[:, 0], rtol=1e-6, atol=0), r          # the device divides by reciprocal
        assert float(got_sc[5]) == 1.0
        deq.append(got_codes.float() * got_sc.unsqueeze(-1))
    q = torch.randn(len(ctxs), hi, di, device=dev).to(BF)
    w = torch.rand(len(ctxs), hi, device=dev)
    row_req = torch.arange(len(ctxs), dtype=torch.int32, device=dev)
    pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device=dev)
    scores = ops.dsa_index(q, w, cache, table, row_req, pos, max(ctxs), k_scale=kscale)
    torch.cuda.synchronize()
    ops.check_status()
    for r, n in enumerate(ctxs):
        want = index_scores_reference(q[r], w[r], deq[r])
        err = (scores[r, :n] - want).abs().max().item()
        assert err <= 6e-3 * want.abs().max().item() + 2e-2, (r, err, want.abs().max().item())
        assert torch.isinf(scores[r, n:]).all(), r
