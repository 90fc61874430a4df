"""Table routing and the block-32 Hadamard rotation (plain and int8-coded) against their PyTorch oracles, bit for bit."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def test_hadamard32_rows_bitwise_and_involution(dev):
    from dgpp_b200.ops import core as ops, reference as ref

    torch.manual_seed(1)
    x = (torch.randn(21, 1024, device=dev) * 3).to(BF)
    got = ops.hadamard32_rows(x)
    assert torch.equal(got, ref.hadamard32(x))
    # H32 / sqrt(32) is its own inverse (up to the two bf16 roundings)
    back = ops.hadamard32_rows(got)
    assert (back.float() - x.float()).abs().max().item() <= 0.05 * x.float().abs().max().item()
    # decode slot layout: every (period)-th row keeps its staged content
    y = ops.hadamard32_rows(x, period=3)
    want = ref.hadamard32(x)
    skip = torch.arange(21, device=dev) % 3 == 2
    assert torch.equal(y[skip], x[skip]) and torch.equal(y[~skip], want[~skip])


def test_hadamard32_int8_codes_bitwise(dev):
    from dgpp_b200.ops import core as ops, reference as ref

    torch.manual_seed(2)
    x = (torch.randn(9, 512, device=dev) * torch.rand(9, 1, device=dev) * 10).to(BF)
    x[4] = 0
    codes, scales = ops.hadamard32_quant_int8(x)
    wc, ws = ref.hadamard32_quant_int8(x)
    assert torch.equal(scales, ws) and torch.equal(codes, wc)


def test_moe_hash_routes(dev):
    from dgpp_b200.ops import core as ops, reference as ref

    torch.manual_seed(3)
    T, E, k, vocab = 50, 64, 6, 300
    tid2eid = torch.stack([torch.sort(torch.randperm(E, device=dev)[:k]).values for _ in range(vocab)]).to(torch.int32)
    tokens = torch.randint(0, vocab, (T,), device=dev, dtype=torch.int32)
    tokens[7] = -1                                   # padding rows read table row 0
    scores = torch.sigmoid(torch.randn(T, E, device=dev))
    for norm in (True, False):
        ids, w = ops.moe_hash_routes(tokens, tid2eid, scores, scaling=2.5, norm_topk=norm)
        wi, ww = ref.moe_hash_routes(tokens, tid2eid, scores, scaling=2.5, norm_topk=norm)
        assert torch.equal(ids, wi) and torch.allclose(w, ww, rtol=1e-6, atol=0)


def test_segment_copy_and_bounded_stream_wait(dev):
    from dgpp_b200.ops import core as ops

    torch.manual_seed(5)
    srcs = [torch.randn(n, device=dev) for n in (4, 1024, 70000, 16)]
    dsts = [torch.zeros_like(s) for s in srcs]
    ops.segment_copy(list(zip(srcs, dsts)))
    assert ops.stream_wait(5.0) is True
    for s, d in zip(srcs, dsts):
        assert torch.equal(s, d)
    # a deadline that is already over while work is queued: the wait reports "pending" instead of blocking
    a = torch.randn(8192, 8192, device=dev)
    for _ in range(20):
        a = a @ a.t() * 1e-4
    pending = ops.stream_wait(0.0)
    assert pending in (True, False)          # (True only if the queue drained before the first poll)
    assert ops.stream_wait(30.0) is True


def test_releasable_range_commit_release_keeps_addresses(dev):
    from dgpp_b200.utils.vmm import ReleasableRange

    r = ReleasableRange(64 << 20)
    try:
        g = r.granule
        assert r.size >= 64 << 20 and r.size % g == 0 and r.committed() == 0
        free0 = torch.cuda.mem_get_info()[0]
        r.commit(0, 3 * g)
        assert r.committed() == 3 * g
        a = r.tensor(0, 3 * g, torch.float32)
        a.fill_(1.5)
        assert float(a.sum()) == 1.5 * (3 * g // 4)
        ptr = a.data_ptr()
        r.release(g, g)                                    # the middle granule goes back to the device
        assert r.committed() == 2 * g
        b = r.tensor(0, g, torch.float32)
        assert b.data_ptr() == ptr and float(b[17]) == 1.5    # what stayed committed kept its contents and address
        r.commit(g, g)                                     # recommit: fresh memory at the same address
        c = r.tensor(g, g, torch.float32)
        c.zero_()
        assert float(c.sum()) == 0.0 and c.data_ptr() == ptr + g
        torch.cuda.synchronize()
        r.release(0, r.size)
        assert r.committed() == 0
        assert torch.cuda.mem_get_info()[0] >= free0 - (1 << 20)
    finally:
        r.close()


def test_ngpt_norms_and_gated_residual_kernels(dev):
    from dgpp_b200.ops import core as ops, reference as ref

    torch.manual_seed(9)
    x = (torch.randn(13, 4096, device=dev) * 2).to(BF)
    assert torch.equal(ops.justnorm(x), ref.justnorm(x))
    a, b = (torch.randn(7, 7168, device=dev)).to(BF), (torch.randn(7, 7168, device=dev) * 3).to(BF)
    alpha = (torch.rand(7168, device=dev) * 0.2).to(BF)
    got, want = ops.slerp_alpha(a, b, alpha, 1.7), ref.slerp_alpha(a, b, alpha, 1.7)
    assert (got.float() - want.float()).abs().max().item() <= 2 ** -9            # at most one bf16 ulp of a unit-norm row
    assert (got != want).float().mean().item() < 0.01
    hc, H, rows = 4, 1024, 9
    t = torch.randn(rows, 64, device=dev).to(BF) * 4
    assert torch.equal(ops.gr_gate_act(t.clone(), hc), ref.gr_gate_act(t, hc))
    logits, rn = torch.randn(rows, hc * H, device=dev).to(BF), torch.randn(rows, hc * H, device=dev).to(BF)
    gm, wm = ops.gr_mix_finish(logits, rn, hc), ref.gr_mix_finish(logits, rn, hc)
    assert (gm.float() - wm.float()).abs().max().item() <= 2 ** -7 and (gm != wm).float().mean().item() < 0.01
    R = torch.randn(rows, hc * H, device=dev).to(BF)
    w_inj, y = (torch.randn(hc, hc * H, device=dev) * 0.02).to(BF), torch.randn(rows, H, device=dev).to(BF)
    gc, wc = ops.gr_combine(R.clone(), rn, w_inj, y, hc), ref.gr_combine(R, rn, w_inj, y, hc)
    assert (gc.float() - wc.float()).abs().max().item() <= 0.07 and (gc != wc).float().mean().item() < 0.02


def test_hyper_connection_coefficients_and_fold(dev):
    from dgpp_b200.ops import core as ops, reference as ref

    torch.manual_seed(12)
    tokens, n, D = 11, 4, 1024
    streams = torch.randn(tokens, n, D, device=dev).to(BF)
    fn = (torch.randn((2 + n) * n, n * D, device=dev) * 0.05).to(BF)
    base = torch.randn((2 + n) * n, device=dev) * 0.5
    scale = torch.tensor([0.7, 1.3, 2.0], device=dev)
    col, post, comb = ops.mhc_compute(streams, fn, base, scale, iters=20)
    wcol, wpost, wcomb = ref.mhc_compute(streams, fn, base, scale, iters=20)
    assert (post.float() - wpost.float()).abs().max().item() <= 2 ** -6
    assert (comb.float() - wcomb.float()).abs().max().item() <= 2 ** -7
    assert (col.float() - wcol.float()).abs().max().item() <= 0.02 * wcol.float().abs().max().item()
    # the mixer is close to doubly stochastic after the Sinkhorn passes
    c = comb.float()
    assert (c.sum(-2) - 1).abs().max().item() < 0.02 and (c.sum(-1) - 1).abs().max().item() < 0.05
    h = torch.randn(tokens, D, device=dev).to(BF)
    got = ops.mhc_fold(streams, h, post, comb)
    want = ref.mhc_fold(streams, h, post, comb)
    assert (got.float() - want.float()).abs().max().item() <= 2 ** -5 and (got != want).float().mean().item() < 0.01
    inplace = streams.clone()
    ops.mhc_fold(inplace, h, post, comb, out=inplace)
    assert torch.equal(inplace, got)


def test_hashed_bigram_embedding_add(dev):
    """Device-side bigram hash + table gather + add against the host formula (64-bit product, modulo the table size)."""
    from dgpp_b200.ops import core as ops

    torch.manual_seed(4)
    rows, hidden, table_rows = 77, 1024, 4099
    tokens = torch.randint(0, 151936, (rows,), dtype=torch.int32, device=dev)
    prev = torch.randint(0, 151936, (rows,), dtype=torch.int32, device=dev)
    table = torch.randn(table_rows, hidden, device=dev).to(BF)
    x = torch.randn(rows, hidden, device=dev).to(BF)
    ids = (prev.long() * 1000003 + tokens.long() * 7919 + 12345) % table_rows
    want = (x.float() + table[ids].float()).to(BF)
    got = ops.ple_embed_add(tokens, prev, table, x.clone())
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(got, want)
