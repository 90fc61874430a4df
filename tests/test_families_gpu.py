"""Looped-hypersphere and gated-residual families on the GPU: kernel runners against their PyTorch oracles."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def _drive(r, m, vocab, dev, close):
    """Two requests: chunked prefill, batched teacher-forced decode through the graph, reset and repeat."""
    from dgpp_b200.ops import core as ops

    g = torch.Generator().manual_seed(2)
    a = torch.randint(0, vocab, (110,), generator=g).tolist()
    b = torch.randint(0, vocab, (37,), generator=g).tolist()
    la = r.prefill(1, a[:100], chunk=64).clone()
    lb = r.prefill(0, b[:30], chunk=16).clone()
    want_a = m.forward_reference(torch.tensor(a, device=dev))
    want_b = m.forward_reference(torch.tensor(b, device=dev))
    torch.cuda.synchronize()
    ops.check_status()
    close(la[-1], want_a[99], "prefill a")
    close(lb[-1], want_b[29], "prefill b")
    for s in range(4):
        out = r.decode([1, 0], [a[100 + s], b[30 + s]])
        close(out[0], want_a[100 + s], f"decode a {s}")
        close(out[1], want_b[30 + s], f"decode b {s}")
    assert r.lengths[:2] == [34, 104]
    torch.cuda.synchronize()
    ops.check_status()
    r.reset(0)
    assert torch.equal(r.prefill(0, b[:30], chunk=16), lb)


def test_dory_loops_on_the_hypersphere(dev):
    from dgpp_b200.models.dory import DoryConfig, DoryModel, DoryRunner

    cfg = DoryConfig(layers=2, loops=3, hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2048)
    m = DoryModel.random_init(cfg, dev, seed=4)
    r = DoryRunner(m, max_rows=64, slots=2, max_seq_len=256, device=dev)
    assert len(r.kv.layers) == 6                     # one cache layer per (loop, layer)

    def close(got, want, what):
        err = (got - want).abs().max().item()
        assert err <= 0.06 * want.abs().max().item() + 0.02, (what, err)

    _drive(r, m, cfg.vocab, dev, close)


@pytest.mark.parametrize("moe", [False, True])
def test_flash_next_gated_residual_branches(dev, moe):
    from dgpp_b200.models.flash_next import FlashNextConfig, FlashNextModel, FlashNextRunner
    from dgpp_b200.models.moe import MoEConfig

    cfg = FlashNextConfig(layers=4, hidden=512, full_every=2, hc=4, gr_rank=128, q_heads=4, kv_heads=2, head_dim=128,
                          gdn_k_heads=2, gdn_v_heads=4, ffn=1024, vocab=2048, ple_rows=1024,
                          moe=MoEConfig(hidden=512, experts=16, top_k=2, moe_ffn=512, shared_ffn=512) if moe else None)
    m = FlashNextModel.random_init(cfg, dev, seed=5)
    r = FlashNextRunner(m, max_rows=64, slots=2, max_seq_len=256, device=dev)

    def close(got, want, what):
        if moe:
            cos = torch.nn.functional.cosine_similarity(got.float(), want.float(), dim=0).item()
            assert cos >= 0.985, (what, cos)
            return
        err = (got - want).abs().max().item()
        assert err <= 0.06 * want.abs().max().item() + 0.02, (what, err)

    _drive(r, m, cfg.vocab, dev, close)
    assert r.last_token[1] != 0                      # the bigram hash carries over between passes


def test_family_runner_behind_the_scheduler(dev):
    """The generic runner adapter: three concurrent requests through the scheduler emit the tokens the runner emits for
    each request alone."""
    from dgpp_b200.engine.adapters import RunnerEngine
    from dgpp_b200.models.dory import DoryConfig, DoryModel, DoryRunner
    from dgpp_b200.ops import core as ops
    from dgpp_b200.runtime import rt

    cfg = DoryConfig(layers=2, loops=2, hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2048)
    m = DoryModel.random_init(cfg, dev, seed=6)
    g = torch.Generator().manual_seed(5)
    reqs = {f"r{i}": torch.randint(0, cfg.vocab, (20 + 33 * i,), generator=g).tolist() for i in range(3)}
    want = {}
    for rid, p in reqs.items():
        one = DoryRunner(m, max_rows=64, slots=1, max_seq_len=512, device=dev)
        tok = int(torch.argmax(one.prefill(0, p, chunk=64)[-1]))
        seq = [tok]
        for _ in range(5):
            tok = int(torch.argmax(one.decode([0], [tok])[0]))
            seq.append(tok)
        want[rid] = seq
    eng = RunnerEngine(DoryRunner(m, max_rows=64, slots=3, max_seq_len=512, device=dev), max_context=384, prefill_chunk=64)
    sc = rt.SchedulerConfig()
    sc.prefix_cache = False
    s = rt.Scheduler(eng, sc)
    for rid, p in reqs.items():
        s.submit(rid, p, 6)
    s.run(100000)
    got = {}
    for kind, x, a, b in s.events():
        if kind == "token":
            got.setdefault(x, []).append(a)
    torch.cuda.synchronize()
    ops.check_status()
    assert got == want


def test_flash_next_pooled_key_sparse_attention(dev):
    """The pooled-key kernels against the oracle's kept sets, then the runner with the sparse full-attention layers:
    select_k large enough to keep every block checks the whole path under the family's bound; a small select_k drops
    blocks, where a near-tie between two blocks' scores may resolve differently, so that case is judged over all rows."""
    from dgpp_b200.engine.kv_cache import PagedKV
    from dgpp_b200.models.flash_next import FlashNextConfig, FlashNextModel, FlashNextRunner, QsaConfig, qsa_keep_reference
    from dgpp_b200.ops import core as ops
    from dgpp_b200.ops import reference as ref

    g = torch.Generator(device=dev).manual_seed(9)
    T, ih, di, page, k = 203, 4, 128, 16, 3
    kv = PagedKV(1, 1, 128, 40, 2, 16, page, True, dev)
    assert kv.reserve(1, T)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    req = torch.ones(T, dtype=torch.int32, device=dev)
    inv, _ = ref.rope_inv_freq(di, 1e4, dev)
    qn = (0.1 * torch.randn(di, device=dev, generator=g)).to(torch.bfloat16)
    kn = (0.1 * torch.randn(di, device=dev, generator=g)).to(torch.bfloat16)
    iqk0 = torch.randn(T, (ih + 1) * di, device=dev, generator=g).to(torch.bfloat16)
    iqk = iqk0.clone()
    raw, comp = torch.zeros(40, page, di, dtype=torch.bfloat16, device=dev), torch.zeros(40, di, dtype=torch.bfloat16, device=dev)
    ops.msa_index_prep(iqk, pos, req, kv.block_table, inv, qn, None, raw, ih, di, di, 1e-6, one_plus_w=True, raw_key=True)
    ops.qsa_compress(raw, comp, pos, req, kv.block_table, inv, kn, di, 1e-6, one_plus_w=True)
    sel = ops.qsa_select(iqk, comp, kv.block_table, req, pos, ih, di, page, k, 32, copies=2)
    torch.cuda.synchronize()
    ops.check_status()
    table = kv.block_table[1].long()
    assert torch.equal(raw[table[pos.long() // page], pos.long() % page], iqk0.view(T, ih + 1, di)[:, ih])     # raw keys
    assert torch.equal(iqk.view(T, ih + 1, di)[:, ih], iqk0.view(T, ih + 1, di)[:, ih])
    iq = iqk.float().view(T, ih + 1, di)[:, :ih].contiguous()
    keep = qsa_keep_reference(iq, iqk0.float().view(T, ih + 1, di)[:, ih].contiguous(), kn, inv, page, k, 1e-6)
    got = torch.zeros(T, keep.shape[1] + 1, dtype=torch.bool, device=dev)
    got.scatter_(1, torch.where(sel[:, 0] >= 0, sel[:, 0], torch.full_like(sel[:, 0], keep.shape[1])).long(), True)
    assert (got[:, :-1] != keep).any(-1).float().mean().item() <= 0.02
    assert torch.equal(sel[:, 0], sel[:, 1])
    valid = sel[:, 0] >= 0
    asc = torch.where(valid[:, 1:], sel[:, 0, 1:] > sel[:, 0, :-1], torch.ones_like(valid[:, 1:]))
    assert bool(asc.all()) and int(valid.sum(-1).max()) == k + 1

    for select_k in (16, 2):
        cfg = FlashNextConfig(layers=4, hidden=512, full_every=2, hc=4, gr_rank=128, q_heads=4, kv_heads=2, head_dim=128,
                              gdn_k_heads=2, gdn_v_heads=4, ffn=1024, vocab=2048, ple_rows=1024, page=16,
                              qsa=QsaConfig(index_heads=4, index_dim=128, select_k=select_k))
        m = FlashNextModel.random_init(cfg, dev, seed=5)
        r = FlashNextRunner(m, max_rows=64, slots=2, max_seq_len=256, device=dev)
        gg = torch.Generator().manual_seed(2)
        a = torch.randint(0, cfg.vocab, (110,), generator=gg).tolist()
        b = torch.randint(0, cfg.vocab, (40,), generator=gg).tolist()
        la = r.prefill(1, a[:100], chunk=64).clone()
        lb = r.prefill(0, b[:30], chunk=16).clone()
        want_a = m.forward_reference(torch.tensor(a, device=dev))
        want_b = m.forward_reference(torch.tensor(b, device=dev))
        cosines = []

        def close(got_l, want_l, what):
            cos = torch.nn.functional.cosine_similarity(got_l.float(), want_l.float(), dim=0).item()
            cosines.append(cos)
            if select_k >= 16:
                err = (got_l - want_l).abs().max().item()
                assert err <= 0.06 * want_l.abs().max().item() + 0.02, (what, err)

        close(la[-1], want_a[99], "prefill a")
        close(lb[-1], want_b[29], "prefill b")
        for s in range(8):
            out = r.decode([1, 0], [a[100 + s], b[30 + s]])
            close(out[0], want_a[100 + s], f"decode a {s}")
            close(out[1], want_b[30 + s], f"decode b {s}")
        torch.cuda.synchronize()
        ops.check_status()
        assert sum(1 for c in cosines if c >= 0.98) >= 0.75 * len(cosines) and min(cosines) >= 0.5, cosines


def test_family_checkpoint_round_trip_on_the_device(dev, tmp_path):
    """A written family checkpoint loads onto the GPU (expert matrices restacked for the grouped GEMM) and its runner
    gives the logits of the original model's runner bit for bit."""
    from dgpp_b200.loaders.family_io import load_family, runner_for, save_family
    from dgpp_b200.models.mimo import MimoConfig, MimoModel
    from dgpp_b200.models.moe import MoEConfig

    cfg = MimoConfig(layers=4, hidden=512, q_heads=8, kv_heads=2, swa_kv_heads=4, head_dim=128, rotary_dim=64, window=24,
                     ffn=1024, vocab=2048, moe=MoEConfig(hidden=512, experts=16, top_k=2, moe_ffn=512))
    m = MimoModel.random_init(cfg, dev, seed=8)
    save_family(m, str(tmp_path / "ck"))
    back = load_family(str(tmp_path / "ck"), dev)
    assert back.layers[1].moe.gu_q is not None
    a = torch.randint(0, cfg.vocab, (70,), generator=torch.Generator().manual_seed(1)).tolist()
    outs = []
    for model in (m, back):
        r = runner_for(model, 64, 2, 256, dev)
        lg = [r.prefill(0, a[:60], chunk=32).clone()]
        for s in range(3):
            lg.append(r.decode([0], [a[60 + s]]).clone())
        outs.append(torch.cat(lg))
    assert torch.equal(outs[0], outs[1])
