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


def test_hybrid_engine_behind_the_scheduler_with_state_snapshots(dev):
    """Requests sharing a long prefix: the second one attaches the cached KV blocks AND the recurrent-state snapshot
    taken at the cut; its tokens equal those of a run without any prefix cache."""
    from dgpp_b200.engine.adapters import HybridEngine
    from dgpp_b200.models.hybrid import HybridConfig, HybridModel, HybridRunner
    from dgpp_b200.ops import core as ops
    from dgpp_b200.runtime import rt

    cfg = HybridConfig(layers=4, hidden=512, full_every=4, q_heads=4, kv_heads=2, head_dim=128, gdn_k_heads=2,
                       gdn_v_heads=4, gdn_dk=128, gdn_dv=128, ffn=1024, vocab=2048)
    m = HybridModel.random_init(cfg, dev, seed=7, std=0.05)
    g = torch.Generator().manual_seed(3)
    shared = torch.randint(0, cfg.vocab, (300,), generator=g).tolist()
    reqs = {"a": shared + torch.randint(0, cfg.vocab, (21,), generator=g).tolist(),
            "b": shared + torch.randint(0, cfg.vocab, (35,), generator=g).tolist(),
            "c": torch.randint(0, cfg.vocab, (90,), generator=g).tolist()}

    def run(prefix: bool, order):
        r = HybridRunner(m, max_rows=64, slots=2, max_seq_len=512, device=dev)
        eng = HybridEngine(r, snapshot_every=128, prefill_chunk=64)
        sc = rt.SchedulerConfig()
        sc.prefix_cache = prefix
        sc.prefix_min_tokens = 16
        s = rt.Scheduler(eng, sc)
        out = {}
        for rid in order:                       # one after the other, so that "b" can hit what "a" published
            s.submit(rid, reqs[rid], 6)
            s.run(100000)
            for kind, x, a, b in s.events():
                if kind == "token":
                    out.setdefault(x, []).append(a)
        ops.check_status()
        return out, s.meters(), eng

    plain, m0, _ = run(False, ["a", "b", "c"])
    cached, m1, eng = run(True, ["a", "b", "c"])
    assert m0["prefix_hit_tokens"] == 0
    # the chain matches 256 + tokens (4 blocks of 64), snapshots exist at 128 and 256 -> 256 tokens are reused
    assert m1["prefix_hit_tokens"] == 256 and eng.snapshots_restored == 1 and eng.snapshots_taken >= 2
    assert cached == plain and all(len(v) == 6 for v in cached.values())


@pytest.mark.parametrize("moe,depth,P", [(False, 3, 2), (True, 2, 2), (True, 3, 5)])
def test_mtp_speculation_emits_the_plain_greedy_sequence(dev, moe, depth, P):
    """Draft with the MTP head, verify 1 + depth rows in one pass, commit / roll back on the device: the emitted tokens
    equal plain greedy decoding token for token, whatever was accepted.  Forced drafts cover full and partial accepts; five requests at depth 3 make 20 verify rows
    (the 32-row MoE blocks)."""
    from dgpp_b200.models.hybrid import HybridConfig, HybridModel, HybridRunner
    from dgpp_b200.models.moe import MoEConfig
    from dgpp_b200.ops import core as ops

    ops.PIN_SPLIT_ROWS = True
    cfg = HybridConfig(layers=4, hidden=512, full_every=4, q_heads=4, kv_heads=2, head_dim=128, gdn_k_heads=2,
                       gdn_v_heads=4, gdn_dk=128, gdn_dv=128, ffn=1024, vocab=2048, mtp=True,
                       moe=MoEConfig(experts=16, top_k=2, moe_ffn=512, shared_ffn=512) if moe else None)
    m = HybridModel.random_init(cfg, dev, seed=9, std=0.05)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (45, 70, 33, 51, 64)[:P]]
    N = 18

    plain = HybridRunner(m, max_rows=64, slots=P, max_seq_len=256, device=dev)
    want = []
    for s, p in enumerate(prompts):
        tok = int(torch.argmax(plain.prefill(s, p, chunk=32)[0]))
        seq = [tok]
        for _ in range(N + 4):
            tok = int(torch.argmax(plain.decode([s], [tok])[0]))
            seq.append(tok)
        want.append(seq)

    def run(forced):
        r = HybridRunner(m, max_rows=64, slots=P, max_seq_len=256, device=dev)
        r.enable_spec(depth)
        pend, got = [], []
        for s, p in enumerate(prompts):
            pend.append(int(torch.argmax(r.prefill(s, p, chunk=32)[0])))
            got.append([pend[-1]])
        step = 0
        while min(len(x) for x in got) < N:
            drafts = None
            if forced:
                drafts = []
                for s in range(P):
                    nxt = want[s][len(got[s]):len(got[s]) + depth]
                    nxt = nxt + [0] * (depth - len(nxt))
                    keep = (step + s) % (depth + 1)               # accept `keep` drafts, then a wrong one
                    drafts.append([t if i < keep else (t + 1) % cfg.vocab for i, t in enumerate(nxt)])
            outs = r.spec_step(list(range(P)), pend, drafts=drafts)
            for s in range(P):
                assert 1 <= len(outs[s]) <= depth + 1
                if forced:
                    assert len(outs[s]) == (step + s) % (depth + 1) + 1, (step, s, outs[s])
                got[s] += outs[s]
                pend[s] = outs[s][-1]
            step += 1
        torch.cuda.synchronize()
        ops.check_status()
        return got, r

    for forced in (True, False):
        got, r = run(forced)
        for s in range(P):
            n = min(len(got[s]), len(want[s]))
            assert got[s][:n] == want[s][:n], (forced, s)
            assert r.lengths[s] == len(prompts[s]) + len(got[s]) - 1


def test_decode_of_more_than_16_rows_uses_the_wide_blocks(dev):
    """20 live requests decode in one pass (tensor-core attention, 32-row MoE blocks): the logits of every row equal
    those of the same request decoded alone on a second runner."""
    from dgpp_b200.models.hybrid import HybridConfig, HybridModel, HybridRunner
    from dgpp_b200.models.moe import MoEConfig
    from dgpp_b200.ops import core as ops

    cfg = HybridConfig(layers=4, hidden=512, full_every=4, q_heads=4, kv_heads=2, head_dim=128, gdn_k_heads=2,
                       gdn_v_heads=4, gdn_dk=128, gdn_dv=128, ffn=1024, vocab=2048,
                       moe=MoEConfig(experts=16, top_k=2, moe_ffn=512, shared_ffn=512))
    m = HybridModel.random_init(cfg, dev, seed=5, std=0.05)
    n = 20
    many = HybridRunner(m, max_rows=64, slots=n, max_seq_len=128, device=dev)
    one = HybridRunner(m, max_rows=64, slots=1, max_seq_len=128, device=dev)
    assert len(many.moe_wide) == len(many.moe) > 0 and not one.moe_wide
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab, (9 + 3 * s,), generator=g).tolist() for s in range(n)]
    nxt = torch.randint(0, cfg.vocab, (2, n), generator=g).tolist()
    for s, p in enumerate(prompts):
        many.prefill(s, p, chunk=32)
    got = [many.decode(list(range(n)), nxt[k]).clone() for k in range(2)]
    for s in (0, 7, 19):
        one.reset(0)
        one.prefill(0, prompts[s], chunk=32)
        for k in range(2):
            want = one.decode([0], [nxt[k][s]])[0]
            assert (got[k][s] - want).abs().max().item() <= 0.03 * want.abs().max().item() + 0.02, (s, k)
    torch.cuda.synchronize()
    ops.check_status()


@pytest.mark.parametrize("moe", [False, True])
def test_decode_width_block_scaled_linears(dev, moe):
    """NVFP4 weights: decode passes of up to 16 rows run their projections block-scaled (norm kernels emit the
    three-term rows); logits stay within the oracle's tolerance, prefill keeps the exact path."""
    from dgpp_b200.models.hybrid import HybridConfig, HybridModel, HybridRunner
    from dgpp_b200.models.moe import MoEConfig
    from dgpp_b200.ops import core as ops

    cfg = HybridConfig(layers=4, hidden=512, full_every=4, q_heads=4, kv_heads=2, head_dim=128, gdn_k_heads=2,
                       gdn_v_heads=4, gdn_dk=128, gdn_dv=128, ffn=1024, vocab=2048,
                       moe=MoEConfig(hidden=512, experts=16, top_k=2, moe_ffn=512, shared_ffn=512) if moe else None)
    m = HybridModel.random_init(cfg, dev, seed=5, std=0.05, fmt="nvfp4")
    g = torch.Generator().manual_seed(1)
    a = torch.randint(0, cfg.vocab, (60,), generator=g).tolist()
    want = m.forward_reference(torch.tensor(a, device=dev))
    outs = {}
    for fp4 in (True, False):
        r = HybridRunner(m, max_rows=64, slots=2, max_seq_len=256, device=dev)
        r.decode_fp4 = fp4
        r.prefill(0, a[:50], chunk=32)
        r.prefill(1, a[:44], chunk=32)
        outs[fp4] = [r.decode([0, 1], [a[50 + s], a[44 + s]])[0].clone() for s in range(5)]
        assert bool(r.dq.bufs) == fp4
    torch.cuda.synchronize()
    ops.check_status()
    for s in range(5):
        for fp4 in (True, False):
            got, ref_row = outs[fp4][s], want[50 + s]
            if moe:
                cos = torch.nn.functional.cosine_similarity(got.float(), ref_row.float(), dim=0).item()
                assert cos >= 0.98, (fp4, s, cos)
            else:
                err = (got - ref_row).abs().max().item()
                assert err <= 0.08 * ref_row.abs().max().item() + 0.03, (fp4, s, err)
