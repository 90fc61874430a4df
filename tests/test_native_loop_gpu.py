"""The native decode loop (graph replays with two steps in flight, per-step pinned mailbox, stop ids, status read) emits
the tokens of the Python-driven loop."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def test_native_decode_loop_matches_python_loop_and_stops(dev):
    from dgpp_b200.engine.llm_engine import LLMEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel
    from dgpp_b200.ops import core as ops

    cfg = DenseConfig.tiny(hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2048, layers=3)
    model = DenseModel.random_init(cfg, device=dev, seed=3, std=0.05)
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (40, 17, 90)]
    eng = LLMEngine(model, max_batch=4, max_seq_len=512, prefill_chunk=64)
    want = eng.generate(prompts, max_tokens=40)
    for inflight in (1, 2, 4):
        got = eng.generate(prompts, max_tokens=40, native_loop=True, inflight=inflight)
        assert got == want, inflight
    ops.check_status()
    # stop ids: row 0 stops at its 10th token, the others run on; a row's output ends with its stop id
    stop = want[0][9]
    first = [seq.index(stop) if stop in seq[1:] or seq[0] == stop else None for seq in want]
    got = eng.generate(prompts, max_tokens=40, native_loop=True, stop_ids=[stop])
    for s, seq in enumerate(want):
        cut = next((i for i in range(1, len(seq)) if seq[i] == stop), None)
        if cut is None:
            # the loop ends once EVERY row has stopped, so a row without the stop id runs to the end
            assert got[s] == seq[:len(got[s])] and len(got[s]) >= 10
        else:
            assert got[s] == seq[:cut + 1], (s, cut)
    # the engine stays usable: bookkeeping followed the launched steps
    again = eng.generate(prompts, max_tokens=12, native_loop=True)
    assert again == [seq[:12] for seq in want]


def test_group_prefill_first_tokens_match_single_request_prefill(dev):
    """Several requests' prompt runs in one pass (rows of different requests, per-row attention): the greedy first tokens
    and the following decode tokens equal those of one-request-at-a-time prefill."""
    from dgpp_b200.engine.adapters import KernelEngine
    from dgpp_b200.engine.llm_engine import LLMEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel
    from dgpp_b200.ops import core as ops
    from dgpp_b200.runtime import rt

    cfg = DenseConfig.tiny(hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2048, layers=3)
    model = DenseModel.random_init(cfg, device=dev, seed=4, std=0.05)
    g = torch.Generator().manual_seed(9)
    prompts = {f"r{i}": torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for i, n in enumerate((150, 20, 33, 64, 9))}

    def run(group):
        keng = KernelEngine(LLMEngine(model, max_batch=6, max_seq_len=512, prefill_chunk=128))
        sc = rt.SchedulerConfig()
        sc.prefix_cache = False
        sc.prefill_budget_idle = sc.prefill_budget_busy = sc.prefill_chunk = 128
        sc.prefill_group_max = group
        s = rt.Scheduler(keng, sc)
        for rid, p in prompts.items():
            s.submit(rid, p, 6)
        s.run(100000)
        ops.check_status()
        ev = s.events()
        return {rid: [a for kind, r, a, b in ev if kind == "token" and r == rid] for rid in prompts}, s.meters()

    one, m1 = run(1)
    grp, m6 = run(6)
    assert m6["prefill_calls"] < m1["prefill_calls"] and m6["prefill_tokens"] == m1["prefill_tokens"]
    same = sum(one[r] == grp[r] for r in prompts)
    # prefill rows of a group pass take the per-row attention kernel instead of the chunk kernel: near ties may differ
    assert same >= len(prompts) - 1, (one, grp)
