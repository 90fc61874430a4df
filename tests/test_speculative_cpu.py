"""Speculative decoding control on CPU: lookup drafts, verify schedule, accept / rollback judgement, and an
end-to-end check that lookup-speculative greedy decoding of the reference model emits exactly the plain greedy
tokens while running fewer target passes."""
import torch

from dgpp_b200.runtime import rt


def test_lookup_draft_proposes_the_latest_continuation():
    d = rt.LookupDraft(2, 3)
    d.append([1, 2, 3, 4, 9, 1, 2, 3, 5, 7, 1, 2, 3])
    assert d.propose(3) == [5, 7, 1]          # the most recent "1 2 3" was followed by 5 7 1
    assert d.propose(1) == [5]
    d.push(5)
    assert d.propose(2) == [7, 1]
    e = rt.LookupDraft(2, 4)
    e.append([4, 5, 6])
    assert e.propose(4) == []                  # nothing repeats yet


def test_judge_accepts_prefix_and_counts_kept_rows():
    acc, emitted, keep = rt.spec_judge(10, [5, 6, 7], [5, 6, 9, 1])
    assert (acc, emitted, keep) == (2, [5, 6, 9], 13)          # rows at positions 10, 11, 12 stay
    acc, emitted, keep = rt.spec_judge(10, [5, 6, 7], [5, 6, 7, 8])
    assert (acc, emitted, keep) == (3, [5, 6, 7, 8], 14)
    acc, emitted, keep = rt.spec_judge(10, [5, 6, 7], [4, 0, 0, 0])
    assert (acc, emitted, keep) == (0, [4], 11)
    acc, emitted, keep = rt.spec_judge(10, [], [4])
    assert (acc, emitted, keep) == (0, [4], 11)
    # a stop token inside the accepted run ends the emission there
    acc, emitted, keep = rt.spec_judge(10, [5, 6, 7], [5, 6, 7, 8], stop_ids=[6])
    assert emitted == [5, 6] and acc == 2 and keep == 12
    # the remaining token budget caps the step
    acc, emitted, keep = rt.spec_judge(10, [5, 6, 7], [5, 6, 7, 8], budget=2)
    assert emitted == [5, 6] and keep == 12


def test_schedule_adapts():
    s = rt.VerifySchedule(0, 6, 2)
    for _ in range(5):
        s.observe(s.draft_len(), s.draft_len())
    assert s.draft_len() == 6 and s.acceptance() == 1.0
    for _ in range(30):
        s.observe(max(s.draft_len(), 1), 0)
    assert s.draft_len() == 0
    assert s.proposed_total() > s.accepted_total() > 0


def test_lookup_speculation_equals_plain_greedy():
    from dgpp_b200.models.dense import DenseConfig, DenseModel

    cfg = DenseConfig.tiny(hidden=64, q_heads=2, kv_heads=1, head_dim=32, ffn=128, vocab=64, layers=2, weight_fmt="bf16")
    model = DenseModel.random_init(cfg, device="cpu", seed=3, std=0.3)

    def target_picks(tokens, n_rows):
        """Greedy picks of the last n_rows rows of one causal pass over `tokens` (a fresh pass: the oracle has no cache)."""
        logits = model.forward_reference(torch.tensor(tokens))[0]
        return logits[-n_rows:].argmax(-1).tolist()

    prompt = [3, 9, 4, 3, 9, 4, 3, 9]
    plain = list(prompt)
    for _ in range(24):
        plain.append(target_picks(plain, 1)[0])

    seq, passes = list(prompt), 0
    draft, sched = rt.LookupDraft(2, 4), rt.VerifySchedule(0, 5, 3)
    draft.append(seq)
    while len(seq) < len(plain):
        k = sched.draft_len()
        d = draft.propose(k) if k else []
        picks = target_picks(seq + d, len(d) + 1)
        passes += 1
        acc, emitted, keep = rt.spec_judge(len(seq) - 1, d, picks, budget=len(plain) - len(seq))
        sched.observe(len(d), acc)
        seq += emitted
        draft.append(emitted)
        assert keep == len(seq) - 1 + (0 if emitted else 0) or keep <= len(seq)
    assert seq == plain
    assert passes < 24          # a tiny random model falls into loops: most drafts land


def test_confidence_scheduled_verify_depth():
    """Depth = leading drafts whose prefix survival still beats lambda * row; lambda never drops below the plain-step
    rate and follows committed tokens over modelled time; a batch shares one depth by mean survival."""
    import math

    from dgpp_b200.runtime import rt

    logit = lambda p: math.log(p / (1 - p))
    d = rt.ConfidenceDepth(base_ms=20.0, row_ms=1.0, ema=0.5)
    assert abs(d.lambda_() - 1 / 21.0) < 1e-12 and d.floor() == d.lambda_()
    conf = [logit(0.9), logit(0.8), logit(0.5), logit(0.05), logit(0.99)]
    # survivals 0.9, 0.72, 0.36, 0.018, ...; threshold 1/21 = 0.0476: three drafts pay, the fourth does not, and the
    # confident fifth behind it cannot be reached
    assert d.depth(conf) == 3
    assert d.depth(conf, accept_scale=0.5) == 2                      # 0.45, 0.18, 0.045
    assert d.depth([]) == 0 and d.depth([logit(0.01)]) == 0
    # good steps raise lambda (4 tokens over 20 + 4 rows), which shortens the depth; bad steps cannot push it under the floor
    for _ in range(20):
        d.observe(4 * 8, 4 * 8)                                      # eight requests: 32 tokens over 20 + 32 ms
    assert abs(d.lambda_() - 32 / 52.0) < 1e-3 and d.depth(conf) == 2          # threshold 0.615: 0.9, 0.72 pay, 0.36 does not
    for _ in range(60):
        d.observe(0, 4)
    assert d.lambda_() == d.floor() and d.depth(conf) == 3
    # batch: means 0.9, (0.72 + 0.09) / 2, ... against 0.0476
    sure, unsure = [logit(0.9), logit(0.8), logit(0.9)], [logit(0.9), logit(0.1), logit(0.01)]
    assert d.depth_batch([sure, unsure]) == 3 and d.depth(unsure) == 2
    hi = rt.ConfidenceDepth(base_ms=1.0, row_ms=1.0)                 # threshold 0.5
    assert hi.depth_batch([sure, unsure]) == 1 and hi.depth(sure) == 3 and hi.depth_batch([]) == 0
