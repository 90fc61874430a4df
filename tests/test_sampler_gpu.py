"""Device sampler against the host oracle: identical tokens, log-probabilities and alternatives, bit for bit."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def _oracle(rt, logits_row, p, counts, pos, allowed=None, candidates=128):
    return rt.sample_reference(logits_row, p.temperature, p.top_k, p.top_p, p.min_p, p.repetition_penalty,
                               p.presence_penalty, p.frequency_penalty, p.seed, p.top_logprobs, p.logit_bias, counts, pos,
                               allowed, candidates, True)


@pytest.mark.parametrize("vocab", [1000, 4096, 151936])
def test_device_sampler_matches_oracle(dev, vocab):
    from dgpp_b200.runtime import rt
    from dgpp_b200.sampling.device import DeviceSampler, SamplingParams

    torch.manual_seed(vocab)
    rnd = random.Random(vocab)
    rows = 12
    s = DeviceSampler(vocab, rows, slots=4, device=dev)
    logits = (torch.randn(rows, vocab, device=dev) * 3.0).contiguous()
    logits[3, 17] = logits[3, 900] = logits[3].max() + 1.0          # exact tie: lowest id wins
    params = [
        SamplingParams(),                                                    # greedy
        SamplingParams(top_logprobs=5),                                      # greedy + alternatives
        SamplingParams(temperature=0.7, top_k=40, seed=1),
        SamplingParams(temperature=1.0, top_k=2, seed=2, top_logprobs=3),    # the tie row
        SamplingParams(temperature=0.9, top_p=0.9, seed=3),
        SamplingParams(temperature=1.3, min_p=0.05, seed=4, top_logprobs=20),
        SamplingParams(temperature=0.8, top_k=50, top_p=0.95, min_p=0.01, seed=5),
        SamplingParams(temperature=1.0, seed=6),                             # unfiltered: may need the host's width
        SamplingParams(temperature=0.6, top_k=20, repetition_penalty=1.3, presence_penalty=0.5, frequency_penalty=0.2, seed=7),
        SamplingParams(temperature=0.5, top_k=10, seed=8, logit_bias={5: 4.0, 77: -100.0, 123: 2.5}),
        SamplingParams(temperature=2.0, top_p=0.5, seed=9),
        SamplingParams(temperature=0.3, top_k=200, seed=10),                 # k above the candidate width
    ]
    params[3].temperature = 1.0
    slots = [-1, -1, 0, -1, 1, -1, 2, -1, 3, -1, -1, -1]
    seen = {sl: [rnd.randrange(vocab) for _ in range(50)] + [int(logits[r].argmax())] * 3
            for r, sl in enumerate(slots) if sl >= 0}
    for sl, ids in seen.items():
        s.count(sl, ids)
    positions = [100 + r for r in range(rows)]
    got = s.sample(logits, params, slots, positions, count_picks=False)
    host = logits.cpu()
    n_dev = 0
    for r in range(rows):
        counts = {}
        for i in seen.get(slots[r], []):
            counts[i] = counts.get(i, 0) + 1
        tok, lp, top, width = _oracle(rt, host[r].tolist(), params[r], counts, positions[r])
        assert got[r].token == tok, (r, got[r], tok)
        assert got[r].logprob == lp, (r, got[r].logprob, lp)
        assert [(a, b) for a, b in got[r].top] == [(a, b) for a, b in top], r
        if not params[r].greedy:
            assert got[r].on_device == (width <= 128), (r, width)
        n_dev += got[r].on_device
    assert n_dev >= 6          # unfiltered / top-p rows over a large vocabulary need the host's wider prefixes


def test_device_sampler_mask_and_counts(dev):
    from dgpp_b200.runtime import rt
    from dgpp_b200.sampling.device import DeviceSampler, SamplingParams

    vocab = 5000
    torch.manual_seed(0)
    s = DeviceSampler(vocab, 2, slots=2, device=dev)
    logits = torch.randn(2, vocab, device=dev)
    allowed = torch.zeros(2, vocab, dtype=torch.bool)
    allowed[0, 100:164] = True
    allowed[1, ::7] = True
    import numpy as np

    pad = np.zeros((2, (vocab + 31) // 32 * 32), dtype=np.uint8)
    pad[:, :vocab] = allowed.numpy()
    words = np.packbits(pad, axis=1, bitorder="little").view(np.uint32)        # bit i of word i // 32 = token i
    masks = torch.from_numpy(words.view(np.int32).copy()).to(dev)
    params = [SamplingParams(), SamplingParams(temperature=1.0, top_k=30, seed=3)]
    got = s.sample(logits, params, [0, 1], [7, 8], masks=masks)
    for r in range(2):
        tok, lp, top = rt.sample_reference(logits[r].cpu().tolist(), params[r].temperature, params[r].top_k, 1.0, 0.0, 1.0,
                                           0.0, 0.0, params[r].seed, 0, {}, {}, 7 + r, allowed[r].to(torch.uint8).tolist())
        assert got[r].token == tok and bool(allowed[r, tok])
        assert got[r].logprob == lp
    # the picks were counted for the slots
    assert int(s.counts[0, got[0].token]) == 1 and int(s.counts[1, got[1].token]) == 1


@pytest.mark.parametrize("vocab,world", [(4096, 4), (151936, 8), (1000, 2)])
def test_sharded_candidate_fold_picks_the_unsharded_tokens(dev, vocab, world):
    """Vocabulary-sharded head: per-slice candidate tables (step 1 on every slice, emulated here by running the slices one
    after the other on one GPU) folded by the merge kernel give the token of the unsharded sampler on the full row; the
    log-probability differs only by the slice-wise order of the log-sum-exp fold."""
    from dgpp_b200.sampling.device import DeviceSampler, SamplingParams

    torch.manual_seed(vocab + world)
    rows = 10
    s = DeviceSampler(vocab, rows, slots=4, device=dev)
    logits = (torch.randn(rows, vocab, device=dev) * 3.0).contiguous()
    logits[3, 17] = logits[3, vocab - 5] = logits[3].max() + 1.0         # exact tie across two slices: lowest id wins
    params = [
        SamplingParams(), SamplingParams(top_logprobs=5), SamplingParams(temperature=0.7, top_k=40, seed=1),
        SamplingParams(temperature=1.0, top_k=2, seed=2, top_logprobs=3), SamplingParams(temperature=0.9, top_p=0.9, seed=3),
        SamplingParams(temperature=1.3, min_p=0.05, seed=4, top_logprobs=20),
        SamplingParams(temperature=0.8, top_k=50, top_p=0.95, min_p=0.01, seed=5),
        SamplingParams(temperature=0.6, top_k=20, repetition_penalty=1.3, presence_penalty=0.5, frequency_penalty=0.2, seed=7),
        SamplingParams(temperature=0.5, top_k=10, seed=8, logit_bias={5: 4.0, vocab - 3: 6.0, 123: 2.5}),
        SamplingParams(temperature=0.3, top_k=100, seed=10),
    ]
    slots = [-1, -1, 0, -1, 1, -1, 2, 3, -1, -1]
    for sl in (0, 1, 2, 3):
        s.count(sl, [int(logits[slots.index(sl)].argmax())] * 3 + [7, vocab - 1])
    positions = [50 + r for r in range(rows)]
    want = s.sample(logits, params, slots, positions, count_picks=False)
    per = (vocab + world - 1) // world
    tabs = []
    for w in range(world):
        lo, hi = w * per, min(vocab, (w + 1) * per)
        c, m, n = s.local_tables(logits[:, lo:hi], lo, params, slots, positions)
        tabs.append((c.clone(), m.clone(), n.clone()))
    got = s.merge_tables(torch.stack([t[0] for t in tabs]), torch.stack([t[1] for t in tabs]),
                         torch.stack([t[2] for t in tabs]), params, slots, count_picks=False)
    for r in range(rows):
        if not (want[r].on_device and got[r].on_device):
            continue                                   # a row the candidate prefix does not resolve: host path in both
        assert got[r].token == want[r].token, (r, got[r], want[r])
        assert abs(got[r].logprob - want[r].logprob) < 1e-4, r
        assert [a for a, _ in got[r].top] == [a for a, _ in want[r].top], r
    assert sum(g.on_device for g in got) >= 8
