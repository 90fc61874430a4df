"""Numerics contract of the dense engine on the GPU: the same prompt gives the same greedy tokens whatever the prefill
chunking, whether a position is reached by decoding or by prefilling, and whatever the decode batch width.  Decode runs
the block-scaled FP4 path on three residual NVFP4 activation terms while prefill runs the exact W4A16 kernel, so where
two paths disagree the disagreement must be a near-tie of the top two logits (margin printed, bounded); rows of one
decode batch fed the same prompt must agree exactly.
(reference rule: docs/testing.md:468-487 near-tie classification; tests/cuda/qwen35_forward_test.cpp.)
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
MARGIN = 0.05


@pytest.fixture(scope="module")
def setup():
    from dgpp_b200.models.dense import DenseConfig, DenseModel

    dev = torch.device("cuda", 0)
    cfg = DenseConfig.tiny(layers=3, hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=768, vocab=4096)
    model = DenseModel.random_init(cfg, device=dev, seed=0, std=0.05)
    g = torch.Generator().manual_seed(21)
    prompt = torch.randint(0, cfg.vocab, (300,), generator=g).tolist()
    return dev, cfg, model, prompt


def _engine(model, chunk, batch=1):
    from dgpp_b200.engine.llm_engine import LLMEngine
    return LLMEngine(model, max_batch=batch, max_seq_len=512, prefill_chunk=chunk)


def _last_logits(eng, tokens):
    eng.kv.release(0)
    assert eng.kv.reserve(0, len(tokens) + 2)
    eng.prefill(0, tokens)
    torch.cuda.synchronize()
    return eng.runner.logits[0].clone()


def _agree(a_tok, b_tok, logits, what):
    """Equal, or a near-tie between exactly these two candidates in `logits`."""
    if a_tok == b_tok:
        return 0.0
    margin = abs(float(logits[a_tok] - logits[b_tok]))
    top2 = torch.topk(logits, 2).indices.tolist()
    assert {a_tok, b_tok} == set(top2) and margin < MARGIN, f"{what}: {a_tok} vs {b_tok}, margin {margin:.4f}, top2 {top2}"
    print(f"{what}: near-tie {a_tok} / {b_tok}, margin {margin:.4f}")
    return margin


def test_prefill_chunking_gives_the_same_tokens(setup):
    dev, cfg, model, prompt = setup
    outs, logits = {}, {}
    for chunk in (64, 256, 512):
        eng = _engine(model, chunk)
        outs[chunk] = eng.generate([prompt], max_tokens=8)[0]
        logits[chunk] = _last_logits(eng, prompt)
    # prefill itself is the same exact kernel on different row groupings: first tokens and last-position logits agree
    # to accumulation order of the attention tiles
    for chunk in (64, 256):
        assert (logits[chunk] - logits[512]).abs().max().item() < 2e-2 * logits[512].abs().max().item()
        for i, (a, b) in enumerate(zip(outs[chunk], outs[512])):
            if a != b:
                ctx = prompt + outs[512][:i]
                _agree(a, b, _last_logits(_engine(model, 512), ctx), f"chunk {chunk} vs whole at token {i}")
                break


def test_decoded_position_equals_prefilled_position(setup):
    dev, cfg, model, prompt = setup
    eng = _engine(model, 512)
    toks = eng.generate([prompt], max_tokens=10)[0]
    worst = 0.0
    for i in range(1, len(toks)):
        # token i was picked by a decode step; the same position reached by prefilling prompt + tokens[:i]
        lg = _last_logits(eng, prompt + toks[:i])
        worst = max(worst, _agree(toks[i], int(lg.argmax()), lg, f"decode vs prefill at token {i}"))
    print(f"largest near-tie margin between the decode and the prefill arithmetic: {worst:.4f}")


def test_rows_of_a_decode_batch_are_identical_and_match_width_one(setup):
    dev, cfg, model, prompt = setup
    one = _engine(model, 512, batch=1).generate([prompt], max_tokens=10)[0]
    eng8 = _engine(model, 512, batch=8)
    rows = eng8.generate([prompt] * 8, max_tokens=10)
    assert all(r == rows[0] for r in rows), "rows of one batch fed the same prompt differ"
    for i, (a, b) in enumerate(zip(rows[0], one)):
        if a != b:
            lg = _last_logits(_engine(model, 512), prompt + one[:i])
            _agree(a, b, lg, f"batch 8 vs batch 1 at token {i}")
            break
