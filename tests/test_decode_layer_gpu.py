"""Persistent decode-layer kernel (csrc/kernels/decode_layer.cu) against the per-operator launch sequence.

The kernel keeps the rounding points and reduction orders of the stand-alone kernels, so with the same split-K
partition a decode step through it reproduces their logits bit for bit; where the partitions differ the logits
agree to fp32 summation order.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


def _engines(dev, max_batch, **cfg_kw):
    from dgpp_b200.engine.llm_engine import LLMEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel

    base = dict(layers=3, hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=768, vocab=4096)
    base.update(cfg_kw)
    cfg = DenseConfig.tiny(**base)
    model = DenseModel.random_init(cfg, device=dev, seed=0, std=0.05)
    mk = lambda fused, graphs: LLMEngine(model, max_batch=max_batch, max_seq_len=256, prefill_chunk=64,
                                         fused_decode=fused, use_graphs=graphs)
    return cfg, model, mk


def _run(eng, prompts, steps):
    """Prefill, then `steps` decode steps; returns the per-step logits (clones) and picked ids."""
    b = len(prompts)
    for s in range(b):
        eng.kv.release(s)
    firsts = torch.zeros(b, dtype=torch.int32, device=eng.dev)
    for s, p in enumerate(prompts):
        assert eng.kv.reserve(s, len(p) + steps + 2)
        firsts[s:s + 1].copy_(eng.prefill(s, p))
    eng.start_decode(list(range(b)), firsts)
    logits, ids = [], []
    for _ in range(steps):
        eng.decode_step(b)
        torch.cuda.synchronize()
        logits.append(eng.runner.logits[:b].clone())
        ids.append(eng.d_tokens[:b].clone())
    return logits, ids


@pytest.mark.parametrize("rows,att_splits", [(5, None), (1, None), (3, 1)])
def test_fused_step_bitwise_equals_operator_sequence(dev, rows, att_splits):
    from dgpp_b200.ops import core as ops

    cfg, model, mk = _engines(dev, max_batch=rows)
    a, b = mk(False, False), mk(True, False)
    if att_splits is not None:
        a.runner.decode_splits = b.runner.decode_splits = att_splits
    assert b.runner._fused_ok(rows) and not a.runner._fused_ok(rows)
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (70, 33, 64, 17, 90)[:rows]]
    la, ia = _run(a, prompts, 5)
    lb, ib = _run(b, prompts, 5)
    ops.check_status()
    for step, (x, y) in enumerate(zip(la, lb)):
        assert torch.isfinite(y).all()
        assert torch.equal(x, y), f"step {step}: max |diff| {(x - y).abs().max().item()}"
    for x, y in zip(ia, ib):
        assert torch.equal(x, y)


def test_fused_step_in_graph_and_split_k(dev):
    """Wider projections (split-K inside the kernel differs from the operator sequence's policy): logits agree to
    summation order, greedy tokens agree away from near-ties; graph replays are deterministic."""
    from dgpp_b200.ops import core as ops

    cfg, model, mk = _engines(dev, max_batch=4, hidden=2048, q_heads=16, kv_heads=4, ffn=2048, layers=2)
    a, b = mk(False, False), mk(True, True)
    g = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (40, 33, 64, 17)]
    la, ia = _run(a, prompts, 4)
    lb, ib = _run(b, prompts, 4)
    lb2, ib2 = _run(b, prompts, 4)
    ops.check_status()
    assert b.launches_per_step() < a.runner.m.cfg.layers * 6 + 8
    for x, y in zip(lb, lb2):
        assert torch.equal(x, y)
    x, y = la[0], lb[0]
    scale = x.abs().max().item()
    assert (x - y).abs().max().item() <= 2e-2 * scale
    top2 = torch.topk(x, 2, dim=-1)
    margin = top2.values[:, 0] - top2.values[:, 1]
    same = ia[0] == ib[0]
    assert bool((same | (margin < 0.05)).all())
