"""Session cursor over the kernel engine: piecewise feeding equals one-shot prefill, rollback re-derives the same
continuation, a fork shares full KV blocks and continues like its parent."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_session_on_the_kernel_engine():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dgpp_b200.engine.llm_engine import LLMEngine
    from dgpp_b200.engine.session import Session
    from dgpp_b200.models.dense import DenseConfig, DenseModel
    from dgpp_b200.ops import core as ops

    dev = torch.device("cuda:0")
    cfg = DenseConfig.tiny(hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2048, layers=3)
    model = DenseModel.random_init(cfg, device=dev, seed=4, std=0.05)
    eng = LLMEngine(model, max_batch=3, max_seq_len=512, prefill_chunk=128)
    p = torch.randint(0, cfg.vocab, (150,), generator=torch.Generator().manual_seed(2)).tolist()
    one = Session(eng, 0)
    first_one = one.feed(p)
    s = Session(eng, 1)
    s.feed(p[:40])
    s.feed(p[40:141])
    first = s.feed(p[141:])
    assert s.position == 150
    # chunk boundaries move with the pieces; the pick agrees unless the top two logits are a near tie
    lg = eng.runner.logits[0].float()
    assert first == first_one or (lg.topk(2).values.diff().abs().item() < 0.05 * lg.abs().max().item())
    mark = s.checkpoint()
    a = s.generate(6)
    s.rollback(mark)
    assert eng.lengths[1] == 150 and s.pending is None
    s.feed([a[0]])
    assert s.generate(5) == a[1:6]                   # the same rows recomputed over the same cache: bit-equal picks
    page = eng.kv.page
    f = s.fork(2)
    full = s.position // page
    assert f.position == s.position and eng.kv.req_blocks[2][:full] == eng.kv.req_blocks[1][:full]
    assert all(eng.kv.alloc.refcount(b) >= 2 for b in eng.kv.req_blocks[1][:full])
    ga, gb = s.generate(4), f.generate(4)
    lg = eng.runner.logits[0].float()
    assert ga[0] == gb[0] or ga == gb or lg.topk(2).values.diff().abs().item() < 0.05 * lg.abs().max().item()
    torch.cuda.synchronize()
    ops.check_status()
    for x in (one, s, f):
        x.close()
    assert eng.kv.free_blocks() == eng.kv.num_blocks
