"""Low-rank adapter kernel and the adapted decode path on the GPU against PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


@pytest.mark.parametrize("rows,n,k,r", [(1, 512, 256, 8), (8, 5120, 5120, 16), (37, 1000, 17408, 64), (130, 384, 1024, 3)])
def test_lora_apply_matches_reference(rows, n, k, r):
    from dgpp_b200.adapters.lora import lora_reference
    from dgpp_b200.ops import core as ops
    g = torch.Generator(device="cuda").manual_seed(rows + n)
    x = torch.randn(rows, k, device="cuda", generator=g).to(BF)
    a = (torch.randn(r, k, device="cuda", generator=g) * 0.05).to(BF)
    b = (torch.randn(n, r, device="cuda", generator=g) * 0.05).to(BF)
    big = torch.randn(rows, n + 64, device="cuda", generator=g).to(BF)
    out = big[:, 32:32 + n]                                   # a column slice: row stride != n
    want = lora_reference(x, a, b, out, 0.5)
    before = big.clone()
    ops.lora_apply(x, a, b, out, 0.5)
    torch.cuda.synchronize()
    ops.check_status()
    err = (out.float() - want.float()).abs().max().item()
    scale = want.float().abs().max().item()
    assert err <= 2 ** -7 * scale + 1e-6, (err, scale)      # one bf16 rounding of the sum
    assert torch.equal(big[:, :32], before[:, :32]) and torch.equal(big[:, 32 + n:], before[:, 32 + n:])
    # run-to-run identical
    out2 = before[:, 32:32 + n].clone()
    ops.lora_apply(x, a, b, out2, 0.5)
    assert torch.equal(out2, out)


def test_engine_with_adapter_follows_the_adapted_reference():
    from dgpp_b200.adapters import lora
    from dgpp_b200.engine.llm_engine import LLMEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel
    cfg = DenseConfig.tiny(hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2048, layers=2)
    m = DenseModel.random_init(cfg, device="cuda", seed=0, std=0.05)
    t = lora.random_adapter_tensors(cfg, 8, ["q_proj", "v_proj", "o_proj", "up_proj", "down_proj"], seed=4, std=0.2)
    ad = lora.bind_adapter(t, cfg, 8, 16.0, "cuda")
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    eng = LLMEngine(m, max_batch=2, max_seq_len=256, prefill_chunk=64)
    plain = eng.generate([prompt], max_tokens=8)[0]
    eng.set_adapter(ad)
    adapted = eng.generate([prompt], max_tokens=8)[0]
    eng.set_adapter(None)
    again = eng.generate([prompt], max_tokens=8)[0]
    assert again == plain and adapted != plain               # the adapter changes the output and comes off cleanly
    # teacher-forced: at every step the engine's token is (near-)optimal under the adapted reference model
    toks = torch.tensor(prompt + adapted[:-1], device="cuda")
    logits, _ = m.forward_reference(toks, lora=ad)
    logits = logits[len(prompt) - 1:].float()
    for i, tok in enumerate(adapted):
        top = logits[i].max().item()
        assert logits[i, tok].item() >= top - 0.35 * (logits[i].std().item()), (i, tok)
