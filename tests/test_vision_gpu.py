"""Vision tower on the GPU (tcgen05 GEMMs + the operand kernels) against its fp32 PyTorch oracle, and the image
embedding splice of the CUDA engine."""
import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def test_vision_kernels_match_torch():
    from dgpp_b200.ops import core as ops

    torch.manual_seed(0)
    x = torch.randn(37, 320, device="cuda").to(BF)
    w, b = (1 + 0.1 * torch.randn(320, device="cuda")).to(BF), (0.1 * torch.randn(320, device="cuda")).to(BF)
    want = torch.nn.functional.layer_norm(x.float(), (320,), w.float(), b.float(), 1e-6)
    assert (ops.layernorm(x, w, b, 1e-6).float() - want).abs().max() < 0.03
    res = torch.randn(37, 320, device="cuda").to(BF)
    for act, fn in ((0, lambda t: t), (1, torch.nn.functional.gelu),
                    (2, lambda t: torch.nn.functional.gelu(t, approximate="tanh"))):
        y = x.clone()
        ops.bias_act(y, b, resid=res, act=act)
        assert (y.float() - (fn(x.float() + b.float()) + res.float())).abs().max() < 0.03
    s = torch.randn(50, 128, device="cuda").to(BF) * 3
    want = torch.softmax(s[:, :100].float(), -1)
    ops.softmax_rows(s, 100)
    torch.cuda.synchronize()
    assert (s[:, :100].float() - want).abs().max() < 0.01 and (s[:, 100:] == 0).all()
    ops.check_status()


@pytest.mark.parametrize("h,w", [(56, 84), (140, 196)])
def test_vision_tower_matches_oracle(h, w):
    from dgpp_b200.models.vision import VisionConfig, VisionTower
    from dgpp_b200.ops import core as ops

    vc = VisionConfig(hidden=256, heads=4, layers=2, mlp=512, out_hidden=384)
    tower = VisionTower.random_init(vc, device="cuda", seed=2)
    canvas = torch.randint(0, 256, (h, w, 3), dtype=torch.uint8, device="cuda")
    got = tower.forward(canvas)
    torch.cuda.synchronize()
    ops.check_status()
    want = tower.forward_reference(canvas)
    assert got.shape == want.shape == (tower.tokens_of(h, w), 384)
    err = (got.float() - want).abs().max().item()
    assert err <= 0.03 * want.abs().max().item() + 0.02, (err, want.abs().max().item())
    cos = torch.nn.functional.cosine_similarity(got.float().flatten(), want.flatten(), dim=0).item()
    assert cos > 0.999, cos
    assert torch.equal(got, tower.forward(canvas))           # run-to-run identical


def test_kernel_engine_splices_image_rows():
    from dgpp_b200.engine.adapters import KernelEngine
    from dgpp_b200.engine.llm_engine import LLMEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel

    cfg = DenseConfig.tiny(vocab=4096)
    model = DenseModel.random_init(cfg, device="cuda", seed=0, std=0.05)
    eng = KernelEngine(LLMEngine(model, max_batch=2, max_seq_len=512, prefill_chunk=8))
    prompt = [5, 9, 77, 1234, 42, 7, 300, 8, 15, 16, 99, 3000, 17, 4, 21, 1000, 2000, 3]
    assert eng.reserve(0, len(prompt) + 4)
    eng.open(0, "plain")
    want = eng.prefill(0, prompt, 0, True)
    want_next = eng.step_batch([0])[0]
    eng.close(0)
    # positions 6..11 become pseudo image ids; their rows are the original tokens' embeddings (chunks of 8 cut the span)
    pseudo = prompt[:6] + [cfg.vocab + 77 + j for j in range(6)] + prompt[12:]
    eng.set_embeds("img", [(6, model.embed[torch.tensor(prompt[6:12], device="cuda")].clone())])
    assert eng.reserve(1, len(prompt) + 4)
    eng.open(1, "img")
    assert eng.prefill(1, pseudo, 0, True) == want
    assert eng.step_batch([1])[0] == want_next
    eng.close(1)
    # the spans are consumed by their request: the next request in the slot sees plain token embeddings
    assert eng.reserve(1, len(prompt) + 4)
    eng.open(1, "later")
    assert eng.prefill(1, prompt, 0, True) == want
