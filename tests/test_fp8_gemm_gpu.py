"""Native FP8 linear: e4m3 activations (per token and 128 columns) x e4m3 weights (per 128 x 128 block) on tcgen05
kind::f8f6f4 with the scales promoted per K block, against fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def test_fp8_activation_quantiser_round_trip(dev):
    from dgpp_b200.ops import core as ops

    torch.manual_seed(1)
    x = (torch.randn(37, 1024, device=dev) * torch.rand(37, 1, device=dev) * 8).to(BF)
    x[3, 128:256] = 0
    xa = ops.fp8_act_quant(x)
    torch.cuda.synchronize()
    back = xa.dequant()
    # e4m3 keeps 3 mantissa bits: relative error per element <= 2^-4, against the block maximum
    blocks = x.float().view(37, 8, 128)
    tol = blocks.abs().amax(-1, keepdim=True) * 2.0 ** -4 + 1e-6
    assert ((back.view(37, 8, 128) - blocks).abs() <= tol).all()
    assert torch.equal(back[3, 128:256], torch.zeros(128, device=dev))


@pytest.mark.parametrize("rows,n,k,splits", [(1, 512, 1024, None), (8, 1024, 4096, None), (8, 1024, 4096, 1), (100, 640, 2048, None),
                                             (300, 384, 1024, None), (16, 4096, 7168, 4)])
def test_gemm_fp8_matches_fp32_reference(dev, rows, n, k, splits):
    from dgpp_b200.ops import core as ops
    from dgpp_b200.quant.formats import quantize

    torch.manual_seed(2)
    w = quantize(torch.randn(n, k, device=dev) * 0.05, "fp8")
    x = torch.randn(rows, k, device=dev).to(BF)
    xa = ops.fp8_act_quant(x)
    out = ops.gemm_fp8(xa, w, splits=splits)
    torch.cuda.synchronize()
    ops.check_status()
    # exact reference of what the kernel computes: dequantised operands, fp32 accumulation
    wd = w.payload.view(torch.float8_e4m3fn).float().view(n, k)
    sc = w.scale.repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)
    want = xa.dequant() @ (wd * sc).t()
    err = (out.float() - want).abs().max().item()
    assert err <= 1e-2 * want.abs().max().item() + 1e-3, err
    # and against the bf16-activation converter path (the activation rounding is the only difference)
    base = ops.gemm_tc(x, w)
    assert (out.float() - base.float()).abs().max().item() <= 6e-2 * base.float().abs().max().item()
    # deterministic
    assert torch.equal(out, ops.gemm_fp8(xa, w, splits=splits))
