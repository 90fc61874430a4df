"""BF12: the lossless 12-bit resident form of a bf16 matrix (codec side; the kernel side is a GPU test)."""
import torch

from dgpp_b200.quant.formats import QuantLinear, bf12_decode, bf12_encode, bf12_layout, quantize


def _bits(t):
    return t.view(torch.int16)


def test_roundtrip_is_bit_exact_with_outliers():
    torch.manual_seed(0)
    w = (torch.randn(200, 1024) * 0.02).to(torch.bfloat16)
    w[3, 5] = 0.0                     # exponent field 0: outside any trained row's window
    w[7, 100] = 1e-30
    w[9] = 0                          # an all-zero row packs with base 0 and no escapes
    w[11, 1023] = 3e20
    w[199, 0] = float("inf")
    w[198, 1] = -0.0
    q = bf12_encode(w)
    assert q is not None and q.fmt == "bf12" and (q.n, q.k) == (200, 1024)
    assert torch.equal(_bits(bf12_decode(q)), _bits(w))
    assert torch.equal(q.dequant(), w.float()) or torch.isinf(w).any()
    # 12 bits a weight plus the side tables
    assert q.nbytes < 0.76 * w.numel() * 2
    _, off_rows, _ = bf12_layout(200, 1024)
    starts = q.scale[off_rows:off_rows + 201 * 4].view(torch.int32)
    assert starts[0] == 0 and (starts[1:] >= starts[:-1]).all()
    assert int(starts[10]) - int(starts[9]) == 0
    assert 0 < int(starts[-1]) < 200


def test_escapes_are_column_sorted_per_row():
    torch.manual_seed(1)
    w = (torch.randn(4, 256) * 0.02).to(torch.bfloat16)
    w[2, 200] = 1e25
    w[2, 17] = 1e-25
    w[2, 255] = 0.0
    q = bf12_encode(w, max_escape_fraction=1.0)
    _, off_rows, off_esc = bf12_layout(4, 256)
    starts = q.scale[off_rows:off_rows + 5 * 4].view(torch.int32).tolist()
    esc = q.scale[off_esc:off_esc + starts[-1] * 4].view(torch.int32)
    cols = [(int(v) >> 16) & 0xFFFF for v in esc[starts[2]:starts[3]]]
    assert cols == sorted(cols) and {17, 200, 255} <= set(cols)
    assert torch.equal(_bits(bf12_decode(q)), _bits(w))


def test_wide_rows_keep_bf16():
    # exponents spread over 60 octaves: most weights would escape, the packing is refused
    torch.manual_seed(2)
    w = (torch.randn(16, 256) * torch.exp2(torch.randint(-30, 30, (16, 256)).float())).to(torch.bfloat16)
    assert bf12_encode(w) is None
    q = quantize(w.float(), "bf12")
    assert isinstance(q, QuantLinear) and q.fmt == "bf16"
    q = quantize(torch.randn(16, 256) * 0.02, "bf12")
    assert q.fmt == "bf12"


def test_model_pack_and_export_roundtrip(tmp_path):
    from dgpp_b200.models.dense import DenseConfig, DenseModel

    cfg = DenseConfig.plumbing_fp32(weight_fmt="bf16", head_fmt="bf16")
    m = DenseModel.random_init(cfg, device="cpu", seed=3)
    want = m.head.payload.clone()
    saved = m.pack_bf12()
    assert m.head.fmt == "bf12" and saved > 0.2 * want.numel() * 2
    assert torch.equal(_bits(bf12_decode(m.head)), _bits(want))
