"""GPTQ / AutoRound repack: symmetric files land in the int4 layout code for code, files with other zero points in the
int8 layout; values equal the GPTQ decode up to the bf16 rounding of the scales; refusals."""
import pytest
import torch

from dgpp_b200.loaders.gptq import gptq_dequant, pack_gptq, repack_gptq, unpack_int4_words


def test_word_unpacking_orders_nibbles_ascending():
    w = torch.tensor([[0x76543210, -1]], dtype=torch.int32)
    assert unpack_int4_words(w, 0)[:, 0].tolist() == [0, 1, 2, 3, 4, 5, 6, 7] and unpack_int4_words(w, 0)[:, 1].tolist() == [15] * 8
    assert unpack_int4_words(w, 1)[0].tolist() == [0, 1, 2, 3, 4, 5, 6, 7] + [15] * 8


@pytest.mark.parametrize("group,sym,off", [(128, True, 1), (64, True, 0), (-1, True, 1), (128, False, 1), (256, False, 0)])
def test_repack_matches_the_gptq_decode(group, sym, off):
    torch.manual_seed(3)
    n, k = 48, 512
    w = torch.randn(n, k) * 0.05 + (0.0 if sym else 0.02)
    qw, qz, sc = pack_gptq(w, group, sym, off)
    assert qw.shape == (k // 8, n) and sc.dtype == torch.float16
    want = gptq_dequant(qw, qz, sc, group, off)
    assert (want - w).abs().max().item() < 0.06               # the test writer itself is a sane 4-bit quantiser
    g_idx = torch.arange(k) // (k if group == -1 else group)
    m = repack_gptq(qw, qz, sc, group, g_idx=g_idx, zero_offset=off)
    assert m.fmt == ("int4" if sym else "int8") and (m.n, m.k) == (n, k)
    assert m.scale.shape == (n, k // 64) and m.scale.dtype == torch.bfloat16
    got = m.dequant()
    assert (got - want).abs().max().item() <= 2.0 ** -8 * want.abs().max().item()      # bf16 scales only
    # with scales that bf16 holds exactly the repack is exact
    sc2 = sc.to(torch.bfloat16).to(torch.float16)
    assert torch.equal(repack_gptq(qw, qz, sc2, group, zero_offset=off).dequant(), gptq_dequant(qw, qz, sc2, group, off))


def test_refusals():
    qw, qz, sc = pack_gptq(torch.randn(16, 256), 128, True)
    with pytest.raises(NotImplementedError, match="activation-ordered"):
        repack_gptq(qw, qz, sc, 128, g_idx=torch.randperm(256) // 128)
    with pytest.raises(ValueError, match="multiples of 64"):
        repack_gptq(qw, qz[:, :], sc, 32)
    with pytest.raises(ValueError, match="disagree"):
        repack_gptq(qw, qz, sc[:1], 128)
    with pytest.raises(NotImplementedError, match="4-bit"):
        repack_gptq(qw, qz, sc, 128, bits=8)
