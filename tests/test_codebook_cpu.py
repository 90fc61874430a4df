"""NF4I8 / Mixed346 codebook matrices: the row bit streams (codes that straddle words included) and the exact repack
into the int8 layout."""
import pytest
import torch

from dgpp_b200.loaders.codebook import (GAUSS3_LEVELS, NF4I8_LEVELS, code_levels, codebook_dequant, encode_codebook,
                                        pack_stream, repack_codebook, unpack_stream)


@pytest.mark.parametrize("bits", [3, 4, 6])
def test_stream_round_trip_and_word_layout(bits):
    g = torch.Generator().manual_seed(bits)
    codes = torch.randint(0, 1 << bits, (5, 256), generator=g, dtype=torch.uint8)
    words = pack_stream(codes, bits)
    assert words.shape == (5, 256 * bits // 32) and words.dtype == torch.int32
    assert torch.equal(unpack_stream(words, 256, bits), codes)
    # code k sits at bit k * bits of the row's little-endian stream
    row = 0
    for wd in reversed(words[2].tolist()):
        row = (row << 32) | (wd & 0xFFFFFFFF)
    for k in (0, 1, 10, 11, 21, 255):
        assert (row >> (k * bits)) & ((1 << bits) - 1) == int(codes[2, k])
    with pytest.raises(ValueError):
        unpack_stream(words, 128, bits)


@pytest.mark.parametrize("bits", [3, 4, 6])
def test_repack_is_exact(bits):
    g = torch.Generator().manual_seed(10 + bits)
    w = torch.randn(24, 384, generator=g) * 0.05
    idx, sc = encode_codebook(w, bits)
    want = codebook_dequant(idx, sc, 384, bits)
    q = repack_codebook(idx, sc, 384, bits)
    assert q.fmt == "int8" and q.n == 24 and q.k == 384
    assert torch.equal(q.dequant().float(), want)
    # the encoder is a sane quantiser: error shrinks with the code width
    rel = ((want - w).norm() / w.norm()).item()
    assert rel < {3: 0.25, 4: 0.13, 6: 0.04}[bits], rel


def test_tables_and_refusals():
    assert code_levels(4).tolist() == list(NF4I8_LEVELS) and code_levels(3).tolist() == list(GAUSS3_LEVELS)
    assert code_levels(6)[0].item() == -32 and code_levels(6)[63].item() == 31
    with pytest.raises(ValueError):
        code_levels(5)
    idx, sc = encode_codebook(torch.randn(4, 256), 4)
    with pytest.raises(ValueError):
        repack_codebook(idx, sc.float(), 256, 4)
    with pytest.raises(ValueError):
        repack_codebook(idx[:, :-1], sc, 256, 4)
    zero_idx, zero_sc = encode_codebook(torch.zeros(2, 128), 4)
    assert float(codebook_dequant(zero_idx, zero_sc, 128, 4).abs().max()) == 0.0
