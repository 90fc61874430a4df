"""Codebook-quantised checkpoints (NF4I8 and Mixed346) re-expressed in this engine's int8 layout.

Both formats store, for a weight W [N, K], one dense little-endian bit stream of codes per row
(`weight_indices` int32 [N, K * bits / 32]: code k occupies bits [k * bits, (k + 1) * bits) of the row's stream, so a
3- or 6-bit code may straddle two words) and one bf16 scale per 128 codes; a code is an index into a fixed table of
int8 levels and the value is level * scale:

    NF4I8      4 bits   levels round(127 x NF4)
    Mixed346   3 bits   Gaussian Lloyd-Max levels;  4 bits  the NF4I8 table;  6 bits  level = code - 32

Every level is an integer in [-127, 127], so the int8 layout of the kernels here (offset-binary byte, value =
(byte - 128) * scale, one bf16 scale per 64 input channels) holds the matrix exactly: byte = level + 128, the scale of
a 128-group repeated over its two 64-blocks.  Storage grows to one byte per weight; nothing is rounded.
The checkpoints rotate the routed experts' inputs by a 32-wide Hadamard transform before quantising; that is a
property of the layer (`ops.hadamard32_rows` on the activations), not of the matrix.
(reference counterparts: src/models/quant_matrix.hpp kNf4i8Codebook / kGauss3Codebook / packed_code_level,
 src/loaders/packq_quant.hpp packq_field / packq_encode_row_m346.)
"""
from __future__ import annotations

import torch

from ..quant.formats import QuantLinear

NF4I8_LEVELS = (-127, -88, -67, -50, -36, -23, -12, 0, 10, 20, 31, 43, 56, 71, 92, 127)
GAUSS3_LEVELS = (-127, -79, -45, -14, 14, 45, 79, 127)
GROUP = 128


def code_levels(bits: int) -> torch.Tensor:
    """int16 table: the level of every code of a `bits`-wide stream."""
    if bits == 3:
        return torch.tensor(GAUSS3_LEVELS, dtype=torch.int16)
    if bits == 4:
        return torch.tensor(NF4I8_LEVELS, dtype=torch.int16)
    if bits == 6:
        return torch.arange(64, dtype=torch.int16) - 32
    raise ValueError(f"codebook formats store 3-, 4- or 6-bit codes (got {bits})")


def unpack_stream(words: torch.Tensor, k: int, bits: int) -> torch.Tensor:
    """int32 [N, K * bits / 32] row streams -> uint8 codes [N, K]."""
    n = words.shape[0]
    if words.shape[1] * 32 != k * bits:
        raise ValueError(f"a row of {k} codes of {bits} bits takes {k * bits // 32} words, the tensor has {words.shape[1]}")
    w = words.to(torch.int64) & 0xFFFFFFFF
    # one spare word so that the two-word read of a straddling code stays inside
    w = torch.cat([w, torch.zeros(n, 1, dtype=torch.int64, device=w.device)], dim=1)
    bit = torch.arange(k, device=w.device, dtype=torch.int64) * bits
    lo, off = bit // 32, bit % 32
    both = w[:, lo] | (w[:, lo + 1] << 32)
    return ((both >> off) & ((1 << bits) - 1)).to(torch.uint8)


def pack_stream(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """uint8 codes [N, K] -> int32 row streams (the inverse of `unpack_stream`; for tests and synthetic files)."""
    n, k = codes.shape
    assert (k * bits) % 32 == 0
    nbits = ((codes.to(torch.int64).unsqueeze(-1) >> torch.arange(bits, dtype=torch.int64)) & 1).reshape(n, k * bits)
    v = (nbits.view(n, k * bits // 32, 32) << torch.arange(32, dtype=torch.int64)).sum(-1)
    return torch.where(v >= 2 ** 31, v - 2 ** 32, v).to(torch.int32)


def codebook_dequant(weight_indices: torch.Tensor, scales: torch.Tensor, k: int, bits: int) -> torch.Tensor:
    """fp32 [N, K] values (the oracle of `repack_codebook`)."""
    lv = code_levels(bits).to(weight_indices.device)[unpack_stream(weight_indices, k, bits).long()].float()
    return lv * scales.float().repeat_interleave(GROUP, dim=1)


def repack_codebook(weight_indices: torch.Tensor, scales: torch.Tensor, k: int, bits: int = 4) -> QuantLinear:
    """One NF4I8 (bits 4) or Mixed346 (bits 3 / 4 / 6) matrix as an int8 QuantLinear, exactly."""
    n = weight_indices.shape[0]
    if k % GROUP:
        raise ValueError(f"codebook formats need K to be a multiple of {GROUP} (got {k})")
    if tuple(scales.shape) != (n, k // GROUP) or scales.dtype != torch.bfloat16:
        raise ValueError(f"scales must be bf16 [{n}, {k // GROUP}] (got {scales.dtype} {tuple(scales.shape)})")
    level = code_levels(bits).to(weight_indices.device)[unpack_stream(weight_indices, k, bits).long()]
    byte = (level + 128).to(torch.uint8).contiguous()
    return QuantLinear("int8", n, k, byte, scales.repeat_interleave(GROUP // 64, dim=1).contiguous())


def encode_codebook(w: torch.Tensor, bits: int):
    """Round-to-nearest encoder of the formats: fp32 W [N, K] -> (weight_indices int32, scales bf16 [N, K / 128]).
    The scale maps the group's absolute maximum onto the largest level; every value takes its nearest level (ties to
    the lower code)."""
    n, k = w.shape
    lv = code_levels(bits).float()
    blk = w.float().view(n, k // GROUP, GROUP)
    s = (blk.abs().amax(-1) / float(lv.abs().max())).to(torch.bfloat16)
    s = torch.where(s.float() > 0, s, torch.ones_like(s))
    x = blk / s.float().unsqueeze(-1)
    codes = (x.unsqueeze(-1) - lv).abs().argmin(-1).to(torch.uint8).view(n, k)
    return pack_stream(codes, bits), s
