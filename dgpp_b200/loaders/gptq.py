"""GPTQ / AutoRound 4-bit checkpoints re-expressed in this engine's packed-integer layouts.

A GPTQ linear stores, for a weight W [N, K] (out features N, in features K) and group size g along K:
    qweight  int32 [K / 8, N]      eight 4-bit codes q per word, consecutive k in ascending nibbles
    qzeros   int32 [K / g, N / 8]  eight 4-bit zero points per word, consecutive n in ascending nibbles
    scales   fp16  [K / g, N]
    g_idx    int32 [K]             group of every input channel (k // g unless the file was made with activation order)
and decodes as W[n, k] = (q - (z + zero_offset)) * s, zero_offset = 1 for the original GPTQ writer (it stores z - 1),
0 for the v2 / AutoRound writers.

The kernels here read offset-binary codes with one bf16 scale per 64 input channels: value = (code - 8) * scale for
int4, (code - 128) * scale for int8.  A symmetric file (every zero point 8, what AutoRound writes by default) maps onto
the int4 layout code for code; a file with other zero points maps onto the int8 layout with code = q - zero + 128,
which holds every q - zero in [-15, 15].  Both are exact in the codes; the fp16 scales are rounded to bf16 (relative
2^-9, two orders below the 4-bit rounding they scale).  Group sizes that are multiples of 64 (or one group per row)
repeat their scale over the 64-blocks they cover.  Activation-ordered files (a non-monotone g_idx) would need the
input channels permuted at run time and are refused.
(reference counterparts: src/loaders/gptq_repack.cpp, the int4 AutoRound views of src/models/quant_matrix.hpp.)
"""
from __future__ import annotations

from typing import Optional

import torch

from ..quant.formats import QuantLinear, pack_nibbles


def unpack_int4_words(words: torch.Tensor, axis: int) -> torch.Tensor:
    """int32 words holding eight 4-bit codes each (ascending nibbles) -> uint8 codes, the packed axis 8x longer."""
    w = words.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(0, 32, 4, device=words.device, dtype=torch.int64)
    axis = axis % w.dim()
    codes = (w.unsqueeze(axis + 1) >> shifts.view([-1 if d == axis + 1 else 1 for d in range(w.dim() + 1)])) & 0xF
    shape = list(w.shape)
    shape[axis] *= 8
    return codes.reshape(shape).to(torch.uint8)


def gptq_dequant(qweight, qzeros, scales, group_size: int, zero_offset: int = 1) -> torch.Tensor:
    """fp32 [N, K] values of a GPTQ linear (the oracle of `repack_gptq`)."""
    q = unpack_int4_words(qweight, 0).t().float()                       # [N, K]
    z = unpack_int4_words(qzeros, 1).t().float() + zero_offset          # [N, K / g]
    s = scales.t().float()                                              # [N, K / g]
    n, k = q.shape
    g = k if group_size in (-1, 0) else group_size
    return ((q.view(n, k // g, g) - z.unsqueeze(-1)) * s.unsqueeze(-1)).view(n, k)


def repack_gptq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, group_size: int,
                g_idx: Optional[torch.Tensor] = None, zero_offset: int = 1, bits: int = 4) -> QuantLinear:
    """One GPTQ / AutoRound linear as a QuantLinear in the int4 (symmetric files) or int8 (other zero points) layout."""
    if bits != 4:
        raise NotImplementedError(f"GPTQ repack handles 4-bit files (got {bits} bits)")
    k, n = qweight.shape[0] * 8, qweight.shape[1]
    g = k if group_size in (-1, 0) else int(group_size)
    if k % 64 or g % 64 or k % g:
        raise ValueError(f"GPTQ repack needs K and the group size to be multiples of 64 (K={k}, group {g})")
    if tuple(scales.shape) != (k // g, n) or tuple(qzeros.shape) != (k // g, n // 8):
        raise ValueError(f"GPTQ tensors disagree: qweight {tuple(qweight.shape)}, qzeros {tuple(qzeros.shape)}, "
                         f"scales {tuple(scales.shape)} for group {g}")
    if g_idx is not None:
        want = torch.arange(k, device=g_idx.device) // g
        if not torch.equal(g_idx.to(want.dtype), want):
            raise NotImplementedError("activation-ordered GPTQ files (g_idx is not k // group) are not supported")
    q = unpack_int4_words(qweight, 0).t().contiguous()                  # [N, K] codes 0..15
    z = (unpack_int4_words(qzeros, 1).t().to(torch.int16) + zero_offset)          # [N, K / g]
    s = scales.t().to(torch.bfloat16).repeat_interleave(g // 64, dim=1).contiguous()    # [N, K / 64]
    if bool((z == 8).all()):
        return QuantLinear("int4", n, k, pack_nibbles(q).contiguous(), s)
    code = q.view(n, k // g, g).to(torch.int16) - z.unsqueeze(-1) + 128
    assert int(code.min()) >= 0 and int(code.max()) <= 255
    return QuantLinear("int8", n, k, code.to(torch.uint8).view(n, k).contiguous(), s)


def pack_gptq(w: torch.Tensor, group_size: int, symmetric: bool, zero_offset: int = 1):
    """Quantise fp32 W [N, K] the way a GPTQ writer lays it out (round to nearest, no error feedback): returns
    (qweight, qzeros, scales).  For tests and synthetic checkpoints."""
    n, k = w.shape
    g = k if group_size in (-1, 0) else group_size
    blk = w.float().view(n, k // g, g)
    if symmetric:
        s = (blk.abs().amax(-1) / 7.0).clamp_min(1e-8)
        z = torch.full_like(s, 8.0)
    else:
        lo, hi = blk.amin(-1).clamp_max(0), blk.amax(-1).clamp_min(0)
        s = ((hi - lo) / 15.0).clamp_min(1e-8)
        z = torch.round(-lo / s).clamp(0, 15)
    s = s.to(torch.float16)
    q = torch.round(blk / s.float().unsqueeze(-1) + z.unsqueeze(-1)).clamp(0, 15).to(torch.int64).view(n, k)
    zs = (z.to(torch.int64) - zero_offset) & 0xF
    shifts = torch.arange(0, 32, 4, dtype=torch.int64)

    def words(codes, axis):          # pack eight consecutive entries of `axis` into one int32
        c = codes.movedim(axis, -1)
        c = c.reshape(*c.shape[:-1], c.shape[-1] // 8, 8)
        v = (c << shifts).sum(-1)
        v = torch.where(v >= 2 ** 31, v - 2 ** 32, v).to(torch.int32)
        return v.movedim(-1, axis)

    return words(q.t().contiguous(), 0), words(zs.t().contiguous(), 1), s.t().contiguous()
