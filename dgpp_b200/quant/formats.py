"""Checkpoint weight formats, as PyTorch reference codecs.

Every quantised weight keeps the byte layout of the safetensors checkpoints the engine reads
(reference: src/models/quant_matrix.hpp:2-209 describes the same layouts):

==========  ==============================  =============================================
format      payload                         scales
==========  ==============================  =============================================
``nvfp4``   e2m1, 2 codes/byte [N, K/2]     e4m3 per 16 along K [N, K/16] + fp32 per tensor
            (low nibble = even k)
``mxfp4``   e2m1 packed [N, K/2]            e8m0 per 32 along K [N, K/32]
``fp8``     e4m3 bytes [N, K]               fp32 per 128x128 block [ceil(N/128), K/128]
``mxfp8``   e4m3 bytes [N, K]               e8m0 per 32 along K [N, K/32]
``int4``    offset-binary, 2 codes/byte     bf16 per 64 along K [N, K/64]
``int8``    offset-binary bytes [N, K]      bf16 per 64 along K [N, K/64]
``bf16``    bf16 [N, K]                     --
``bf12``    sign + mantissa bytes [N, K]    one side buffer: exponent nibbles [N, K/2], row bases
            (lossless resident form of       [N], escape row starts [N + 1] uint32, escapes
            a bf16 matrix, see bf12_encode)  ((column << 16) | bf16 bits)
==========  ==============================  =============================================

The quantisers here are used to build random-init models of a given format and as the oracle the
CUDA kernels are tested against; ``QuantLinear.dequant()`` never runs on a serving path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_E2M1_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
# a tie on an odd boundary index rounds up (to the even code), on an even index it rounds down
_E2M1_TIE_UP = (False, True, False, True, False, True, False)


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """Round fp32 values (already divided by their scale) to e2m1 codes 0..15, ties to the even code."""
    a = x.abs().float()
    code = torch.zeros_like(a, dtype=torch.uint8)
    for i, b in enumerate(_E2M1_BOUNDS):
        code += ((a >= b) if _E2M1_TIE_UP[i] else (a > b)).to(torch.uint8)
    sign = (x < 0).to(torch.uint8) << 3
    return code | sign


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=code.device)
    mag = lut[(code & 7).long()]
    return torch.where((code & 8) != 0, -mag, mag)


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] codes -> [..., K/2] bytes, low nibble = even index."""
    lo = codes[..., 0::2]
    hi = codes[..., 1::2]
    return (lo | (hi << 4)).to(torch.uint8)


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    lo = packed & 0xF
    hi = packed >> 4
    return torch.stack((lo, hi), dim=-1).flatten(-2)


def e8m0_decode(e: torch.Tensor) -> torch.Tensor:
    return torch.exp2(e.float() - 127.0)


@dataclass
class QuantLinear:
    """One quantised [N, K] matrix in checkpoint layout."""

    fmt: str
    n: int
    k: int
    payload: torch.Tensor                 # uint8 / bf16, see module docstring
    scale: Optional[torch.Tensor] = None  # block scales (uint8 codes, fp32 or bf16 depending on fmt)
    alpha: float = 1.0                    # per-tensor fp32 multiplier (nvfp4 global scale)
    scale_tiled: Optional[torch.Tensor] = None  # nvfp4: the same scale bytes in tcgen05.cp atom order (see tile_scales)

    def to(self, device) -> "QuantLinear":
        return QuantLinear(self.fmt, self.n, self.k, self.payload.to(device),
                           None if self.scale is None else self.scale.to(device), self.alpha,
                           None if self.scale_tiled is None else self.scale_tiled.to(device))

    def tiled_scales(self) -> torch.Tensor:
        """Scale bytes permuted for the block-scaled tensor-core kernel (built once, cached)."""
        if self.scale_tiled is None:
            assert self.fmt == "nvfp4"
            self.scale_tiled = tile_scales(self.scale.view(self.n, self.k // 16))
        return self.scale_tiled

    @property
    def nbytes(self) -> int:
        b = self.payload.numel() * self.payload.element_size()
        if self.scale is not None:
            b += self.scale.numel() * self.scale.element_size()
        return b

    def dequant(self) -> torch.Tensor:
        """fp32 [N, K] values of the stored weights (oracle only)."""
        f, n, k = self.fmt, self.n, self.k
        if f in ("bf16", "fp32"):
            return self.payload.float()
        if f == "nvfp4":
            v = e2m1_decode(unpack_nibbles(self.payload)).view(n, k // 16, 16)
            s = self.scale.view(torch.float8_e4m3fn).float().view(n, k // 16, 1)
            return (v * s).view(n, k) * self.alpha
        if f == "mxfp4":
            v = e2m1_decode(unpack_nibbles(self.payload)).view(n, k // 32, 32)
            return (v * e8m0_decode(self.scale).view(n, k // 32, 1)).view(n, k)
        if f == "fp8":
            v = self.payload.view(torch.float8_e4m3fn).float()
            s = self.scale.repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)[:, :k]
            return v * s
        if f == "mxfp8":
            v = self.payload.view(torch.float8_e4m3fn).float().view(n, k // 32, 32)
            return (v * e8m0_decode(self.scale).view(n, k // 32, 1)).view(n, k)
        if f == "bf12":
            return bf12_decode(self).float()
        if f in ("int4", "int8"):
            bits = 4 if f == "int4" else 8
            codes = unpack_nibbles(self.payload) if bits == 4 else self.payload
            v = (codes.float() - float(1 << (bits - 1))).view(n, k // 64, 64)
            return (v * self.scale.float().view(n, k // 64, 1)).view(n, k)
        raise ValueError(f"unknown format {f}")

    def dequant_bf16_exact(self) -> torch.Tensor:
        """What the tensor-core path multiplies with: per-element values before the fp32 tensor scale,
        rounded the way the converter warps round (exact for fp4, bf16(e4m3*scale) for fp8)."""
        if self.fmt == "nvfp4":
            return (self.dequant() / self.alpha).to(torch.bfloat16)
        return self.dequant().to(torch.bfloat16)


def _up16(v: int) -> int:
    return (v + 15) & ~15


def bf12_layout(n: int, k: int):
    """Byte offsets of (row bases, escape row starts, escapes) inside a BF12 side buffer; the exponent nibbles
    start at 0.  Every part starts on a 16-byte boundary (the nibble plane is a TMA source)."""
    off_base = _up16(n * (k // 2))
    off_rows = off_base + _up16(n)
    off_esc = off_rows + _up16((n + 1) * 4)
    return off_base, off_rows, off_esc


def bf12_encode(w: torch.Tensor, max_escape_fraction: float = 1.0 / 64) -> Optional["QuantLinear"]:
    """Pack a bf16 matrix [N, K] (K % 128 == 0, K <= 65536) into the lossless 12-bit resident form.

    A bf16 weight's sign and mantissa do not compress, its exponent does: almost every weight of a trained row lies
    inside a window of 15 consecutive exponents.  Stored per weight: the sign + mantissa byte as is, and a 4-bit
    exponent code against the row's base (the window start that covers most of the row).  Code 15 is the escape:
    the weight's true bits sit in a per-row, column-sorted side table.  0.75 of the bf16 bytes, every value
    bit-for-bit the original.  Returns None when more than `max_escape_fraction` of the weights would escape (the
    packing would not pay; the matrix keeps its bf16 form).
    (reference counterpart: src/kernels/bf12_gemv.hpp -- same idea, a lane-owned layout for a CUDA-core GEMV there;
     here two TMA planes feeding the converter warps of the tensor-core GEMM.)"""
    assert w.dtype == torch.bfloat16 and w.dim() == 2
    n, k = w.shape
    assert k % 128 == 0 and k <= 65536, "bf12: K must be a multiple of 128 and at most 65536"
    dev = w.device
    off_base, off_rows, off_esc = bf12_layout(n, k)
    sm = torch.empty(n, k, dtype=torch.uint8, device=dev)
    ex = torch.empty(n, k // 2, dtype=torch.uint8, device=dev)
    base = torch.empty(n, dtype=torch.uint8, device=dev)
    counts = torch.zeros(n, dtype=torch.int64, device=dev)
    esc_parts = []
    step = max(1, (1 << 24) // k)                          # rows per pass: bounds the int32 temporaries
    for r0 in range(0, n, step):
        bits = w[r0:r0 + step].contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
        e = (bits >> 7) & 0xFF
        rows = bits.shape[0]
        hist = torch.zeros(rows, 256 + 15, dtype=torch.int64, device=dev)
        hist.scatter_add_(1, e.long(), torch.ones_like(e, dtype=torch.int64))
        cs = torch.cat((torch.zeros(rows, 1, dtype=torch.int64, device=dev), hist.cumsum(1)), 1)
        inside = cs[:, 15:15 + 256] - cs[:, 0:256]         # weights with exponent in [b, b + 14], b = 0..255
        # exponent 255 + code must stay a byte: bases above 241 gain nothing
        b = inside[:, :242].argmax(1).to(torch.int32)
        code = e - b.unsqueeze(1)
        out = (code < 0) | (code > 14)
        code = torch.where(out, torch.full_like(code, 15), code).to(torch.uint8)
        sm[r0:r0 + rows] = (((bits >> 8) & 0x80) | (bits & 0x7F)).to(torch.uint8)
        ex[r0:r0 + rows] = pack_nibbles(code)
        base[r0:r0 + rows] = b.to(torch.uint8)
        counts[r0:r0 + rows] = out.sum(1)
        rr, cc = out.nonzero(as_tuple=True)                # row-major: column-sorted within each row
        esc_parts.append(((cc.to(torch.int64) << 16) | bits[rr, cc].to(torch.int64)).to(torch.int64))
    total = int(counts.sum())
    if total > max_escape_fraction * n * k:
        return None
    esc = torch.cat(esc_parts) if esc_parts else torch.zeros(0, dtype=torch.int64, device=dev)
    starts = torch.zeros(n + 1, dtype=torch.int64, device=dev)
    starts[1:] = counts.cumsum(0)
    aux = torch.zeros(off_esc + max(16, _up16(total * 4)), dtype=torch.uint8, device=dev)
    aux[:n * (k // 2)] = ex.flatten()
    aux[off_base:off_base + n] = base
    aux[off_rows:off_rows + (n + 1) * 4] = starts.to(torch.int32).view(torch.uint8)
    if total:
        # (values above 2^31 wrap to the same 32 bits through int64 -> int32)
        aux[off_esc:off_esc + total * 4] = esc.to(torch.int32).view(torch.uint8)
    return QuantLinear("bf12", n, k, sm, aux)


def bf12_decode(q: "QuantLinear") -> torch.Tensor:
    """The bf16 matrix a BF12 form holds, bit for bit."""
    assert q.fmt == "bf12"
    n, k = q.n, q.k
    off_base, off_rows, off_esc = bf12_layout(n, k)
    aux = q.scale
    code = unpack_nibbles(aux[:n * (k // 2)].view(n, k // 2)).to(torch.int32)
    base = aux[off_base:off_base + n].to(torch.int32).unsqueeze(1)
    s = q.payload.to(torch.int32)
    bits = ((s & 0x80) << 8) | ((base + code) << 7) | (s & 0x7F)
    starts = aux[off_rows:off_rows + (n + 1) * 4].view(torch.int32).to(torch.int64)
    total = int(starts[-1])
    if total:
        esc = aux[off_esc:off_esc + total * 4].view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        rows = torch.repeat_interleave(torch.arange(n, device=aux.device), starts[1:] - starts[:-1])
        bits[rows, esc >> 16] = (esc & 0xFFFF).to(torch.int32)
    bits = torch.where(bits >= 0x8000, bits - 0x10000, bits).to(torch.int16)
    return bits.view(torch.bfloat16)


def mxfp4_as_nvfp4(w: "QuantLinear") -> Optional["QuantLinear"]:
    """Re-express an MXFP4 matrix (e2m1 codes, one e8m0 power-of-two scale per 32 elements) in the NVFP4 layout
    (same e2m1 code bytes, one e4m3 scale per 16 elements, fp32 tensor scale) WITHOUT changing any value, so that
    the block-scaled tensor-core GEMM (and its grouped expert mode) can stream MXFP4 checkpoints as stored.
    A power of two 2^p is an exact e4m3 value for p in [-9, 8]; the tensor scale recentres the matrix's exponent
    range into that window (largest scale -> 2^8).  Returns None when the range of one matrix is wider than the
    window (18 octaves), in which case the converter GEMM keeps serving it."""
    assert w.fmt == "mxfp4"
    e = w.scale.view(w.n, w.k // 32).to(torch.int32)
    if bool((e == 0).any()):
        # scale 2^-127 cannot be kept; fine when those blocks are all zero (the usual meaning), otherwise refuse
        by_block = w.payload.view(w.n, w.k // 32, 16)
        if bool((by_block[e == 0] != 0).any()):
            return None
    used = e[e > 0] if bool((e > 0).any()) else e
    hi = int(used.max())
    lo = int(used.min())
    if hi - lo > 17:
        return None
    shift = hi - 127 - 8                      # tensor scale 2^shift, block scales 2^(e - 127 - shift) in [2^-9, 2^8]
    p = (e - 127 - shift).clamp(min=-9)       # e == 0 blocks (2^-127, all-zero in practice) land on the smallest value
    val = torch.exp2(p.float())
    code = val.to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(code.view(torch.float8_e4m3fn).float(), val), "a power of two in the window is exact in e4m3"
    scale16 = code.repeat_interleave(2, dim=1).contiguous()
    return QuantLinear("nvfp4", w.n, w.k, w.payload, scale16.view(-1) if w.scale.dim() == 1 else scale16,
                       float(2.0 ** shift))


def tile_scales(sf: torch.Tensor) -> torch.Tensor:
    """[rows, K/16] e4m3 bytes -> flat bytes ordered [row_tile][stage][step][m % 32][m / 32][factor], i.e. one
    512-byte atom per (128-row tile, K=64 step) with factor i of row m at byte (m % 32) * 16 + (m / 32) * 4 + i,
    four atoms (one 256-K pipeline stage) contiguous.  Rows are padded to a multiple of 128 with zeros."""
    rows, groups = sf.shape
    assert groups % 16 == 0, "K must be a multiple of 256"
    tiles = (rows + 127) // 128
    pad = tiles * 128 - rows
    if pad:
        sf = torch.cat([sf, torch.zeros(pad, groups, dtype=sf.dtype, device=sf.device)])
    v = sf.view(tiles, 4, 32, groups // 16, 4, 4)          # [tile][m/32][m%32][stage][step][factor]
    return v.permute(0, 3, 4, 2, 1, 5).contiguous().view(-1)


def untile_scales(flat: torch.Tensor, rows: int, groups: int, row_tile: int = 128) -> torch.Tensor:
    """Inverse of the atom order for token tiles of `row_tile` rows (activation scales): returns [rows, K/16]."""
    atoms = 2 if row_tile > 128 else 1
    tiles = flat.numel() // ((groups // 16) * 4 * atoms * 512)
    v = flat.view(tiles, groups // 16, 4, atoms, 32, 4, 4)  # [tile][stage][step][atom][m%32][m/32][factor]
    v = v.permute(0, 3, 5, 4, 1, 2, 6).contiguous()         # [tile][atom][m/32][m%32][stage][step][factor]
    full = v.view(tiles, atoms * 128, groups)
    return full[:, :row_tile].reshape(tiles * row_tile, groups)[:rows]


def quantize(w: torch.Tensor, fmt: str) -> QuantLinear:
    """Quantise an fp32/bf16 [N, K] matrix into `fmt` (see module docstring)."""
    n, k = w.shape
    wf = w.float()
    if fmt == "bf16":
        return QuantLinear("bf16", n, k, w.to(torch.bfloat16).contiguous())
    if fmt == "fp32":
        return QuantLinear("fp32", n, k, wf.contiguous())
    if fmt == "bf12":
        wb = w.to(torch.bfloat16).contiguous()
        return bf12_encode(wb) or QuantLinear("bf16", n, k, wb)
    if fmt == "nvfp4":
        assert k % 16 == 0
        amax = wf.abs().max().clamp_min(1e-12)
        gs = (amax / (6.0 * 448.0)).item()
        blk = wf.view(n, k // 16, 16)
        sb = (blk.abs().amax(-1) / 6.0 / gs).clamp(max=448.0)
        sb8 = sb.to(torch.float8_e4m3fn)
        sbf = sb8.float().clamp_min(2.0 ** -9).unsqueeze(-1)
        codes = e2m1_encode(blk / (sbf * gs))
        return QuantLinear("nvfp4", n, k, pack_nibbles(codes.view(n, k)).contiguous(),
                           sb8.view(torch.uint8).contiguous(), gs)
    if fmt == "mxfp4":
        assert k % 32 == 0
        blk = wf.view(n, k // 32, 32)
        amax = blk.abs().amax(-1).clamp_min(2.0 ** -126)
        e = (torch.floor(torch.log2(amax)) - 2.0).clamp(-127, 127)
        codes = e2m1_encode(blk / torch.exp2(e).unsqueeze(-1))
        return QuantLinear("mxfp4", n, k, pack_nibbles(codes.view(n, k)).contiguous(),
                           (e + 127).to(torch.uint8).contiguous())
    if fmt == "fp8":
        assert k % 128 == 0
        nb = (n + 127) // 128
        pad = nb * 128 - n
        wp = torch.nn.functional.pad(wf, (0, 0, 0, pad)) if pad else wf
        blk = wp.view(nb, 128, k // 128, 128)
        s = (blk.abs().amax((1, 3)) / 448.0).clamp_min(1e-12)
        q = (blk / s.view(nb, 1, k // 128, 1)).clamp(-448, 448).to(torch.float8_e4m3fn)
        q = q.view(nb * 128, k)[:n]
        return QuantLinear("fp8", n, k, q.view(torch.uint8).contiguous(), s.float().contiguous())
    if fmt == "mxfp8":
        assert k % 32 == 0
        blk = wf.view(n, k // 32, 32)
        amax = blk.abs().amax(-1).clamp_min(2.0 ** -126)
        e = (torch.floor(torch.log2(amax)) - 8.0).clamp(-127, 127)
        q = (blk / torch.exp2(e).unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
        return QuantLinear("mxfp8", n, k, q.view(n, k).view(torch.uint8).contiguous(),
                           (e + 127).to(torch.uint8).contiguous())
    if fmt in ("int4", "int8"):
        assert k % 64 == 0
        bits = 4 if fmt == "int4" else 8
        qmax = float((1 << (bits - 1)) - 1)
        blk = wf.view(n, k // 64, 64)
        s = (blk.abs().amax(-1) / qmax).clamp_min(1e-12).to(torch.bfloat16)
        q = torch.round(blk / s.float().unsqueeze(-1)).clamp(-qmax - 1, qmax) + float(1 << (bits - 1))
        codes = q.to(torch.uint8).view(n, k)
        payload = pack_nibbles(codes) if bits == 4 else codes
        return QuantLinear(fmt, n, k, payload.contiguous(), s.contiguous())
    raise ValueError(f"unknown format {fmt}")


def random_quant_linear(n: int, k: int, fmt: str, device, std: float = 0.02,
                        generator: Optional[torch.Generator] = None, chunk_rows: int = 8192) -> QuantLinear:
    """N(0, std) weights quantised to `fmt`, generated in row chunks so a 27B-class model can be
    initialised on one device without an fp32 copy of a whole matrix.  nvfp4 uses the analytic
    global scale of the distribution (std * 5.5 sigma) so chunks share one tensor scale."""
    if fmt == "nvfp4":
        gs = (5.5 * std) / (6.0 * 448.0)
        payloads, scales = [], []
        for r0 in range(0, n, chunk_rows):
            r = min(chunk_rows, n - r0)
            w = torch.randn(r, k, device=device, dtype=torch.float32, generator=generator) * std
            blk = w.view(r, k // 16, 16)
            sb8 = (blk.abs().amax(-1) / 6.0 / gs).clamp(max=448.0).to(torch.float8_e4m3fn)
            sbf = sb8.float().clamp_min(2.0 ** -9).unsqueeze(-1)
            codes = e2m1_encode(blk / (sbf * gs))
            payloads.append(pack_nibbles(codes.view(r, k)))
            scales.append(sb8.view(torch.uint8))
        return QuantLinear("nvfp4", n, k, torch.cat(payloads).contiguous(), torch.cat(scales).contiguous(), gs)
    if fmt == "bf12":      # the side tables index the whole matrix: encode once, over the assembled bf16 rows
        w = torch.cat([(torch.randn(min(chunk_rows, n - r0), k, device=device, dtype=torch.float32,
                                    generator=generator) * std).to(torch.bfloat16) for r0 in range(0, n, chunk_rows)])
        return bf12_encode(w) or QuantLinear("bf16", n, k, w)
    if fmt == "fp8":
        chunk_rows = max(128, chunk_rows // 128 * 128)
    parts = []
    for r0 in range(0, n, chunk_rows):
        r = min(chunk_rows, n - r0)
        w = torch.randn(r, k, device=device, dtype=torch.float32, generator=generator) * std
        parts.append(quantize(w, fmt))
    if len(parts) == 1:
        return parts[0]
    return QuantLinear(fmt, n, k, torch.cat([p.payload for p in parts]).contiguous(),
                       None if parts[0].scale is None else torch.cat([p.scale for p in parts]).contiguous(),
                       parts[0].alpha)
