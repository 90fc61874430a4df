"""Inline image inputs of the chat endpoint: data-URI decoding, PNG / PPM decoders, and the processor geometry that
turns decoded RGB into the patch canvas a vision tower expects.

Only inline `data:` URIs are accepted: resolving remote URLs is deliberately not part of the serving path.  PNG is
decoded here (zlib + the five scanline filters, 8 / 16-bit gray, RGB, palette, with or without alpha, non-interlaced);
binary PPM / PGM as the trivial lossless carrier used by tests and tools; JPEG (sequential and progressive Huffman
streams, grey / YCbCr / RGB) and lossless WebP (VP8L, plain or in the extended container) go through the native decoders
of the runtime library.  Lossy and animated WebP are refused with a 400 that names the content part and the reason.
A decode error carries the API field of the part.
(reference counterparts: src/serve/image_inputs.cpp prepare_image / resize_image, common/image_input.hpp; the
 reference decodes through stb_image / simplewebp.)
"""
from __future__ import annotations

import base64
import binascii
import struct
import zlib
from dataclasses import dataclass
from typing import Tuple

import numpy as np

MAX_IMAGE_BYTES = 32 << 20
MAX_IMAGE_SIDE = 8192


class ImageInputError(ValueError):
    def __init__(self, message: str, param: str):
        super().__init__(message)
        self.param = param


@dataclass
class ImagePreprocess:
    """grid: canvas granularity in pixels (patch size x spatial merge); one visual token per grid cell.
    pad_to_grid: round the canvas UP to the grid and paint the remainder black; otherwise resize to the NEAREST
    multiple (ties to even), never pad, and refuse extreme aspect ratios / sides below the grid."""
    grid: int = 28
    min_tokens: int = 4
    max_tokens: int = 1024
    pad_to_grid: bool = False
    max_aspect: float = 200.0


def decode_data_uri(url: str, param: str) -> Tuple[str, bytes]:
    if not isinstance(url, str) or not url.startswith("data:"):
        raise ImageInputError("only inline data: URIs are accepted for images (remote URLs are not fetched)", param)
    head, sep, payload = url[5:].partition(",")
    if not sep:
        raise ImageInputError("malformed data URI", param)
    mime = head.split(";")[0].strip().lower()
    if ";base64" not in head:
        raise ImageInputError("image data URIs must be base64 encoded", param)
    if len(payload) > MAX_IMAGE_BYTES * 4 // 3 + 8:
        raise ImageInputError("the image is too large", param)
    try:
        data = base64.b64decode(payload, validate=True)
    except (binascii.Error, ValueError):
        raise ImageInputError("the image payload is not valid base64", param) from None
    return mime, data


def _paeth(a, b, c):
    p = a.astype(np.int16) + b.astype(np.int16) - c.astype(np.int16)
    pa, pb, pc = np.abs(p - a), np.abs(p - b), np.abs(p - c)
    return np.where((pa <= pb) & (pa <= pc), a, np.where(pb <= pc, b, c)).astype(np.uint8)


def decode_png(data: bytes, param: str = "image_url") -> np.ndarray:
    """-> uint8 [H, W, 3]; alpha is composited over white."""
    if data[:8] != b"\x89PNG\r\n\x1a\n":
        raise ImageInputError("not a PNG stream", param)
    pos, idat, plte, trns, hdr = 8, [], None, None, None
    while pos + 8 <= len(data):
        n, typ = struct.unpack(">I4s", data[pos:pos + 8])
        body = data[pos + 8:pos + 8 + n]
        if len(body) != n or pos + 12 + n > len(data):
            raise ImageInputError("truncated PNG chunk", param)
        if zlib.crc32(typ + body) & 0xFFFFFFFF != struct.unpack(">I", data[pos + 8 + n:pos + 12 + n])[0]:
            raise ImageInputError("PNG chunk checksum mismatch", param)
        pos += 12 + n
        if typ == b"IHDR":
            hdr = struct.unpack(">IIBBBBB", body)
        elif typ == b"PLTE":
            plte = np.frombuffer(body, np.uint8).reshape(-1, 3)
        elif typ == b"tRNS":
            trns = np.frombuffer(body, np.uint8)
        elif typ == b"IDAT":
            idat.append(body)
        elif typ == b"IEND":
            break
    if hdr is None or not idat:
        raise ImageInputError("PNG without a header or image data", param)
    w, h, depth, ctype, _, _, interlace = hdr
    if not (0 < w <= MAX_IMAGE_SIDE and 0 < h <= MAX_IMAGE_SIDE):
        raise ImageInputError(f"image side outside 1..{MAX_IMAGE_SIDE}", param)
    if interlace:
        raise ImageInputError("interlaced PNG is not supported", param)
    chans = {0: 1, 2: 3, 3: 1, 4: 2, 6: 4}.get(ctype)
    if chans is None or depth not in (8, 16) or (ctype == 3 and depth != 8):
        raise ImageInputError(f"unsupported PNG colour type {ctype} / bit depth {depth}", param)
    bpp = chans * depth // 8
    stride = w * bpp
    try:
        raw = zlib.decompress(b"".join(idat))
    except zlib.error:
        raise ImageInputError("corrupt PNG data stream", param) from None
    if len(raw) != h * (stride + 1):
        raise ImageInputError("PNG data stream has the wrong length", param)
    rows = np.frombuffer(raw, np.uint8).reshape(h, stride + 1)
    out = np.zeros((h, stride), np.uint8)
    prev = np.zeros(stride, np.uint8)
    for y in range(h):
        f, line = int(rows[y, 0]), rows[y, 1:]
        if f == 0:
            cur = line.copy()
        elif f == 2:
            cur = line + prev
        elif f in (1, 3, 4):
            # left-neighbour filters: pixel by pixel along the row, vectorised over the bytes of one pixel
            cur = np.zeros(stride, np.uint8)
            left, upleft = np.zeros(bpp, np.uint8), np.zeros(bpp, np.uint8)
            for x in range(0, stride, bpp):
                up = prev[x:x + bpp]
                if f == 1:
                    pred = left
                elif f == 3:
                    pred = ((left.astype(np.uint16) + up) >> 1).astype(np.uint8)
                else:
                    pred = _paeth(left, up, upleft)
                left = line[x:x + bpp] + pred
                cur[x:x + bpp] = left
                upleft = up
        else:
            raise ImageInputError("unknown PNG filter", param)
        out[y] = cur
        prev = cur
    px = out.reshape(h, w, chans, depth // 8)[..., 0]     # 16-bit samples: keep the high byte
    if ctype == 3:
        if plte is None or int(px.max()) >= len(plte):
            raise ImageInputError("PNG palette index out of range", param)
        rgb = plte[px[..., 0]]
        if trns is not None:
            a = np.full(len(plte), 255, np.uint8)
            a[:len(trns)] = trns
            return _over_white(rgb, a[px[..., 0]])
        return rgb.copy()
    if ctype == 0:
        return np.repeat(px, 3, axis=2)
    if ctype == 2:
        return px.copy()
    if ctype == 4:
        return _over_white(np.repeat(px[..., :1], 3, axis=2), px[..., 1])
    return _over_white(px[..., :3], px[..., 3])


def _over_white(rgb: np.ndarray, alpha: np.ndarray) -> np.ndarray:
    a = alpha.astype(np.uint16)[..., None]
    return ((rgb.astype(np.uint16) * a + 255 * (255 - a) + 127) // 255).astype(np.uint8)


def decode_ppm(data: bytes, param: str = "image_url") -> np.ndarray:
    """Binary PPM (P6) / PGM (P5), maxval 255 -> uint8 [H, W, 3]."""
    fields, pos = [], 0
    while len(fields) < 4:
        while pos < len(data) and data[pos:pos + 1].isspace():
            pos += 1
        if data[pos:pos + 1] == b"#":
            while pos < len(data) and data[pos:pos + 1] != b"\n":
                pos += 1
            continue
        start = pos
        while pos < len(data) and not data[pos:pos + 1].isspace():
            pos += 1
        if start == pos:
            raise ImageInputError("truncated PNM header", param)
        fields.append(data[start:pos])
    pos += 1
    magic = fields[0]
    try:
        w, h, mx = int(fields[1]), int(fields[2]), int(fields[3])
    except ValueError:
        raise ImageInputError("malformed PNM header", param) from None
    ch = {b"P6": 3, b"P5": 1}.get(magic)
    if ch is None or mx != 255 or not (0 < w <= MAX_IMAGE_SIDE and 0 < h <= MAX_IMAGE_SIDE):
        raise ImageInputError("unsupported PNM variant", param)
    if len(data) - pos < w * h * ch:
        raise ImageInputError("truncated PNM pixels", param)
    px = np.frombuffer(data, np.uint8, w * h * ch, pos).reshape(h, w, ch)
    return np.repeat(px, 3, axis=2) if ch == 1 else px.copy()


def decode_jpeg(data: bytes, param: str = "image_url") -> np.ndarray:
    """RGB uint8 [h, w, 3] through the runtime library's decoder (grey images are replicated to three channels)."""
    from ..runtime import rt

    try:
        w, h, ch, px = rt.decode_jpeg(data)
    except ValueError as e:
        raise ImageInputError(str(e), param) from None
    a = np.frombuffer(px, np.uint8).reshape(h, w, ch)
    return np.repeat(a, 3, axis=2) if ch == 1 else a.copy()


def decode_webp(data: bytes, param: str = "image_url") -> np.ndarray:
    """RGB uint8 [h, w, 3] of a lossless WebP file; alpha is composited over white like PNG alpha."""
    from ..runtime import rt

    try:
        w, h, px = rt.decode_webp(data)
    except ValueError as e:
        raise ImageInputError(str(e), param) from None
    if not (0 < w <= MAX_IMAGE_SIDE and 0 < h <= MAX_IMAGE_SIDE):
        raise ImageInputError(f"image side outside 1..{MAX_IMAGE_SIDE}", param)
    a = np.frombuffer(px, np.uint8).reshape(h, w, 4)
    if int(a[..., 3].min()) == 255:
        return a[..., :3].copy()
    return _over_white(a[..., :3], a[..., 3])


def decode_image(data: bytes, param: str = "image_url") -> np.ndarray:
    if data[:8] == b"\x89PNG\r\n\x1a\n":
        return decode_png(data, param)
    if data[:2] in (b"P6", b"P5"):
        return decode_ppm(data, param)
    if data[:3] == b"\xff\xd8\xff":
        return decode_jpeg(data, param)
    if data[:4] == b"RIFF" and data[8:12] == b"WEBP":
        return decode_webp(data, param)
    raise ImageInputError("unrecognised image format (PNG, JPEG, lossless WebP and binary PPM are accepted)", param)


def _round_half_even(x: float) -> int:
    return int(np.rint(x))


def canvas_size(width: int, height: int, pp: ImagePreprocess, param: str = "image_url") -> Tuple[int, int]:
    """(canvas_w, canvas_h) in pixels, both multiples of pp.grid, with min_tokens <= cells <= max_tokens."""
    g = pp.grid
    if max(width, height) / max(1, min(width, height)) > pp.max_aspect:
        raise ImageInputError("the image's aspect ratio is too extreme", param)
    if not pp.pad_to_grid and min(width, height) < g // 2:
        raise ImageInputError(f"image sides must be at least {g // 2} pixels", param)
    rnd = (lambda v: -(-int(np.ceil(v)) // g) * g) if pp.pad_to_grid else (lambda v: max(g, _round_half_even(v / g) * g))
    cw, ch = rnd(width), rnd(height)
    cells = (cw // g) * (ch // g)
    if cells > pp.max_tokens:
        s = (pp.max_tokens * g * g / (width * height)) ** 0.5
        cw = max(g, int(width * s) // g * g)
        ch = max(g, int(height * s) // g * g)
    elif cells < pp.min_tokens:
        s = (pp.min_tokens * g * g / (width * height)) ** 0.5
        cw = -(-int(np.ceil(width * s)) // g) * g
        ch = -(-int(np.ceil(height * s)) // g) * g
    return cw, ch


def resize_image(rgb: np.ndarray, pp: ImagePreprocess, param: str = "image_url") -> np.ndarray:
    """Decoded RGB -> uint8 canvas [H', W', 3] whose sides are multiples of the grid (bicubic, antialiased)."""
    import torch
    import torch.nn.functional as F

    h, w, _ = rgb.shape
    cw, ch = canvas_size(w, h, pp, param)
    if pp.pad_to_grid and cw >= w and ch >= h:
        out = np.zeros((ch, cw, 3), np.uint8)
        out[:h, :w] = rgb
        return out
    if (cw, ch) == (w, h):
        return np.ascontiguousarray(rgb)
    t = torch.from_numpy(np.ascontiguousarray(rgb)).permute(2, 0, 1).unsqueeze(0).float()
    t = F.interpolate(t, size=(ch, cw), mode="bicubic", align_corners=False, antialias=True)
    return t.round().clamp(0, 255).to(torch.uint8)[0].permute(1, 2, 0).contiguous().numpy()


def prepare_image(image_url, pp: ImagePreprocess, param: str = "image_url") -> np.ndarray:
    """An `image_url` content part's value ({"url": "data:..."} or the URL string) -> canvas uint8 [H', W', 3]."""
    url = image_url.get("url") if isinstance(image_url, dict) else image_url
    _, data = decode_data_uri(url, param)
    return resize_image(decode_image(data, param), pp, param)


def encode_png(rgb: np.ndarray) -> bytes:
    """Minimal PNG writer (RGB, 8 bit, filter 0): tools and tests build requests with it."""
    h, w, _ = rgb.shape
    raw = b"".join(b"\x00" + rgb[y].tobytes() for y in range(h))

    def chunk(typ: bytes, body: bytes) -> bytes:
        return struct.pack(">I", len(body)) + typ + body + struct.pack(">I", zlib.crc32(typ + body) & 0xFFFFFFFF)

    return (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0)) +
            chunk(b"IDAT", zlib.compress(raw)) + chunk(b"IEND", b""))
