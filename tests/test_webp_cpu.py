"""Lossless WebP decoder of the runtime library against Pillow's decoder on files Pillow wrote: every transform kind
(predictor, cross-colour, subtract-green, colour indexing at each packing width), backward references, the colour
cache, alpha, the extended container, plus refusals of damaged and unsupported files.
(reference counterpart: src/serve/image_inputs.cpp, WebP through a third-party decoder)"""
import io
import struct

import numpy as np
import pytest

from dgpp_b200.runtime import rt
from dgpp_b200.serve.image_inputs import ImageInputError, decode_image

PIL = pytest.importorskip("PIL.Image")
from PIL import features  # noqa: E402

pytestmark = pytest.mark.skipif(not features.check("webp"), reason="Pillow without WebP")


def _encode(arr, mode, **kw):
    b = io.BytesIO()
    PIL.fromarray(arr, mode).save(b, "WEBP", lossless=True, exact=True, **kw)
    return b.getvalue()


def _native(data):
    w, h, px = rt.decode_webp(data)
    return np.frombuffer(px, np.uint8).reshape(h, w, 4)


def _pillow(data):
    return np.asarray(PIL.open(io.BytesIO(data)).convert("RGBA"))


def _photo(h, w, seed=0):
    rng = np.random.default_rng(seed)
    y, x = np.mgrid[0:h, 0:w]
    p = np.stack([(x * 1.2) % 256, (y * 1.7) % 256, ((x + y) * 0.8) % 256], -1).astype(int)
    return (p + rng.integers(-6, 6, p.shape)).clip(0, 255).astype(np.uint8)


@pytest.mark.parametrize("method", [0, 3, 6])
@pytest.mark.parametrize("quality", [0, 75, 100])
def test_photo_like_matches_pillow(method, quality):
    data = _encode(_photo(150, 200), "RGB", method=method, quality=quality)
    got = _native(data)
    assert np.array_equal(got, _pillow(data))
    assert np.array_equal(got[..., :3], _photo(150, 200)) and int(got[..., 3].min()) == 255


@pytest.mark.parametrize("colors", [2, 3, 4, 9, 16, 17, 200])
def test_palette_images(colors):
    rng = np.random.default_rng(colors)
    table = rng.integers(0, 256, (colors, 3), dtype=np.uint8)
    img = table[rng.integers(0, colors, (61, 83))]
    data = _encode(img, "RGB")
    assert np.array_equal(_native(data)[..., :3], img)


def test_alpha_noise_and_odd_sizes():
    rng = np.random.default_rng(1)
    photo = _photo(70, 90)
    y, x = np.mgrid[0:70, 0:90]
    rgba = np.concatenate([photo, ((x + y) % 256).astype(np.uint8)[..., None]], -1)
    data = _encode(rgba, "RGBA")
    assert b"VP8X" in data[:32] or b"VP8L" in data[:32]
    assert np.array_equal(_native(data), rgba)
    for shape in ((1, 1), (1, 300), (300, 1), (5, 7), (64, 97)):
        img = rng.integers(0, 256, shape + (3,), dtype=np.uint8)
        assert np.array_equal(_native(_encode(img, "RGB"))[..., :3], img)
    flat = np.full((40, 300, 3), 200, np.uint8)
    assert np.array_equal(_native(_encode(flat, "RGB"))[..., :3], flat)
    big = np.kron(_photo(100, 120), np.ones((5, 5, 1), np.uint8))          # long backward references
    assert np.array_equal(_native(_encode(big, "RGB", method=6, quality=100))[..., :3], big)


def test_decode_image_routes_webp_and_composites_alpha():
    photo = _photo(32, 48)
    assert np.array_equal(decode_image(_encode(photo, "RGB")), photo)
    rgba = np.concatenate([photo, np.full((32, 48, 1), 0, np.uint8)], -1)
    rgba[:16, :, 3] = 255
    out = decode_image(_encode(rgba, "RGBA"))
    assert np.array_equal(out[:16], photo[:16]) and int(out[16:].min()) == 255      # transparent half shows white


def test_refusals():
    good = _encode(_photo(40, 40), "RGB")
    with pytest.raises(ValueError, match="webp"):
        rt.decode_webp(good[:len(good) // 2])
    with pytest.raises(ValueError, match="RIFF"):
        rt.decode_webp(b"RIFX" + good[4:])
    b = io.BytesIO()
    PIL.fromarray(_photo(40, 40), "RGB").save(b, "WEBP", quality=80)           # lossy
    with pytest.raises(ImageInputError, match="lossy") as e:
        decode_image(b.getvalue(), "messages[0].content[1].image_url")
    assert e.value.param == "messages[0].content[1].image_url"
    # a header that claims 16384 x 16384 is refused before any allocation of that size
    hdr = 0x2f | ((16383) << 8) | ((16383) << 22)
    body = struct.pack("<Q", hdr)[:5] + b"\x00" * 8
    data = b"RIFF" + struct.pack("<I", 4 + 8 + len(body)) + b"WEBPVP8L" + struct.pack("<I", len(body)) + body
    with pytest.raises(ValueError, match="side"):
        rt.decode_webp(data)
    rng = np.random.default_rng(0)
    ok = bad = 0
    for _ in range(300):                      # random damage: either decodes to the stated size or is refused cleanly
        buf = bytearray(good)
        for _ in range(int(rng.integers(1, 4))):
            buf[int(rng.integers(20, len(buf)))] = int(rng.integers(0, 256))
        try:
            w, h, px = rt.decode_webp(bytes(buf))
            assert len(px) == w * h * 4
            ok += 1
        except ValueError:
            bad += 1
    assert bad > 0
