"""Native JPEG decoder against an independent decoder (Pillow, used only to make and check test files): sequential and
progressive streams, all common chroma layouts, restart markers, optimised tables, odd sizes; refusals; the chat image
path accepts a JPEG data URI."""
import base64
import io

import numpy as np
import pytest

from dgpp_b200.runtime import rt

Image = pytest.importorskip("PIL.Image")


def _picture(w, h, grey=False, seed=0):
    rng = np.random.default_rng(seed)
    y, x = np.mgrid[0:h, 0:w]
    a = np.stack([128 + 100 * np.sin(x / 9.0) * np.cos(y / 7.0), 128 + 90 * np.cos(x / 13.0 + y / 5.0),
                  128 + 80 * np.sin((x + y) / 11.0)], -1) + rng.normal(0, 6, (h, w, 3))
    a = np.clip(a, 0, 255).astype(np.uint8)
    return a[..., 0] if grey else a


def _encode(a, **kw):
    b = io.BytesIO()
    Image.fromarray(a).save(b, "JPEG", **kw)
    return b.getvalue()


def _decode(data):
    w, h, c, px = rt.decode_jpeg(data)
    a = np.frombuffer(px, np.uint8).reshape(h, w, c)
    return a[..., 0] if c == 1 else a


CASES = [dict(quality=90, subsampling=0), dict(quality=85, subsampling=1), dict(quality=80, subsampling=2),
         dict(quality=80, subsampling=2, progressive=True), dict(quality=95, subsampling=0, progressive=True),
         dict(quality=70, optimize=True), dict(quality=85, subsampling=2, restart_marker_blocks=3), dict(quality=25)]


@pytest.mark.parametrize("size", [(64, 48), (97, 61), (8, 8), (1, 1), (33, 130)])
@pytest.mark.parametrize("grey", [False, True])
def test_decoder_agrees_with_an_independent_decoder(size, grey):
    for kw in CASES:
        data = _encode(_picture(*size, grey=grey), **kw)
        want = np.asarray(Image.open(io.BytesIO(data)))
        got = _decode(data)
        assert got.shape == want.shape, kw
        d = np.abs(got.astype(int) - want.astype(int))
        # inverse transform, chroma filter and colour conversion round differently: a few levels at most, rarely
        assert d.max() <= 4 and (d.size < 64 or d.mean() <= 0.25), (kw, d.max(), d.mean())


def test_refusals_name_the_reason():
    good = _encode(_picture(40, 30), quality=80)
    for bad, why in ((b"", "SOI"), (good[:2] + b"\xff\xd9", "frame"), (b"\x89PNG", "SOI")):
        with pytest.raises(ValueError, match=why):
            rt.decode_jpeg(bad)
    cmyk = io.BytesIO()
    Image.fromarray(np.zeros((8, 8, 4), np.uint8), "CMYK").save(cmyk, "JPEG")
    with pytest.raises(ValueError, match="components"):
        rt.decode_jpeg(cmyk.getvalue())
    sof = good.index(b"\xff\xc0")
    arith = good[:sof] + b"\xff\xc9" + good[sof + 2:]
    with pytest.raises(ValueError, match="arithmetic"):
        rt.decode_jpeg(arith)
    # a file cut inside its entropy-coded data still decodes (the missing part reads as zero bits) to the right size
    big = _encode(_picture(200, 150), quality=80)
    w, h, c, px = rt.decode_jpeg(big[:len(big) * 2 // 3])
    assert (w, h, c, len(px)) == (200, 150, 3, 200 * 150 * 3)


def test_damaged_files_never_take_the_process_down():
    rng = np.random.default_rng(5)
    for kw in (dict(quality=60, subsampling=2, restart_marker_blocks=1), dict(quality=60, subsampling=2, progressive=True)):
        data = bytearray(_encode(_picture(24, 20), **kw))
        for _ in range(300):
            buf = bytearray(data)
            for _ in range(int(rng.integers(1, 5))):
                buf[int(rng.integers(0, len(buf)))] = int(rng.integers(0, 256))
            try:
                w, h, c, px = rt.decode_jpeg(bytes(buf))
                assert len(px) == w * h * c
            except ValueError:
                pass


def test_chat_image_part_accepts_a_jpeg_data_uri():
    from dgpp_b200.serve.image_inputs import ImagePreprocess, decode_image, prepare_image

    a = _picture(56, 42)
    data = _encode(a, quality=92, subsampling=0)
    rgb = decode_image(data)
    assert rgb.shape == (42, 56, 3) and np.abs(rgb.astype(int) - a.astype(int)).mean() < 6
    grey = decode_image(_encode(_picture(30, 30, grey=True), quality=90))
    assert grey.shape == (30, 30, 3) and (grey[..., 0] == grey[..., 2]).all()
    out = prepare_image("data:image/jpeg;base64," + base64.b64encode(data).decode(), ImagePreprocess(), "p")
    assert out is not None
