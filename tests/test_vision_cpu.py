"""Image inputs, the vision tower's oracle, the embedding splice and the chat endpoint with image parts (CPU).
(Model of the reference's tests/unit/image_inputs_test.cpp and tests/host/*_vision_frontend_test.cpp.)"""
import base64
import http.client
import json
import struct
import zlib

import numpy as np
import pytest
import torch

from dgpp_b200.runtime import rt
from dgpp_b200.serve.image_inputs import (ImageInputError, ImagePreprocess, canvas_size, decode_image, decode_png,
                                          encode_png, prepare_image, resize_image)


def _chunk(t, b):
    return struct.pack(">I", len(b)) + t + b + struct.pack(">I", zlib.crc32(t + b) & 0xFFFFFFFF)


def _png(rows_bytes, w, h, depth, ctype, extra=b""):
    return (b"\x89PNG\r\n\x1a\n" + _chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, depth, ctype, 0, 0, 0)) + extra +
            _chunk(b"IDAT", zlib.compress(rows_bytes)) + _chunk(b"IEND", b""))


def _filtered_png(rgb):
    """RGB PNG that uses filters 0..4 on successive rows."""
    h, w, _ = rgb.shape
    raw, prev = b"", np.zeros(w * 3, np.int16)
    for y in range(h):
        line = rgb[y].reshape(-1).astype(np.int16)
        f = y % 5
        left = np.concatenate([np.zeros(3, np.int16), line[:-3]])
        ul = np.concatenate([np.zeros(3, np.int16), prev[:-3]])
        if f == 0:
            enc = line
        elif f == 1:
            enc = line - left
        elif f == 2:
            enc = line - prev
        elif f == 3:
            enc = line - ((left + prev) >> 1)
        else:
            p = left + prev - ul
            pa, pb, pc = abs(p - left), abs(p - prev), abs(p - ul)
            enc = line - np.where((pa <= pb) & (pa <= pc), left, np.where(pb <= pc, prev, ul))
        raw += bytes([f]) + (enc & 255).astype(np.uint8).tobytes()
        prev = line
    return _png(raw, w, h, 8, 2)


def test_png_decoder_filters_palette_alpha_and_16_bit():
    rng = np.random.default_rng(0)
    img = rng.integers(0, 256, (23, 31, 3), dtype=np.uint8)
    assert np.array_equal(decode_png(encode_png(img)), img)
    assert np.array_equal(decode_png(_filtered_png(img)), img)
    # palette with transparency: index 1 is fully transparent -> white
    pal = bytes([10, 20, 30, 200, 100, 50])
    idx = np.array([[0, 1, 0], [1, 0, 1]], np.uint8)
    raw = b"".join(b"\x00" + idx[y].tobytes() for y in range(2))
    out = decode_png(_png(raw, 3, 2, 8, 3, _chunk(b"PLTE", pal) + _chunk(b"tRNS", bytes([255, 0]))))
    assert out[0, 0].tolist() == [10, 20, 30] and out[0, 1].tolist() == [255, 255, 255]
    # 16-bit gray keeps the high byte; gray + alpha composites over white
    g16 = np.array([[0x1234, 0xFF00]], ">u2")
    assert decode_png(_png(b"\x00" + g16.tobytes(), 2, 1, 16, 0))[0, :, 0].tolist() == [0x12, 0xFF]
    ga = bytes([0, 100, 255, 100, 0])      # filter, (gray 100, alpha 255), (gray 100, alpha 0)
    assert decode_png(_png(ga, 2, 1, 8, 4))[0, :, 0].tolist() == [100, 255]


def test_image_errors_name_the_part():
    with pytest.raises(ImageInputError) as e:
        prepare_image({"url": "https://example.com/cat.png"}, ImagePreprocess(), "messages[0].content[1].image_url")
    assert e.value.param == "messages[0].content[1].image_url" and "data:" in str(e.value)
    for bad in ("data:image/png;base64,@@@", "data:image/png,abcd", "data:image/png;base64"):
        with pytest.raises(ImageInputError):
            prepare_image(bad, ImagePreprocess(), "p")
    with pytest.raises(ImageInputError, match="jpeg"):             # a JPEG signature with nothing decodable behind it
        decode_image(b"\xff\xd8\xff\xe0" + b"0" * 32)
    with pytest.raises(ImageInputError, match="lossy"):
        decode_image(b"RIFF\x18\x00\x00\x00WEBPVP8 \x0c\x00\x00\x00" + b"\x00" * 12)
    good = encode_png(np.zeros((8, 8, 3), np.uint8))
    broken = bytearray(good)
    broken[40] ^= 1                      # inside IDAT: checksum mismatch
    with pytest.raises(ImageInputError):
        decode_png(bytes(broken))
    with pytest.raises(ImageInputError):
        decode_png(good[:30])
    ppm = b"P6\n# c\n2 1\n255\n" + bytes([1, 2, 3, 4, 5, 6])
    assert decode_image(ppm).tolist() == [[[1, 2, 3], [4, 5, 6]]]


def test_canvas_geometry():
    pp = ImagePreprocess(grid=28, min_tokens=4, max_tokens=64)
    assert canvas_size(90, 60, pp) == (84, 56)                # nearest multiples of the grid
    assert canvas_size(53, 37, pp) == (84, 56)                # 2 x 1 cells would be under min_tokens: scaled up
    cw, ch = canvas_size(4000, 3000, pp)
    assert cw % 28 == 0 and ch % 28 == 0 and (cw // 28) * (ch // 28) <= 64
    cw, ch = canvas_size(30, 30, pp)
    assert (cw // 28) * (ch // 28) >= 4
    with pytest.raises(ImageInputError):
        canvas_size(10000, 10, pp)
    pad = ImagePreprocess(grid=28, pad_to_grid=True)
    img = np.full((30, 40, 3), 200, np.uint8)
    out = resize_image(img, pad)
    assert out.shape == (56, 56, 3) and out[29, 39, 0] == 200 and out[30, 0, 0] == 0 and out[0, 40, 0] == 0
    out = resize_image(img, pp)
    assert out.shape[0] % 28 == 0 and out.shape[1] % 28 == 0 and abs(int(out[10, 10, 0]) - 200) <= 1


def test_vision_tower_oracle_shapes_and_patch_order():
    from dgpp_b200.models.vision import VisionConfig, VisionTower

    vc = VisionConfig(hidden=64, heads=2, layers=1, mlp=96, out_hidden=48)
    tower = VisionTower.random_init(vc, device="cpu", seed=1)
    py, px = tower.patch_positions(56, 84, "cpu")
    assert py.tolist()[:8] == [0, 0, 1, 1, 0, 0, 1, 1] and px.tolist()[:8] == [0, 1, 0, 1, 2, 3, 2, 3]
    canvas = torch.randint(0, 256, (56, 84, 3), dtype=torch.uint8)
    out = tower.forward_reference(canvas)
    assert out.shape == (tower.tokens_of(56, 84), 48) == (6, 48) and torch.isfinite(out).all()
    assert torch.equal(out, tower.forward_reference(canvas))
    other = canvas.clone()
    other[0:14, 0:14] = 255 - other[0:14, 0:14]           # one patch changes: attention spreads it to every token
    assert (tower.forward_reference(other) - out).abs().max() > 0


def test_embedding_spans_replace_token_rows():
    from dgpp_b200.engine.adapters import ReferenceEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel

    cfg = DenseConfig.plumbing_fp32()
    m = DenseModel.random_init(cfg, device="cpu", seed=0)
    prompt = [5, 9, 77, 1234, 42, 7, 300, 8, 15, 16]
    a = ReferenceEngine(m, slots=2, num_blocks=64, block_tokens=16, max_context=256)
    assert a.reserve(0, len(prompt) + 1)
    a.open(0, "plain")
    want = a.prefill(0, prompt, 0, True)
    # the same prompt with positions 3..6 as pseudo image ids whose rows are the embeddings of the original tokens,
    # prefilled in two chunks that cut through the span
    b = ReferenceEngine(m, slots=2, num_blocks=64, block_tokens=16, max_context=256)
    pseudo = prompt[:3] + [cfg.vocab + 1000 + j for j in range(4)] + prompt[7:]
    b.set_embeds("img", [(3, m.embed[torch.tensor(prompt[3:7])].clone())])
    assert b.reserve(1, len(prompt) + 1)
    b.open(1, "img")
    assert b.prefill(1, pseudo[:5], 0, False) == -1
    assert b.prefill(1, pseudo[5:], 5, True) == want
    # without the spans the pad embedding is used instead: the hidden state differs
    c = ReferenceEngine(m, slots=2, num_blocks=64, block_tokens=16, max_context=256)
    assert c.reserve(0, len(prompt) + 1)
    c.open(0, "none")
    c.prefill(0, pseudo, 0, True)
    assert not torch.equal(c.k[0, c.blocks[0][0], 4], a.k[0, a.blocks[0][0], 4])
    assert torch.allclose(b.k[0, b.blocks[1][0], :10], a.k[0, a.blocks[0][0], :10])


def _post(port, body):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=60)
    c.request("POST", "/v1/chat/completions", json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, json.loads(data)


def test_chat_endpoint_with_image_parts():
    from dgpp_b200.engine.adapters import ReferenceEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel
    from dgpp_b200.serve.app import Server, tiny_vision_frontend

    tok = rt.Tokenizer.byte_level([], [("<|im_start|>", 256, True), ("<|im_end|>", 257, True)], rt.SplitPattern.Qwen2)
    cfg = DenseConfig.plumbing_fp32()
    eng = ReferenceEngine(DenseModel.random_init(cfg, device="cpu", seed=0), slots=2, num_blocks=128, max_context=1024)
    plain = Server(eng, tok, model_name="vl", eos_ids=[257])
    srv = Server(eng, tok, model_name="vl", eos_ids=[257], vision=tiny_vision_frontend(cfg, "cpu"))
    port = srv.start()
    try:
        rng = np.random.default_rng(3)
        img = rng.integers(0, 256, (60, 90, 3), dtype=np.uint8)
        url = "data:image/png;base64," + base64.b64encode(encode_png(img)).decode()
        msg = lambda u: {"model": "vl", "max_tokens": 4, "messages": [{"role": "user", "content": [
            {"type": "text", "text": "what is "}, {"type": "image_url", "image_url": {"url": u}},
            {"type": "text", "text": " ?"}]}]}
        st, a = _post(port, msg(url))
        assert st == 200, a
        text_only = len(tok.encode(srv.template.render_json(json.dumps(
            {"messages": [{"role": "user", "content": "what is  ?"}], "add_generation_prompt": True}))))
        grid_tokens = (56 // 28) * (84 // 28)                 # 60 x 90 -> canvas 56 x 84 -> 6 visual tokens
        assert a["usage"]["prompt_tokens"] == text_only + grid_tokens + 2
        st, b = _post(port, msg(url))
        assert st == 200 and b["choices"][0]["message"]["content"] == a["choices"][0]["message"]["content"]
        # a broken image answers 400 and names the part
        st, e = _post(port, msg("data:image/png;base64,AAAA"))
        assert st == 400 and e["error"]["param"] == "messages[0].content[1].image_url"
        st, e = _post(port, msg("https://example.com/x.png"))
        assert st == 400 and "data:" in e["error"]["message"]
    finally:
        srv.stop()
    # a server without a vision frontend refuses image parts instead of silently dropping them
    port = plain.start()
    try:
        st, e = _post(port, msg(url))
        assert st == 400 and e["error"]["param"] == "messages"
    finally:
        plain.stop()
