"""Per-rank resident weight image: round trip, key binding, damage detection (CPU tensors)."""
import os

import torch

from dgpp_b200.loaders import resident_image as ri
from dgpp_b200.models.dense import DenseConfig, DenseModel


def _same(a, b):
    return (a is None and b is None) or (a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b))


def test_round_trip_key_and_damage(tmp_path):
    cfg = DenseConfig.tiny(sliding_window=32, attn_sinks=True, qk_norm=True)
    m = DenseModel.random_init(cfg, device="cpu", seed=1, std=0.05, tp_rank=1, tp_size=2)
    key = ri.image_key("ckpt@abc", cfg, 1, 2)
    assert key != ri.image_key("ckpt@abc", cfg, 0, 2) and key != ri.image_key("ckpt@abd", cfg, 1, 2)
    path = str(tmp_path / "img.bin")
    size = ri.save_image(m, path, key)
    assert size == os.path.getsize(path) and size % 4096 == 0
    back = ri.load_image(path, key, device="cpu")
    assert back is not None and back.cfg == cfg and back.tp_rank == 1 and back.tp_size == 2
    assert _same(back.embed, m.embed) and _same(back.final_norm, m.final_norm)
    for a, b in zip(m.layers, back.layers):
        assert b.window == a.window == 32 and _same(a.sink, b.sink) and _same(a.q_norm, b.q_norm)
        for nm in ("qkv", "o", "gate_up", "down"):
            wa, wb = getattr(a, nm), getattr(b, nm)
            assert (wa.fmt, wa.n, wa.k, wa.alpha) == (wb.fmt, wb.n, wb.k, wb.alpha)
            assert _same(wa.payload, wb.payload) and _same(wa.scale, wb.scale) and _same(wa.tiled_scales(), wb.scale_tiled)
    toks = torch.randint(0, cfg.vocab, (12,))
    la, _ = m.forward_reference(toks, all_reduce=lambda x: x)
    lb, _ = back.forward_reference(toks, all_reduce=lambda x: x)
    assert torch.equal(la, lb)
    # another key (other checkpoint / rank) does not adopt the file
    assert ri.load_image(path, ri.image_key("ckpt@abd", cfg, 1, 2), device="cpu") is None
    # one flipped byte in the tensor area is caught by the CRC; with verify off the caller owns the risk
    raw = bytearray(open(path, "rb").read())
    raw[-5000] ^= 0x40
    open(path, "wb").write(bytes(raw))
    assert ri.load_image(path, key, device="cpu") is None
    assert ri.load_image(path, key, device="cpu", verify=False) is not None
    # a truncated file is refused
    open(path, "wb").write(bytes(raw[: len(raw) // 2]))
    assert ri.load_image(path, key, device="cpu") is None
    assert ri.load_image(str(tmp_path / "absent.bin"), key, device="cpu") is None


def test_load_or_build_builds_once(tmp_path):
    cfg = DenseConfig.tiny()
    calls = []

    def build():
        calls.append(1)
        return DenseModel.random_init(cfg, device="cpu", seed=3, std=0.05)

    m1, hit1 = ri.load_or_build(build, str(tmp_path), "src", cfg, device="cpu")
    m2, hit2 = ri.load_or_build(build, str(tmp_path), "src", cfg, device="cpu")
    assert (hit1, hit2) == (False, True) and len(calls) == 1
    assert torch.equal(m1.layers[1].down.payload, m2.layers[1].down.payload)
