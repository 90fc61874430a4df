"""Checkpoint loaders on CPU: safetensors round trip through the native reader / writer, header validation,
sharded index, hub-cache resolution, architecture detection, shard slices, dense-model binding with TP slicing."""
import json
import os
import struct

import pytest
import torch

from dgpp_b200.loaders.checkpoint import load_dense, open_checkpoint, save_dense, write_safetensors
from dgpp_b200.models.dense import DenseConfig, DenseModel
from dgpp_b200.runtime import rt


def test_safetensors_round_trip_and_metadata(tmp_path):
    t = {"a.weight": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int32),
         "c.codes": torch.randint(0, 255, (4, 8), dtype=torch.uint8), "empty": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, {"format": "pt", "note": "hello"})
    f = rt.SafetensorsFile(p)
    assert f.names() == sorted(t)
    assert f.metadata()["note"] == "hello"
    assert f.info("a.weight") == {"name": "a.weight", "dtype": "BF16", "shape": [3, 5], "nbytes": 30}
    view, owner = f.view("b")
    assert bytes(view) == t["b"].numpy().tobytes()
    with pytest.raises(KeyError):
        f.info("missing")


def _raw(path, header: dict, data: bytes):
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + data)


def test_safetensors_rejects_bad_headers(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    _raw(p, {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4)          # outside the file
    with pytest.raises(RuntimeError, match="outside"):
        rt.SafetensorsFile(p)
    _raw(p, {"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8)          # size mismatch
    with pytest.raises(RuntimeError, match="need"):
        rt.SafetensorsFile(p)
    _raw(p, {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
             "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12)        # overlap
    with pytest.raises(RuntimeError, match="overlap"):
        rt.SafetensorsFile(p)
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(RuntimeError, match="header length"):
        rt.SafetensorsFile(p)


def test_hub_cache_resolution_and_family_detection(tmp_path):
    root = tmp_path / "hub"
    snap = root / "models--acme--tiny" / "snapshots" / "abc123"
    snap.mkdir(parents=True)
    (root / "models--acme--tiny" / "refs").mkdir()
    (root / "models--acme--tiny" / "refs" / "main").write_text("abc123\n")
    assert rt.resolve_model("acme/tiny", str(root)) == str(snap)
    assert rt.resolve_model("acme/tiny@abc123", str(root)) == str(snap)
    assert rt.resolve_model(str(snap)) == str(snap)
    with pytest.raises(RuntimeError, match="not in the hub cache"):
        rt.resolve_model("acme/other", str(root))
    with pytest.raises(RuntimeError):
        rt.resolve_model("not a repo id", str(root))
    fam = lambda **kw: rt.detect_family(json.dumps(kw))
    assert fam(architectures=["Qwen3ForCausalLM"], model_type="qwen3") == "dense_gqa"
    assert fam(architectures=["Qwen3_5ForConditionalGeneration"]) == "qwen_hybrid"
    assert fam(architectures=["Glm4ForCausalLM"], model_type="glm4") == "glm4"
    assert fam(architectures=["GlmDsaForCausalLM"]) == "glm_dsa"
    assert fam(architectures=["DeepseekV4ForCausalLM"]) == "deepseek_v4"
    assert fam(architectures=["MiniMaxM3ForCausalLM"]) == "minimax"
    assert fam(architectures=["MiMoV2ForCausalLM"]) == "mimo"
    with pytest.raises(RuntimeError, match="unsupported architecture"):
        fam(architectures=["Mamba2"])


def test_shard_slices_cover_extent_without_overlap():
    for extent, world, gran in [(151936, 8, 1), (40, 8, 1), (17408, 8, 16), (10, 4, 1), (7, 3, 1)]:
        prev = 0
        for r in range(world):
            b, e = rt.shard_slice(rt.Split.Rows, world, r, extent, gran)
            assert b == prev and b % gran == 0 and e >= b
            prev = e
        assert prev == extent
    assert rt.shard_slice(rt.Split.Replicated, 8, 3, 100) == (0, 100)
    assert [rt.expert_slice(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    with pytest.raises(RuntimeError, match="granule"):
        rt.shard_slice(rt.Split.Cols, 2, 0, 100, 16)


@pytest.mark.parametrize("fmt,shard_layers", [("bf16", 0), ("nvfp4", 1), ("mxfp4", 0), ("fp8", 2), ("mxfp8", 0), ("int4", 1),
                                              ("int8", 0)])
def test_dense_checkpoint_round_trip_and_tp_slices(tmp_path, fmt, shard_layers):
    heads = (8, 4) if fmt == "fp8" else (4, 2)       # fp8 128 x 128 blocks: rank slices must stay block aligned
    cfg = DenseConfig.tiny(hidden=256, q_heads=heads[0], kv_heads=heads[1], head_dim=64, ffn=512, vocab=512, layers=3, weight_fmt=fmt)
    model = DenseModel.random_init(cfg, device="cpu", seed=1, std=0.05)
    d = str(tmp_path / "ckpt")
    save_dense(model, d, shard_layers=shard_layers)
    ck = open_checkpoint(d)
    assert ck.family == "dense_gqa"
    assert os.path.exists(os.path.join(d, "model.safetensors.index.json")) == (shard_layers > 0)
    back = load_dense(d, device="cpu")
    assert back.cfg.weight_fmt == fmt and back.cfg.layers == 3
    for a, b in zip(model.layers, back.layers):
        for name in ("qkv", "o", "gate_up", "down"):
            wa, wb = getattr(a, name), getattr(b, name)
            assert torch.equal(wa.payload, wb.payload) and wa.alpha == pytest.approx(wb.alpha)
            assert torch.equal(wa.dequant(), wb.dequant())
    assert torch.equal(model.embed, back.embed) and torch.equal(model.head.payload, back.head.payload)
    # the TP shards loaded from disk are the shards random_init builds for that rank
    for r in range(2):
        want = DenseModel.random_init(cfg, device="cpu", seed=1, std=0.05, tp_rank=r, tp_size=2)
        got = load_dense(d, device="cpu", tp_rank=r, tp_size=2)
        for a, b in zip(want.layers, got.layers):
            for name in ("qkv", "o", "gate_up", "down"):
                wa, wb = getattr(a, name), getattr(b, name)
                if fmt == "bf16":
                    assert torch.equal(wa.payload, wb.payload), name
                else:   # shards of a quantised tensor are slices of the FULL tensor's codes
                    full = getattr(model.layers[0], name)
                    assert wb.n == wa.n and wb.k == wa.k
        ids = torch.randint(0, cfg.vocab, (5,))
    # the reloaded model computes the same logits
    ids = torch.randint(0, cfg.vocab, (6,))
    assert torch.equal(model.forward_reference(ids)[0], back.forward_reference(ids)[0])
