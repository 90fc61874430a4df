"""Low-rank adapters on CPU: manifest + digest check, tensor-parallel slicing, reference forward equivalence with
merged weights.  (Model of the reference's tests: tests/test_adapters.cpp, tests/test_low_rank.cpp.)"""
import json
import os

import pytest
import torch

from dgpp_b200.adapters import lora
from dgpp_b200.models.dense import DenseConfig, DenseModel
from dgpp_b200.quant.formats import quantize

TARGETS = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


def _cfg(**kw):
    return DenseConfig.plumbing_fp32(**kw)


def test_manifest_roundtrip_and_digest_check(tmp_path):
    cfg = _cfg()
    t = lora.random_adapter_tensors(cfg, rank=4, targets=["q_proj", "down_proj"], seed=1)
    d = str(tmp_path / "ad")
    lora.save_adapter(d, t, rank=4, alpha=8.0, targets=["q_proj", "down_proj"])
    ad = lora.load_adapter(d, cfg, device="cpu")
    assert ad.rank == 4 and ad.scale == 2.0 and len(ad.layers) == cfg.layers
    assert [p.col0 for p in ad.pairs(0, "qkv")] == [0] and len(ad.pairs(1, "down")) == 1 and ad.pairs(0, "o") == []
    assert torch.equal(ad.pairs(0, "qkv")[0].a, t["layers.0.q_proj.lora_A"])
    # one flipped byte in the tensor file -> refused
    path = os.path.join(d, "adapter.safetensors")
    raw = bytearray(open(path, "rb").read())
    raw[-1] ^= 1
    open(path, "wb").write(bytes(raw))
    with pytest.raises(ValueError, match="digest"):
        lora.load_adapter(d, cfg, device="cpu")
    # unknown target in the manifest -> refused
    man = json.load(open(os.path.join(d, "adapter_manifest.json")))
    man["targets"].append("router")
    json.dump(man, open(os.path.join(d, "adapter_manifest.json"), "w"))
    with pytest.raises(ValueError, match="unknown targets"):
        lora.load_adapter(d, cfg, device="cpu")


def test_reference_forward_equals_merged_weights():
    """With fp32 weights, adding the adapter at run time equals running the model with W + scale * B A."""
    cfg = _cfg()
    torch.manual_seed(0)
    m = DenseModel.random_init(cfg, device="cpu", seed=3, std=0.05)
    t = {k: v.float() for k, v in lora.random_adapter_tensors(cfg, 4, TARGETS, seed=2, std=0.1).items()}
    ad = lora.bind_adapter(t, cfg, 4, 8.0, "cpu")
    for L in ad.layers:                       # keep the adapter in fp32 for an exact comparison
        for pairs in L.values():
            for p in pairs:
                p.a, p.b = p.a.float(), p.b.float()
    ad2 = lora.bind_adapter(t, cfg, 4, 8.0, "cpu")
    toks = torch.randint(0, cfg.vocab, (9,))
    got, _ = m.forward_reference(toks, lora=ad2)
    base, _ = m.forward_reference(toks)
    assert (got - base).abs().max() > 0.1     # the adapter does something
    # merged model
    d, nq, nkv = cfg.head_dim, cfg.q_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
    bf = lambda x: x.to(torch.bfloat16).float()
    for i, L in enumerate(m.layers):
        g = lambda n, s: bf(t[f"layers.{i}.{n}.lora_{s}"])
        w = L.qkv.dequant().float()
        w[:nq] += 2.0 * g("q_proj", "B") @ g("q_proj", "A")
        w[nq:nq + nkv] += 2.0 * g("k_proj", "B") @ g("k_proj", "A")
        w[nq + nkv:] += 2.0 * g("v_proj", "B") @ g("v_proj", "A")
        L.qkv = quantize(w, "fp32")
        L.o = quantize(L.o.dequant().float() + 2.0 * g("o_proj", "B") @ g("o_proj", "A"), "fp32")
        w = L.gate_up.dequant().float()
        w[:cfg.ffn] += 2.0 * g("gate_proj", "B") @ g("gate_proj", "A")
        w[cfg.ffn:] += 2.0 * g("up_proj", "B") @ g("up_proj", "A")
        L.gate_up = quantize(w, "fp32")
        L.down = quantize(L.down.dequant().float() + 2.0 * g("down_proj", "B") @ g("down_proj", "A"), "fp32")
    merged, _ = m.forward_reference(toks)
    # (the reference linear rounds its input to bf16, the adapter path does not: small differences remain)
    assert (got - merged).abs().max() < 0.05 * (got - base).abs().max()


def test_tensor_parallel_slices_sum_to_the_unsharded_update():
    cfg = _cfg(q_heads=4, kv_heads=2, ffn=512)
    t = lora.random_adapter_tensors(cfg, 4, TARGETS, seed=5, std=0.1)
    full = lora.bind_adapter(t, cfg, 4, 4.0, "cpu")
    parts = [lora.bind_adapter(t, cfg, 4, 4.0, "cpu", tp_rank=r, tp_size=2) for r in range(2)]
    d = cfg.head_dim
    x = torch.randn(3, cfg.hidden).to(torch.bfloat16)
    # column-split: the ranks' output columns tile the unsharded output (q | k | v per rank)
    out_full = torch.zeros(3, (cfg.q_heads + 2 * cfg.kv_heads) * d, dtype=torch.bfloat16)
    full.apply(0, "qkv", x, out_full)
    nq, nkv = cfg.q_heads * d, cfg.kv_heads * d
    for r, ad in enumerate(parts):
        o = torch.zeros(3, (nq + 2 * nkv) // 2, dtype=torch.bfloat16)
        ad.apply(0, "qkv", x, o)
        want = torch.cat([out_full[:, r * nq // 2:(r + 1) * nq // 2], out_full[:, nq + r * nkv // 2: nq + (r + 1) * nkv // 2],
                          out_full[:, nq + nkv + r * nkv // 2: nq + nkv + (r + 1) * nkv // 2]], dim=1)
        assert torch.equal(o, want)
    # row-split: the ranks' updates add up to the unsharded one (fp32 sum, then compare loosely: bf16 partials)
    act = torch.randn(3, cfg.ffn).to(torch.bfloat16)
    want = torch.zeros(3, cfg.hidden, dtype=torch.bfloat16)
    full.apply(0, "down", act, want)
    acc = torch.zeros(3, cfg.hidden)
    for r, ad in enumerate(parts):
        o = torch.zeros(3, cfg.hidden, dtype=torch.bfloat16)
        ad.apply(0, "down", act[:, r * cfg.ffn // 2:(r + 1) * cfg.ffn // 2].contiguous(), o)
        acc += o.float()
    assert torch.allclose(acc, want.float(), rtol=2e-2, atol=2e-2)
