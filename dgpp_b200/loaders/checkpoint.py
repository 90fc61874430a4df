"""Checkpoints: safetensors directories read through the native mmap reader, bound to model weights as stored.

* ``open_checkpoint(spec)`` resolves a directory or ``org/name`` hub-cache id, parses ``config.json`` and detects
  the model family natively.
* ``load_dense`` binds a Hugging Face style dense GQA decoder (Qwen3 / GLM-4 / Llama naming) to ``DenseModel``.
  Quantised tensors are sliced for the tensor-parallel rank and uploaded byte for byte: NVFP4
  (``weight`` packed e2m1 + ``weight_scale`` e4m3 per 16 + fp32 global), MXFP4 (e8m0 per 32), FP8 block
  (``weight_scale_inv`` fp32 per 128 x 128), bf16.  K slices must start on a scale-group boundary.
* ``save_dense`` writes the same layout (round-trip tests, synthetic checkpoints for the serving app).
(reference counterparts: src/loaders/safetensors.hpp, src/models/qwen/binding35.cpp, loader35.cpp,
 src/models/quant_matrix.hpp:99-143,279-281.)
"""
from __future__ import annotations

import json
import os
import warnings
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..models.dense import DenseConfig, DenseLayer, DenseModel, padded_q_heads
from ..quant.formats import QuantLinear
from ..runtime import rt

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64,
    "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
    "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2, "F8_E8M0": torch.uint8,
}
_NAMES = {v: k for k, v in _DTYPES.items() if k != "F8_E8M0"}


@dataclass
class OpenCheckpoint:
    dir: str
    config: dict
    family: str
    ckpt: "rt.Checkpoint"

    def names(self) -> List[str]:
        return self.ckpt.names()

    def has(self, name: str) -> bool:
        return self.ckpt.has(name)

    def tensor(self, name: str) -> torch.Tensor:
        """Zero-copy CPU tensor over the file mapping (read-only: clone or upload before writing)."""
        info = self.ckpt.info(name)
        view, owner = self.ckpt.view(name)
        dt = _DTYPES[info["dtype"]]
        if info["nbytes"] == 0:
            return torch.empty(info["shape"], dtype=dt)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.frombuffer(view, dtype=torch.uint8)
        t = t.view(dt).view(info["shape"])
        t._dgpp_owner = owner          # keeps the mapping alive as long as the tensor
        return t


def open_checkpoint(spec: str, cache_root: str = "") -> OpenCheckpoint:
    d = rt.resolve_model(spec, cache_root)
    with open(os.path.join(d, "config.json")) as f:
        raw = f.read()
    return OpenCheckpoint(d, json.loads(raw), rt.detect_family(raw), rt.Checkpoint(d))


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    items = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        items.append((name, _NAMES[t.dtype], list(t.shape), t.view(torch.uint8).reshape(-1).numpy()))
    rt.write_safetensors(path, items, metadata or {})


# ---------------------------------------------------------------------------------------------------- dense GQA
def dense_config_from_hf(cfg: dict, weight_fmt: Optional[str] = None) -> DenseConfig:
    cfg = cfg.get("text_config", cfg)
    q = cfg.get("quantization_config") or {}
    fmt = weight_fmt or {"nvfp4": "nvfp4", "mxfp4": "mxfp4", "fp8": "fp8", "mxfp8": "mxfp8", "int4": "int4", "int8": "int8"}.get(
        str(q.get("quant_algo") or q.get("quant_method") or q.get("format") or "").lower().replace("-", ""), "bf16")
    if not weight_fmt and str(q.get("format", "")).lower() == "pack-quantized":
        groups = q.get("config_groups") or {}
        bits = next((g.get("weights", {}).get("num_bits") for g in groups.values() if g.get("weights")), 4)
        fmt = "int8" if bits == 8 else "int4"
    heads = cfg["num_attention_heads"]
    rope = cfg.get("rope_scaling") or {}
    hd = cfg.get("head_dim") or cfg["hidden_size"] // heads
    return DenseConfig(
        layers=cfg["num_hidden_layers"], hidden=cfg["hidden_size"], q_heads=heads,
        kv_heads=cfg.get("num_key_value_heads", heads), head_dim=hd, ffn=cfg["intermediate_size"],
        vocab=cfg["vocab_size"], rope_theta=float(cfg.get("rope_theta", 1e4)),
        rot_dim=int(hd * cfg["partial_rotary_factor"]) if cfg.get("partial_rotary_factor") else None,
        eps=float(cfg.get("rms_norm_eps", 1e-6)), qk_norm=bool(cfg.get("qk_norm", cfg.get("use_qk_norm", False))),
        weight_fmt=fmt, head_fmt="bf16",
        yarn_factor=float(rope.get("factor", 1.0)) if rope.get("type", rope.get("rope_type")) == "yarn" else 1.0,
        yarn_original_max_pos=int(rope.get("original_max_position_embeddings", 0)),
        name=str(cfg.get("_name_or_path") or cfg.get("model_type") or "dense"))


_GROUP = {"nvfp4": 16, "mxfp4": 32, "fp8": 128, "mxfp8": 32, "int8": 64, "int4": 64, "bf16": 1, "fp32": 1}


def _read_linear(ck: OpenCheckpoint, prefix: str, fmt: str, rows: Optional[Tuple[int, int]], cols: Optional[Tuple[int, int]],
                 device) -> QuantLinear:
    """One [N, K] projection sliced to rows [r0, r1) and / or K columns [c0, c1), still in storage format."""
    if fmt in ("int4", "int8"):
        # pack-quantized release: offset-binary codes packed little-endian into int32 words (8 or 4 per word) in
        # `.weight_packed` (or plain bytes in `.weight`), one bf16 scale per 64 in `.weight_scale`
        name = prefix + (".weight_packed" if ck.has(prefix + ".weight_packed") else ".weight")
        raw = ck.tensor(name)
        per_byte = 2 if fmt == "int4" else 1
        by = raw.view(torch.uint8).view(raw.shape[0], -1)
        n_full, k_full = by.shape[0], by.shape[1] * per_byte
        r0, r1 = rows or (0, n_full)
        c0, c1 = cols or (0, k_full)
        if c0 % 64 or c1 % 64:
            raise ValueError(f"{prefix}: K slice [{c0}, {c1}) does not start / end on a 64-wide scale group")
        payload = by[r0:r1, c0 // per_byte:c1 // per_byte].contiguous().to(device)
        sc = ck.tensor(prefix + ".weight_scale")
        if sc.shape[1] * 64 != k_full:
            raise ValueError(f"{prefix}: scales of group size {k_full // sc.shape[1]}; this engine streams group 64")
        s = sc[r0:r1, c0 // 64:c1 // 64].to(torch.bfloat16).contiguous().to(device)
        return QuantLinear(fmt, r1 - r0, c1 - c0, payload, s)
    w = ck.tensor(prefix + ".weight")
    n_full = w.shape[0]
    r0, r1 = rows or (0, n_full)
    if fmt in ("bf16", "fp32"):
        c0, c1 = cols or (0, w.shape[1])
        dt = torch.float32 if fmt == "fp32" else torch.bfloat16
        return QuantLinear(fmt, r1 - r0, c1 - c0, w[r0:r1, c0:c1].to(dt).contiguous().to(device))
    k_full = w.shape[1] * (2 if fmt in ("nvfp4", "mxfp4") else 1)
    c0, c1 = cols or (0, k_full)
    g = _GROUP[fmt]
    if c0 % g or c1 % g:
        raise ValueError(f"{prefix}: K slice [{c0}, {c1}) does not start / end on a {g}-wide scale group")
    if fmt in ("nvfp4", "mxfp4"):
        payload = w.view(torch.uint8)[r0:r1, c0 // 2:c1 // 2].contiguous().to(device)
        s = ck.tensor(prefix + ".weight_scale").view(torch.uint8)[r0:r1, c0 // g:c1 // g].contiguous().to(device)
        alpha = 1.0
        if fmt == "nvfp4":
            if ck.has(prefix + ".weight_scale_2"):
                alpha = float(ck.tensor(prefix + ".weight_scale_2").float().reshape(-1)[0])
            elif ck.has(prefix + ".weight_global_scale"):
                alpha = 1.0 / float(ck.tensor(prefix + ".weight_global_scale").float().reshape(-1)[0])
        return QuantLinear(fmt, r1 - r0, c1 - c0, payload, s, alpha)
    if fmt == "mxfp8":
        payload = w.view(torch.uint8)[r0:r1, c0:c1].contiguous().to(device)
        s = ck.tensor(prefix + ".weight_scale").view(torch.uint8)[r0:r1, c0 // 32:c1 // 32].contiguous().to(device)
        return QuantLinear(fmt, r1 - r0, c1 - c0, payload, s)
    if fmt == "fp8":
        if r0 % 128 or (r1 % 128 and r1 != n_full):
            raise ValueError(f"{prefix}: fp8 block rows [{r0}, {r1}) must be aligned to 128")
        payload = w.view(torch.uint8)[r0:r1, c0:c1].contiguous().to(device)
        s = ck.tensor(prefix + ".weight_scale_inv").float()[r0 // 128:(r1 + 127) // 128, c0 // 128:(c1 + 127) // 128]
        return QuantLinear(fmt, r1 - r0, c1 - c0, payload, s.contiguous().to(device))
    raise ValueError(f"unsupported weight format {fmt}")


def _pad(w: QuantLinear, rows: int = 0, cols: int = 0) -> QuantLinear:
    """Appends zero rows / zero K columns in storage format (zero codes, zero block scales): padding channels that
    keep a tensor-parallel shard on the GEMM's K granule contribute exact zeros."""
    if not rows and not cols:
        return w
    assert w.fmt in ("nvfp4", "mxfp4", "bf16", "fp32"), "padding is defined on fp4 / unquantised shards"
    pay, sc = w.payload, w.scale
    if w.fmt in ("nvfp4", "mxfp4"):
        grp = 16 if w.fmt == "nvfp4" else 32
        sc = sc.view(w.n, w.k // grp)
        if cols:
            pay = torch.cat([pay, pay.new_zeros(w.n, cols // 2)], 1)
            sc = torch.cat([sc, sc.new_zeros(w.n, cols // grp)], 1)
        if rows:
            pay = torch.cat([pay, pay.new_zeros(rows, pay.shape[1])])
            sc = torch.cat([sc, sc.new_zeros(rows, sc.shape[1])])
        return QuantLinear(w.fmt, w.n + rows, w.k + cols, pay.contiguous(), sc.contiguous(), w.alpha)
    if cols:
        pay = torch.cat([pay, pay.new_zeros(w.n, cols)], 1)
    if rows:
        pay = torch.cat([pay, pay.new_zeros(rows, pay.shape[1])])
    return QuantLinear(w.fmt, w.n + rows, w.k + cols, pay.contiguous())


def _cat(parts: List[QuantLinear]) -> QuantLinear:
    """Stack projections along N (q|k|v, gate|up).  NVFP4 tensors keep their own global scale, so differing
    globals are folded into the e4m3 block scales only when they are equal; otherwise the caller keeps them apart."""
    p0 = parts[0]
    if len({round(p.alpha, 12) for p in parts}) != 1:
        raise ValueError("projections with different NVFP4 global scales cannot be stacked without re-encoding")
    payload = torch.cat([p.payload for p in parts])
    scale = None if p0.scale is None else torch.cat([p.scale for p in parts])
    return QuantLinear(p0.fmt, sum(p.n for p in parts), p0.k, payload, scale, p0.alpha)


def load_dense(spec: str, device="cuda", tp_rank: int = 0, tp_size: int = 1, weight_fmt: Optional[str] = None,
               cache_root: str = "") -> DenseModel:
    ck = open_checkpoint(spec, cache_root)
    cfg = dense_config_from_hf(ck.config, weight_fmt)
    W, r, d, H = tp_size, tp_rank, cfg.head_dim, cfg.hidden
    assert cfg.q_heads % W == 0 and cfg.kv_heads % W == 0 and cfg.ffn % W == 0 and cfg.vocab % W == 0
    hq_l, hkv_l, ffn_l, vl = cfg.q_heads // W, cfg.kv_heads // W, cfg.ffn // W, cfg.vocab // W
    adt = torch.float32 if cfg.weight_fmt == "fp32" else torch.bfloat16
    dev = torch.device(device)

    def vec(name):
        return ck.tensor(name).to(adt).to(dev)

    fmt = cfg.weight_fmt
    # the same padding DenseModel.random_init applies to tensor-parallel NVFP4 shards
    q_pad = (padded_q_heads(cfg, W) - hq_l) * d
    ffn_pad = (-ffn_l) % 256 if (W > 1 and fmt in ("nvfp4", "mxfp4")) else 0
    layers = []
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        q = _read_linear(ck, p + "self_attn.q_proj", fmt, (r * hq_l * d, (r + 1) * hq_l * d), None, dev)
        k = _read_linear(ck, p + "self_attn.k_proj", fmt, (r * hkv_l * d, (r + 1) * hkv_l * d), None, dev)
        v = _read_linear(ck, p + "self_attn.v_proj", fmt, (r * hkv_l * d, (r + 1) * hkv_l * d), None, dev)
        o = _read_linear(ck, p + "self_attn.o_proj", fmt, None, (r * hq_l * d, (r + 1) * hq_l * d), dev)
        g = _read_linear(ck, p + "mlp.gate_proj", fmt, (r * ffn_l, (r + 1) * ffn_l), None, dev)
        u = _read_linear(ck, p + "mlp.up_proj", fmt, (r * ffn_l, (r + 1) * ffn_l), None, dev)
        dn = _read_linear(ck, p + "mlp.down_proj", fmt, None, (r * ffn_l, (r + 1) * ffn_l), dev)
        qn = vec(p + "self_attn.q_norm.weight") if cfg.qk_norm and ck.has(p + "self_attn.q_norm.weight") else None
        kn = vec(p + "self_attn.k_norm.weight") if cfg.qk_norm and ck.has(p + "self_attn.k_norm.weight") else None
        layers.append(DenseLayer(vec(p + "input_layernorm.weight"), vec(p + "post_attention_layernorm.weight"),
                                 _cat([_pad(q, rows=q_pad), k, v]), _pad(o, cols=q_pad),
                                 _cat([_pad(g, rows=ffn_pad), _pad(u, rows=ffn_pad)]), _pad(dn, cols=ffn_pad), qn, kn))
    embed = vec("model.embed_tokens.weight")
    head_name = "lm_head" if ck.has("lm_head.weight") else "model.embed_tokens"
    head = _read_linear(ck, head_name, cfg.head_fmt, (r * vl, (r + 1) * vl), None, dev)
    m = DenseModel(cfg, embed, layers, vec("model.norm.weight"), head, tp_rank, tp_size)
    m._init_rope(dev)
    return m


def save_dense(model: DenseModel, out_dir: str, shard_layers: int = 0) -> None:
    """Write an unsharded (tp_size 1) DenseModel as config.json + safetensors (one file, or one file per
    `shard_layers` layers with an index)."""
    assert model.tp_size == 1
    cfg = model.cfg
    os.makedirs(out_dir, exist_ok=True)
    d = cfg.head_dim
    nq, nkv = cfg.q_heads * d, cfg.kv_heads * d
    groups: Dict[str, Dict[str, torch.Tensor]] = {}

    def put(file: str, prefix: str, w: QuantLinear, r0: int, r1: int):
        g = groups.setdefault(file, {})
        if w.fmt == "bf12":      # a resident form only: checkpoints carry the bf16 tensor it stands for
            from ..quant.formats import bf12_decode
            w = QuantLinear("bf16", w.n, w.k, bf12_decode(w))
        if w.fmt in ("bf16", "fp32"):
            g[prefix + ".weight"] = w.payload[r0:r1]
            return
        if w.fmt == "fp8":
            g[prefix + ".weight"] = w.payload[r0:r1].view(torch.float8_e4m3fn)
            g[prefix + ".weight_scale_inv"] = w.scale[r0 // 128:(r1 + 127) // 128]
            return
        if w.fmt in ("int4", "int8"):
            g[prefix + ".weight_packed"] = w.payload[r0:r1].contiguous().view(torch.int32)
            g[prefix + ".weight_scale"] = w.scale.view(w.n, -1)[r0:r1]
            return
        g[prefix + ".weight"] = w.payload[r0:r1].view(torch.float8_e4m3fn) if w.fmt == "mxfp8" else w.payload[r0:r1]
        sc = w.scale.view(w.n, -1)[r0:r1]
        g[prefix + ".weight_scale"] = sc.view(torch.float8_e4m3fn) if w.fmt == "nvfp4" else sc
        if w.fmt == "nvfp4":
            g[prefix + ".weight_scale_2"] = torch.tensor([w.alpha], dtype=torch.float32)

    for i, L in enumerate(model.layers):
        f = "model.safetensors" if shard_layers <= 0 else f"model-{i // shard_layers:05d}.safetensors"
        p = f"model.layers.{i}."
        put(f, p + "self_attn.q_proj", L.qkv, 0, nq)
        put(f, p + "self_attn.k_proj", L.qkv, nq, nq + nkv)
        put(f, p + "self_attn.v_proj", L.qkv, nq + nkv, nq + 2 * nkv)
        put(f, p + "self_attn.o_proj", L.o, 0, L.o.n)
        put(f, p + "mlp.gate_proj", L.gate_up, 0, cfg.ffn)
        put(f, p + "mlp.up_proj", L.gate_up, cfg.ffn, 2 * cfg.ffn)
        put(f, p + "mlp.down_proj", L.down, 0, L.down.n)
        g = groups[f]
        g[p + "input_layernorm.weight"] = L.in_norm
        g[p + "post_attention_layernorm.weight"] = L.post_norm
        if L.q_norm is not None:
            g[p + "self_attn.q_norm.weight"] = L.q_norm
            g[p + "self_attn.k_norm.weight"] = L.k_norm
    first = "model.safetensors" if shard_layers <= 0 else "model-00000.safetensors"
    g = groups.setdefault(first, {})
    g["model.embed_tokens.weight"] = model.embed
    g["model.norm.weight"] = model.final_norm
    put(first, "lm_head", model.head, 0, model.head.n)
    weight_map = {}
    for f, tensors in groups.items():
        write_safetensors(os.path.join(out_dir, f), tensors, {"format": "pt"})
        weight_map.update({n: f for n in tensors})
    if shard_layers > 0:
        with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as fh:
            json.dump({"metadata": {}, "weight_map": weight_map}, fh)
    hf = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": cfg.layers,
          "hidden_size": cfg.hidden, "num_attention_heads": cfg.q_heads, "num_key_value_heads": cfg.kv_heads,
          "head_dim": cfg.head_dim, "intermediate_size": cfg.ffn, "vocab_size": cfg.vocab, "rope_theta": cfg.rope_theta,
          "rms_norm_eps": cfg.eps, "qk_norm": cfg.qk_norm}
    if cfg.weight_fmt not in ("bf16", "fp32"):
        hf["quantization_config"] = {"quant_algo": cfg.weight_fmt.upper()}
    if cfg.weight_fmt == "fp32":
        hf["torch_dtype"] = "float32"
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(hf, fh)
