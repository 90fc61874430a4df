"""Per-rank resident weight image: the rank's already sliced, padded and tiled weights in one file on local disk.

A restart then skips checkpoint parsing, tensor-parallel slicing and scale tiling: the file is read in large
sequential chunks into a pinned staging buffer and copied to the device tensor by tensor, each verified by CRC-32C.

Layout:  8-byte magic ``DGPPIMG1`` | u64 header length | header JSON | padding to 4096 | tensor bytes (each 4096-aligned)
Header:  {"key": <cache key>, "config": {...DenseConfig...}, "tp_rank", "tp_size",
          "tensors": [{"name", "dtype", "shape", "offset", "nbytes", "crc32c"}, ...],
          "linears": {"layers.0.qkv": {"fmt", "n", "k", "alpha"}, ...}}
The cache key binds an image to what it was built from (checkpoint identity + config digest + rank / world +
format version); a key mismatch, a truncated file or a CRC failure makes ``load_image`` return None and the caller
falls back to the checkpoint.
(reference counterparts: src/loaders/resident_image.cpp pre-sliced per-rank image with hash verification,
 src/loaders/resident_stream.hpp streaming builder, DGPP_RESIDENT_CACHE / _DIR / _VERIFY switches.)
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import os
import struct
from typing import Dict, Optional, Tuple

import torch

from ..models.dense import DenseConfig, DenseLayer, DenseModel
from ..quant.formats import QuantLinear
from ..runtime import rt

MAGIC = b"DGPPIMG1"
ALIGN = 4096
_DT = {"uint8": torch.uint8, "bfloat16": torch.bfloat16, "float32": torch.float32, "int32": torch.int32,
       "float16": torch.float16, "int8": torch.int8}


def image_key(source_id: str, cfg: DenseConfig, tp_rank: int, tp_size: int) -> str:
    """Identity of an image: what it was built from and for whom."""
    blob = json.dumps({"src": source_id, "cfg": dataclasses.asdict(cfg), "rank": tp_rank, "world": tp_size, "v": 1},
                      sort_keys=True)
    return hashlib.sha256(blob.encode()).hexdigest()


def _model_tensors(m: DenseModel) -> Tuple[Dict[str, torch.Tensor], Dict[str, dict]]:
    tensors: Dict[str, torch.Tensor] = {"embed": m.embed, "final_norm": m.final_norm}
    linears: Dict[str, dict] = {}

    def put_linear(name: str, w: QuantLinear):
        linears[name] = {"fmt": w.fmt, "n": w.n, "k": w.k, "alpha": float(w.alpha)}
        tensors[name + ".payload"] = w.payload
        if w.scale is not None:
            tensors[name + ".scale"] = w.scale
        if w.fmt == "nvfp4":
            tensors[name + ".scale_tiled"] = w.tiled_scales()

    put_linear("head", m.head)
    for i, L in enumerate(m.layers):
        p = f"layers.{i}."
        tensors[p + "in_norm"], tensors[p + "post_norm"] = L.in_norm, L.post_norm
        for nm in ("q_norm", "k_norm", "sink"):
            t = getattr(L, nm)
            if t is not None:
                tensors[p + nm] = t
        for nm in ("qkv", "o", "gate_up", "down"):
            put_linear(p + nm, getattr(L, nm))
    return tensors, linears


def save_image(model: DenseModel, path: str, key: str) -> int:
    """Write the image of this rank's model; returns the file size.  The file appears atomically (temp + rename)."""
    tensors, linears = _model_tensors(model)
    table, blobs, off = [], [], 0
    for name, t in tensors.items():
        raw = t.detach().contiguous().cpu().view(torch.uint8).reshape(-1).numpy().tobytes()
        table.append({"name": name, "dtype": str(t.dtype).replace("torch.", ""), "shape": list(t.shape), "offset": off,
                      "nbytes": len(raw), "crc32c": rt.crc32c(raw)})
        blobs.append(raw)
        off += (len(raw) + ALIGN - 1) // ALIGN * ALIGN
    header = json.dumps({"key": key, "config": dataclasses.asdict(model.cfg), "tp_rank": model.tp_rank,
                         "tp_size": model.tp_size, "tensors": table, "linears": linears}).encode()
    head_len = 16 + len(header)
    data0 = (head_len + ALIGN - 1) // ALIGN * ALIGN
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(MAGIC + struct.pack("<Q", len(header)) + header)
        f.write(b"\0" * (data0 - head_len))
        for raw in blobs:
            f.write(raw)
            f.write(b"\0" * ((-len(raw)) % ALIGN))
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)
    return os.path.getsize(path)


def load_image(path: str, key: str, device="cuda", verify: bool = True, chunk_bytes: int = 256 << 20) -> Optional[DenseModel]:
    """Rebuild the rank's model from its image, or None when the image is absent, stale or damaged."""
    try:
        f = open(path, "rb", buffering=0)
    except OSError:
        return None
    with f:
        head = f.read(16)
        if len(head) != 16 or head[:8] != MAGIC:
            return None
        (hlen,) = struct.unpack("<Q", head[8:])
        if hlen > (64 << 20):
            return None
        raw = f.read(hlen)
        if len(raw) != hlen:
            return None
        try:
            hdr = json.loads(raw)
        except ValueError:
            return None
        if hdr.get("key") != key:
            return None
        data0 = (16 + hlen + ALIGN - 1) // ALIGN * ALIGN
        size = os.fstat(f.fileno()).st_size
        dev = torch.device(device)
        pinned = dev.type == "cuda"
        out: Dict[str, torch.Tensor] = {}
        stage = torch.empty(chunk_bytes, dtype=torch.uint8, pin_memory=pinned) if pinned else None
        for t in hdr["tensors"]:
            n = t["nbytes"]
            if data0 + t["offset"] + n > size:
                return None
            dt = _DT[t["dtype"]]
            dst = torch.empty(n, dtype=torch.uint8, device=dev)
            f.seek(data0 + t["offset"])
            crc, done = 0, 0
            while done < n:
                m = min(chunk_bytes, n - done)
                if stage is not None:
                    buf = stage[:m].numpy()
                    got = f.readinto(memoryview(buf))
                    if got != m:
                        return None
                    if verify:
                        crc = rt.crc32c(buf.tobytes(), crc)
                    dst[done:done + m].copy_(stage[:m], non_blocking=True)
                    torch.cuda.current_stream().synchronize()      # the staging buffer is reused by the next chunk
                else:
                    b = f.read(m)
                    if len(b) != m:
                        return None
                    if verify:
                        crc = rt.crc32c(b, crc)
                    dst[done:done + m] = torch.frombuffer(bytearray(b), dtype=torch.uint8)
                done += m
            if verify and n and crc != t["crc32c"]:
                return None
            out[t["name"]] = dst.view(dt).view(t["shape"]) if n else torch.empty(t["shape"], dtype=dt, device=dev)

    def linear(name: str) -> QuantLinear:
        info = hdr["linears"][name]
        return QuantLinear(info["fmt"], info["n"], info["k"], out[name + ".payload"], out.get(name + ".scale"),
                           info["alpha"], out.get(name + ".scale_tiled"))

    cfg = DenseConfig(**hdr["config"])
    layers = []
    for i in range(cfg.layers):
        p = f"layers.{i}."
        layers.append(DenseLayer(out[p + "in_norm"], out[p + "post_norm"], linear(p + "qkv"), linear(p + "o"),
                                 linear(p + "gate_up"), linear(p + "down"), out.get(p + "q_norm"), out.get(p + "k_norm"),
                                 out.get(p + "sink"), cfg.layer_window(i)))
    m = DenseModel(cfg, out["embed"], layers, out["final_norm"], linear("head"), hdr["tp_rank"], hdr["tp_size"])
    m._init_rope(dev)
    return m


def load_or_build(build_fn, cache_dir: str, source_id: str, cfg: DenseConfig, device="cuda", tp_rank: int = 0,
                  tp_size: int = 1, verify: bool = True) -> Tuple[DenseModel, bool]:
    """The model from its resident image when one matches, else ``build_fn()`` (whose result is then cached).
    Returns (model, came_from_image)."""
    key = image_key(source_id, cfg, tp_rank, tp_size)
    path = os.path.join(cache_dir, f"image-{key[:16]}-r{tp_rank}of{tp_size}.bin")
    m = load_image(path, key, device, verify)
    if m is not None:
        return m, True
    m = build_fn()
    os.makedirs(cache_dir, exist_ok=True)
    save_image(m, path, key)
    return m, False
