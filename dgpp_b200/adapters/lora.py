"""Runtime low-rank adapters (LoRA) for the dense decoder.

An adapter is a directory with ``adapter_manifest.json`` and one safetensors file:

    {"format": "dgpp-lora-1", "rank": 16, "alpha": 32.0, "file": "adapter.safetensors",
     "sha256": "<hex digest of the file>", "targets": ["q_proj", "v_proj", "down_proj", ...]}

Tensors follow the PEFT naming: ``layers.{i}.{target}.lora_A`` [rank, in] and ``layers.{i}.{target}.lora_B``
[out, rank] in bf16; targets are q_proj / k_proj / v_proj / o_proj / gate_proj / up_proj / down_proj.  The file's
digest is checked before anything is bound.  The update of one projection is ``scale * (x A^T) B^T`` with
``scale = alpha / rank``, added to the projection's bf16 output by ``ops.lora_apply`` (fp32 rank-r intermediate).

Tensor parallelism: B is sliced with the rows of a column-split projection (q/k/v, gate/up: the update lands in the
rank's own output columns); A is sliced with the columns of a row-split projection (o, down): each rank adds the
update computed from its slice into its partial output and the projection's all-reduce sums them, so adapters add
no collective.  Zero padding of the model (padded query heads / intermediate channels) is mirrored with zero rows /
columns.
(reference counterparts: src/adapters/manifest.hpp sha256-checked artifact, src/adapters/runtime.hpp
 Runtime::project / Runtime::add, src/models/glm_dsa/modification_targets.cpp target table.)
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..models.dense import DenseConfig, DenseModel, padded_q_heads

BF = torch.bfloat16
TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


@dataclass
class LoraPair:
    a: torch.Tensor        # [rank, K_local] bf16
    b: torch.Tensor        # [N_local, rank] bf16
    col0: int              # first output column (of the fused local projection) the update is added to


@dataclass
class LoraAdapter:
    """Adapter bound to one tensor-parallel rank of one model: per layer, per fused projection, the list of pairs."""
    rank: int
    scale: float
    layers: List[Dict[str, List[LoraPair]]] = field(default_factory=list)   # proj in {"qkv", "o", "gate_up", "down"}
    name: str = "adapter"

    def pairs(self, layer: int, proj: str) -> List[LoraPair]:
        return self.layers[layer].get(proj, []) if layer < len(self.layers) else []

    def apply(self, layer: int, proj: str, x: torch.Tensor, out: torch.Tensor, scratch=None) -> None:
        """out[:, cols] += scale * (x A^T) B^T for every pair of (layer, proj).  CUDA tensors use the kernel;
        CPU tensors the PyTorch restatement (the oracle of the kernel)."""
        for p in self.pairs(layer, proj):
            view = out[:, p.col0:p.col0 + p.b.shape[0]]
            if x.is_cuda:
                from ..ops import core as ops
                ops.lora_apply(x, p.a, p.b, view, self.scale, scratch=scratch)
            else:
                view.copy_(lora_reference(x, p.a, p.b, view, self.scale))


def lora_reference(x, a, b, out, scale: float) -> torch.Tensor:
    """fp32 restatement: bf16(out + scale * (x A^T) B^T) with the rank-r intermediate in fp32."""
    y = x.float() @ a.float().t()
    return (out.float() + scale * (y @ b.float().t())).to(out.dtype)


def save_adapter(out_dir: str, tensors: Dict[str, torch.Tensor], rank: int, alpha: float, targets: List[str]) -> None:
    from ..loaders.checkpoint import write_safetensors
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "adapter.safetensors")
    write_safetensors(path, {k: v.to(BF) for k, v in tensors.items()}, {"format": "dgpp-lora-1"})
    manifest = {"format": "dgpp-lora-1", "rank": rank, "alpha": alpha, "file": "adapter.safetensors",
                "sha256": _sha256(path), "targets": list(targets)}
    with open(os.path.join(out_dir, "adapter_manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1)


def random_adapter_tensors(cfg: DenseConfig, rank: int, targets: List[str], seed: int = 0, std: float = 0.05):
    """Unsharded random adapter tensors of the right shapes (tests, benchmarks)."""
    g = torch.Generator().manual_seed(seed)
    d = cfg.head_dim
    dims = {"q_proj": (cfg.hidden, cfg.q_heads * d), "k_proj": (cfg.hidden, cfg.kv_heads * d),
            "v_proj": (cfg.hidden, cfg.kv_heads * d), "o_proj": (cfg.q_heads * d, cfg.hidden),
            "gate_proj": (cfg.hidden, cfg.ffn), "up_proj": (cfg.hidden, cfg.ffn), "down_proj": (cfg.ffn, cfg.hidden)}
    out = {}
    for i in range(cfg.layers):
        for t in targets:
            k, n = dims[t]
            out[f"layers.{i}.{t}.lora_A"] = (torch.randn(rank, k, generator=g) * std).to(BF)
            out[f"layers.{i}.{t}.lora_B"] = (torch.randn(n, rank, generator=g) * std).to(BF)
    return out


def _rows(t: torch.Tensor, lo: int, hi: int, pad: int) -> torch.Tensor:
    s = t[lo:hi]
    return torch.cat([s, s.new_zeros(pad, s.shape[1])]) if pad else s


def _cols(t: torch.Tensor, lo: int, hi: int, pad: int) -> torch.Tensor:
    s = t[:, lo:hi]
    return torch.cat([s, s.new_zeros(s.shape[0], pad)], dim=1) if pad else s


def bind_adapter(tensors: Dict[str, torch.Tensor], cfg: DenseConfig, rank: int, alpha: float, device, tp_rank: int = 0,
                 tp_size: int = 1, name: str = "adapter") -> LoraAdapter:
    """Slice unsharded adapter tensors for one tensor-parallel rank, mirroring the model's own slicing and padding."""
    W, r, d = tp_size, tp_rank, cfg.head_dim
    hq_l, hkv_l, ffn_l = cfg.q_heads // W, max(cfg.kv_heads // W, 1), cfg.ffn // W
    ffn_pad = (-ffn_l) % 256 if (W > 1 and cfg.weight_fmt in ("nvfp4", "mxfp4")) else 0
    q_pad = (padded_q_heads(cfg, W) - hq_l) * d
    nq_l, nkv_l, I_l = hq_l * d + q_pad, hkv_l * d, ffn_l + ffn_pad
    up = lambda t: t.to(BF).contiguous().to(device)
    ad = LoraAdapter(rank=rank, scale=float(alpha) / rank, name=name)
    for i in range(cfg.layers):
        L: Dict[str, List[LoraPair]] = {}

        def get(t):
            a, b = tensors.get(f"layers.{i}.{t}.lora_A"), tensors.get(f"layers.{i}.{t}.lora_B")
            if (a is None) != (b is None):
                raise ValueError(f"adapter: layers.{i}.{t} has only one of lora_A / lora_B")
            if a is not None and (a.shape[0] != rank or b.shape[1] != rank):
                raise ValueError(f"adapter: layers.{i}.{t} rank {a.shape[0]} / {b.shape[1]} != manifest rank {rank}")
            return a, b

        for t, lo, hi, pad, col0 in (("q_proj", r * hq_l * d, (r + 1) * hq_l * d, q_pad, 0),
                                     ("k_proj", r * hkv_l * d, (r + 1) * hkv_l * d, 0, nq_l),
                                     ("v_proj", r * hkv_l * d, (r + 1) * hkv_l * d, 0, nq_l + nkv_l)):
            a, b = get(t)
            if a is not None:
                L.setdefault("qkv", []).append(LoraPair(up(a), up(_rows(b, lo, hi, pad)), col0))
        a, b = get("o_proj")
        if a is not None:
            L.setdefault("o", []).append(LoraPair(up(_cols(a, r * hq_l * d, (r + 1) * hq_l * d, q_pad)), up(b), 0))
        for t, col0 in (("gate_proj", 0), ("up_proj", I_l)):
            a, b = get(t)
            if a is not None:
                L.setdefault("gate_up", []).append(LoraPair(up(a), up(_rows(b, r * ffn_l, (r + 1) * ffn_l, ffn_pad)), col0))
        a, b = get("down_proj")
        if a is not None:
            L.setdefault("down", []).append(LoraPair(up(_cols(a, r * ffn_l, (r + 1) * ffn_l, ffn_pad)), up(b), 0))
        ad.layers.append(L)
    return ad


def load_adapter(adapter_dir: str, cfg: DenseConfig, device="cuda", tp_rank: int = 0, tp_size: int = 1) -> LoraAdapter:
    """Read, verify (sha256) and bind an adapter directory."""
    from ..loaders.checkpoint import _DTYPES  # noqa: F401  (dtype table of the reader)
    from ..runtime import rt
    with open(os.path.join(adapter_dir, "adapter_manifest.json")) as f:
        man = json.load(f)
    if man.get("format") != "dgpp-lora-1":
        raise ValueError(f"adapter: unknown format {man.get('format')!r}")
    unknown = [t for t in man.get("targets", []) if t not in TARGETS]
    if unknown:
        raise ValueError(f"adapter: unknown targets {unknown}")
    path = os.path.join(adapter_dir, man["file"])
    digest = _sha256(path)
    if digest != man["sha256"]:
        raise ValueError(f"adapter: {man['file']} digest {digest[:12]}.. does not match the manifest {man['sha256'][:12]}..")
    st = rt.SafetensorsFile(path)
    tensors = {}
    for name in st.names():
        info = st.info(name)
        view, owner = st.view(name)
        t = torch.frombuffer(bytearray(view), dtype=torch.uint8).view(_DTYPES[info["dtype"]]).view(info["shape"])
        tensors[name] = t
    have = {n.split(".")[2] for n in tensors}
    if not have <= set(man["targets"]):
        raise ValueError(f"adapter: tensors for {sorted(have - set(man['targets']))} are not listed in the manifest")
    return bind_adapter(tensors, cfg, int(man["rank"]), float(man["alpha"]), device, tp_rank, tp_size,
                        name=os.path.basename(os.path.normpath(adapter_dir)))


def merged_reference_weights(w: torch.Tensor, a: torch.Tensor, b: torch.Tensor, scale: float) -> torch.Tensor:
    """W + scale * B A in fp32 (what the adapter is equivalent to on an unquantised weight)."""
    return w.float() + scale * (b.float() @ a.float())
