"""Checkpoints of the smaller model families in this library's own layout: one safetensors file holding every weight
under its path in the model object (`layers.3.qkv.payload`, `layers.3.moe.experts_gu.5.scale`, ...) plus a
`config.json` that names the family (`model_type` = "dgpp-<family>") and carries the configuration and the format of
every quantised matrix.  `save_family` writes one; `load_family` rebuilds the model on a device.  Quantised payloads
and scales travel byte for byte.  The fixture writer of the per-family load / bind / forward checks, and the hand-off
format between a conversion script and the server for these families.
(reference counterparts: src/models/*/loader.cpp + binding.cpp per family, tools' fixture writers; there every family
 binds its publisher's tensor names, which this build does for the dense family only.)
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Callable, Dict, Iterator, Tuple

import torch

from ..quant.formats import QuantLinear
from .checkpoint import open_checkpoint, write_safetensors


def _registry() -> Dict[str, Tuple[type, type]]:
    from ..models.dory import DoryConfig, DoryModel
    from ..models.flash_next import FlashNextConfig, FlashNextModel
    from ..models.glm_flash import GlmFlashConfig, GlmFlashModel
    from ..models.mimo import MimoConfig, MimoModel
    from ..models.minimax import MinimaxConfig, MinimaxModel

    return {"glm_flash": (GlmFlashConfig, GlmFlashModel), "dory": (DoryConfig, DoryModel),
            "flash_next": (FlashNextConfig, FlashNextModel), "minimax": (MinimaxConfig, MinimaxModel),
            "mimo": (MimoConfig, MimoModel)}


def _nested() -> Dict[str, type]:
    from ..models.engram import EngramConfig
    from ..models.flash_next import QsaConfig
    from ..models.moe import MoEConfig

    return {"moe": MoEConfig, "engram": EngramConfig, "qsa": QsaConfig}


# fields that are rebuilt from the stored ones (stacked expert views, kernel views of the shared expert)
_DERIVED = {"gu_q", "gu_sf", "gu_alpha", "down_q", "down_sf", "down_alpha", "shared_gu_k", "shared_down_k", "shared_stacked"}


def _children(obj: Any) -> Iterator[Tuple[str, Any, Callable[[Any], None]]]:
    """(name, value, setter) of every member of a container node."""
    if isinstance(obj, (list, tuple)):
        for i, v in enumerate(obj):
            yield str(i), v, (lambda nv, i=i: obj.__setitem__(i, nv))
    elif isinstance(obj, dict):
        for k, v in obj.items():
            yield str(k), v, (lambda nv, k=k: obj.__setitem__(k, nv))
    else:
        for k, v in vars(obj).items():
            if k.startswith("_") or k in ("cfg", "c") or k in _DERIVED:
                continue
            yield k, v, (lambda nv, k=k: setattr(obj, k, nv))


def _walk(obj: Any, prefix: str = "") -> Iterator[Tuple[str, Any, Callable[[Any], None]]]:
    """Leaves (tensors and quantised matrices) of a model object tree, depth first in attribute order."""
    for name, v, setter in _children(obj):
        path = f"{prefix}{name}"
        if isinstance(v, (torch.Tensor, QuantLinear)):
            yield path, v, setter
        elif isinstance(v, (list, tuple, dict)) or dataclasses.is_dataclass(v) or (hasattr(v, "__dict__") and not callable(v)
                                                                                   and type(v).__module__.startswith("dgpp_b200")):
            yield from _walk(v, path + ".")


def _family_of(model: Any) -> str:
    for name, (_, cls) in _registry().items():
        if type(model) is cls:
            return name
    raise ValueError(f"{type(model).__name__} is not one of the families with a native checkpoint layout")


def _cfg_dict(cfg: Any) -> dict:
    return json.loads(json.dumps(dataclasses.asdict(cfg)))          # tuples become lists, nested dataclasses dicts


def _cfg_build(cls: type, d: dict) -> Any:
    nested, kw = _nested(), {}
    names = {f.name: f for f in dataclasses.fields(cls)}
    for k, v in d.items():
        if k not in names:
            raise ValueError(f"{cls.__name__} has no field {k!r}")
        if isinstance(v, dict) and k in nested:
            v = _cfg_build(nested[k], v)
        elif isinstance(v, list) and isinstance(names[k].default, tuple):
            v = tuple(v)
        kw[k] = v
    return cls(**kw)


def save_family(model: Any, out_dir: str) -> None:
    family = _family_of(model)
    tensors: Dict[str, torch.Tensor] = {}
    quant: Dict[str, dict] = {}
    for path, v, _ in _walk(model):
        if isinstance(v, QuantLinear):
            tensors[path + ".payload"] = v.payload
            if v.scale is not None:
                tensors[path + ".scale"] = v.scale
            quant[path] = {"fmt": v.fmt, "n": v.n, "k": v.k, "alpha": float(v.alpha)}
        else:
            tensors[path] = v
    os.makedirs(out_dir, exist_ok=True)
    extra = {}
    if getattr(model, "engram", None) is not None:
        extra["engram_pad_class"] = int(model.engram.pad_class)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump({"model_type": f"dgpp-{family}", "architectures": [type(model).__name__], "config": _cfg_dict(model.cfg),
                   "quant": quant, **extra}, f, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors, {"format": "pt"})


def load_family(spec: str, device="cuda") -> Any:
    """Rebuilds the model a `save_family` directory holds.  The object tree comes from the family's own constructor
    (every member then takes the stored bytes), so the configuration alone decides which tensors must exist: a missing
    or mis-shaped one is an error that names it."""
    ck = open_checkpoint(spec)
    mt = ck.config.get("model_type", "")
    if not mt.startswith("dgpp-") or mt[5:] not in _registry():
        raise ValueError(f"{spec}: model_type {mt!r} is not a native family checkpoint")
    cfg_cls, model_cls = _registry()[mt[5:]]
    cfg = _cfg_build(cfg_cls, ck.config["config"])
    model = model_cls.random_init(cfg, "cpu", seed=0)
    quant = ck.config.get("quant", {})
    seen = set()
    for path, v, setter in _walk(model):
        if isinstance(v, QuantLinear):
            meta = quant.get(path)
            if meta is None or not ck.has(path + ".payload"):
                raise ValueError(f"{spec}: quantised matrix {path} is missing")
            if (meta["n"], meta["k"]) != (v.n, v.k):
                raise ValueError(f"{spec}: {path} is {meta['n']} x {meta['k']}, the configuration wants {v.n} x {v.k}")
            scale = ck.tensor(path + ".scale").clone().to(device) if ck.has(path + ".scale") else None
            setter(QuantLinear(meta["fmt"], v.n, v.k, ck.tensor(path + ".payload").clone().to(device), scale, meta["alpha"]))
            seen.update((path + ".payload", path + ".scale"))
        else:
            if not ck.has(path):
                raise ValueError(f"{spec}: tensor {path} is missing")
            t = ck.tensor(path)
            if tuple(t.shape) != tuple(v.shape) or t.dtype != v.dtype:
                raise ValueError(f"{spec}: {path} is {t.dtype} {tuple(t.shape)}, the configuration wants {v.dtype} {tuple(v.shape)}")
            setter(t.clone().to(device))
            seen.add(path)
    stray = [n for n in ck.names() if n not in seen]
    if stray:
        raise ValueError(f"{spec}: tensors the configuration does not use: {stray[:4]}{' ...' if len(stray) > 4 else ''}")
    if getattr(model, "engram", None) is not None:
        model.engram.pad_class = int(ck.config.get("engram_pad_class", model.engram.pad_class))
    _restack(model, device)
    return model


def _restack(obj: Any, device) -> None:
    """Expert matrices of block-scaled formats are stacked for the grouped GEMM once they sit on a GPU."""
    from ..models.moe import MoEWeights

    if isinstance(obj, MoEWeights):
        if torch.device(device).type == "cuda" and obj.experts_gu and obj.experts_gu[0].fmt in ("nvfp4", "mxfp4"):
            obj.stack()
        return
    for _, v, _s in _children(obj):
        if isinstance(v, (list, tuple, dict)) or dataclasses.is_dataclass(v) or (hasattr(v, "__dict__") and not callable(v)
                                                                                 and type(v).__module__.startswith("dgpp_b200")):
            _restack(v, device)


def runner_for(model: Any, max_rows: int, slots: int, max_seq_len: int, device="cuda") -> Any:
    """The kernel runner of a family model (what `engine.adapters.RunnerEngine` drives)."""
    from ..models.dory import DoryRunner
    from ..models.flash_next import FlashNextRunner
    from ..models.glm_flash import GlmFlashRunner
    from ..models.mimo import MimoRunner
    from ..models.minimax import MinimaxRunner

    cls = {"glm_flash": GlmFlashRunner, "dory": DoryRunner, "flash_next": FlashNextRunner, "minimax": MinimaxRunner,
           "mimo": MimoRunner}[_family_of(model)]
    return cls(model, max_rows, slots, max_seq_len, device)


def tiny_model(family: str, device="cpu", seed: int = 0, vocab: int = 4096) -> Any:
    """A small random-init model of `family` (the shapes the server's `--model <family>-tiny` choices use)."""
    from ..models.moe import MoEConfig

    cfg_cls, model_cls = _registry()[family]
    moe = MoEConfig(hidden=512, experts=16, top_k=2, moe_ffn=512, shared_ffn=512)
    if family == "glm_flash":
        cfg = cfg_cls(layers=4, hidden=512, vocab=vocab, mla_every=2, k_heads=2, v_heads=4, heads=8, q_lora=256, kv_lora=128,
                      nope=64, rope=32, v_dim=64, ffn=1024, moe=moe)
    elif family == "dory":
        cfg = cfg_cls(vocab=vocab)
    elif family == "flash_next":
        cfg = cfg_cls(vocab=vocab, moe=moe)
    elif family == "minimax":
        cfg = cfg_cls(vocab=vocab, moe_layers=[False, True, True, True],
                      moe=MoEConfig(hidden=512, experts=16, top_k=2, moe_ffn=512, shared_ffn=512, routed_scaling=2.0,
                                    swiglu_limit=7.0, swiglu_alpha=1.702))
    else:
        cfg = cfg_cls(vocab=vocab, moe=MoEConfig(hidden=512, experts=16, top_k=2, moe_ffn=512))
    return model_cls.random_init(cfg, device, seed=seed)


def main(argv=None) -> int:
    """Writes a small random-init checkpoint of one family: a fixture for the load / forward checks and for
    `python -m dgpp_b200.serve.app --family-dir DIR`."""
    import argparse

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--family", required=True, choices=sorted(_registry()))
    ap.add_argument("--out", required=True)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--vocab", type=int, default=4096)
    ap.add_argument("--check", action="store_true", help="load the directory back and compare the oracle logits of a short prompt")
    a = ap.parse_args(argv)
    model = tiny_model(a.family, "cpu", a.seed, a.vocab)
    save_family(model, a.out)
    report = {"family": a.family, "out": a.out, "tensors": sum(1 for _ in _walk(model))}
    if a.check:
        back = load_family(a.out, "cpu")
        t = torch.arange(3, 19) % a.vocab
        report["round_trip_equal"] = bool(torch.equal(back.forward_reference(t), model.forward_reference(t)))
    print(json.dumps(report))
    return 0 if report.get("round_trip_equal", True) else 1


if __name__ == "__main__":
    raise SystemExit(main())
