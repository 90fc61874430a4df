"""ctypes binding of ``libdgpp_kernels.so`` (plain C ABI, no torch headers).

The library is loaded lazily.  On a machine with a GPU a missing library is an error, never a
silent fallback: the ops in this package are the CUDA kernels, the PyTorch restatements live in
``dgpp_b200.ops.reference`` and are only used as test oracles and on CPU-only hosts.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libdgpp_kernels.so"

P = C.c_void_p
I = C.c_int
L = C.c_int64
F = C.c_float

_SIGNATURES = {
    "dgpp_status_read": [P],
    "dgpp_status_clear": [],
    "dgpp_embed_gather": [P, P, P, I, I, I, P],
    "dgpp_rmsnorm": [P, P, P, P, P, I, I, F, I, P],
    "dgpp_swiglu": [P, P, I, I, F, F, P],
    "dgpp_argmax": [P, I, L, I, I, I, P, P, P],
    "dgpp_copy_bytes": [P, P, L, P],
    "dgpp_add_bf16": [P, P, P, L, P],
    "dgpp_gemv_quant": [I, P, P, P, F, P, P, I, I, I, L, L, P],
    "dgpp_rope_kv_write": [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, F, I, I, P],
    "dgpp_attn_decode": [P, L, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P],
    "dgpp_attn_decode_sink": [P, L, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P, P],
    "dgpp_attn_decode_sparse": [P, L, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P, I, I, P],
    "dgpp_engram_embed": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, L, P],
    "dgpp_engram_gate": [P, P, P, P, I, I, I, F, P],
    "dgpp_msa_index_prep": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P],
    "dgpp_qsa_compress": [P, P, P, P, P, P, P, I, I, I, I, I, F, I, P],
    "dgpp_qsa_select": [P, L, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P],
    "dgpp_msa_index_select": [P, L, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P],
    "dgpp_attn_decode_tc": [P, L, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P, I, I, P],
    "dgpp_attn_prefill_tc": [P, L, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P],
    "dgpp_attn_prefill_tc256": [P, L, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P],
    "dgpp_decode_advance": [P, P, P, P, P, I, I, P],
    "dgpp_act_quant_nvfp4": [I, P, L, P, P, P, P, P, P, P, I, I, I, I, I, F, F, F, I, P],
    "dgpp_attn_combine_quant": [P, P, I, I, I, P, P, P, P, I, I, I, I, I, P],
    "dgpp_act_quant_nvfp4_cluster": [I, P, L, P, P, P, P, P, P, P, I, I, I, I, I, I, F, F, F, I, P, P, I, P],
    "dgpp_gemm_fp4_set_prefetch": [P, L],
    "dgpp_gemm_fp4_set_preload": [I],
    "dgpp_vis_patchify": [P, P, I, I, I, I, P, P, P],
    "dgpp_layernorm": [P, P, P, P, I, I, F, P],
    "dgpp_bias_act": [P, P, P, I, I, I, P],
    "dgpp_vis_qkv_split_rope": [P, P, P, P, P, P, P, I, I, I, I, F, P],
    "dgpp_softmax_rows": [P, I, I, I, P],
    "dgpp_gemm_fp4_set_trace": [P],
    "dgpp_gemm_fp4": [I, P, P, P, I, I, P, P, F, P, P, P, I, I, I, I, I, P, P, P, P],
    "dgpp_graph_begin_capture": [P],
    "dgpp_graph_launch": [P, P],
    "dgpp_graph_destroy": [P],
    "dgpp_gemm_tc": [I, I, I, P, L, P, P, F, P, P, P, I, I, I, I, I, P, P, P],
    "dgpp_gemm_tc_push": [I, I, I, P, L, P, P, F, I, I, I, P, P],
    "dgpp_gemm_tc_ag": [I, I, I, P, P, P, F, P, P, I, I, I, I, I, P, P, P],
}


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def load():
    """Return the loaded kernel library, building nothing (see ``dgpp_b200.build``)."""
    global _LIB
    if _LIB is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: run `python -m dgpp_b200.build` (nvcc, sm_100a) before using CUDA ops")
        lib = C.CDLL(str(_LIB_PATH), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL") else C.DEFAULT_MODE)
        lib.dgpp_last_error.restype = C.c_char_p
        lib.dgpp_last_error.argtypes = []
        lib.dgpp_status_device_ptr.restype = P
        lib.dgpp_status_device_ptr.argtypes = []
        _LIB = lib
    return _LIB


def declare(name: str, argtypes) -> None:
    """Register the signature of an exported function (used by modules that add kernels)."""
    _SIGNATURES[name] = list(argtypes)


def _fn(name: str):
    lib = load()
    fn = getattr(lib, name)
    if not getattr(fn, "_dgpp_typed", False):
        fn.argtypes = _SIGNATURES[name]
        fn.restype = I
        fn._dgpp_typed = True
    return fn


def ptr(t) -> int | None:
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def stream_ptr(stream=None) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return stream.cuda_stream


def call(name: str, *args) -> None:
    rc = _fn(name)(*args)
    if rc != 0:
        raise RuntimeError(f"{name}: {load().dgpp_last_error().decode()}")


def check_status(clear: bool = True) -> None:
    """Synchronise and raise if any kernel reported a bounded-wait expiry or bad argument."""
    buf = (C.c_int * 4)()
    call("dgpp_status_read", C.cast(buf, P))
    if buf[0] != 0:
        if clear:
            call("dgpp_status_clear")
        raise RuntimeError(f"device status code={buf[0]} count={buf[1]} detail={buf[2]}")
