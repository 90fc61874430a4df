"""Releasable device ranges (csrc/engine/vmm_range.cu): a fixed virtual address range whose physical backing is committed
and released granule by granule.  ``ReleasableRange.tensor`` gives a torch view that stays valid across commits and
releases (touching a released part is an error, as with any unmapped address).
(reference counterpart: src/loaders/releasable_range.cpp.)
"""
from __future__ import annotations

import torch

from ..ops import _lib
from ..ops._lib import I, L, P, call

_lib.declare("dgpp_vmm_commit", [P, L, L])
_lib.declare("dgpp_vmm_release", [P, L, L])
_lib.declare("dgpp_vmm_destroy", [P])


class _Raw:
    """CUDA array interface over a raw device span (uint8)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class ReleasableRange:
    def __init__(self, nbytes: int):
        lib = _lib.load()
        lib.dgpp_vmm_create.restype = P
        lib.dgpp_vmm_create.argtypes = [L]
        for name in ("dgpp_vmm_ptr", "dgpp_vmm_size", "dgpp_vmm_granule", "dgpp_vmm_committed"):
            getattr(lib, name).restype = L
            getattr(lib, name).argtypes = [P]
        self._lib = lib
        self.handle = lib.dgpp_vmm_create(int(nbytes))
        if not self.handle:
            raise RuntimeError("vmm_create: " + lib.dgpp_last_error().decode())
        self.ptr, self.size, self.granule = lib.dgpp_vmm_ptr(self.handle), lib.dgpp_vmm_size(self.handle), lib.dgpp_vmm_granule(self.handle)

    def commit(self, offset: int, nbytes: int) -> None:
        call("dgpp_vmm_commit", self.handle, int(offset), int(nbytes))

    def release(self, offset: int, nbytes: int) -> None:
        call("dgpp_vmm_release", self.handle, int(offset), int(nbytes))

    def committed(self) -> int:
        return int(self._lib.dgpp_vmm_committed(self.handle))

    def tensor(self, offset: int, nbytes: int, dtype=torch.uint8) -> torch.Tensor:
        """View of [offset, offset + nbytes) (must be committed before it is touched)."""
        t = torch.as_tensor(_Raw(self.ptr + offset, nbytes), device="cuda")
        return t.view(dtype)

    def close(self) -> None:
        if self.handle:
            call("dgpp_vmm_destroy", self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
