"""Loader of the native host runtime (pybind11 module ``_dgpp_rt`` built in-tree by ``dgpp_b200.build``)."""
from __future__ import annotations

import importlib.util
import sys

from .build import rt_module_path


def _load():
    path = rt_module_path()
    if not path.exists():
        raise ImportError(f"{path} is missing: run `python -m dgpp_b200.build`")
    name = "_dgpp_rt"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, str(path))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


rt = _load()
