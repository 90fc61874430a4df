"""Every module of the package imports on a machine without a GPU (signature tables, dataclasses, lazy library loads)."""
import importlib
import pkgutil

import dgpp_b200


def test_every_module_imports():
    failed = []
    for m in pkgutil.walk_packages(dgpp_b200.__path__, "dgpp_b200."):
        if m.name.endswith("__main__"):
            continue
        try:
            importlib.import_module(m.name)
        except Exception as e:          # noqa: BLE001 - the test reports every module that fails, with its reason
            failed.append((m.name, repr(e)))
    assert not failed, failed
