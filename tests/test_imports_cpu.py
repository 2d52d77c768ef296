"""Every module of the package imports on a machine without a GPU (command-line tools and benchmark modules import
their GPU-only dependencies inside the functions that need them)."""

import importlib
import pkgutil

import kohakuwullm_b200


def test_every_module_imports_without_a_gpu():
    failed = []
    count = 0
    for info in pkgutil.walk_packages(kohakuwullm_b200.__path__, "kohakuwullm_b200."):
        leaf = info.name.rsplit(".", 1)[-1]
        if leaf.startswith("_kwu_"):          # the ctypes libraries, not Python modules
            continue
        try:
            importlib.import_module(info.name)
            count += 1
        except Exception as exc:  # noqa: BLE001
            failed.append(f"{info.name}: {type(exc).__name__}: {exc}")
    assert not failed, failed
    assert count > 120
