"""Dynamic import helpers. Parity target: ``verl/utils/import_utils.py``."""

from __future__ import annotations

import importlib
import importlib.util
import os
import sys
from functools import cache

__all__ = ["is_package_available", "load_extern_object", "load_extern_type", "import_external_libs", "deprecated",
           "load_class_from_fqn"]


@cache
def is_package_available(name: str) -> bool:
    try:
        return importlib.util.find_spec(name) is not None
    except Exception:
        return False


def load_extern_object(module_path: str, object_name: str):
    """Load ``object_name`` from a python file path or a ``pkg://dotted.module`` reference."""
    if module_path.startswith("pkg://"):
        mod = importlib.import_module(module_path[len("pkg://"):])
    else:
        path = os.path.expanduser(module_path[len("file://"):] if module_path.startswith("file://") else module_path)
        if not os.path.exists(path):
            raise FileNotFoundError(f"Custom module file '{path}' not found.")
        name = f"custom_module_{abs(hash(os.path.abspath(path)))}"
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    if not hasattr(mod, object_name):
        raise AttributeError(f"'{object_name}' not found in module '{module_path}'.")
    return getattr(mod, object_name)


load_extern_type = load_extern_object


def load_class_from_fqn(fqn: str, description: str = "class"):
    mod, _, name = fqn.rpartition(".")
    return getattr(importlib.import_module(mod), name)


def import_external_libs(libs=None) -> None:
    if not libs:
        return
    for lib in ([libs] if isinstance(libs, str) else libs):
        importlib.import_module(lib)


def deprecated(replacement: str = ""):
    import functools
    import warnings

    def deco(fn):
        @functools.wraps(fn)
        def wrapped(*a, **k):
            warnings.warn(f"{fn.__name__} is deprecated" + (f"; use {replacement}" if replacement else ""),
                          DeprecationWarning, stacklevel=2)
            return fn(*a, **k)

        return wrapped

    return deco
