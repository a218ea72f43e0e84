"""Loader of the C++ host runtime (`_lib/_runtime*.so`): KV pool, NVMe prefix cache, scheduler core, op log,
safetensors reader, memory guard.  Built in-tree by `python -m spark_engine_b200.build`."""
import glob
import importlib.util
import os

_here = os.path.dirname(os.path.abspath(__file__))
_mod = None


def rt():
    global _mod
    if _mod is None:
        paths = glob.glob(os.path.join(_here, "_lib", "_runtime*.so"))
        if not paths:
            from .build import build_runtime
            build_runtime()
            paths = glob.glob(os.path.join(_here, "_lib", "_runtime*.so"))
        spec = importlib.util.spec_from_file_location("_runtime", paths[0])
        _mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_mod)
    return _mod
