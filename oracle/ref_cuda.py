"""Loader of oracle/_ref/int2_tc_ops_ref.so: the reference's own CUDA extension, compiled unmodified for
sm_100a by `oracle/build_ref.sh --cuda` (TEST INFRASTRUCTURE ONLY; None when it has not been built)."""
import importlib.machinery
import importlib.util
import os

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "int2_tc_ops_ref.so")
_mod = None


def load():
    global _mod
    if _mod is None:
        if not os.path.exists(_PATH):
            return None
        import torch  # noqa: F401  (the extension links against libtorch)
        loader = importlib.machinery.ExtensionFileLoader("int2_tc_ops_ref", _PATH)
        spec = importlib.util.spec_from_file_location("int2_tc_ops_ref", _PATH, loader=loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
        _mod = mod
    return _mod
