"""`import applegpu_runtime as gpu` — the reference's package name, served by applegpu_runtime_b200.

Code written against the reference's Python surface (python/applegpu_runtime/__init__.py:3-125), its own test files
included (python/tests/test_transformer_ops.py, test_batched_ops.py, test_attention.py, test_fusion.py), imports this
name; every public name resolves to the B200 implementation. Nothing is implemented here.
"""
import applegpu_runtime_b200 as _impl
from applegpu_runtime_b200 import *  # noqa: F401,F403
from applegpu_runtime_b200 import __version__  # noqa: F401


def __getattr__(name):
    return getattr(_impl, name)


def __dir__():
    return sorted(set(globals()) | set(dir(_impl)))
