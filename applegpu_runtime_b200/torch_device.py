"""torch device "applegpu": the C++ PrivateUse1 backend of this package, over device-memory buffers.

    from applegpu_runtime_b200 import torch_device
    torch_device.load()
    model = model.to("applegpu")

Mirrors what the reference's python/applegpu_runtime/cpp_backend.py:1-78 does for its C++ backend (load the
extension, expose a `torch.applegpu` device module, rename PrivateUse1, generate the tensor methods); the extension
itself is csrc/shim/torch_privateuse1.cpp, built by build_torch_shim.py. A process can name PrivateUse1 once, so this
backend and the Python tensor-subclass frontend (torch_backend.py, which needs no device registration) can be
used together, but two different PrivateUse1 extensions cannot.
"""
import sys
import types

from . import _lib, build_torch_shim

_loaded = None


def load(build=True):
    """Load (building it first if it is missing or stale) the backend and register device "applegpu". Idempotent."""
    global _loaded
    if _loaded is not None:
        return _loaded
    import torch
    lib = _lib.load()       # the extension's NEEDED entry for libapplegpu_b200.so resolves to this same file
    path = build_torch_shim.build() if build else build_torch_shim.OUT
    mod = types.ModuleType("torch.applegpu")
    hooks = dict(device_count=lambda: 1, is_available=lambda: True, current_device=lambda: 0, set_device=lambda d: None,
                 synchronize=lambda d=None: lib.applegpu_eager_synchronize(), _exchange_device=lambda d: 0,
                 _maybe_exchange_device=lambda d: 0, _is_in_bad_fork=lambda: False, manual_seed_all=lambda s: None,
                 manual_seed=lambda s: None, is_initialized=lambda: True, init=lambda: None)
    for name, fn in hooks.items():
        setattr(mod, name, fn)
    sys.modules["torch.applegpu"] = mod
    torch.applegpu = mod
    torch.ops.load_library(path)
    torch.utils.rename_privateuse1_backend("applegpu")
    torch.utils.generate_methods_for_privateuse1_backend()
    _loaded = path
    return path


def launch_count():
    """Kernels this library has launched so far in the process (each aten op routed to the device adds to it)."""
    return int(_lib.load().applegpu_launch_count())
