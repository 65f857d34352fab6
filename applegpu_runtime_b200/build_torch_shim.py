"""Builds the PrivateUse1 ("applegpu") PyTorch backend of this package.

csrc/shim/torch_privateuse1.cpp is compiled with g++ against the installed torch headers and linked with
libapplegpu_b200.so (the C-ABI library next to this file) into libapplegpu_torch.so, also next to this file. The
upstream recipe it stands in for is backend_cpp/setup.py:50-64 (one C++ source, the C header directory, the runtime's
library). torch_device.load() builds it on first use when it is missing or older than its source.

    python -m applegpu_runtime_b200.build_torch_shim
"""
import os
import subprocess
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(PKG, "csrc", "shim", "torch_privateuse1.cpp")
OUT = os.path.join(PKG, "libapplegpu_torch.so")


def build(force=False):
    lib = os.path.join(PKG, "libapplegpu_b200.so")
    if not os.path.exists(lib):
        raise RuntimeError("libapplegpu_b200.so is not built: run make -C applegpu_runtime_b200/csrc first")
    headers = [os.path.join(PKG, "..", "include", h) for h in ("applegpu_b200_ffi.h", "applegpu_b200_ext.h")]
    newest = max(os.path.getmtime(p) for p in [SRC] + headers)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= newest:
        return OUT
    import torch
    from torch.utils import cpp_extension
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-Wno-unused-function", "-fvisibility=hidden",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI), "-I" + sysconfig.get_paths()["include"]]
    for inc in cpp_extension.include_paths():
        cmd += ["-isystem", inc]
    cmd += [SRC, "-o", OUT, "-L" + torch_lib, "-lc10", "-ltorch", "-ltorch_cpu", "-Wl,-rpath," + torch_lib,
            "-L" + PKG, "-lapplegpu_b200", "-Wl,-rpath,$ORIGIN"]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
