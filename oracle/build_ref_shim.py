"""Builds the reference's own PrivateUse1 C++ shim against this repository's C-ABI library.

Test infrastructure only (the drop-in check of the boundary): the reference's
backend_cpp/applegpu_backend.cpp is compiled from where it lies in a checkout of the reference,
unmodified, with g++ and the installed torch headers, and linked against
applegpu_runtime_b200/libapplegpu_b200.so instead of the reference's Rust static library
(backend_cpp/setup.py:50-64 is the upstream recipe: same single source file, same include directory).
The output goes to oracle/_ref/applegpu_backend.so, which is not tracked. Nothing in the package
loads it; tests/test_gpu_privateuse1_shim.py does, and skips when it is absent.

    python oracle/build_ref_shim.py [path-to-reference-checkout]
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref", "applegpu_backend.so")


def build(reference_root, force=False):
    src = os.path.join(reference_root, "backend_cpp", "applegpu_backend.cpp")
    if not os.path.exists(src):
        return None
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(src):
        return OUT
    import torch
    from torch.utils import cpp_extension
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    pkg = os.path.join(ROOT, "applegpu_runtime_b200")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-w",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I" + os.path.join(reference_root, "backend_cpp"), "-I" + sysconfig.get_paths()["include"]]
    for inc in cpp_extension.include_paths():
        cmd += ["-isystem", inc]
    cmd += [src, "-o", OUT, "-L" + torch_lib, "-lc10", "-ltorch", "-ltorch_cpu", "-Wl,-rpath," + torch_lib,
            "-L" + pkg, "-lapplegpu_b200", "-Wl,-rpath,$ORIGIN/../../applegpu_runtime_b200"]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("APPLEGPU_REFERENCE_ROOT", "")
    out = build(ref, force=True) if ref else None
    print(out or "reference checkout not found: pass its path")
    sys.exit(0 if out else 1)
