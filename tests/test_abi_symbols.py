"""The C-ABI library loads and exports every symbol the headers declare (no compute calls)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROTO = re.compile(r"^APPLEGPU_API\s+[\w\s\*]+?\b(applegpu_\w+)\s*\(", re.M)


def _declared(header):
    with open(os.path.join(ROOT, "include", header)) as f:
        return PROTO.findall(f.read())


def test_headers_declare_the_reference_surface():
    names = _declared("applegpu_b200_ffi.h")
    # the 56 prototypes of the reference's backend_cpp/applegpu_ffi.h:11-92
    assert len(names) == 56
    for n in ("applegpu_ffi_init", "applegpu_ffi_matmul_out", "applegpu_ffi_read_f32", "applegpu_eager_matmul_ex",
              "applegpu_eager_create_view", "applegpu_eager_layer_norm", "applegpu_eager_find_by_data_ptr"):
        assert n in names


def test_library_exports_every_declared_symbol():
    from applegpu_runtime_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    declared = _declared("applegpu_b200_ffi.h") + _declared("applegpu_b200_ext.h")
    assert len(declared) > 100
    missing = [n for n in declared if not hasattr(lib, n)]
    assert not missing, missing


def test_python_binding_covers_both_headers():
    from applegpu_runtime_b200 import _lib
    bound = set(_lib.REFERENCE_SYMBOLS) | set(_lib.EXT_SYMBOLS)
    declared = set(_declared("applegpu_b200_ffi.h") + _declared("applegpu_b200_ext.h"))
    assert declared == bound
    assert set(_declared("applegpu_b200_ffi.h")) == set(_lib.REFERENCE_SYMBOLS)


def test_no_product_module_imports_the_oracle():
    pkg = os.path.join(ROOT, "applegpu_runtime_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cc", ".cu", ".h", ".cuh")):
                with open(os.path.join(dirpath, fn)) as f:
                    text = f.read()
                assert "import oracle" not in text and "from oracle" not in text and "msl_ref" not in text, fn


def test_reference_shim_links_against_the_library():
    """Every applegpu_* symbol the reference's PrivateUse1 shim leaves undefined (a build of its unmodified
    source, oracle/build_ref_shim.py) is exported by this library."""
    import shutil
    import subprocess
    import pytest
    shim = os.path.join(ROOT, "oracle", "_ref", "applegpu_backend.so")
    if not os.path.exists(shim) or not shutil.which("nm"):
        pytest.skip("shim not built here")
    from applegpu_runtime_b200 import _lib
    out = subprocess.run(["nm", "-D", "--undefined-only", shim], capture_output=True, text=True, check=True).stdout
    needed = sorted({ln.split()[-1] for ln in out.splitlines() if ln.split() and ln.split()[-1].startswith("applegpu_")})
    assert len(needed) >= 25
    lib = ctypes.CDLL(_lib.LIB_PATH)
    assert not [n for n in needed if not hasattr(lib, n)]
    assert set(needed) <= set(_lib.REFERENCE_SYMBOLS)
