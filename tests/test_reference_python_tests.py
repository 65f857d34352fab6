"""The reference's own Python test files against this implementation, through the `applegpu_runtime` alias package.

python/tests/test_transformer_ops.py, test_batched_ops.py, test_attention.py and test_fusion.py of the reference
import `applegpu_runtime as gpu` and nothing else of the project, so they can be pointed at this repository
unmodified. They are not copied here: where a checkout of the reference is present (APPLEGPU_REFERENCE_ROOT, or a
`reference` directory beside the repository) the CPU test checks that every `gpu.<name>` and every tensor method those
files use exists on the alias, and the GPU test runs the files themselves with pytest. Without a checkout both skip;
the same cases, restated, are in tests/test_gpu_ops.py and tests/test_gpu_matmul.py.
"""
import ast
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("APPLEGPU_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))
FILES = ["test_transformer_ops.py", "test_batched_ops.py", "test_attention.py", "test_fusion.py"]
PATHS = [os.path.join(REF, "python", "tests", f) for f in FILES]
needs_checkout = pytest.mark.skipif(not all(os.path.exists(p) for p in PATHS), reason="no checkout of the reference next to the repository")


def test_alias_package_serves_the_b200_implementation():
    import applegpu_runtime as gpu
    import applegpu_runtime_b200 as impl
    assert gpu.from_numpy is impl.from_numpy and gpu.GpuTensor is impl.GpuTensor and gpu.gpt2_forward is impl.gpt2_forward
    assert gpu.LIB_PATH.endswith("libapplegpu_b200.so")


@needs_checkout
def test_every_name_the_reference_tests_use_exists():
    import applegpu_runtime as gpu
    module_names, method_names = set(), set()
    for path in PATHS:
        tree = ast.parse(open(path).read())
        for node in ast.walk(tree):
            if isinstance(node, ast.Attribute) and isinstance(node.value, ast.Name) and node.value.id == "gpu":
                module_names.add(node.attr)
            # methods called on results of gpu.* calls or on local tensors: t.gelu(), x.to_numpy(), a @ b ...
            if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute):
                base = node.func.value
                while isinstance(base, ast.Attribute):
                    base = base.value
                if not (isinstance(base, ast.Name) and base.id in ("gpu", "np", "math", "pytest", "torch")):
                    method_names.add(node.func.attr)
    missing = sorted(n for n in module_names if not hasattr(gpu, n))
    assert not missing, missing
    tensor_methods = {m for m in method_names if not hasattr(__import__("numpy").ndarray, m) and not hasattr(list, m) and not hasattr(str, m)}
    missing_methods = sorted(m for m in tensor_methods if not hasattr(gpu.GpuTensor, m))
    assert not missing_methods, missing_methods


@needs_checkout
@pytest.mark.gpu
def test_reference_python_tests_run_unmodified():
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", "--rootdir", ROOT] + PATHS, env=env, cwd=ROOT, capture_output=True, text=True, timeout=1800)
    assert r.returncode == 0, r.stdout[-6000:] + r.stderr[-2000:]
