"""Host-visible mode of the C-ABI, and the reference's own PrivateUse1 shim running on this library.

Upstream every pointer the ABI returns is host memory too (shared Metal buffers): its C++ shim
(backend_cpp/applegpu_backend.cpp:264-342, :691-749) copies with memcpy and builds CPU views over
them. APPLEGPU_HOST_VISIBLE=1 backs the buffer pool with managed memory so that code runs unchanged.
The second test loads a build of that shim (oracle/build_ref_shim.py, unmodified reference source
linked against this library) and drives the same flows as python/tests/test_cpp_backend.py:15-371:
empty / copy round trips, add / mul / mm / addmm / relu, nn.Linear, embedding, layer_norm, gelu,
softmax, views, and the MLP of the first benchmark configuration, each against PyTorch CPU.
Each case runs in a child process: the mode is chosen before the device context exists and the
PrivateUse1 backend can be renamed once per process.
"""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "oracle", "_ref", "applegpu_backend.so")

pytestmark = pytest.mark.gpu


def _run(code, timeout=600):
    env = dict(os.environ, APPLEGPU_HOST_VISIBLE="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], env=env, cwd=ROOT, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-3000:] + "\n" + r.stderr[-6000:]
    return r.stdout


def test_host_visible_pointers_through_ctypes():
    out = _run("""
        import ctypes
        import numpy as np
        from applegpu_runtime_b200 import _lib
        lib = _lib.load()
        assert lib.applegpu_eager_init()
        assert lib.applegpu_host_visible() == 1
        assert lib.applegpu_set_host_visible(0) == -1          # the context exists in the other mode
        rng = np.random.default_rng(0)
        a = rng.standard_normal((300, 200)).astype(np.float32)
        b = rng.standard_normal((200, 150)).astype(np.float32)
        u64 = ctypes.c_uint64
        def alloc(x):
            dims = (u64 * x.ndim)(*x.shape)
            tid = u64(0)
            p = lib.applegpu_eager_alloc(dims, x.ndim, 0, ctypes.byref(tid))
            assert p
            ctypes.memmove(p, x.ctypes.data, x.nbytes)          # host write through the returned pointer
            return tid.value, p
        ia, pa = alloc(a); ib, pb = alloc(b)
        oid = u64(0)
        pc = lib.applegpu_eager_matmul(ia, ib, ctypes.byref(oid))
        assert pc, lib.applegpu_eager_last_error()
        rid = u64(0)
        pr = lib.applegpu_eager_relu(oid.value, ctypes.byref(rid))
        lib.applegpu_eager_flush_and_wait()
        c = np.frombuffer(ctypes.string_at(pr, 300 * 150 * 4), np.float32).reshape(300, 150)   # host read
        ref = np.maximum(a.astype(np.float64) @ b.astype(np.float64), 0)
        assert np.max(np.abs(c - ref)) / np.max(np.abs(ref)) < 1e-5
        # write again on the host after the device used the buffer, run again, read again
        a2 = (a * 0.5).astype(np.float32)
        ctypes.memmove(pa, a2.ctypes.data, a2.nbytes)
        oid2 = u64(0)
        pc2 = lib.applegpu_eager_matmul(ia, ib, ctypes.byref(oid2))
        lib.applegpu_eager_synchronize()
        c2 = np.frombuffer(ctypes.string_at(pc2, 300 * 150 * 4), np.float32).reshape(300, 150)
        ref2 = a2.astype(np.float64) @ b.astype(np.float64)
        assert np.max(np.abs(c2 - ref2)) / np.max(np.abs(ref2)) < 1e-5
        # bf16 operands on the tensor-core path read managed memory through TMA after the prefetch
        import applegpu_runtime_b200 as gpu
        from oracle import msl_ref as R
        x = rng.standard_normal((512, 256)).astype(np.float32); w = rng.standard_normal((256, 384)).astype(np.float32)
        gx = gpu.from_bytes(R.to_bf16(x).tobytes(), [512, 256], "bfloat16"); gw = gpu.from_bytes(R.to_bf16(w).tobytes(), [256, 384], "bfloat16")
        y = (gx @ gw).to_numpy()
        refy = R.from_bf16(R.to_bf16(x)).astype(np.float64) @ R.from_bf16(R.to_bf16(w)).astype(np.float64)
        assert np.max(np.abs(y - refy)) / np.max(np.abs(refy)) < 2e-2
        assert gpu.pipeline_status() == 0
        for t in (ia, ib, oid.value, rid.value, oid2.value):
            lib.applegpu_eager_free(t)
        print("ok", lib.applegpu_launch_count())
    """)
    assert out.strip().startswith("ok")


_SHIM_PRELUDE = """
    import ctypes, sys, types
    import torch
    import torch.nn.functional as F
    from applegpu_runtime_b200 import _lib
    lib = _lib.load()                                   # the shim's NEEDED entry resolves to this same file
    mod = types.ModuleType("torch.applegpu")            # what torch asks of a renamed PrivateUse1 backend module
    for name, fn in dict(device_count=lambda: 1, is_available=lambda: True, current_device=lambda: 0, set_device=lambda d: None,
                         synchronize=lambda d=None: lib.applegpu_eager_flush_and_wait(), _exchange_device=lambda d: 0,
                         _maybe_exchange_device=lambda d: 0, _is_in_bad_fork=lambda: False, manual_seed_all=lambda s: None,
                         manual_seed=lambda s: None).items():
        setattr(mod, name, fn)
    sys.modules["torch.applegpu"] = mod
    torch.applegpu = mod
    torch.ops.load_library(SHIM)
    torch.utils.rename_privateuse1_backend("applegpu")
    torch.utils.generate_methods_for_privateuse1_backend()
    assert lib.applegpu_host_visible() == 1
    dev = "applegpu"
    def close(a, b, tol=1e-5):
        a = a.cpu().double(); b = b.cpu().double()
        assert a.shape == b.shape, (a.shape, b.shape)
        return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30)) <= tol
"""


@pytest.mark.skipif(not os.path.exists(SHIM), reason="oracle/_ref/applegpu_backend.so not built (needs a checkout of the reference at build time)")
def test_reference_privateuse1_shim_runs_on_this_library():
    out = _run("SHIM = %r\n" % SHIM + textwrap.dedent(_SHIM_PRELUDE) + textwrap.dedent("""
        torch.manual_seed(0)
        # allocation and copies through the returned pointers
        t = torch.empty(3, 4, device=dev)
        assert t.device.type == "applegpu" and t.shape == (3, 4) and t.dtype == torch.float32
        for dt in (torch.float32, torch.float16, torch.int32):
            assert torch.empty(2, 3, device=dev, dtype=dt).dtype == dt
        src = torch.randn(5, 7)
        assert torch.equal(src.to(dev).cpu(), src)
        g = torch.empty(5, 7, device=dev); g.copy_(src)
        assert torch.equal(g.cpu(), src)
        launches0 = lib.applegpu_launch_count()
        # elementwise, matmul, addmm, relu against PyTorch CPU
        a, b = torch.randn(33, 65), torch.randn(33, 65)
        ga, gb = a.to(dev), b.to(dev)
        assert close(ga + gb, a + b) and close(ga * gb, a * b) and close(ga - gb, a - b)
        assert close(torch.relu(ga), torch.relu(a)) and close(-ga, -a)
        m1, m2, bias = torch.randn(40, 24), torch.randn(24, 56), torch.randn(56)
        assert close(torch.mm(m1.to(dev), m2.to(dev)), m1 @ m2)
        w = torch.randn(56, 24)
        assert close(torch.addmm(bias.to(dev), m1.to(dev), w.to(dev).t()), torch.addmm(bias, m1, w.t()))
        # the first benchmark configuration: Linear(64,128) -> ReLU -> Linear(128,10), batch 32, float32, seed 0
        torch.manual_seed(0)
        mlp = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 10))
        x = torch.randn(32, 64)
        with torch.no_grad():
            want = mlp(x)
            import copy
            got = copy.deepcopy(mlp).to(dev)(x.to(dev))
        assert got.device.type == "applegpu" and close(got, want)
        # transformer-forward ops of the shim
        with torch.no_grad():
            table = torch.randn(50, 32); idx = torch.randint(0, 50, (4, 9))
            assert torch.equal(F.embedding(idx.to(dev), table.to(dev)).cpu(), F.embedding(idx, table))
            h = torch.randn(6, 11, 32); gam, bet = torch.randn(32), torch.randn(32)
            assert close(F.layer_norm(h.to(dev), (32,), gam.to(dev), bet.to(dev), 1e-5), F.layer_norm(h, (32,), gam, bet, 1e-5), 1e-4)
            assert close(F.gelu(h.to(dev), approximate="tanh"), F.gelu(h, approximate="tanh"), 1e-4)
            assert close(torch.softmax(h.to(dev), -1), torch.softmax(h, -1), 1e-5)
            q, k = torch.randn(3, 10, 16), torch.randn(3, 16, 10)
            assert close(torch.bmm(q.to(dev), k.to(dev)), torch.bmm(q, k))
            gh = h.to(dev)
            assert close(gh.transpose(1, 2).contiguous(), h.transpose(1, 2).contiguous())
            assert close(gh[:, 2:7, :] * 2.0, h[:, 2:7, :] * 2.0)
        # a pre-LN transformer block with causal attention, written with the torch ops the shim registers
        def block(x_ids, p, heads):
            x = F.embedding(x_ids, p["wte"]) + p["wpe"][: x_ids.shape[1]]
            B, T, D = x.shape
            h = F.layer_norm(x, (D,), p["ln1_g"], p["ln1_b"], 1e-5)
            qkv = F.linear(h.reshape(B * T, D), p["w_qkv"], p["b_qkv"]).reshape(B, T, 3, heads, D // heads)
            q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3).reshape(B * heads, T, D // heads) for i in range(3))
            att = torch.bmm(q, k.transpose(1, 2)) * (1.0 / (D // heads) ** 0.5) + p["mask"]
            ctx = torch.bmm(torch.softmax(att, -1), v).reshape(B, heads, T, D // heads).permute(0, 2, 1, 3).reshape(B * T, D)
            x = x + F.linear(ctx, p["w_o"], p["b_o"]).reshape(B, T, D)
            h = F.layer_norm(x, (D,), p["ln2_g"], p["ln2_b"], 1e-5)
            ff = F.linear(F.gelu(F.linear(h.reshape(B * T, D), p["w_fc"], p["b_fc"]), approximate="tanh"), p["w_pr"], p["b_pr"])
            return x + ff.reshape(B, T, D)
        torch.manual_seed(1)
        D, heads, T, B = 64, 4, 24, 3
        p = {"wte": torch.randn(97, D) * 0.02, "wpe": torch.randn(32, D) * 0.02, "ln1_g": torch.ones(D), "ln1_b": torch.zeros(D),
             "ln2_g": torch.ones(D), "ln2_b": torch.zeros(D), "w_qkv": torch.randn(3 * D, D) * 0.02, "b_qkv": torch.zeros(3 * D),
             "w_o": torch.randn(D, D) * 0.02, "b_o": torch.zeros(D), "w_fc": torch.randn(4 * D, D) * 0.02, "b_fc": torch.zeros(4 * D),
             "w_pr": torch.randn(D, 4 * D) * 0.02, "b_pr": torch.zeros(D),
             "mask": torch.triu(torch.full((T, T), -1e9), diagonal=1)}
        ids = torch.randint(0, 97, (B, T))
        with torch.no_grad():
            want = block(ids, p, heads)
            got = block(ids.to(dev), {k: v.to(dev) for k, v in p.items()}, heads)
        assert got.device.type == "applegpu" and close(got, want, 1e-4)
        assert lib.applegpu_launch_count() > launches0 + 40, "the ops did not reach the CUDA kernels"
        assert lib.applegpu_pipeline_status() == 0
        print("ok", lib.applegpu_launch_count() - launches0)
    """))
    assert out.strip().splitlines()[-1].startswith("ok")
