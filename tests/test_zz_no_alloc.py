"""The allocation-free attention entry point (applegpu_attention_noalloc) against the regular
eager attention entry point, through the C ABI.

Some callers of this library may not allocate device memory at the moment they need attention
(fixed-budget serving loops, plugins whose host owns all device buffers). Their entry point keeps
its score matrix in a fixed array inside the library instead of taking it from the buffer pool.
It launches the same kernels on the same layouts as applegpu_eager_attention, so the two must
agree to the tolerance the other attention tests use; this file checks that on two calls in a
row (the second call finds the first call's data in the shared scratch) and checks the size
limit. It is named to be collected last so a failure here cannot hide any other test."""
import ctypes

import numpy as np
import pytest

from oracle import msl_ref as R

pytestmark = pytest.mark.gpu
F32, BF16 = 0, 10
SCRATCH_BYTES = 64 << 20


@pytest.fixture()
def lib(gpu_dev):
    from applegpu_runtime_b200 import _lib
    return _lib.load()


def _eager(lib, arr, code):
    arr = np.ascontiguousarray(arr)
    d = (ctypes.c_uint64 * arr.ndim)(*arr.shape)
    tid = ctypes.c_uint64()
    p = lib.applegpu_eager_alloc(d, arr.ndim, code, ctypes.byref(tid))
    assert p, lib.applegpu_eager_last_error()
    assert lib.applegpu_eager_upload(tid.value, arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes) == 0
    return tid.value, p


def _read(lib, tid, shape, np_dtype):
    out = np.empty(shape, np_dtype)
    assert lib.applegpu_eager_download(tid, out.ctypes.data_as(ctypes.c_void_p), out.nbytes) == 0, lib.applegpu_eager_last_error()
    return out


def _both_paths(lib, q, k, v, code, np_dtype, causal):
    """Returns (regular entry point output, allocation-free entry point output) as raw arrays."""
    iq, pq = _eager(lib, q, code); ik, pk = _eager(lib, k, code); iv, pv = _eager(lib, v, code)
    bh, tq, dk = q.shape; tk = k.shape[1]; dv = v.shape[2]
    oid = ctypes.c_uint64()
    assert lib.applegpu_eager_attention(iq, ik, iv, causal, ctypes.byref(oid)), lib.applegpu_eager_last_error()
    regular = _read(lib, oid.value, (bh, tq, dv), np_dtype)
    out_id, p_out = _eager(lib, np.zeros((bh, tq, dv), np_dtype), code)     # caller-owned output buffer
    stream = lib.applegpu_stream()
    rc = lib.applegpu_attention_noalloc(pq, pk, pv, p_out, code, bh, tq, tk, dk, dv, causal, stream)
    assert rc == 0, lib.applegpu_ffi_last_error()
    noalloc = _read(lib, out_id, (bh, tq, dv), np_dtype)
    for t in (iq, ik, iv, oid.value, out_id):
        lib.applegpu_eager_free(t)
    return regular, noalloc


def test_noalloc_attention_matches_regular_entry_point_twice_in_a_row(lib):
    rng = np.random.default_rng(0)
    # two calls in a row with different shapes and masks: the second finds the first's scores in the scratch
    for causal, shape in ((True, (6, 200, 64)), (False, (4, 136, 64))):
        q, k, v = (rng.standard_normal(shape).astype(np.float32) for _ in range(3))
        regular, noalloc = _both_paths(lib, q, k, v, F32, np.float32, causal)
        np.testing.assert_allclose(noalloc, regular, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(noalloc, R.attention(q, k, v, causal), rtol=1e-4, atol=1e-5)   # the bar of test_gpu_matmul.py


def test_noalloc_attention_bf16_tensor_core_path_twice_in_a_row(lib, gpu_dev):
    rng = np.random.default_rng(1)
    for causal in (True, False):
        q, k, v = (R.to_bf16(rng.standard_normal((12, 256, 64)).astype(np.float32)) for _ in range(3))
        regular, noalloc = _both_paths(lib, q, k, v, BF16, np.uint16, causal)
        a, b = R.from_bf16(noalloc), R.from_bf16(regular)
        assert np.max(np.abs(a - b)) <= 2e-2 * np.max(np.abs(b))            # bf16 bar; in practice identical
        ref = R.attention(R.from_bf16(q), R.from_bf16(k), R.from_bf16(v), causal)
        assert np.max(np.abs(a - ref)) <= 2e-2 * np.max(np.abs(ref))
        # the entry point's OWN status word (its GEMMs do not write the one pipeline_status() reads)
        assert lib.applegpu_attention_noalloc_status(lib.applegpu_stream()) == 0
    assert gpu_dev.pipeline_status() == 0


def test_noalloc_attention_allocates_nothing_and_accepts_the_default_stream(lib, gpu_dev):
    """The property the entry point exists for: after one warm-up call (which resolves the scratch address)
    a further call leaves the pool statistics and the device's free-memory figure unchanged. Also the one
    success path the other tests do not take: cuda_stream = NULL (the legacy default stream)."""
    import torch
    rng = np.random.default_rng(2)
    q, k, v = (R.to_bf16(rng.standard_normal((8, 192, 64)).astype(np.float32)) for _ in range(3))
    iq, pq = _eager(lib, q, BF16); ik, pk = _eager(lib, k, BF16); iv, pv = _eager(lib, v, BF16)
    io, po = _eager(lib, np.zeros((8, 192, 64), np.uint16), BF16)
    stream = lib.applegpu_stream()
    assert lib.applegpu_attention_noalloc(pq, pk, pv, po, BF16, 8, 192, 192, 64, 64, True, stream) == 0      # warm-up
    gpu_dev.synchronize()
    want = _read(lib, io, (8, 192, 64), np.uint16)
    stats0 = gpu_dev.pool_stats()
    free0 = torch.cuda.mem_get_info(lib.applegpu_device())[0]
    assert lib.applegpu_attention_noalloc(pq, pk, pv, po, BF16, 8, 192, 192, 64, 64, True, stream) == 0
    assert lib.applegpu_attention_noalloc_status(stream) == 0
    stats1 = gpu_dev.pool_stats()
    free1 = torch.cuda.mem_get_info(lib.applegpu_device())[0]
    for key in ("misses", "live_bytes", "pooled_bytes", "live_buffers"):
        assert stats1[key] == stats0[key], key
    assert free1 == free0
    # NULL stream: the runtime stream is non-blocking, so order the two by hand
    gpu_dev.synchronize()
    assert lib.applegpu_attention_noalloc(pq, pk, pv, po, BF16, 8, 192, 192, 64, 64, True, None) == 0, lib.applegpu_ffi_last_error()
    assert lib.applegpu_attention_noalloc_status(None) == 0
    got = _read(lib, io, (8, 192, 64), np.uint16)
    assert np.array_equal(got, want)
    for t in (iq, ik, iv, io):
        lib.applegpu_eager_free(t)


def test_noalloc_attention_rejects_problems_larger_than_its_scratch(lib):
    q, pq = _eager(lib, np.zeros((1, 8, 8), np.float32), F32)
    too_many_rows = SCRATCH_BYTES // (4 * 8) + 1       # batch_heads * q_len * kv_len * 4 bytes just over the limit
    rc = lib.applegpu_attention_noalloc(pq, pq, pq, pq, F32, 1, too_many_rows, 8, 8, 8, False, None)
    assert rc == -1
    msg = lib.applegpu_ffi_last_error()
    assert b"exceeds the built-in scratch" in msg and str(SCRATCH_BYTES).encode() in msg
    assert lib.applegpu_attention_noalloc(pq, pq, pq, pq, 5, 1, 8, 8, 8, 8, False, None) == -1   # int32 is not a float dtype
    lib.applegpu_eager_free(q)
