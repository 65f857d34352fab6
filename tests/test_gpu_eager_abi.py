"""The eager flavour and the raw graph flavour, driven through ctypes exactly as a C caller
would. Restates crates/core/tests/backend_ffi_integration.rs:50-160 and eager_integration.rs:12-210
(alloc / register / op / eval / read, views, in-place ops, pool recycling) with explicit
upload / download in place of pointer pokes (the data pointers are device pointers)."""
import ctypes

import numpy as np
import pytest

from oracle import msl_ref as R

pytestmark = pytest.mark.gpu
F32, I32 = 0, 5


@pytest.fixture()
def lib(gpu_dev):
    from applegpu_runtime_b200 import _lib
    return _lib.load()


def dims(*d):
    return (ctypes.c_uint64 * max(len(d), 1))(*d), len(d)


def eager_tensor(lib, arr, code=F32):
    arr = np.ascontiguousarray(arr)
    d, nd = dims(*arr.shape)
    tid = ctypes.c_uint64()
    p = lib.applegpu_eager_alloc(d, nd, code, ctypes.byref(tid))
    assert p, lib.applegpu_eager_last_error()
    assert lib.applegpu_eager_upload(tid.value, arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes) == 0
    return tid.value, p


def eager_read(lib, tid, dtype=np.float32):
    d = (ctypes.c_uint64 * 8)(); nd = ctypes.c_uint32()
    assert lib.applegpu_eager_shape(tid, d, ctypes.byref(nd)) == 0
    shape = [int(d[i]) for i in range(nd.value)]
    out = np.empty(shape, dtype)
    assert lib.applegpu_eager_download(tid, out.ctypes.data_as(ctypes.c_void_p), out.nbytes) == 0, lib.applegpu_eager_last_error()
    return out


def test_graph_flavour_alloc_register_matmul_eval_read(lib):
    # backend_ffi_integration.rs:97-130
    ids = []
    for data in ([1, 2, 3, 4], [5, 6, 7, 8]):
        tid = ctypes.c_uint64()
        p = lib.applegpu_ffi_alloc(16, F32, ctypes.byref(tid))
        assert p and tid.value
        arr = np.array(data, np.float32)
        assert lib.applegpu_ffi_upload(tid.value, arr.ctypes.data_as(ctypes.c_void_p), 16) == 0
        d, nd = dims(2, 2)
        assert lib.applegpu_ffi_register_tensor(tid.value, d, nd, F32) == 0
        ids.append(tid.value)
    c = lib.applegpu_ffi_matmul(ids[0], ids[1])
    assert c >= 100000
    d = (ctypes.c_uint64 * 8)(); nd = ctypes.c_uint32()
    assert lib.applegpu_ffi_shape(c, d, ctypes.byref(nd)) == 0 and [d[0], d[1]] == [2, 2]
    assert lib.applegpu_ffi_eval(c) == 0
    out = (ctypes.c_float * 4)()
    assert lib.applegpu_ffi_read_f32(c, out, 4) == 0
    assert list(out) == [19.0, 22.0, 43.0, 50.0]
    for i in ids + [c]:
        lib.applegpu_ffi_free(i)


def test_graph_flavour_out_variants_write_into_the_reserved_buffer(lib):
    a = np.arange(6, dtype=np.float32).reshape(2, 3); b = np.ones((2, 3), np.float32)
    ids = []
    for arr in (a, b):
        d, nd = dims(*arr.shape)
        t = lib.applegpu_ffi_from_host(arr.ctypes.data_as(ctypes.c_void_p), d, nd, F32)
        assert t
        ids.append(t)
    out_id = ctypes.c_uint64()
    p = lib.applegpu_ffi_add_out(ids[0], ids[1], ctypes.byref(out_id))
    assert p and out_id.value
    assert lib.applegpu_ffi_eval(out_id.value) == 0
    got = np.empty((2, 3), np.float32)
    assert lib.applegpu_ffi_read_bytes(out_id.value, got.ctypes.data_as(ctypes.c_void_p), got.nbytes) == 0
    assert np.array_equal(got, a + b)
    s_id = ctypes.c_uint64()
    assert lib.applegpu_ffi_scalar_mul_out(out_id.value, 0.5, ctypes.byref(s_id))
    m_id = ctypes.c_uint64()
    assert lib.applegpu_ffi_mean_all_out(s_id.value, ctypes.byref(m_id))
    v = (ctypes.c_float * 1)()
    assert lib.applegpu_ffi_read_f32(m_id.value, v, 1) == 0
    assert abs(v[0] - float(((a + b) * 0.5).mean())) < 1e-6
    t_id = ctypes.c_uint64()
    assert lib.applegpu_ffi_threshold_backward_out(ids[1], ids[0], 2.5, ctypes.byref(t_id))
    tb = (ctypes.c_float * 6)()
    assert lib.applegpu_ffi_read_f32(t_id.value, tb, 6) == 0
    assert list(tb) == [0, 0, 0, 1, 1, 1]
    dst = ctypes.c_uint64()
    assert lib.applegpu_ffi_alloc(24, F32, ctypes.byref(dst))
    assert lib.applegpu_ffi_copy(out_id.value, dst.value) == 0
    d, nd = dims(2, 3)
    assert lib.applegpu_ffi_register_tensor(dst.value, d, nd, F32) == 0
    cp = (ctypes.c_float * 6)()
    assert lib.applegpu_ffi_read_f32(dst.value, cp, 6) == 0 and list(cp) == (a + b).reshape(-1).tolist()


def test_eager_binary_ops_and_broadcast(lib):
    a = np.arange(12, dtype=np.float32).reshape(3, 4); b = np.array([1, 2, 3, 4], np.float32)
    ia, _ = eager_tensor(lib, a); ib, _ = eager_tensor(lib, b)
    for name, fn in (("add", np.add), ("sub", np.subtract), ("mul", np.multiply), ("div", np.divide)):
        oid = ctypes.c_uint64()
        p = getattr(lib, f"applegpu_eager_{name}")(ia, ib, ctypes.byref(oid))
        assert p, lib.applegpu_eager_last_error()
        lib.applegpu_eager_flush_and_wait()
        assert np.array_equal(eager_read(lib, oid.value), fn(a, b))
        assert lib.applegpu_eager_find_by_data_ptr(p) == oid.value
        lib.applegpu_eager_free(oid.value)
    oid = ctypes.c_uint64()
    assert lib.applegpu_eager_relu(lib.applegpu_eager_find_by_data_ptr(lib.applegpu_eager_neg(ia, ctypes.byref(oid))), ctypes.byref(oid))
    assert np.array_equal(eager_read(lib, oid.value), np.maximum(-a, 0))


def test_eager_views_share_storage_and_honour_offsets(lib):
    # eager_integration.rs views + test_cpp_backend.py:252-263 (slice offset regression)
    x = np.arange(24, dtype=np.float32).reshape(4, 6)
    ix, px = eager_tensor(lib, x)
    shape, nd = dims(4, 2); strides, _ = dims(6, 1)
    vid = ctypes.c_uint64()
    pv = lib.applegpu_eager_create_view(ix, shape, strides, nd, 2, ctypes.byref(vid))     # x[:, 2:4]
    assert pv == px + 2 * 4
    assert np.array_equal(eager_read(lib, vid.value), x[:, 2:4])
    oid = ctypes.c_uint64()
    assert lib.applegpu_eager_add(vid.value, vid.value, ctypes.byref(oid))
    assert np.array_equal(eager_read(lib, oid.value), 2 * x[:, 2:4])
    # transpose view feeding matmul must be rejected: "matmul requires contiguous inputs" (eager.rs:422-425)
    tshape, _ = dims(6, 4); tstr, _ = dims(1, 6)
    tid = ctypes.c_uint64()
    assert lib.applegpu_eager_create_view(ix, tshape, tstr, 2, 0, ctypes.byref(tid))
    mm = ctypes.c_uint64()
    assert not lib.applegpu_eager_matmul(tid.value, ix, ctypes.byref(mm))
    assert b"matmul requires contiguous inputs" in lib.applegpu_eager_last_error()
    # matmul_ex takes the base tensor plus a transpose flag instead (eager.rs:485-560)
    assert lib.applegpu_eager_matmul_ex(ix, ix, True, False, ctypes.byref(mm)), lib.applegpu_eager_last_error()
    np.testing.assert_allclose(eager_read(lib, mm.value), x.T @ x, rtol=1e-6)
    assert lib.applegpu_eager_matmul_ex(ix, ix, False, True, ctypes.byref(mm))
    np.testing.assert_allclose(eager_read(lib, mm.value), x @ x.T, rtol=1e-6)
    # freeing the base keeps the view alive (refcounted buffer, eager.rs:143-149)
    lib.applegpu_eager_free(ix)
    assert np.array_equal(eager_read(lib, vid.value), x[:, 2:4])


def test_eager_inplace_and_reductions(lib):
    a = np.arange(6, dtype=np.float32).reshape(2, 3); b = np.ones((2, 3), np.float32)
    ia, _ = eager_tensor(lib, a); ib, _ = eager_tensor(lib, b)
    assert lib.applegpu_eager_add_inplace(ia, ib) == 0
    assert lib.applegpu_eager_add_scaled_inplace(ia, ib, -0.5) == 0
    assert np.array_equal(eager_read(lib, ia), a + 1 - 0.5)
    oid = ctypes.c_uint64()
    assert lib.applegpu_eager_sum_dim(ia, -1, False, ctypes.byref(oid))
    np.testing.assert_allclose(eager_read(lib, oid.value), (a + 0.5).sum(-1))
    assert lib.applegpu_eager_sum_dim(ia, 0, True, ctypes.byref(oid))
    got = eager_read(lib, oid.value)
    assert got.shape == (1, 3)
    np.testing.assert_allclose(got, (a + 0.5).sum(0, keepdims=True))
    assert lib.applegpu_eager_mean_all(ia, ctypes.byref(oid))
    np.testing.assert_allclose(eager_read(lib, oid.value), [(a + 0.5).mean()])
    assert lib.applegpu_eager_scalar_mul(ia, 2.0, ctypes.byref(oid))
    assert np.array_equal(eager_read(lib, oid.value), (a + 0.5) * 2)


def test_eager_gpt2_ops(lib):
    rng = np.random.default_rng(0)
    w = rng.standard_normal((11, 8)).astype(np.float32); idx = np.array([[3, 0], [10, 3]], np.int32)
    iw, _ = eager_tensor(lib, w); ii, _ = eager_tensor(lib, idx, I32)
    oid = ctypes.c_uint64()
    assert lib.applegpu_eager_embedding(iw, ii, ctypes.byref(oid))
    assert np.array_equal(eager_read(lib, oid.value), R.embedding(w, idx))          # shape idx.shape + [D] (eager.rs:972-975)
    x = rng.standard_normal((5, 8)).astype(np.float32); g = rng.standard_normal(8).astype(np.float32); b = rng.standard_normal(8).astype(np.float32)
    ix, _ = eager_tensor(lib, x); ig, _ = eager_tensor(lib, g); ib, _ = eager_tensor(lib, b)
    assert lib.applegpu_eager_layer_norm(ix, ig, ib, 1e-5, ctypes.byref(oid))
    np.testing.assert_allclose(eager_read(lib, oid.value), R.layer_norm(x, g, b), rtol=1e-5, atol=1e-6)
    assert lib.applegpu_eager_gelu(ix, ctypes.byref(oid))
    np.testing.assert_allclose(eager_read(lib, oid.value), R.gelu(x), rtol=1e-5, atol=1e-7)
    assert lib.applegpu_eager_softmax(ix, ctypes.byref(oid))
    np.testing.assert_allclose(eager_read(lib, oid.value), R.softmax(x), rtol=1e-5)
    assert lib.applegpu_eager_softmax_causal(ix, ctypes.byref(oid))
    np.testing.assert_allclose(eager_read(lib, oid.value), R.softmax_causal(x), rtol=1e-5)
    assert lib.applegpu_eager_argmax(ix, ctypes.byref(oid))
    assert np.array_equal(eager_read(lib, oid.value, np.int32), R.argmax(x))
    assert lib.applegpu_eager_quantize(ix, 3, 0.1, 0, ctypes.byref(oid))
    assert np.array_equal(eager_read(lib, oid.value, np.int8), R.quantize(x, "int8", 0.1))
    assert lib.applegpu_eager_linear(ix, iw, 0, 0, 1, True, ctypes.byref(oid)), lib.applegpu_eager_last_error()  # gelu(x @ w^T)
    np.testing.assert_allclose(eager_read(lib, oid.value), R.gelu((x @ w.T).astype(np.float32)), rtol=1e-5, atol=1e-6)
    q = rng.standard_normal((2, 6, 8)).astype(np.float32)
    iq, _ = eager_tensor(lib, q)
    assert lib.applegpu_eager_attention(iq, iq, iq, True, ctypes.byref(oid)), lib.applegpu_eager_last_error()
    np.testing.assert_allclose(eager_read(lib, oid.value), R.attention(q, q, q, True), rtol=1e-4, atol=1e-5)


def test_eager_errors_do_not_poison_the_runtime(lib):
    oid = ctypes.c_uint64()
    assert not lib.applegpu_eager_add(987654321, 987654322, ctypes.byref(oid))
    assert b"not found" in lib.applegpu_eager_last_error()
    a, _ = eager_tensor(lib, np.ones((2, 3), np.float32)); b, _ = eager_tensor(lib, np.ones((4, 5), np.float32))
    assert not lib.applegpu_eager_matmul(a, b, ctypes.byref(oid))
    assert b"mismatch" in lib.applegpu_eager_last_error()
    assert lib.applegpu_eager_add(a, a, ctypes.byref(oid))             # still usable afterwards
    assert np.array_equal(eager_read(lib, oid.value), np.full((2, 3), 2, np.float32))


def test_pool_recycles_buffers_and_reports_stats(lib, gpu_dev):
    # pool_integration.rs / eager_integration.rs pool recycling
    gpu_dev.synchronize()
    s0 = gpu_dev.pool_stats()
    d, nd = dims(1024, 1024)
    tid = ctypes.c_uint64()
    p1 = lib.applegpu_eager_alloc(d, nd, F32, ctypes.byref(tid))
    lib.applegpu_eager_free(tid.value)
    p2 = lib.applegpu_eager_alloc(d, nd, F32, ctypes.byref(tid))
    s1 = gpu_dev.pool_stats()
    assert p1 == p2 and s1["hits"] >= s0["hits"] + 1
    lib.applegpu_eager_free(tid.value)
    assert gpu_dev.pool_stats()["pooled_bytes"] >= 4 << 20
    gpu_dev.pool_drain()
    assert gpu_dev.pool_stats()["pooled_bytes"] == 0


def test_allocation_failure_is_reported_not_fatal(lib):
    # host-side fault injection: the next device allocation reports failure
    lib.applegpu_pool_drain()
    lib.applegpu_pool_fail_next(1)
    d, nd = dims(3, 1000)
    tid = ctypes.c_uint64()
    assert not lib.applegpu_eager_alloc(d, nd, F32, ctypes.byref(tid))
    assert b"Failed to allocate GPU buffer" in lib.applegpu_eager_last_error()
    assert lib.applegpu_eager_alloc(d, nd, F32, ctypes.byref(tid))     # the runtime carries on
    lib.applegpu_eager_free(tid.value)


# ── compiled-graph executor (crates/core/src/compiled_graph.rs wire format) ──
def _op(code, inputs, out_dims=(), params=(), dtype=F32):
    import struct
    b = struct.pack("<BB", code, len(inputs)) + b"".join(struct.pack("<H", i) for i in inputs)
    b += struct.pack("<B", len(out_dims)) + b"".join(struct.pack("<Q", d) for d in out_dims)
    b += struct.pack("<BB", dtype, len(params)) + b"".join(struct.pack("<f", p) for p in params)
    return b


def _run_graph(lib, ops, input_ids, outputs):
    buf = (ctypes.c_uint8 * len(ops)).from_buffer_copy(ops)
    tids = (ctypes.c_uint64 * len(input_ids))(*input_ids)
    oix = (ctypes.c_uint16 * len(outputs))(*outputs)
    out_t = (ctypes.c_uint64 * len(outputs))()
    out_p = (ctypes.c_void_p * len(outputs))()
    n = lib.applegpu_eager_execute_graph(buf, len(ops), tids, len(input_ids), oix, len(outputs), out_t, out_p)
    return n, list(out_t), list(out_p)


def test_compiled_graph_runs_an_mlp_forward_and_backward_fragment(lib):
    """Linear -> ReLU -> Linear and a ReLU-backward fragment, the op mix torch.compile hands the reference
    (addmm, transpose views, relu, threshold_backward, scalar_mul, sum_dim, mean_all, view, identity)."""
    rng = np.random.default_rng(11)
    x = rng.standard_normal((32, 64)).astype(np.float32)
    w1 = (rng.standard_normal((128, 64)) * 0.1).astype(np.float32); b1 = rng.standard_normal(128).astype(np.float32)
    w2 = (rng.standard_normal((10, 128)) * 0.1).astype(np.float32); b2 = rng.standard_normal(10).astype(np.float32)
    ids = [eager_tensor(lib, a)[0] for a in (x, w1, b1, w2, b2)]      # node table slots 0..4
    ops = b"".join([
        _op(11, [1], (64, 128)),                  # 5: w1^T (view)
        _op(13, [2, 0, 5], (32, 128)),            # 6: addmm(b1, x, w1^T)
        _op(5, [6], (32, 128)),                   # 7: relu
        _op(11, [3], (128, 10)),                  # 8: w2^T
        _op(13, [4, 7, 8], (32, 10)),             # 9: logits
        _op(9, [9], (1,)),                        # 10: mean_all
        _op(7, [7, 6], (32, 128), (0.0,)),        # 11: threshold_backward(grad = h, input = pre-activation)
        _op(10, [11], (128,), (0.0, 0.0)),        # 12: sum over dim 0
        _op(8, [12], (128,), (0.5,)),             # 13: scalar_mul
        _op(12, [13], (8, 16)),                   # 14: view
        _op(255, [14]),                           # 15: identity
        _op(1, [9, 9], (32, 10)),                 # 16: sub -> zeros
        _op(6, [16], (32, 10)),                   # 17: neg
    ])
    n, out_ids, out_ptrs = _run_graph(lib, ops, ids, [9, 10, 15, 17, 0])
    assert n == 5, lib.applegpu_eager_last_error()
    assert all(out_ptrs[:4]) and out_ids[4] == ids[0]                 # an input may be returned as an output
    pre = x @ w1.T + b1
    h = np.maximum(pre, 0)
    logits = h @ w2.T + b2
    np.testing.assert_allclose(eager_read(lib, out_ids[0]), logits, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(eager_read(lib, out_ids[1]), [logits.mean()], rtol=1e-4, atol=1e-5)
    g = np.where(pre > 0, h, 0).sum(0) * 0.5
    np.testing.assert_allclose(eager_read(lib, out_ids[2]), g.reshape(8, 16), rtol=1e-4, atol=1e-4)
    assert not eager_read(lib, out_ids[3]).any()


def test_compiled_graph_rejects_malformed_streams(lib):
    x = eager_tensor(lib, np.ones((2, 2), np.float32))[0]
    n, _, _ = _run_graph(lib, _op(5, [0], (2, 2))[:-1], [x], [1])                  # truncated
    assert n == -1 and b"truncated" in lib.applegpu_eager_last_error()
    n, _, _ = _run_graph(lib, _op(5, [3], (2, 2)), [x], [1])                       # input index past the table
    assert n == -1 and b"out of range" in lib.applegpu_eager_last_error()
    n, _, _ = _run_graph(lib, _op(99, [0], (2, 2)), [x], [1])
    assert n == -1 and b"unsupported op: 99" in lib.applegpu_eager_last_error()
    n, _, _ = _run_graph(lib, _op(5, [0], (2, 2)), [x], [7])
    assert n == -1 and b"output 7 out of range" in lib.applegpu_eager_last_error()


def test_a_bounded_wait_that_runs_out_is_reported_and_the_device_stays_usable(lib, gpu_dev):
    """Every mbarrier wait of the tcgen05 kernels is bounded and reports through the pipeline status word. Here a
    test-only kernel waits (for at most a millisecond) on a barrier nothing arrives at: the wait gives up, the
    kernel returns, the word carries the code, every blocking point of the library reports it as an error and
    clears it, and the next launch runs normally. Nothing faults, traps or spins without a limit."""
    gpu_dev.synchronize()
    assert gpu_dev.pipeline_status() == 0
    # 1. the explicit poll sees the code and clears the word
    assert lib.applegpu_test_wait_runs_out(77, 1000) == 0
    assert gpu_dev.pipeline_status() == 77
    assert gpu_dev.pipeline_status() == 0
    # 2. a blocking read turns the code into an error instead of handing back bytes as a result
    a, _ = eager_tensor(lib, np.ones((4, 4), np.float32))
    assert lib.applegpu_test_wait_runs_out(78, 1000) == 0
    out = np.empty((4, 4), np.float32)
    assert lib.applegpu_eager_download(a, out.ctypes.data_as(ctypes.c_void_p), out.nbytes) == -1
    assert b"pipeline wait timed out (code 78)" in lib.applegpu_eager_last_error()
    assert lib.applegpu_eager_download(a, out.ctypes.data_as(ctypes.c_void_p), out.nbytes) == 0       # cleared: the next read succeeds
    # 3. a marker wait reports it too
    assert lib.applegpu_test_wait_runs_out(79, 1000) == 0
    m = lib.applegpu_marker_record()
    assert m and lib.applegpu_marker_wait(m) == -1
    assert b"code 79" in lib.applegpu_ffi_last_error()
    # 4. the tensor-core path works afterwards (a stale word would make its waits bail out)
    rng = np.random.default_rng(0)
    x = R.to_bf16(rng.standard_normal((256, 128)).astype(np.float32)); w = R.to_bf16(rng.standard_normal((128, 256)).astype(np.float32))
    gx = gpu_dev.from_bytes(x.tobytes(), [256, 128], "bfloat16"); gw = gpu_dev.from_bytes(w.tobytes(), [128, 256], "bfloat16")
    got = (gx @ gw).to_numpy()
    ref = R.from_bf16(x).astype(np.float64) @ R.from_bf16(w).astype(np.float64)
    assert np.max(np.abs(got - ref)) <= 2e-2 * np.max(np.abs(ref))
    assert gpu_dev.pipeline_status() == 0
    lib.applegpu_eager_free(a)
