"""Batched matmul and attention parity. fp32 runs the CUDA-core kernel (true fp32, reference
tolerance rtol=atol=1e-4: python/tests/test_batched_ops.py:20-54); bf16/f16 run the tcgen05 kernel
and are held to the north-star bar of 2e-2 relative to an fp32 product of the same rounded inputs."""
import numpy as np
import pytest

from oracle import msl_ref as R

pytestmark = pytest.mark.gpu


def bf16_round(x):
    return R.from_bf16(R.to_bf16(np.asarray(x, np.float32)))


def up(gpu, x, dtype):
    if dtype == "bfloat16":
        return gpu.from_bytes(R.to_bf16(x).tobytes(), list(x.shape), "bfloat16")
    return gpu.from_numpy(x.astype(dtype))


def rounded(x, dtype):
    return bf16_round(x) if dtype == "bfloat16" else x.astype(np.float16).astype(np.float32)


def rel_err(got, ref):
    return float(np.max(np.abs(got.astype(np.float64) - ref)) / max(1e-30, float(np.max(np.abs(ref)))))


@pytest.fixture(autouse=True)
def _status_clean(gpu_dev):
    yield
    assert gpu_dev.pipeline_status() == 0, "a bounded wait in the tcgen05 pipeline gave up"


@pytest.mark.parametrize("shape_a,shape_b", [((2, 2), (2, 2)), ((5, 7), (7, 3)), ((64, 64), (64, 64)), ((130, 70), (70, 129)),
                                             ((4, 33, 17), (4, 17, 9)), ((4, 33, 17), (17, 9)), ((2, 3, 8, 5), (2, 3, 5, 4)), ((3, 1, 8, 5), (4, 5, 6))])
def test_matmul_f32_matches_oracle(gpu_dev, shape_a, shape_b):
    rng = np.random.default_rng(sum(shape_a))
    a = rng.standard_normal(shape_a).astype(np.float32); b = rng.standard_normal(shape_b).astype(np.float32)
    got = (gpu_dev.from_numpy(a) @ gpu_dev.from_numpy(b)).to_numpy()
    np.testing.assert_allclose(got, np.matmul(a.astype(np.float64), b.astype(np.float64)), rtol=1e-4, atol=1e-4)
    if a.ndim <= 3 and b.ndim <= 3 and (a.ndim == b.ndim or b.ndim == 2):
        np.testing.assert_allclose(got, R.matmul(a, b), rtol=1e-5, atol=1e-5)   # same k-ascending fp32 accumulation


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 256, 128), (256, 512, 256), (1024, 768, 768), (200, 136, 72), (1, 64, 64),
                                    (8, 2304, 768), (129, 264, 200), (384, 50257 // 8 * 8, 64), (64, 3072, 768), (1000, 1000, 1000)])
def test_matmul_half_tcgen05_b_nmajor(gpu_dev, dtype, m, n, k):
    """B stored [K, N] (the layout of every GPT-2 Conv1D weight): MN-major operand path."""
    rng = np.random.default_rng(m * 31 + n * 7 + k)
    a = rng.standard_normal((m, k)).astype(np.float32); b = rng.standard_normal((k, n)).astype(np.float32)
    ga, gb = up(gpu_dev, a, dtype), up(gpu_dev, b, dtype)
    from applegpu_runtime_b200 import _lib
    assert _lib.load().applegpu_matmul_path(ga.id, gb.id, False) == b"tcgen05"
    got = (ga @ gb).to_numpy().astype(np.float32)
    ref = np.matmul(rounded(a, dtype).astype(np.float64), rounded(b, dtype).astype(np.float64))
    assert rel_err(got, ref) <= 2e-2
    # against the oracle in the same storage type the only difference is summation order
    assert rel_err(got, ref) <= 6e-3


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 300, 96), (77, 50257, 64), (512, 1024, 768)])
def test_matmul_half_tcgen05_b_kmajor(gpu_dev, dtype, m, n, k):
    """B given as transpose([N, K]) — a tied embedding or K in Q.K^T: K-major operand path, no copy."""
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32); bt = rng.standard_normal((n, k)).astype(np.float32)
    ga, gbt = up(gpu_dev, a, dtype), up(gpu_dev, bt, dtype)
    got = (ga @ gpu_dev.transpose(gbt)).to_numpy().astype(np.float32)
    ref = np.matmul(rounded(a, dtype).astype(np.float64), rounded(bt, dtype).astype(np.float64).T)
    assert rel_err(got, ref) <= 6e-3


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("m,n,k,kmajor", [(4096, 768, 256, False), (2100, 2312, 136, False), (4224, 776, 64, False), (8192, 2304, 768, False),
                                           (4096, 1000, 200, True), (2100, 50257, 64, True)])
def test_matmul_cta_pair_tiles(gpu_dev, dtype, m, n, k, kmajor):
    """Shapes large enough for the 256 x 256 CTA-pair kernel (cta_group::2): ragged M (a peer CTA partly or
    wholly past the last row), ragged N, both B layouts; checked against fp64 and against the single-CTA kernel."""
    rng = np.random.default_rng(m + 3 * n + 7 * k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((n, k) if kmajor else (k, n)).astype(np.float32)
    ga, gb = up(gpu_dev, a, dtype), up(gpu_dev, b, dtype)
    gpu_dev.set_matmul_path("tcgen05_pair")
    try:
        got = (ga @ (gpu_dev.transpose(gb) if kmajor else gb)).to_numpy().astype(np.float32)
    finally:
        gpu_dev.set_matmul_path("auto")
    bb = rounded(b, dtype).astype(np.float64)
    ref = np.matmul(rounded(a, dtype).astype(np.float64), bb.T if kmajor else bb)
    assert rel_err(got, ref) <= 6e-3
    gpu_dev.set_matmul_path("tcgen05_1cta")
    try:
        one = (ga @ (gpu_dev.transpose(gb) if kmajor else gb)).to_numpy().astype(np.float32)
    finally:
        gpu_dev.set_matmul_path("auto")
    assert rel_err(got, one.astype(np.float64)) <= 1e-3


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("m,n,k", [(8192, 768, 768), (2048, 768, 3072), (4100, 776, 200), (300, 200, 64)])
def test_matmul_cta_pair_192_wide_tiles_kmajor(gpu_dev, dtype, m, n, k):
    """The 256 x 192 CTA-pair tile (K-major weights: N = 768 fills 74 CTA pairs in 1.73 waves instead of 2.6 or 1.3),
    pinned; bias and residual in the epilogue, ragged M and N, against fp64 and against the single-CTA kernel."""
    rng = np.random.default_rng(m + 3 * n + 7 * k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((n, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    res = rng.standard_normal((m, n)).astype(np.float32)
    ga, gw, gb, gr = up(gpu_dev, a, dtype), up(gpu_dev, w, dtype), up(gpu_dev, bias, dtype), up(gpu_dev, res, dtype)
    ref = rounded(a, dtype).astype(np.float64) @ rounded(w, dtype).astype(np.float64).T + rounded(bias, dtype).astype(np.float64) + rounded(res, dtype).astype(np.float64)
    outs = {}
    for tile in ("pair192", "s128"):
        gpu_dev.set_gemm_tile(tile)
        try:
            y = gr + gpu_dev.add_bias(ga @ gpu_dev.transpose(gw), gb)
            assert "fused_linear[bias,residual,]" in y.plan()
            outs[tile] = y.to_numpy().astype(np.float32)
        finally:
            gpu_dev.set_gemm_tile("auto")
    assert rel_err(outs["pair192"], ref) <= 6e-3
    assert rel_err(outs["pair192"], outs["s128"].astype(np.float64)) <= 1e-3
    assert gpu_dev.pipeline_status() == 0


@pytest.fixture
def pair_path(gpu_dev):
    gpu_dev.set_matmul_path("tcgen05_pair")
    yield
    gpu_dev.set_matmul_path("auto")


def test_matmul_cta_pair_batched_and_epilogues(gpu_dev, pair_path):
    rng = np.random.default_rng(77)
    a = rng.standard_normal((12, 512, 64)).astype(np.float32); b = rng.standard_normal((12, 64, 520)).astype(np.float32)
    got = (up(gpu_dev, a, "bfloat16") @ up(gpu_dev, b, "bfloat16")).to_numpy()
    assert rel_err(got, np.matmul(bf16_round(a).astype(np.float64), bf16_round(b).astype(np.float64))) <= 6e-3
    x = bf16_round(rng.standard_normal((4100, 128))); w = bf16_round(rng.standard_normal((128, 776)) * 0.1)
    bias = bf16_round(rng.standard_normal(776)); res = bf16_round(rng.standard_normal((4100, 776)))
    gx, gw, gb, gr = (up(gpu_dev, t, "bfloat16") for t in (x, w, bias, res))
    y1 = gpu_dev.gelu(gpu_dev.add_bias(gx @ gw, gb)).to_numpy()
    ref = R.gelu((x.astype(np.float64) @ w.astype(np.float64) + bias).astype(np.float32))
    assert rel_err(y1, ref.astype(np.float64)) <= 1.5e-2
    y2 = (gr + gpu_dev.add_bias(gx @ gw, gb)).to_numpy()
    assert rel_err(y2, x.astype(np.float64) @ w.astype(np.float64) + bias + res) <= 1.5e-2


def test_matmul_half_batched_and_broadcast(gpu_dev):
    rng = np.random.default_rng(5)
    a = rng.standard_normal((6, 200, 64)).astype(np.float32); b = rng.standard_normal((6, 64, 136)).astype(np.float32)
    got = (up(gpu_dev, a, "bfloat16") @ up(gpu_dev, b, "bfloat16")).to_numpy()
    assert rel_err(got, np.matmul(bf16_round(a).astype(np.float64), bf16_round(b).astype(np.float64))) <= 6e-3
    w = rng.standard_normal((64, 72)).astype(np.float32)
    got = (up(gpu_dev, a, "bfloat16") @ up(gpu_dev, w, "bfloat16")).to_numpy()      # stride-0 batch on B (lazy.rs:2402-2403)
    assert rel_err(got, np.matmul(bf16_round(a).astype(np.float64), bf16_round(w).astype(np.float64))) <= 6e-3
    a4 = rng.standard_normal((2, 3, 130, 64)).astype(np.float32); b4 = rng.standard_normal((2, 3, 64, 40)).astype(np.float32)
    got = (up(gpu_dev, a4, "bfloat16") @ up(gpu_dev, b4, "bfloat16")).to_numpy()
    assert rel_err(got, np.matmul(bf16_round(a4).astype(np.float64), bf16_round(b4).astype(np.float64))) <= 6e-3


def test_matmul_simt_and_tcgen05_agree(gpu_dev):
    rng = np.random.default_rng(6)
    a = rng.standard_normal((300, 200)).astype(np.float32); b = rng.standard_normal((200, 264)).astype(np.float32)
    ga, gb = up(gpu_dev, a, "bfloat16"), up(gpu_dev, b, "bfloat16")
    t = (ga @ gb).to_numpy()
    gpu_dev.set_matmul_path("simt")
    try:
        s = (ga @ gb).to_numpy()
    finally:
        gpu_dev.set_matmul_path("auto")
    assert rel_err(t, s.astype(np.float64)) <= 4e-3


def test_matmul_odd_layouts_take_the_cuda_core_kernel(gpu_dev):
    rng = np.random.default_rng(7)
    a = rng.standard_normal((10, 7)).astype(np.float32); b = rng.standard_normal((7, 5)).astype(np.float32)   # rows not 16-byte aligned
    got = (up(gpu_dev, a, "bfloat16") @ up(gpu_dev, b, "bfloat16")).to_numpy()
    assert rel_err(got, np.matmul(bf16_round(a).astype(np.float64), bf16_round(b).astype(np.float64))) <= 1e-2


def test_fused_linear_epilogues(gpu_dev):
    rng = np.random.default_rng(8)
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 1.5e-2)):
        x = rng.standard_normal((192, 128)).astype(np.float32); w = (rng.standard_normal((128, 264)) * 0.1).astype(np.float32)
        bias = rng.standard_normal(264).astype(np.float32); res = rng.standard_normal((192, 264)).astype(np.float32)
        if dtype == "bfloat16":
            x, w, bias, res = map(bf16_round, (x, w, bias, res))
        gx, gw, gb, gr = (up(gpu_dev, t, dtype) for t in (x, w, bias, res))
        y1 = gpu_dev.gelu(gpu_dev.add_bias(gx @ gw, gb))
        assert "fused_linear[bias,gelu,]" in y1.plan()
        ref = R.gelu((x.astype(np.float64) @ w.astype(np.float64) + bias).astype(np.float32))
        assert rel_err(y1.to_numpy(), ref.astype(np.float64)) <= tol
        y2 = gr + gpu_dev.add_bias(gx @ gw, gb)
        assert "fused_linear[bias,residual,]" in y2.plan()
        ref2 = x.astype(np.float64) @ w.astype(np.float64) + bias + res
        assert rel_err(y2.to_numpy(), ref2) <= tol
        y3 = gpu_dev.scalar_mul(gx @ gw, 0.125)
        assert "fused_linear[scale,]" in y3.plan()
        assert rel_err(y3.to_numpy(), 0.125 * (x.astype(np.float64) @ w.astype(np.float64))) <= tol
        # unfused execution gives the same numbers (fp32: identical up to fma ordering)
        gpu_dev.set_fusion(True, False)
        try:
            y4 = gpu_dev.gelu(gpu_dev.add_bias(gx @ gw, gb)).to_numpy()
        finally:
            gpu_dev.set_fusion(True, True)
        assert rel_err(y4, ref.astype(np.float64)) <= tol


def test_matmul_int8_weights(gpu_dev):
    rng = np.random.default_rng(9)
    x = bf16_round(rng.standard_normal((70, 96))); w = (rng.standard_normal((130, 96)) * 0.02).astype(np.float32)
    q, s = gpu_dev.quantize_weight(gpu_dev.from_numpy(w))
    got = gpu_dev.matmul_int8(up(gpu_dev, x, "bfloat16"), q, s).to_numpy()
    rq, rs = R.quantize_rows(w)
    ref = R.from_bf16(R.matmul_int8(R.to_bf16(x), rq, rs, st=2))
    assert rel_err(got, ref.astype(np.float64)) <= 1e-2
    xf = rng.standard_normal((9, 96)).astype(np.float32)
    got = gpu_dev.matmul_int8(gpu_dev.from_numpy(xf), q, s).to_numpy()
    np.testing.assert_allclose(got, R.matmul_int8(xf, rq, rs), rtol=1e-5, atol=1e-6)


def test_matmul_int8_prologue_widening_is_exact_and_one_launch(gpu_dev):
    """The tensor-core kernel reads int8 weights as they lie and widens them in its prologue. Identity activations
    make the product return the widened weights themselves: every int8 value, at every position of the swizzled
    tile, must come out exactly, from a single launch (no separate widening pass, no 16-bit copy of the weights)."""
    rng = np.random.default_rng(11)
    k, n = 384, 700                                            # 6 k-blocks; N is not a multiple of the tile width
    w = rng.integers(-127, 128, (n, k)).astype(np.float32)
    w[:, 0] = 127.0                                            # max |w| = 127 in every row: scale exactly 1
    w[5, 1:129] = np.arange(-127, 1, dtype=np.float32)         # the whole negative range in one row
    q, s = gpu_dev.quantize_weight(gpu_dev.from_numpy(w))
    assert np.array_equal(q.to_numpy(), w.astype(np.int8)) and np.all(s.to_numpy() == 1.0)
    x = np.zeros((2 * k, k), np.float32)
    x[np.arange(2 * k), np.arange(2 * k) % k] = 1.0            # two stacked identities: 768 rows, several row blocks
    for dt in ("bfloat16", "float16"):
        gx = up(gpu_dev, x, dt)
        y = gpu_dev.matmul_int8(gx, q, s)
        launches = gpu_dev.launch_count()
        got = y.to_numpy()
        assert gpu_dev.launch_count() - launches == 1
        assert np.array_equal(got, np.concatenate([w.T, w.T], axis=0))
    assert gpu_dev.pipeline_status() == 0


def test_matmul_int8_weights_on_tensor_cores_with_fused_epilogue(gpu_dev):
    """GPT-2-large-like linear: bf16 activations, per-output-channel int8 weights [N, K]; bias, GELU and
    the residual ride in the epilogue of the same GEMM (weights widened exactly to bf16 on the way)."""
    rng = np.random.default_rng(10)
    m, k, n = 512, 320, 1288
    x = bf16_round(rng.standard_normal((m, k))); w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    bias = bf16_round(rng.standard_normal(n) * 0.1); res = bf16_round(rng.standard_normal((m, n)))
    q, s = gpu_dev.quantize_weight(gpu_dev.from_numpy(w))
    rq, rs = R.quantize_rows(w)
    assert np.array_equal(q.to_numpy(), rq) and np.array_equal(s.to_numpy(), rs)      # quantisation itself is bit-exact
    gx, gb, gr = up(gpu_dev, x, "bfloat16"), up(gpu_dev, bias, "bfloat16"), up(gpu_dev, res, "bfloat16")
    y = gpu_dev.gelu(gpu_dev.add_bias(gpu_dev.matmul_int8(gx, q, s), gb))
    assert "fused_linear[int8,bias,gelu,]" in y.plan()
    wd = rq.astype(np.float64) * rs.astype(np.float64)[:, None]
    ref = R.gelu((x.astype(np.float64) @ wd.T + bias).astype(np.float32)).astype(np.float64)
    assert rel_err(y.to_numpy(), ref) <= 1.5e-2
    y2 = gr + gpu_dev.add_bias(gpu_dev.matmul_int8(gx, q, s), gb)
    assert "fused_linear[int8,bias,residual,]" in y2.plan()
    assert rel_err(y2.to_numpy(), x.astype(np.float64) @ wd.T + bias + res) <= 1.5e-2
    # the CUDA-core kernel computes the same product
    gpu_dev.set_matmul_path("simt")
    try:
        y3 = gpu_dev.matmul_int8(gx, q, s).to_numpy()
    finally:
        gpu_dev.set_matmul_path("auto")
    assert rel_err(gpu_dev.matmul_int8(gx, q, s).to_numpy(), y3.astype(np.float64)) <= 8e-3


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("m,n,k,kmajor", [(300, 50257, 64, True), (1000, 777, 96, True), (512, 1032, 128, False), (5, 40, 64, True)])
def test_matmul_argmax_epilogue_is_bit_exact_with_matmul_then_argmax(gpu_dev, dtype, m, n, k, kmajor):
    """argmax(x @ W) with the logits handle dropped runs as one GEMM whose epilogue takes the row maximum
    (no logits tensor). The indices must equal those of the stored-then-scanned form exactly: same
    rounding of each value to the storage type, lowest column on ties (half-precision logits tie often)."""
    rng = np.random.default_rng(m + n)
    a = (rng.integers(-3, 4, (m, k))).astype(np.float32)            # small integers: exact products, many ties
    b = (rng.integers(-2, 3, (n, k) if kmajor else (k, n))).astype(np.float32)
    ga, gb = up(gpu_dev, a, dtype), up(gpu_dev, b, dtype)
    w = gpu_dev.transpose(gb) if kmajor else gb
    logits = ga @ w
    ref_idx = gpu_dev.argmax(logits).to_numpy()                      # handle held: two kernels
    stored = logits.to_numpy().astype(np.float32)
    assert np.array_equal(ref_idx, R.argmax(stored))
    fused = gpu_dev.argmax(gpu_dev.reshape(ga @ w, [m, n]))
    plan = fused.plan()
    assert "fused_linear[argmax,]" in plan and "argmax_" not in plan.replace("fused_linear[argmax,]", "")
    assert np.array_equal(fused.to_numpy(), ref_idx)
    # random real-valued case as well
    a2 = rng.standard_normal((m, k)).astype(np.float32); b2 = rng.standard_normal(b.shape).astype(np.float32)
    ga2, gb2 = up(gpu_dev, a2, dtype), up(gpu_dev, b2, dtype)
    w2 = gpu_dev.transpose(gb2) if kmajor else gb2
    l2 = ga2 @ w2
    want = gpu_dev.argmax(l2).to_numpy()
    assert np.array_equal(gpu_dev.argmax(ga2 @ w2).to_numpy(), want)


@pytest.mark.parametrize("shape_a,shape_b,bt", [((1024, 1024), (1024, 1024), False), ((3, 520, 768), (3, 768, 1032), False), ((2, 1000, 512), (512, 776), False),
                                                ((2048, 768), (1000, 768), True)])
def test_matmul_f32_split_precision_on_tensor_cores(gpu_dev, shape_a, shape_b, bt):
    """float32 products of at least 2 GFLOP: three bf16 terms per operand, six cross terms accumulated in
    float32 on the tensor cores. Bar: the reference's 1e-4 (python/tests/test_batched_ops.py:20-54); measured
    error is orders of magnitude below it and must match the CUDA-core kernel to 1e-5 of the largest entry."""
    rng = np.random.default_rng(sum(shape_a) + sum(shape_b))
    a = rng.standard_normal(shape_a).astype(np.float32); b = rng.standard_normal(shape_b).astype(np.float32)
    ga, gb = gpu_dev.from_numpy(a), gpu_dev.from_numpy(b)
    w = gpu_dev.transpose(gb) if bt else gb
    got = (ga @ w).to_numpy()
    ref = np.matmul(a.astype(np.float64), (b.T if bt else b).astype(np.float64))
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-4)
    assert rel_err(got, ref) <= 2e-6
    gpu_dev.set_f32_split(False)
    try:
        simt = (ga @ w).to_numpy()
    finally:
        gpu_dev.set_f32_split(True)
    assert rel_err(got, simt.astype(np.float64)) <= 1e-5
    # fused epilogue in float32: bias, GELU, residual
    if a.ndim == 2 and not bt:
        bias = rng.standard_normal(shape_b[-1]).astype(np.float32); res = rng.standard_normal(ref.shape).astype(np.float32)
        y = gpu_dev.from_numpy(res) + gpu_dev.gelu(gpu_dev.add_bias(ga @ gb, gpu_dev.from_numpy(bias)))
        want = R.gelu((ref + bias).astype(np.float32)).astype(np.float64) + res
        np.testing.assert_allclose(y.to_numpy(), want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("m,n,k", [(8, 2304, 768), (1, 768, 768), (16, 3072, 768), (8, 768, 3072), (5, 1000, 200), (8, 1288, 1280)])
def test_matmul_skinny_rows_against_a_weight_matrix(gpu_dev, dtype, m, n, k):
    """A decode step: at most 16 rows against a [K, N] weight. Takes the weight-streaming kernel (column
    slabs x K slabs, partials summed in K order); checked against fp64, against the tensor-core kernel, with a
    fused epilogue, and for run-to-run determinism."""
    rng = np.random.default_rng(m * 7 + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32); b = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    bias = rounded(rng.standard_normal(n).astype(np.float32), dtype); res = rounded(rng.standard_normal((m, n)).astype(np.float32), dtype)
    ga, gb, gbias, gres = up(gpu_dev, a, dtype), up(gpu_dev, b, dtype), up(gpu_dev, bias, dtype), up(gpu_dev, res, dtype)
    ref = np.matmul(rounded(a, dtype).astype(np.float64), rounded(b, dtype).astype(np.float64))
    got = (ga @ gb).to_numpy().astype(np.float32)
    assert rel_err(got, ref) <= 6e-3
    again = (ga @ gb).to_numpy().astype(np.float32)
    assert np.array_equal(got, again)                                     # K-ordered reduction: no dependence on scheduling
    gpu_dev.set_matmul_path("tcgen05")
    try:
        tc = (ga @ gb).to_numpy().astype(np.float32)
    finally:
        gpu_dev.set_matmul_path("auto")
    assert rel_err(got, tc.astype(np.float64)) <= 4e-3
    y = gres + gpu_dev.gelu(gpu_dev.add_bias(ga @ gb, gbias))
    want = R.gelu((ref + bias).astype(np.float32)).astype(np.float64) + res
    assert rel_err(y.to_numpy(), want) <= 1.5e-2


@pytest.mark.parametrize("m,n,k", [(8, 2304, 768), (1, 768, 768), (16, 3072, 768), (8, 768, 3072), (5, 1000, 200), (3, 260, 129), (8, 50257, 768), (12, 1001, 1536)])
def test_matmul_skinny_float32(gpu_dev, m, n, k):
    """The float32 form of the weight-streaming kernel: true fp32 multiply-adds (1e-5 relative of fp64),
    equal to the CUDA-core tile kernel within rounding, deterministic, epilogue fused."""
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32); b = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32); res = rng.standard_normal((m, n)).astype(np.float32)
    ga, gb, gbias, gres = (gpu_dev.from_numpy(x) for x in (a, b, bias, res))
    ref = a.astype(np.float64) @ b.astype(np.float64)
    got = (ga @ gb).to_numpy()
    assert rel_err(got, ref) <= 1e-5
    assert np.array_equal(got, (ga @ gb).to_numpy())
    gpu_dev.set_matmul_path("simt")
    try:
        simt = (ga @ gb).to_numpy()
    finally:
        gpu_dev.set_matmul_path("auto")
    assert rel_err(got, simt.astype(np.float64)) <= 1e-5
    y = gres + gpu_dev.relu(gpu_dev.add_bias(ga @ gb, gbias))
    assert rel_err(y.to_numpy(), np.maximum(ref + bias, 0) + res) <= 1e-5
    # a strided A (rows of a wider matrix) still qualifies
    wide = rng.standard_normal((m, k + 8)).astype(np.float32)
    gs = gpu_dev.slice(gpu_dev.from_numpy(wide), 1, 4, 4 + k)
    assert rel_err((gs @ gb).to_numpy(), wide[:, 4:4 + k].astype(np.float64) @ b.astype(np.float64)) <= 1e-5
    # B stored [N, K] (the tied LM head): the K-major weight-streaming kernel where K is a multiple of 4, else the tile kernel
    gbt = gpu_dev.transpose(gpu_dev.from_numpy(np.ascontiguousarray(b.T)))
    got_t = (ga @ gbt).to_numpy()
    assert rel_err(got_t, ref) <= 1e-5
    assert np.array_equal(got_t, (ga @ gbt).to_numpy())
    yt = gres + gpu_dev.relu(gpu_dev.add_bias(ga @ gbt, gbias))
    assert rel_err(yt.to_numpy(), np.maximum(ref + bias, 0) + res) <= 1e-5


# ── attention ───────────────────────────────────────────────────────────────
@pytest.mark.parametrize("tq,tk,causal", [(1, 70, False), (5, 129, False), (200, 200, True), (64, 64, True), (65, 300, False)])
def test_attention_f32_single_kernel_ragged_and_cached(gpu_dev, tq, tk, causal):
    """Head dim 64 in float32 runs as one kernel (online softmax over 64-key blocks): query / key counts that are
    not multiples of the tile, a single query against a cache, and strided (sliced) operands."""
    rng = np.random.default_rng(tq * 1000 + tk)
    q = rng.standard_normal((2, 3, tq, 64)).astype(np.float32)
    k = rng.standard_normal((2, 3, tk, 64)).astype(np.float32)
    v = rng.standard_normal((2, 3, tk, 64)).astype(np.float32)
    fn = gpu_dev.attention_causal if causal else gpu_dev.attention
    launches = gpu_dev.launch_count()
    got = fn(gpu_dev.from_numpy(q), gpu_dev.from_numpy(k), gpu_dev.from_numpy(v)).to_numpy()
    assert gpu_dev.launch_count() - launches == 1
    ref = R.attention(q, k, v, causal)
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-5)
    # operands that are slices of wider tensors (row pitch 192): still one kernel
    wide = rng.standard_normal((2, 3, tk, 192)).astype(np.float32)
    gw = gpu_dev.from_numpy(wide)
    kk, vv = gpu_dev.slice(gw, 3, 64, 128), gpu_dev.slice(gw, 3, 128, 192)
    got2 = fn(gpu_dev.from_numpy(q), kk, vv).to_numpy() if not causal or tq == tk else None
    if got2 is not None:
        np.testing.assert_allclose(got2, R.attention(q, wide[..., 64:128], wide[..., 128:192], causal), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [(2, 8, 8), (3, 33, 16), (1, 4, 130, 64), (2, 12, 128, 64)])
def test_attention_f32_matches_oracle(gpu_dev, causal, shape):
    rng = np.random.default_rng(len(shape))
    q, k, v = (rng.standard_normal(shape).astype(np.float32) for _ in range(3))
    fn = gpu_dev.attention_causal if causal else gpu_dev.attention
    out = fn(gpu_dev.from_numpy(q), gpu_dev.from_numpy(k), gpu_dev.from_numpy(v))
    assert "fused_attention" in out.plan()
    got = out.to_numpy()
    ref = R.attention(q, k, v, causal)
    assert got.shape == ref.shape and np.all(np.isfinite(got))
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-5)
    if causal:   # row 0 sees only V[0]  (ops.rs:3848-3909, test_batched_ops.py:206-265)
        np.testing.assert_allclose(got[..., 0, :], v[..., 0, :], rtol=1e-5, atol=1e-6)


def test_attention_unfused_composition_agrees(gpu_dev):
    rng = np.random.default_rng(11)
    q, k, v = (rng.standard_normal((2, 4, 40, 16)).astype(np.float32) for _ in range(3))
    fused = gpu_dev.attention_causal(gpu_dev.from_numpy(q), gpu_dev.from_numpy(k), gpu_dev.from_numpy(v)).to_numpy()
    gpu_dev.set_fusion(True, False)
    try:
        out = gpu_dev.attention_causal(gpu_dev.from_numpy(q), gpu_dev.from_numpy(k), gpu_dev.from_numpy(v))
        assert "fused_attention" not in out.plan() and "softmax_causal" in out.plan()
        plain = out.to_numpy()
    finally:
        gpu_dev.set_fusion(True, True)
    np.testing.assert_allclose(fused, plain, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("causal", [True, False])
def test_attention_bf16_within_bar(gpu_dev, causal):
    rng = np.random.default_rng(12)
    shape = (2, 12, 256, 64)
    q, k, v = (bf16_round(rng.standard_normal(shape)) for _ in range(3))
    fn = gpu_dev.attention_causal if causal else gpu_dev.attention
    got = fn(up(gpu_dev, q, "bfloat16"), up(gpu_dev, k, "bfloat16"), up(gpu_dev, v, "bfloat16")).to_numpy()
    ref = R.attention(q, k, v, causal)      # fp32 oracle on the same bf16-rounded inputs
    assert rel_err(got, ref.astype(np.float64)) <= 2e-2


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("causal,shape_q,tk", [(True, (2, 3, 128, 64), 128), (True, (1, 2, 200, 64), 200), (True, (2, 12, 1024, 64), 1024),
                                               (False, (1, 4, 130, 64), 130), (False, (3, 2, 1, 64), 300), (False, (1, 1, 77, 64), 513),
                                               (True, (4, 384, 64), 384), (False, (256, 64), 256), (True, (1, 1, 300, 64), 140)])
def test_attention_single_kernel_matches_oracle_and_composition(gpu_dev, dtype, causal, shape_q, tk):
    """Head dim 64 in f16/bf16 takes the single-kernel path: ragged query / key tails, Tq != Tk,
    a decode-shaped call (Tq = 1), 2-D / 3-D / 4-D leading dims."""
    rng = np.random.default_rng(tk + len(shape_q))
    shape_kv = shape_q[:-2] + (tk, 64)
    q = rounded(rng.standard_normal(shape_q).astype(np.float32), dtype)
    k = rounded(rng.standard_normal(shape_kv).astype(np.float32), dtype)
    v = rounded(rng.standard_normal(shape_kv).astype(np.float32), dtype)
    fn = gpu_dev.attention_causal if causal else gpu_dev.attention
    fused = fn(up(gpu_dev, q, dtype), up(gpu_dev, k, dtype), up(gpu_dev, v, dtype)).to_numpy().astype(np.float32)
    ref = R.attention(q, k, v, causal).astype(np.float64)          # fp32 oracle on the same rounded inputs
    assert np.all(np.isfinite(fused))
    assert rel_err(fused, ref) <= 2e-2
    gpu_dev.set_attention_path("composed")
    try:
        composed = fn(up(gpu_dev, q, dtype), up(gpu_dev, k, dtype), up(gpu_dev, v, dtype)).to_numpy().astype(np.float32)
    finally:
        gpu_dev.set_attention_path("auto")
    assert rel_err(composed, ref) <= 2e-2
    assert rel_err(fused, composed.astype(np.float64)) <= 2e-2
    # the single-kernel form keeps scores in fp32, so it is the closer of the two to the fp32 oracle
    assert rel_err(fused, ref) <= rel_err(composed, ref) + 2e-3
    assert gpu_dev.pipeline_status() == 0


def test_attention_on_strided_head_views(gpu_dev):
    # the GPT-2 driver's layout: Q/K/V are column slices of one [B*T, 3d] matrix viewed as [B, h, T, dh]
    rng = np.random.default_rng(13)
    B, T, h, dh = 2, 64, 4, 64
    d = h * dh
    qkv = bf16_round(rng.standard_normal((B * T, 3 * d)))
    g = up(gpu_dev, qkv, "bfloat16")
    def heads(i):
        t = gpu_dev.slice(g, 1, i * d, (i + 1) * d)
        return gpu_dev.transpose_dims(gpu_dev.reshape(t, [B, T, h, dh]), 1, 2)
    out = gpu_dev.attention_causal(heads(0), heads(1), heads(2))
    out = gpu_dev.reshape(gpu_dev.transpose_dims(out, 1, 2), [B * T, d]).to_numpy()
    hq, hk, hv = (np.ascontiguousarray(qkv[:, i * d:(i + 1) * d].reshape(B, T, h, dh).transpose(0, 2, 1, 3)) for i in range(3))
    ref = R.attention(hq, hk, hv, True).transpose(0, 2, 1, 3).reshape(B * T, d)
    assert rel_err(out, ref.astype(np.float64)) <= 2e-2
