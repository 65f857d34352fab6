"""Chained linears: consecutive fused linears of one evaluation, each reading the previous one's result, go out as ONE
launch of the tensor-core kernel whose tiles wait row block by row block for the tiles that produce their rows
(csrc/kernels/gemm_tc.cu gemm_tc_chain_kernel, csrc/core/exec.cc chain). The reference runs every linear of a block as
its own dispatch (python/applegpu_runtime/models/gpt2.py:101-157); the bar here is that chaining changes nothing: the
results are bit-identical to the separate launches with the same tile shape, and within the 16-bit tolerance (2e-2
relative) of a float64 product of the same rounded inputs."""
import numpy as np
import pytest

from oracle import msl_ref as R

pytestmark = pytest.mark.gpu


def up(gpu, x, dtype):
    if dtype == "bfloat16":
        return gpu.from_bytes(R.to_bf16(x).tobytes(), list(x.shape), "bfloat16")
    return gpu.from_numpy(x.astype(dtype))


def rounded(x, dtype):
    return R.from_bf16(R.to_bf16(np.asarray(x, np.float32))) if dtype == "bfloat16" else x.astype(np.float16).astype(np.float32)


@pytest.fixture(autouse=True)
def _restore(gpu_dev):
    was, rows = gpu_dev.gemm_chain_enabled(), gpu_dev.gemm_chain_min_rows()
    gpu_dev.set_gemm_chain(True, min_rows=0)     # by default only linears of 4096 rows and more are chained
    yield
    gpu_dev.set_gemm_chain(was, min_rows=rows)
    gpu_dev.set_gemm_tile("auto")
    assert gpu_dev.pipeline_status() == 0, "a bounded wait in the tcgen05 pipeline gave up"


def _mlp(gpu, x, ws, bs, acts, residual_at):
    """x -> linear_fused -> ... ; link i adds the input of link `residual_at[i]`'s result when named."""
    outs = []
    h = x
    for i, (w, b, act) in enumerate(zip(ws, bs, acts)):
        res = outs[residual_at[i]] if residual_at.get(i) is not None else None
        h = gpu.linear_fused(h, w, bias=b, act=act, residual=res)
        outs.append(h)
    return h, outs


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("rows", [1000, 256, 2304])
def test_chain_matches_separate_launches(gpu_dev, dtype, rows):
    """Five links (one more than a chain holds), ragged sizes: rows not a multiple of 256, widths that are not multiples
    of the 256-column tile, K that is not a multiple of the 128-deep pipeline stage; bias everywhere, GELU on one link,
    a residual that is an earlier link's result (same rows, row block by row block)."""
    gpu = gpu_dev
    dims = [320, 512, 768, 272, 768, 320]
    rng = np.random.default_rng(rows)
    x = (rng.standard_normal((rows, dims[0])) * 0.5).astype(np.float32)
    ws = [(rng.standard_normal((dims[i], dims[i + 1])) / np.sqrt(dims[i])).astype(np.float32) for i in range(5)]
    bs = [(rng.standard_normal(dims[i + 1]) * 0.1).astype(np.float32) for i in range(5)]
    acts = [None, "gelu", None, None, None]
    residual_at = {3: 1}            # link 3 ([rows, 768]) adds link 1's result ([rows, 768]), two links back in the same chain
    gx = up(gpu, x, dtype)
    gw = [up(gpu, w, dtype) for w in ws]
    gb = [up(gpu, b, dtype) for b in bs]
    for t in [gx] + gw + gb:
        t.eval()

    def run():
        before = gpu.launch_count()
        out, outs = _mlp(gpu, gx, gw, gb, acts, residual_at)
        out.eval()
        mids = [o.to_numpy() for o in outs]     # every intermediate is kept alive and read back too
        return mids, gpu.launch_count() - before

    chained, launches_chained = run()
    chained_again, _ = run()
    gpu.set_gemm_tile("pair256")            # a pinned tile shape (the chained kernel's) also means one launch per linear
    separate, launches_separate = run()
    gpu.set_gemm_tile("auto")
    assert launches_separate == 5
    assert launches_chained == 2            # four links as one launch, the fifth alone
    for a, b, c in zip(chained, separate, chained_again):
        assert np.array_equal(a, b)         # same arithmetic, same order: bit for bit
        assert np.array_equal(a, c)
    # against float64 on the rounded inputs, rounding every stored activation as the device does
    h = rounded(x, dtype).astype(np.float64)
    refs = []
    for i in range(5):
        h = h @ rounded(ws[i], dtype).astype(np.float64) + rounded(bs[i], dtype).astype(np.float64)
        if acts[i] == "gelu":
            h = 0.5 * h * (1.0 + np.tanh(0.7978845608028654 * (h + 0.044715 * h ** 3)))
        if residual_at.get(i) is not None:
            h = h + refs[residual_at[i]]
        h = rounded(h.astype(np.float32), dtype).astype(np.float64)
        refs.append(h)
    for got, ref in zip(chained, refs):
        err = float(np.max(np.abs(got.astype(np.float64) - ref)) / np.max(np.abs(ref)))
        assert err <= 2e-2, err


def test_chain_breaks_where_a_link_does_not_follow(gpu_dev):
    """Two independent linears in one evaluation, then one that reads the first: nothing may be reordered or merged
    wrongly; results equal the unchained evaluation bit for bit."""
    gpu = gpu_dev
    rng = np.random.default_rng(5)
    x = up(gpu, rng.standard_normal((512, 256)).astype(np.float32), "bfloat16")
    y = up(gpu, rng.standard_normal((512, 256)).astype(np.float32), "bfloat16")
    w1 = up(gpu, (rng.standard_normal((256, 512)) / 16).astype(np.float32), "bfloat16")
    w2 = up(gpu, (rng.standard_normal((256, 512)) / 16).astype(np.float32), "bfloat16")
    w3 = up(gpu, (rng.standard_normal((512, 256)) / 22).astype(np.float32), "bfloat16")

    def run():
        a = gpu.linear_fused(x, w1)
        b = gpu.linear_fused(y, w2)              # does not read a
        c = gpu.linear_fused(a, w3, residual=x)  # reads a, which is not the product just before it
        d = gpu.linear_fused(b, w3, residual=c)  # reads b and c
        d.eval()
        return [t.to_numpy() for t in (a, b, c, d)]

    on = run()
    gpu.set_gemm_tile("pair256")
    off = run()
    for p, q in zip(on, off):
        assert np.array_equal(p, q)


def test_gpt2_forward_chained_equals_unchained(gpu_dev):
    """The folded-layer_norm GPT-2 forward (row statistics written by one link and read by the next, cleared by a third)
    with the four linears between two attention kernels chained: logits bit-identical to one launch per linear."""
    gpu = gpu_dev
    from applegpu_runtime_b200.gpt2 import init_gpt2_weights, gpt2_forward
    cfg = {"n_layer": 3, "n_head": 4, "n_embd": 256, "vocab_size": 1003, "n_positions": 512}
    model = init_gpt2_weights(cfg, seed=3, dtype="bfloat16")
    ids = np.random.default_rng(9).integers(0, cfg["vocab_size"], (3, 300))      # 900 rows: a ragged last row block

    def run():
        before = gpu.launch_count()
        logits, _ = gpt2_forward(model, ids)
        logits.eval()
        return logits.to_numpy(), gpu.launch_count() - before

    on, launches_on = run()
    on_again, _ = run()
    gpu.set_gemm_tile("pair256")            # same [K, N] weights, one launch per linear
    off, launches_off = run()
    assert np.array_equal(on, off)
    assert np.array_equal(on, on_again)
    assert launches_on < launches_off       # [proj, FC1, FC2, next QKV] went out together
    assert launches_off - launches_on == 3 + 3 + 2   # blocks 0 and 1: proj, FC1, FC2 and the next QKV as one launch instead of four; the last block has three links


def test_few_rows_are_not_chained(gpu_dev):
    """Below the row threshold (default 4096) the linears stay separate launches, where that is faster."""
    gpu = gpu_dev
    gpu.set_gemm_chain(True, min_rows=4096)
    assert gpu.gemm_chain_applies(8192) and not gpu.gemm_chain_applies(2048)
    rng = np.random.default_rng(2)
    x = up(gpu, rng.standard_normal((512, 256)).astype(np.float32), "bfloat16")
    w1 = up(gpu, (rng.standard_normal((256, 512)) / 16).astype(np.float32), "bfloat16")
    w2 = up(gpu, (rng.standard_normal((512, 256)) / 22).astype(np.float32), "bfloat16")
    for t in (x, w1, w2):
        t.eval()
    before = gpu.launch_count()
    y = gpu.linear_fused(gpu.linear_fused(x, w1), w2)
    y.eval()
    assert gpu.launch_count() - before == 2


def test_chain_with_sms_kept_free(gpu_dev):
    """With SMs kept out of the compute grids (room for a collective on another stream) the chained kernel runs on fewer
    CTA pairs and deals its tiles to those: same results."""
    gpu = gpu_dev
    rng = np.random.default_rng(11)
    x = up(gpu, (rng.standard_normal((1536, 256)) * 0.5).astype(np.float32), "bfloat16")
    ws = [up(gpu, (rng.standard_normal((256, 768)) / 16).astype(np.float32), "bfloat16"),
          up(gpu, (rng.standard_normal((768, 256)) / 28).astype(np.float32), "bfloat16"),
          up(gpu, (rng.standard_normal((256, 512)) / 16).astype(np.float32), "bfloat16")]
    for t in [x] + ws:
        t.eval()

    def run():
        before = gpu.launch_count()
        h = gpu.linear_fused(x, ws[0], act="gelu")
        h = gpu.linear_fused(h, ws[1], residual=x)
        h = gpu.linear_fused(h, ws[2])
        h.eval()
        return h.to_numpy(), gpu.launch_count() - before

    full, n_full = run()
    gpu.set_sm_margin(20)
    try:
        fewer, n_fewer = run()
    finally:
        gpu.set_sm_margin(0)
    assert n_full == 1 and n_fewer == 1
    assert np.array_equal(full, fewer)
