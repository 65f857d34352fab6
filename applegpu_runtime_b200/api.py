"""Python surface over the graph flavour of the C ABI.

Mirrors the names and argument meaning of the reference's PyO3 module
(crates/python/src/lib.rs:105-376 `GpuTensor`, :1259-1382 module functions, re-exported by
python/applegpu_runtime/__init__.py:3-125) for the transformer-forward op set, so code written
against `import applegpu_runtime as gpu` (models/gpt2.py, python/tests/test_transformer_ops.py,
test_batched_ops.py, test_attention.py, test_fusion.py) reads the same here. Ops are recorded
lazily; `.to_numpy()`, `.to_list()`, `eval()` run the pending graph on the GPU. Errors raise
ValueError with the library's message, as the PyO3 module does.
"""
import ctypes
import weakref

import numpy as np

from . import _lib

_DTYPE_CODES = {
    "float32": 0, "float16": 1, "float64": 2, "int8": 3, "int16": 4, "int32": 5, "int64": 6,
    "uint8": 7, "uint32": 8, "bool": 9, "bfloat16": 10,
}
_DTYPE_ALIASES = {"f32": "float32", "f16": "float16", "f64": "float64", "i8": "int8", "i16": "int16", "i32": "int32",
                  "i64": "int64", "u8": "uint8", "u32": "uint32", "bool_": "bool", "bf16": "bfloat16"}
_CODE_NAMES = {v: k for k, v in _DTYPE_CODES.items()}
_NP_OF = {
    "float32": np.float32, "float16": np.float16, "float64": np.float64, "int8": np.int8, "int16": np.int16,
    "int32": np.int32, "int64": np.int64, "uint8": np.uint8, "uint32": np.uint32, "bool": np.bool_,
    "bfloat16": np.uint16,  # raw bits; numpy has no bfloat16
}
_SIZES = {"float32": 4, "float16": 2, "float64": 8, "int8": 1, "int16": 2, "int32": 4, "int64": 8, "uint8": 1, "uint32": 4,
          "bool": 1, "bfloat16": 2}

_initialized = False
_dry = False


def _canon_dtype(name):
    name = _DTYPE_ALIASES.get(name, name)
    if name not in _DTYPE_CODES:
        raise ValueError(f"Unknown dtype: {name}")
    return name


def _L():
    return _lib.load()


def _err():
    m = _L().applegpu_ffi_last_error()
    return m.decode() if m else "unknown error"


def version():
    from . import __version__
    return __version__


def init_backend(dry_run=False):
    """Create the CUDA device context (idempotent). `dry_run=True` gives the metadata-only mode
    used on hosts without a GPU: recording, validation and the fusion plan work, eval does not."""
    global _initialized, _dry
    if _initialized:
        return {"backend": "cuda-sm100a", "device": device_name()}
    lib = _L()
    if dry_run:
        if not lib.applegpu_ffi_init_dry():
            raise RuntimeError("dry-run init refused: a device context already exists")
        _dry = True
    elif not lib.applegpu_ffi_init():
        raise RuntimeError(_err())
    _initialized = True
    return {"backend": "cuda-sm100a", "device": device_name()}


def device_name():
    n = _L().applegpu_device_name()
    return n.decode() if n else ""


def dtype_size(dtype):
    return _SIZES[_canon_dtype(dtype)]


def _dims(seq):
    arr = (ctypes.c_uint64 * max(len(seq), 1))(*[int(x) for x in seq])
    return arr, len(seq)


class GpuTensor:
    """Handle to a tensor id of the lazy runtime. Freed when the Python object dies (the free is
    deferred by the runtime while pending ops still use the tensor)."""

    __slots__ = ("id", "_owns", "__weakref__")

    def __init__(self, tid, owns=True):
        if not tid:
            raise ValueError(_err())
        self.id = int(tid)
        self._owns = owns
        if owns:
            weakref.finalize(self, _finalize, self.id)

    # metadata
    @property
    def shape(self):
        out = (ctypes.c_uint64 * 8)()
        nd = ctypes.c_uint32(0)
        if _L().applegpu_ffi_shape(self.id, out, ctypes.byref(nd)) != 0:
            raise ValueError(_err())
        return [int(out[i]) for i in range(nd.value)]

    @property
    def dtype(self):
        c = _L().applegpu_ffi_dtype(self.id)
        if c < 0:
            raise ValueError(f"Tensor {self.id} not found")
        return _CODE_NAMES[c]

    @property
    def ndim(self):
        return len(self.shape)

    def numel(self):
        n = 1
        for d in self.shape:
            n *= d
        return n

    def is_materialized(self):
        return _L().applegpu_ffi_is_pending(self.id) == 0

    # evaluation / readback
    def eval(self):
        if _L().applegpu_ffi_eval(self.id) != 0:
            raise ValueError(_err())
        return self

    def to_bytes(self):
        n = self.numel() * _SIZES[self.dtype]
        buf = (ctypes.c_uint8 * max(n, 1))()
        if _L().applegpu_ffi_read_bytes(self.id, buf, n) != 0:
            raise ValueError(_err())
        return bytes(buf[:n]) if n else b""

    def to_numpy(self):
        """Evaluates and copies to host. bfloat16 is returned widened to float32."""
        dt = self.dtype
        shape = self.shape
        n = self.numel()
        arr = np.empty(n, dtype=_NP_OF[dt])
        if n:
            if _L().applegpu_ffi_read_bytes(self.id, arr.ctypes.data_as(ctypes.c_void_p), n * _SIZES[dt]) != 0:
                raise ValueError(_err())
        if dt == "bfloat16":
            arr = (arr.astype(np.uint32) << 16).view(np.float32)
        return arr.reshape(shape)

    def to_torch(self):
        import torch
        dt = self.dtype
        if dt == "bfloat16":
            n = self.numel()
            raw = np.empty(n, dtype=np.int16)
            if n and _L().applegpu_ffi_read_bytes(self.id, raw.ctypes.data_as(ctypes.c_void_p), n * 2) != 0:
                raise ValueError(_err())
            return torch.from_numpy(raw).view(torch.bfloat16).reshape(self.shape)
        a = self.to_numpy()
        if a.dtype == np.uint32:
            a = a.astype(np.int64)
        return torch.from_numpy(np.ascontiguousarray(a))

    def to_list(self):
        return self.to_numpy().astype(np.float64 if self.dtype.startswith(("float", "bfloat")) else np.int64).reshape(-1).tolist()

    def plan(self):
        """Kernel launch plan of eval() after the fusion pass, one kernel per line."""
        lib = _L()
        n = lib.applegpu_ffi_plan(self.id, None, 0)
        if n < 0:
            raise ValueError(_err())
        buf = ctypes.create_string_buffer(n + 1)
        lib.applegpu_ffi_plan(self.id, buf, n + 1)
        return buf.value.decode()

    # operators
    def __add__(self, o): return add(self, o)
    def __sub__(self, o): return sub(self, o)
    def __mul__(self, o): return mul(self, o) if isinstance(o, GpuTensor) else scalar_mul(self, float(o))
    def __truediv__(self, o): return div(self, o)
    def __matmul__(self, o): return matmul(self, o)
    def __neg__(self): return neg(self)

    # methods named like the reference's pyclass
    def matmul(self, o): return matmul(self, o)
    def add(self, o): return add(self, o)
    def sub(self, o): return sub(self, o)
    def mul(self, o): return mul(self, o)
    def div(self, o): return div(self, o)
    def neg(self): return neg(self)
    def abs(self): return abs(self)
    def sign(self): return sign(self)
    def sin(self): return sin(self)
    def cos(self): return cos(self)
    def relu(self): return relu(self)
    def gelu(self): return gelu(self)
    def gelu_exact(self): return gelu_exact(self)
    def exp(self): return exp(self)
    def log(self): return log(self)
    def sqrt(self): return sqrt(self)
    def tanh(self): return tanh(self)
    def sigmoid(self): return sigmoid(self)
    def softmax(self): return softmax(self)
    def softmax_causal(self): return softmax_causal(self)
    def layer_norm(self, gamma, beta, eps=1e-5): return layer_norm(self, gamma, beta, eps)
    def transpose(self): return transpose(self)
    def transpose_dims(self, dim0, dim1): return transpose_dims(self, dim0, dim1)
    def reshape(self, shape): return reshape(self, shape)
    def slice(self, dim, start, end): return slice(self, dim, start, end)
    def scalar_mul(self, scale): return scalar_mul(self, scale)
    def add_bias(self, bias): return add_bias(self, bias)
    def argmax(self): return argmax(self)
    def gather(self, dim, index): return gather(self, dim, index)
    def index_select(self, dim, index): return index_select(self, dim, index)
    def cast(self, dtype): return cast(self, dtype)
    def sum(self): return sum(self)
    def mean(self): return mean(self)

    def __repr__(self):
        return f"GpuTensor(id={self.id}, shape={self.shape}, dtype={self.dtype})"


def _finalize(tid):
    try:
        if _lib._lib is not None:
            _lib._lib.applegpu_ffi_free(tid)
    except Exception:
        pass


def destroy(t):
    """Release a tensor now (reference: `destroy`, lib.rs)."""
    if isinstance(t, GpuTensor):
        _L().applegpu_ffi_free(t.id)
        t._owns = False


# ── construction ────────────────────────────────────────────────────────────
def _from_buffer(ptr, shape, dtype):
    if not _initialized:
        init_backend()
    dims, nd = _dims(shape)
    tid = _L().applegpu_ffi_from_host(ptr, dims, nd, _DTYPE_CODES[dtype])
    if not tid:
        raise ValueError(_err())
    return GpuTensor(tid)


def from_numpy(arr):
    arr = np.asarray(arr)
    name = {np.dtype(np.float32): "float32", np.dtype(np.float16): "float16", np.dtype(np.float64): "float64",
            np.dtype(np.int8): "int8", np.dtype(np.int16): "int16", np.dtype(np.int32): "int32", np.dtype(np.int64): "int64",
            np.dtype(np.uint8): "uint8", np.dtype(np.uint32): "uint32", np.dtype(np.bool_): "bool"}.get(arr.dtype)
    if name is None:
        raise ValueError(f"Unsupported numpy dtype: {arr.dtype}")
    a = np.ascontiguousarray(arr)
    t = _from_buffer(a.ctypes.data_as(ctypes.c_void_p), list(a.shape), name)
    _L().applegpu_ffi_synchronize()  # `a` may be a temporary; the copy must land before it dies
    return t


def from_bytes(data, shape, dtype):
    dtype = _canon_dtype(dtype)
    n = 1
    for d in shape:
        n *= d
    if len(data) != n * _SIZES[dtype]:
        raise ValueError(f"from_bytes: {len(data)} bytes given, shape {list(shape)} of {dtype} needs {n * _SIZES[dtype]}")
    buf = (ctypes.c_uint8 * max(len(data), 1)).from_buffer_copy(data if len(data) else b"\0")
    t = _from_buffer(buf, list(shape), dtype)
    _L().applegpu_ffi_synchronize()
    return t


def from_torch(t):
    """Ingests a CPU torch tensor, including torch.bfloat16 (which the reference's from_torch
    lacks: crates/python/src/lib.rs:465-479 has no bfloat16 branch)."""
    import torch
    t = t.detach().contiguous().cpu()
    name = {torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16", torch.float64: "float64",
            torch.int8: "int8", torch.int16: "int16", torch.int32: "int32", torch.int64: "int64", torch.uint8: "uint8",
            torch.bool: "bool"}.get(t.dtype)
    if name is None:
        raise ValueError(f"Unsupported torch dtype: {t.dtype}")
    g = _from_buffer(ctypes.c_void_p(t.data_ptr()), list(t.shape), name)
    _L().applegpu_ffi_synchronize()
    return g


def tensor(values, shape, dtype="float32"):
    dtype = _canon_dtype(dtype)
    return from_numpy(np.asarray(values, dtype=_NP_OF[dtype]).reshape(shape))


def aligned_numpy(shape, dtype="float32"):
    return np.zeros(shape, dtype=_NP_OF[_canon_dtype(dtype)])


from_numpy_shared = from_numpy
from_torch_shared = from_torch


# ── ops ─────────────────────────────────────────────────────────────────────
def _wrap(tid, *srcs):
    if not tid:
        raise ValueError(_err())
    for s in srcs:  # recorders may return an input unchanged (no-op cast / transpose)
        if isinstance(s, GpuTensor) and s.id == tid:
            return s
    return GpuTensor(tid)


def _bin(fn_name):
    def f(a, b):
        return _wrap(getattr(_L(), fn_name)(a.id, b.id), a, b)
    return f


def _un(fn_name):
    def f(a):
        return _wrap(getattr(_L(), fn_name)(a.id), a)
    return f


add = _bin("applegpu_ffi_add")
sub = _bin("applegpu_ffi_sub")
mul = _bin("applegpu_ffi_mul")
div = _bin("applegpu_ffi_div")
matmul = _bin("applegpu_ffi_matmul")
neg = _un("applegpu_ffi_neg")
relu = _un("applegpu_ffi_relu")
exp = _un("applegpu_ffi_exp")
log = _un("applegpu_ffi_log")
sqrt = _un("applegpu_ffi_sqrt")
tanh = _un("applegpu_ffi_tanh")
sin = _un("applegpu_ffi_sin")
cos = _un("applegpu_ffi_cos")
abs = _un("applegpu_ffi_abs")
sign = _un("applegpu_ffi_sign")
sigmoid = _un("applegpu_ffi_sigmoid")
gelu = _un("applegpu_ffi_gelu")
gelu_exact = _un("applegpu_ffi_gelu_exact")
softmax = _un("applegpu_ffi_softmax")
softmax_causal = _un("applegpu_ffi_softmax_causal")
argmax = _un("applegpu_ffi_argmax")
sum = _un("applegpu_ffi_sum")
mean = _un("applegpu_ffi_mean")
transpose = _un("applegpu_ffi_transpose")
embedding = _bin("applegpu_ffi_embedding")
add_bias = _bin("applegpu_ffi_add_bias")


def scalar_mul(t, scale):
    return _wrap(_L().applegpu_ffi_scalar_mul(t.id, float(scale)), t)


def layer_norm(input, gamma, beta, eps=1e-5):
    return _wrap(_L().applegpu_ffi_layer_norm(input.id, gamma.id, beta.id, float(eps)), input)


def transpose_dims(t, dim0, dim1):
    return _wrap(_L().applegpu_ffi_transpose_dims(t.id, int(dim0), int(dim1)), t)


def reshape(t, new_shape):
    dims, nd = _dims(list(new_shape))
    return _wrap(_L().applegpu_ffi_reshape(t.id, dims, nd), t)


def slice(t, dim, start, end):
    return _wrap(_L().applegpu_ffi_slice(t.id, int(dim), int(start), int(end)), t)


def concat(a, b, dim=0):
    return _wrap(_L().applegpu_ffi_concat(a.id, b.id, int(dim)), a, b)


def concat_all(tensors, dim=0):
    if len(tensors) == 0:
        raise ValueError("concat_all requires at least 1 tensor")
    out = tensors[0]
    for t in tensors[1:]:
        out = concat(out, t, dim=dim)
    return out


def gather(input, dim, index):
    return _wrap(_L().applegpu_ffi_gather(input.id, int(dim), index.id), input)


def index_select(input, dim, index):
    return _wrap(_L().applegpu_ffi_index_select(input.id, int(dim), index.id), input)


def cast(t, dtype):
    return _wrap(_L().applegpu_ffi_cast(t.id, _DTYPE_CODES[_canon_dtype(dtype)]), t)


def quantize(t, dtype, scale=0.1, zero_point=0):
    return _wrap(_L().applegpu_ffi_quantize(t.id, _DTYPE_CODES[_canon_dtype(dtype)], float(scale), int(zero_point)), t)


def dequantize(t, dtype, scale=0.1, zero_point=0):
    return _wrap(_L().applegpu_ffi_dequantize(t.id, _DTYPE_CODES[_canon_dtype(dtype)], float(scale), int(zero_point)), t)


def attention(q, k, v):
    return _wrap(_L().applegpu_ffi_attention(q.id, k.id, v.id), q)


def attention_causal(q, k, v):
    return _wrap(_L().applegpu_ffi_attention_causal(q.id, k.id, v.id), q)


def quantize_weight(w):
    """Per-output-channel symmetric int8 for a [N,K] weight: returns (q int8 [N,K], scales f32 [N])."""
    q = ctypes.c_uint64(0)
    s = ctypes.c_uint64(0)
    if _L().applegpu_ffi_quantize_weight(w.id, ctypes.byref(q), ctypes.byref(s)) != 0:
        raise ValueError(_err())
    return GpuTensor(q.value), GpuTensor(s.value)


def matmul_int8(x, q, scales):
    """x [..,M,K] @ (q[N,K] * scales[N])^T with the dequantisation inside the GEMM."""
    return _wrap(_L().applegpu_ffi_matmul_int8(x.id, q.id, scales.id), x)


_ACT_CODES = {None: 0, "none": 0, "gelu": 1, "gelu_exact": 2, "relu": 3}


def linear_fused(x, w, bias=None, residual=None, act=None, ln=None, stats_out=None, stats_zero=None):
    """act(x @ w + bias) + residual as one tensor-core launch with the epilogue named up front, and layer_norm folded
    into the product: `ln=(colsum, stats, eps)` makes the result act(rstd * (x @ w - mean * colsum) + bias) with mean and
    rstd of each row of x taken from `stats` [rows, 2] (int64: sum and sum of squares in 2^-28 fixed point), which equals
    layer_norm(x) @ w0 + b0 when w = gamma[:, None] * w0, colsum = w.sum(0) and bias = beta @ w0 + b0 (see
    gpt2.fold_gpt2_layer_norms); `stats_out` [rows, 2] (int64) receives the (sum, sum of squares) of every stored row
    (added with integer atomics, so the order of addition does not matter; it must hold zeros), `stats_zero` [rows, 2]
    has those rows cleared. 16-bit dtypes on the tensor-core path only."""
    colsum, stats, eps = ln if ln is not None else (None, None, 0.0)
    oid = _L().applegpu_ffi_linear_fused(x.id, w.id, bias.id if bias is not None else 0, residual.id if residual is not None else 0, _ACT_CODES[act],
                                         colsum.id if colsum is not None else 0, stats.id if stats is not None else 0, float(eps),
                                         stats_out.id if stats_out is not None else 0, stats_zero.id if stats_zero is not None else 0)
    return _wrap(oid, x, w, bias, residual, colsum, stats, stats_out, stats_zero)


def eval(t):
    t.eval()


def to_list(t):
    return t.to_list()


def shape(t):
    return t.shape


def synchronize():
    _L().applegpu_ffi_synchronize()


# ── op tapes ────────────────────────────────────────────────────────────────
class Tape:
    """The ops one pass of a host program recorded between `tape_begin` and `tape_end`; `replay` issues
    them again on new inputs with one library call instead of one per op."""

    __slots__ = ("handle", "n_inputs", "n_outputs")

    def __init__(self, handle, n_inputs, n_outputs):
        self.handle, self.n_inputs, self.n_outputs = handle, n_inputs, n_outputs

    def replay(self, inputs):
        if len(inputs) != self.n_inputs:
            raise ValueError(f"the tape takes {self.n_inputs} inputs, got {len(inputs)}")
        ids = (ctypes.c_uint64 * max(1, len(inputs)))(*[t.id for t in inputs])
        out = (ctypes.c_uint64 * max(1, self.n_outputs))()
        if _L().applegpu_ffi_tape_replay(self.handle, ids, len(inputs), out, self.n_outputs) < 0:
            raise ValueError(_err())
        held = {t.id for t in inputs}
        # an output that is one of the inputs is owned by whoever passed it in
        return [GpuTensor(out[i], owns=out[i] not in held) for i in range(self.n_outputs)]


def tape_begin(inputs):
    """Start noting every op call. `inputs` are the tensors that will differ between replays."""
    ids = (ctypes.c_uint64 * max(1, len(inputs)))(*[t.id for t in inputs])
    if _L().applegpu_ffi_tape_begin(ids, len(inputs)) != 0:
        raise ValueError(_err())
    return len(inputs)


def tape_end(n_inputs, outputs):
    ids = (ctypes.c_uint64 * max(1, len(outputs)))(*[t.id for t in outputs])
    h = _L().applegpu_ffi_tape_end(ids, len(outputs))
    if not h:
        raise ValueError(_err())
    return Tape(int(h), n_inputs, len(outputs))


def tape_abort():
    _L().applegpu_ffi_tape_abort()


# ── runtime services ────────────────────────────────────────────────────────
def pool_stats():
    out = (ctypes.c_uint64 * 7)()
    _L().applegpu_pool_stats(out)
    return {"hits": int(out[0]), "misses": int(out[1]), "pooled_bytes": int(out[2]), "bucket_count": int(out[3]),
            "live_bytes": int(out[4]), "peak_live_bytes": int(out[5]), "live_buffers": int(out[6])}


def pool_drain():
    _L().applegpu_pool_drain()


def set_pool_watermark(mb):
    _L().applegpu_pool_set_watermark(int(mb) * 1024 * 1024)


def memory_usage():
    return int(_L().applegpu_memory_usage())


def tensor_count():
    return int(_L().applegpu_tensor_count())


def set_fusion(elementwise_chains=True, patterns=True):
    _L().applegpu_ffi_set_fusion(bool(elementwise_chains), bool(patterns))


def set_matmul_path(mode):
    """'auto', 'simt' (CUDA-core kernel), 'tcgen05' (error if operands are not TMA-compatible),
    'tcgen05_1cta' (single-CTA tiles only) or 'tcgen05_pair' (256 x 256 CTA-pair tiles where the shape allows)."""
    _L().applegpu_set_matmul_path({"auto": 0, "simt": 1, "tcgen05": 2, "tcgen05_1cta": 3, "tcgen05_pair": 4}[mode])


def matmul_path(a, b):
    """Which kernel family `a @ b` would take for these two (materialised) tensors: 'tcgen05' or 'simt'."""
    r = _L().applegpu_matmul_path(a.id, b.id, False)
    if not r:
        raise ValueError("matmul_path: unknown tensor id or not a matrix")
    return r.decode()


_TILE_CODES = {"auto": 0, "pair256": 1256, "pair192": 1192, "pair128": 1128, "s256": 256, "s192": 192, "s128": 128}


def set_gemm_tile(name="auto"):
    """Pin the tile shape of the tensor-core GEMM (a tuning and test override): CTA-pair tiles 256 x {256, 192, 128}
    (192 for K-major weights only) or single-CTA tiles 128 x {256, 192, 128}; "auto" picks by modelled cost."""
    _L().applegpu_set_gemm_tile(_TILE_CODES[name])


def set_sm_margin(n=0):
    """Keep `n` SMs out of the persistent kernels' grids (room for a collective on another stream); 0 uses every SM."""
    _L().applegpu_set_sm_margin(int(n))


def set_gemm_chain(on=True, min_rows=None):
    """Chained linears: consecutive 16-bit fused linears of one evaluation, each reading the previous one's result, go
    out as one tensor-core launch (bit-identical results). On by default; APPLEGPU_GEMM_CHAIN=0 starts with it off.
    `min_rows`: linears with fewer rows stay separate launches (default 4096, where chaining starts to pay)."""
    _L().applegpu_set_gemm_chain(bool(on))
    if min_rows is not None:
        _L().applegpu_set_gemm_chain_min_rows(int(min_rows))


def gemm_chain_enabled():
    return bool(_L().applegpu_gemm_chain_enabled())


def gemm_chain_min_rows():
    return int(_L().applegpu_gemm_chain_min_rows())


def gemm_chain_applies(rows):
    """Whether linears of `rows` rows are chained as things stand."""
    return gemm_chain_enabled() and int(rows) >= gemm_chain_min_rows()


def set_f32_split(on=True):
    """Large float32 matmuls as a three-term bf16 split on the tensor cores (default) or always on CUDA cores."""
    _L().applegpu_set_f32_split(bool(on))


def set_attention_path(mode):
    """'auto' (single-kernel attention when eligible) or 'composed' (GEMM + softmax + GEMM)."""
    _L().applegpu_set_attention_path({"auto": 0, "composed": 1}[mode])


def pipeline_status():
    return int(_L().applegpu_pipeline_status())


def launch_count():
    return int(_L().applegpu_launch_count())


def resolve_kernel(base_name, dtype):
    r = _L().applegpu_resolve_kernel(base_name.encode(), _DTYPE_CODES[_canon_dtype(dtype)])
    return r.decode() if r else None


def profile(enable=True, only=None):
    """Turns per-kernel CUDA-event timing on or off (clears earlier records when turning on). `only`: a list of
    kernel-name prefixes (e.g. ["fused_linear", "matmul"]); just those nodes are bracketed, the rest of the step runs
    as it normally does."""
    lib = _L()
    if enable:
        lib.applegpu_profile_clear()
    lib.applegpu_profile_filter(",".join(only).encode() if only else b"")
    lib.applegpu_profile_enable(bool(enable))


def profile_report():
    """{kernel name: {"launches", "ms", "work"}}; work is flops for contractions, bytes otherwise."""
    lib = _L()
    n = lib.applegpu_profile_report(None, 0)
    buf = ctypes.create_string_buffer(n + 1)
    lib.applegpu_profile_report(buf, n + 1)
    out = {}
    for line in buf.value.decode().splitlines():
        name, cnt, ms, work = line.split()
        out[name] = {"launches": int(cnt), "ms": float(ms), "work": float(work)}
    return out
