"""torch frontend: a tensor subclass whose aten ops are recorded into the lazy graph of this library.

Counterpart of the reference's python/applegpu_runtime/torch_backend.py (the `__torch_dispatch__`
frontend: `ApplegpuTensor` :1823-1960, the aten op table :246-1805, `to_applegpu` :1988, `enable`
:18, CPU fallback for ops outside the table :1914). Same user-facing names and flow:

    import applegpu_runtime_b200.torch_backend as tb
    tb.enable()
    model = tb.to_applegpu(model)              # parameters and buffers become ApplegpuTensors
    y = model(tb.to_applegpu(x)).to_torch_cpu()

Differences in design, made for a discrete 180 GB device instead of unified memory:
* the subclass is a storage-less wrapper (`_make_wrapper_subclass`): no host mirror is allocated
  per tensor, the only copy of the data is the device buffer behind the `GpuTensor`;
* ops are recorded lazily and evaluated when a result leaves the device (`to_torch_cpu`,
  `.item()`, a fallback), so the graph-level rewrites of the library (linear = matmul + bias +
  activation + residual in one tensor-core GEMM, single-kernel attention) fire on torch programs;
* bfloat16 is a first-class dtype;
* `F.scaled_dot_product_attention` without a mask is routed to the library's attention op
  (`__torch_function__`), so the score matrix is never materialised;
* an aten op outside the table raises (`strict`, the default): nothing falls back to the host
  unasked. `enable(strict=False)` opts into the reference's behaviour (the op runs through PyTorch
  CPU), and every such call is counted (`fallback_stats()`).
"""
import collections
import math

import torch
import torch.nn.functional as F

from . import api as gpu

aten = torch.ops.aten

_TORCH_TO_GPU = {torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16", torch.float64: "float64",
                 torch.int8: "int8", torch.int16: "int16", torch.int32: "int32", torch.int64: "int64", torch.uint8: "uint8",
                 torch.bool: "bool"}
_GPU_TO_TORCH = {v: k for k, v in _TORCH_TO_GPU.items()}
_FLOAT = ("float32", "float16", "bfloat16")

_TANH_GELU_MODULES = ("NewGELUActivation", "GELUTanh", "PytorchGELUTanh", "FastGELUActivation")
SUPPORTED_OPS = {}
_fallbacks = collections.Counter()
_strict = True
_enabled = False
_in_fallback = False


def enable(strict=True):
    """Initialise the device and the frontend. By default an aten op outside the table raises;
    `strict=False` lets it run through PyTorch CPU (the reference's fallback), counted in
    `fallback_stats()`."""
    global _enabled, _strict
    gpu.init_backend()
    _enabled = True
    _strict = bool(strict)


def fallback_stats():
    """{aten op name: times it ran through PyTorch CPU} since the last reset_fallback_stats()."""
    return dict(_fallbacks)


def reset_fallback_stats():
    _fallbacks.clear()


def register_op(*aten_ops):
    def deco(fn):
        for op in aten_ops:
            SUPPORTED_OPS[op] = fn
        return fn
    return deco


class ApplegpuTensor(torch.Tensor):
    """torch.Tensor whose data lives in a GpuTensor of this library (reported device: cpu, so that
    index tensors and masks a model builds with `device=x.device` stay ordinary host tensors)."""

    @staticmethod
    def __new__(cls, gpu_tensor, torch_dtype=None, requires_grad=False):
        if torch_dtype is None:
            torch_dtype = _GPU_TO_TORCH[gpu_tensor.dtype]
        r = torch.Tensor._make_wrapper_subclass(cls, tuple(gpu_tensor.shape), dtype=torch_dtype, device="cpu", requires_grad=requires_grad)
        r._gpu_tensor = gpu_tensor
        return r

    @property
    def _gpu(self):
        return self._gpu_tensor

    def __repr__(self):
        g = self._gpu_tensor
        return f"ApplegpuTensor(shape={list(g.shape)}, dtype={g.dtype}, device='applegpu')"

    __str__ = __repr__

    def __reduce_ex__(self, protocol):
        return self.to_torch_cpu().__reduce_ex__(protocol)   # torch.save writes host bytes

    @classmethod
    def from_torch(cls, tensor):
        return cls(gpu.from_torch(tensor), torch_dtype=tensor.dtype)

    def to_torch_cpu(self):
        g = self._gpu_tensor
        t = g.to_torch()
        want = self.dtype
        return t if t.dtype == want else t.to(want)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func is F.scaled_dot_product_attention and not _in_fallback:
            r = _sdpa(*args, **kwargs)
            if r is not NotImplemented:
                return r
        # run the function without torch's default post-processing, which would re-type host results
        # (an argmax index tensor, layer-norm statistics) as storage-less instances of this class
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if _in_fallback:
            return func(*args, **kwargs)
        h = SUPPORTED_OPS.get(func)
        if h is not None:
            r = h(*args, **kwargs)
            if r is not NotImplemented:
                return r
        return _cpu_fallback(func, args, kwargs)


# ── helpers ──────────────────────────────────────────────────────────────────
def _wrap(g, like=None):
    dt = None
    if like is not None and isinstance(like, torch.Tensor) and _TORCH_TO_GPU.get(like.dtype) == g.dtype:
        dt = like.dtype
    return ApplegpuTensor(g, torch_dtype=dt)


def _unwrap(t, dtype=None):
    """GpuTensor of an ApplegpuTensor, or an upload of a host tensor (cast to `dtype` first)."""
    if isinstance(t, ApplegpuTensor):
        g = t._gpu_tensor
        if dtype is not None and g.dtype != dtype:
            g = gpu.cast(g, dtype)
        return g
    if isinstance(t, torch.Tensor):
        if dtype is not None and _TORCH_TO_GPU.get(t.dtype) != dtype:
            t = t.to(_GPU_TO_TORCH[dtype])
        if t.dim() == 0:
            t = t.reshape(1)
        return _upload(t)
    raise TypeError(f"cannot move {type(t)} to the device")


_recording_consts = None     # while compile_forward records: host tensors uploaded on the way (kept alive with the tape)


def _upload(t):
    g = gpu.from_torch(t)
    if _recording_consts is not None:
        _recording_consts.append(g)
    return g


def _scalar_tensor(value, dtype):
    return _upload(torch.tensor([float(value)], dtype=_GPU_TO_TORCH[dtype]))


def _is_dev(t):
    return isinstance(t, ApplegpuTensor)


def _gdtype(*ts):
    for t in ts:
        if _is_dev(t):
            return t._gpu_tensor.dtype
    return "float32"


def _norm_dim(d, n):
    return d + n if d < 0 else d


def _to_cpu_tree(x):
    if isinstance(x, ApplegpuTensor):
        return x.to_torch_cpu()
    if isinstance(x, (list, tuple)):
        return type(x)(_to_cpu_tree(v) for v in x)
    if isinstance(x, dict):
        return {k: _to_cpu_tree(v) for k, v in x.items()}
    return x


def _to_dev_tree(x):
    if isinstance(x, torch.Tensor) and not isinstance(x, ApplegpuTensor) and x.dtype in _TORCH_TO_GPU and x.dtype not in (torch.bool, torch.int64):
        return ApplegpuTensor.from_torch(x)
    if isinstance(x, (list, tuple)):
        return type(x)(_to_dev_tree(v) for v in x)
    return x


def _cpu_fallback(func, args, kwargs):
    """Ops outside the table: evaluate the operands, run PyTorch CPU, move float results back.
    This is the frontend's behaviour upstream too (torch_backend.py:1914); integer and bool
    results (indices, masks) stay on the host, where the handlers pick them up."""
    global _in_fallback
    name = str(func)
    if _strict:
        raise NotImplementedError(f"applegpu torch frontend (strict): {name} is not in the op table")
    _fallbacks[name] += 1
    cargs, ckw = _to_cpu_tree(args), _to_cpu_tree(kwargs)
    was = _in_fallback
    _in_fallback = True
    try:
        out = func(*cargs, **ckw)
    finally:
        _in_fallback = was
    return _to_dev_tree(out)


# ── lifecycle ────────────────────────────────────────────────────────────────
@register_op(aten.detach.default, aten.alias.default, aten.lift_fresh.default)
def _op_detach(a):
    return ApplegpuTensor(a._gpu_tensor, torch_dtype=a.dtype) if _is_dev(a) else NotImplemented


@register_op(aten.clone.default, aten.contiguous.default)
def _op_clone(a, memory_format=None):
    if not _is_dev(a):
        return NotImplemented
    g = a._gpu_tensor
    if g.dtype in _FLOAT:
        return _wrap(gpu.scalar_mul(g, 1.0), a)
    return ApplegpuTensor(g, torch_dtype=a.dtype)   # tensors are immutable values in the graph


@register_op(aten._to_copy.default)
def _op_to_copy(a, dtype=None, layout=None, device=None, pin_memory=None, non_blocking=False, memory_format=None):
    if not _is_dev(a):
        return NotImplemented
    if dtype is None or dtype == a.dtype:
        return ApplegpuTensor(a._gpu_tensor, torch_dtype=a.dtype)
    if dtype not in _TORCH_TO_GPU:
        return NotImplemented
    return ApplegpuTensor(gpu.cast(a._gpu_tensor, _TORCH_TO_GPU[dtype]), torch_dtype=dtype)


@register_op(aten._local_scalar_dense.default)
def _op_item(a):
    return a.to_torch_cpu().reshape(-1)[0].item()


# ── elementwise ──────────────────────────────────────────────────────────────
def _binary(fn, a, b, alpha=1):
    dt = _gdtype(a, b)
    if dt not in _FLOAT:
        return NotImplemented
    like = a if _is_dev(a) else b
    if isinstance(a, (int, float)):
        ga = _scalar_tensor(a, dt)
    else:
        ga = _unwrap(a, dt)
    if isinstance(b, (int, float)):
        if fn is gpu.mul:
            return _wrap(gpu.scalar_mul(ga, float(b)), like)
        if fn is gpu.div:
            return _wrap(gpu.scalar_mul(ga, 1.0 / float(b)), like)
        gb = _scalar_tensor(float(b) * alpha, dt)
    else:
        gb = _unwrap(b, dt)
        if alpha != 1:
            gb = gpu.scalar_mul(gb, float(alpha))
    g = fn(ga, gb)
    return ApplegpuTensor(g, torch_dtype=_GPU_TO_TORCH[g.dtype])


@register_op(aten.add.Tensor, aten.add.Scalar)
def _op_add(a, b, alpha=1):
    return _binary(gpu.add, a, b, alpha)


@register_op(aten.sub.Tensor, aten.sub.Scalar)
def _op_sub(a, b, alpha=1):
    return _binary(gpu.sub, a, b, alpha)


@register_op(aten.rsub.Scalar)
def _op_rsub(a, b, alpha=1):
    return _binary(gpu.sub, b, a, alpha)


@register_op(aten.mul.Tensor, aten.mul.Scalar)
def _op_mul(a, b):
    if isinstance(a, (int, float)):
        a, b = b, a
    if isinstance(b, torch.Tensor) and not _is_dev(b) and b.dim() == 0 and _is_dev(a):
        b = b.item()
    if isinstance(a, torch.Tensor) and not _is_dev(a) and a.dim() == 0 and _is_dev(b):
        a, b = b, a.item()
    return _binary(gpu.mul, a, b)


@register_op(aten.div.Tensor, aten.div.Scalar)
def _op_div(a, b, rounding_mode=None):
    if rounding_mode is not None:
        return NotImplemented
    if isinstance(b, torch.Tensor) and not _is_dev(b) and b.dim() == 0:
        b = b.item()
    return _binary(gpu.div, a, b)


def _unary(fn):
    def h(a, *rest, **kw):
        if not _is_dev(a) or a._gpu_tensor.dtype not in _FLOAT:
            return NotImplemented
        return _wrap(fn(a._gpu_tensor), a)
    return h


for _op, _fn in ((aten.neg.default, gpu.neg), (aten.relu.default, gpu.relu), (aten.exp.default, gpu.exp), (aten.log.default, gpu.log),
                 (aten.sqrt.default, gpu.sqrt), (aten.tanh.default, gpu.tanh), (aten.sigmoid.default, gpu.sigmoid), (aten.abs.default, gpu.abs),
                 (aten.sign.default, gpu.sign), (aten.sin.default, gpu.sin), (aten.cos.default, gpu.cos)):
    SUPPORTED_OPS[_op] = _unary(_fn)


@register_op(aten.gelu.default)
def _op_gelu(a, approximate="none"):
    if not _is_dev(a) or a._gpu_tensor.dtype not in _FLOAT:
        return NotImplemented
    return _wrap(gpu.gelu(a._gpu_tensor) if approximate == "tanh" else gpu.gelu_exact(a._gpu_tensor), a)


@register_op(aten.silu.default)
def _op_silu(a):
    if not _is_dev(a) or a._gpu_tensor.dtype not in _FLOAT:
        return NotImplemented
    g = a._gpu_tensor
    return _wrap(gpu.mul(g, gpu.sigmoid(g)), a)


@register_op(aten.pow.Tensor_Scalar)
def _op_pow(a, exponent):
    if not _is_dev(a) or a._gpu_tensor.dtype not in _FLOAT:
        return NotImplemented
    g = a._gpu_tensor
    if exponent == 2:
        return _wrap(gpu.mul(g, g), a)
    if exponent == 3:
        return _wrap(gpu.mul(gpu.mul(g, g), g), a)
    if exponent == 0.5:
        return _wrap(gpu.sqrt(g), a)
    return NotImplemented


@register_op(aten.reciprocal.default)
def _op_reciprocal(a):
    if not _is_dev(a) or a._gpu_tensor.dtype not in _FLOAT:
        return NotImplemented
    return _wrap(gpu.div(_scalar_tensor(1.0, a._gpu_tensor.dtype), a._gpu_tensor), a)


# ── matmul family ────────────────────────────────────────────────────────────
@register_op(aten.mm.default, aten.bmm.default, aten.matmul.default)
def _op_mm(a, b):
    dt = _gdtype(a, b)
    if dt not in _FLOAT:
        return NotImplemented
    return _wrap(gpu.matmul(_unwrap(a, dt), _unwrap(b, dt)), a if _is_dev(a) else b)


@register_op(aten.addmm.default)
def _op_addmm(bias, a, b, beta=1, alpha=1):
    dt = _gdtype(a, b, bias)
    if dt not in _FLOAT:
        return NotImplemented
    mm = gpu.matmul(_unwrap(a, dt), _unwrap(b, dt))
    if alpha != 1:
        mm = gpu.scalar_mul(mm, float(alpha))
    gb = _unwrap(bias, dt)
    if beta != 1:
        gb = gpu.scalar_mul(gb, float(beta))
    # a [N] bias is the add_bias op (which the linear rewrite absorbs into the GEMM epilogue)
    out = gpu.add_bias(mm, gb) if len(gb.shape) == 1 and gb.shape[0] == mm.shape[-1] else gpu.add(mm, gb)
    return _wrap(out, a if _is_dev(a) else b)


@register_op(aten.linear.default)
def _op_linear(x, w, b=None):
    dt = _gdtype(x, w)
    if dt not in _FLOAT:
        return NotImplemented
    gx = _unwrap(x, dt)
    lead = list(gx.shape[:-1])
    if len(lead) != 1:
        gx = gpu.reshape(gx, [int(math.prod(lead)), gx.shape[-1]])
    out = gpu.matmul(gx, gpu.transpose(_unwrap(w, dt)))
    if b is not None:
        out = gpu.add_bias(out, _unwrap(b, dt))
    if len(lead) != 1:
        out = gpu.reshape(out, lead + [out.shape[-1]])
    return _wrap(out, x if _is_dev(x) else w)


# ── normalisation, softmax, embedding, attention ────────────────────────────
@register_op(aten.native_layer_norm.default)
def _op_native_layer_norm(x, normalized_shape, weight, bias, eps):
    if not _is_dev(x) or len(normalized_shape) != 1 or x._gpu_tensor.dtype not in _FLOAT:
        return NotImplemented
    dt = x._gpu_tensor.dtype
    n = normalized_shape[0]
    gw = _unwrap(weight, dt) if weight is not None else _upload(torch.ones(n, dtype=_GPU_TO_TORCH[dt]))
    gb = _unwrap(bias, dt) if bias is not None else _upload(torch.zeros(n, dtype=_GPU_TO_TORCH[dt]))
    out = _wrap(gpu.layer_norm(x._gpu_tensor, gw, gb, float(eps)), x)
    stat_shape = list(x.shape[:-1]) + [1]
    empty = torch.empty(stat_shape, dtype=torch.float32)      # mean / rstd: only the backward pass reads them
    return out, empty, empty.clone()


@register_op(aten.layer_norm.default)
def _op_layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5, cudnn_enable=True):
    r = _op_native_layer_norm(x, normalized_shape, weight, bias, eps)
    return r if r is NotImplemented else r[0]


@register_op(aten._softmax.default, aten.softmax.int)
def _op_softmax(x, dim, half_to_float_or_dtype=None):
    if not _is_dev(x) or _norm_dim(dim, x.dim()) != x.dim() - 1 or x._gpu_tensor.dtype not in _FLOAT:
        return NotImplemented
    if half_to_float_or_dtype not in (None, False) and half_to_float_or_dtype != x.dtype:
        return NotImplemented
    return _wrap(gpu.softmax(x._gpu_tensor), x)


@register_op(aten.embedding.default)
def _op_embedding(weight, indices, padding_idx=-1, scale_grad_by_freq=False, sparse=False):
    if not _is_dev(weight):
        return NotImplemented
    gi = _unwrap(indices, "int32") if not _is_dev(indices) else _unwrap(indices, "int32")
    return _wrap(gpu.embedding(weight._gpu_tensor, gi), weight)


def _sdpa(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False):
    if attn_mask is not None or dropout_p != 0.0 or enable_gqa or not (_is_dev(query) and _is_dev(key) and _is_dev(value)):
        return NotImplemented
    d = query.shape[-1]
    if scale is not None and abs(scale - 1.0 / math.sqrt(d)) > 1e-9:
        return NotImplemented
    if is_causal and query.shape[-2] != key.shape[-2]:
        return NotImplemented
    q, k, v = query._gpu_tensor, key._gpu_tensor, value._gpu_tensor
    return _wrap(gpu.attention_causal(q, k, v) if is_causal else gpu.attention(q, k, v), query)


@register_op(aten.argmax.default)
def _op_argmax(x, dim=None, keepdim=False):
    if not _is_dev(x) or dim is None or _norm_dim(dim, x.dim()) != x.dim() - 1 or keepdim:
        return NotImplemented
    idx = gpu.argmax(x._gpu_tensor).to_torch()      # int32 on the device; torch's contract is int64 on the host
    return idx.to(torch.int64)


# ── layout ───────────────────────────────────────────────────────────────────
def _infer_shape(shape, numel):
    shape = [int(s) for s in shape]
    if -1 in shape:
        known = 1
        for s in shape:
            if s != -1:
                known *= s
        shape[shape.index(-1)] = numel // max(known, 1)
    return shape


@register_op(aten.view.default, aten._unsafe_view.default, aten.reshape.default, aten._reshape_alias.default)
def _op_view(a, shape, *unused):
    if not _is_dev(a):
        return NotImplemented
    return _wrap(gpu.reshape(a._gpu_tensor, _infer_shape(shape, a.numel())), a)


@register_op(aten.flatten.using_ints)
def _op_flatten(a, start_dim=0, end_dim=-1):
    if not _is_dev(a):
        return NotImplemented
    n = a.dim()
    s, e = _norm_dim(start_dim, n), _norm_dim(end_dim, n)
    shp = list(a.shape)
    return _wrap(gpu.reshape(a._gpu_tensor, shp[:s] + [int(math.prod(shp[s:e + 1]))] + shp[e + 1:]), a)


@register_op(aten.unsqueeze.default)
def _op_unsqueeze(a, dim):
    if not _is_dev(a):
        return NotImplemented
    shp = list(a.shape)
    shp.insert(_norm_dim(dim, a.dim() + 1), 1)
    return _wrap(gpu.reshape(a._gpu_tensor, shp), a)


@register_op(aten.squeeze.dim)
def _op_squeeze(a, dim):
    if not _is_dev(a):
        return NotImplemented
    shp = list(a.shape)
    d = _norm_dim(dim, a.dim())
    if shp[d] == 1:
        shp.pop(d)
    return _wrap(gpu.reshape(a._gpu_tensor, shp), a)


@register_op(aten.t.default)
def _op_t(a):
    if not _is_dev(a) or a.dim() != 2:
        return NotImplemented
    return _wrap(gpu.transpose(a._gpu_tensor), a)


@register_op(aten.transpose.int)
def _op_transpose(a, d0, d1):
    if not _is_dev(a):
        return NotImplemented
    n = a.dim()
    return _wrap(gpu.transpose_dims(a._gpu_tensor, _norm_dim(d0, n), _norm_dim(d1, n)), a)


@register_op(aten.permute.default)
def _op_permute(a, dims):
    if not _is_dev(a):
        return NotImplemented
    n = a.dim()
    want = [_norm_dim(d, n) for d in dims]
    cur = list(range(n))
    g = a._gpu_tensor
    for i in range(n):                      # selection sort by swaps: at most n-1 transposes (views in the executor)
        if cur[i] != want[i]:
            j = cur.index(want[i])
            g = gpu.transpose_dims(g, i, j)
            cur[i], cur[j] = cur[j], cur[i]
    return _wrap(g, a)


@register_op(aten.slice.Tensor)
def _op_slice(a, dim=0, start=None, end=None, step=1):
    if not _is_dev(a) or step != 1:
        return NotImplemented
    d = _norm_dim(dim, a.dim())
    size = a.shape[d]
    s = 0 if start is None else (start + size if start < 0 else start)
    e = size if end is None else (end + size if end < 0 else end)
    s, e = max(0, min(s, size)), max(0, min(e, size))
    if s == 0 and e == size:
        return ApplegpuTensor(a._gpu_tensor, torch_dtype=a.dtype)
    if e <= s:
        return NotImplemented
    return _wrap(gpu.slice(a._gpu_tensor, d, s, e), a)


@register_op(aten.select.int)
def _op_select(a, dim, index):
    if not _is_dev(a):
        return NotImplemented
    d = _norm_dim(dim, a.dim())
    i = index + a.shape[d] if index < 0 else index
    shp = list(a.shape)
    shp.pop(d)
    return _wrap(gpu.reshape(gpu.slice(a._gpu_tensor, d, i, i + 1), shp if shp else [1]), a)


@register_op(aten.split.Tensor)
def _op_split(a, split_size, dim=0):
    if not _is_dev(a):
        return NotImplemented
    d = _norm_dim(dim, a.dim())
    size = a.shape[d]
    return [_op_slice(a, d, s, min(s + split_size, size)) for s in range(0, size, split_size)]


@register_op(aten.split_with_sizes.default)
def _op_split_with_sizes(a, sizes, dim=0):
    if not _is_dev(a):
        return NotImplemented
    d = _norm_dim(dim, a.dim())
    out, s = [], 0
    for n in sizes:
        out.append(_op_slice(a, d, s, s + n))
        s += n
    return out


@register_op(aten.unbind.int)
def _op_unbind(a, dim=0):
    if not _is_dev(a):
        return NotImplemented
    return [_op_select(a, dim, i) for i in range(a.shape[_norm_dim(dim, a.dim())])]


@register_op(aten.cat.default)
def _op_cat(tensors, dim=0):
    dev = [t for t in tensors if _is_dev(t)]
    if not dev:
        return NotImplemented
    dt = dev[0]._gpu_tensor.dtype
    parts = [_unwrap(t, dt) for t in tensors if t.numel() > 0]
    return _wrap(gpu.concat_all(parts, dim=_norm_dim(dim, dev[0].dim())), dev[0])


@register_op(aten.expand.default)
def _op_expand(a, size, implicit=False):
    if not _is_dev(a):
        return NotImplemented
    shp = list(a.shape)
    size = list(size)
    lead = len(size) - len(shp)
    if all(s == -1 or s == shp[i - lead] for i, s in enumerate(size) if i >= lead) and all(s == 1 for s in size[:lead]):
        return _wrap(gpu.reshape(a._gpu_tensor, [1] * lead + shp), a)     # nothing is broadcast: a reshape
    return NotImplemented


# ── moving models and tensors ────────────────────────────────────────────────
def to_applegpu(model_or_tensor, dtype=None):
    """Moves a tensor, or the parameters and buffers of an nn.Module (in place), to the device.
    `dtype` (e.g. torch.bfloat16) converts floating-point data on the way."""
    if not _enabled:
        enable()
    if isinstance(model_or_tensor, torch.Tensor):
        t = model_or_tensor
        if isinstance(t, ApplegpuTensor):
            return t
        if dtype is not None and t.is_floating_point():
            t = t.to(dtype)
        return ApplegpuTensor.from_torch(t)
    module = model_or_tensor
    seen = {}
    # activations written out op by op in Python (HF's `gelu_new`: 0.5 x (1 + tanh(sqrt(2/pi)(x + 0.044715 x^3))))
    # become the aten op of the same function, which the linear rewrite folds into the GEMM epilogue
    for parent in module.modules():
        for name, child in list(parent._modules.items()):
            if child is not None and type(child).__name__ in _TANH_GELU_MODULES:
                parent._modules[name] = torch.nn.GELU(approximate="tanh")
    for mod in module.modules():
        for name, p in list(mod._parameters.items()):
            if p is None:
                continue
            key = id(p)
            if key not in seen:           # tied weights (GPT-2's wte / lm_head) stay one device tensor
                seen[key] = torch.nn.Parameter(to_applegpu(p.detach(), dtype), requires_grad=False)
            mod._parameters[name] = seen[key]
        for name, b in list(mod._buffers.items()):
            if b is None or not b.is_floating_point():
                continue                  # integer / bool buffers (position ids, masks) stay on the host
            key = id(b)
            if key not in seen:
                seen[key] = to_applegpu(b, dtype)
            mod._buffers[name] = seen[key]
    return module


def compile_forward(fn, select=None):
    """Records the ops `fn` issues once per input signature and replays them afterwards.

    The Python side of a forward (module calls, aten dispatch, shape logic) costs several times the
    device time of a GPT-2-small prefill; a replay issues the same ops with one library call
    (`applegpu_ffi_tape_replay`: shapes are re-inferred, fusion runs as usual). The counterpart
    upstream is the compiled-graph path (python/applegpu_runtime/compile_backend.py -> one
    `applegpu_eager_execute_graph` call per forward). `fn` takes tensors (host tensors are moved to
    the device; integer tensors as int32) and returns a tensor, a tuple / list of tensors, or any
    object from which `select` picks those. Requirements, as for any trace: the ops `fn` issues may
    depend on the shapes and dtypes of its inputs, not on their values; tensors `fn` creates on the
    host (position ids, masks) are captured as constants.
    """
    cache = {}

    def run(*args):
        global _recording_consts
        dev = []
        for a in args:
            if not isinstance(a, ApplegpuTensor):
                a = a.to(torch.int32) if not a.is_floating_point() and a.dtype != torch.bool else a
                a = ApplegpuTensor.from_torch(a)
            dev.append(a)
        key = tuple((tuple(a.shape), a.dtype) for a in dev)
        hit = cache.get(key)
        if hit is not None:
            tape, _consts, many = hit
            outs = [ApplegpuTensor(g) for g in tape.replay([a._gpu_tensor for a in dev])]
            return outs if many else outs[0]
        if _recording_consts is not None:
            raise RuntimeError("compile_forward: a recording is already in progress")
        n = gpu.tape_begin([a._gpu_tensor for a in dev])
        _recording_consts = []
        try:
            out = fn(*dev)
            picked = select(out) if select is not None else out
            many = isinstance(picked, (list, tuple))
            outs = list(picked) if many else [picked]
            if not all(isinstance(o, ApplegpuTensor) for o in outs):
                raise TypeError("compile_forward: the function must return device tensors")
            tape = gpu.tape_end(n, [o._gpu_tensor for o in outs])
        except Exception:
            gpu.tape_abort()
            raise
        finally:
            consts, _recording_consts = _recording_consts, None
        cache[key] = (tape, consts, many)
        return outs if many else outs[0]

    run.cache = cache
    return run
