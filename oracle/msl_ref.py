"""TEST INFRASTRUCTURE: numpy front-end of oracle/msl_ref.c (built by oracle/Makefile).

bfloat16 arrays are carried as uint16 bit patterns with `st=2`; `to_bf16` / `from_bf16` convert.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libmsl_ref.so")
_lib = None

ST = {"float32": 0, "float16": 1, "bfloat16": 2}
_NP = {0: np.float32, 1: np.float16, 2: np.uint16}


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE])


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _i64(v):
    return ctypes.c_int64(int(v))


def to_bf16(x):
    """float32 array -> uint16 bf16 bit patterns (round to nearest even)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().ref_convert(_p(x), 0, _p(out), 2, _i64(x.size))
    return out


def from_bf16(bits):
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _st_of(a, st):
    if st is not None:
        return st
    return {np.dtype(np.float32): 0, np.dtype(np.float16): 1, np.dtype(np.uint16): 2}[a.dtype]


def matmul(a, b, st=None):
    st = _st_of(a, st)
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    m, k = a.shape[-2:]; n = b.shape[-1]
    ba = int(np.prod(a.shape[:-2], dtype=np.int64)); bb = int(np.prod(b.shape[:-2], dtype=np.int64))
    batch = max(ba, bb)
    out_shape = (a.shape[:-2] if ba >= bb else b.shape[:-2]) + (m, n)
    out = np.empty(out_shape, a.dtype)
    lib().ref_matmul(_p(a), _p(b), _p(out), _i64(batch), _i64(m), _i64(n), _i64(k),
                     _i64(m * k if ba == batch and ba > 1 or batch == 1 else 0), _i64(k * n if bb == batch and bb > 1 or batch == 1 else 0), st)
    return out


def layer_norm(x, gamma, beta, eps=1e-5, st=None):
    st = _st_of(x, st)
    x = np.ascontiguousarray(x); out = np.empty_like(x)
    cols = x.shape[-1]
    lib().ref_layer_norm(_p(x), _p(np.ascontiguousarray(gamma)), _p(np.ascontiguousarray(beta)), _p(out), _i64(x.size // cols), _i64(cols),
                         ctypes.c_float(eps), st)
    return out


def softmax(x, st=None):
    st = _st_of(x, st)
    x = np.ascontiguousarray(x); out = np.empty_like(x)
    cols = x.shape[-1]
    lib().ref_softmax(_p(x), _p(out), _i64(x.size // cols), _i64(cols), st)
    return out


def softmax_causal(x, st=None):
    st = _st_of(x, st)
    x = np.ascontiguousarray(x); out = np.empty_like(x)
    rows, cols = x.shape[-2:]
    lib().ref_softmax_causal(_p(x), _p(out), _i64(x.size // (rows * cols)), _i64(rows), _i64(cols), st)
    return out


def gelu(x, st=None):
    st = _st_of(x, st)
    x = np.ascontiguousarray(x); out = np.empty_like(x)
    lib().ref_gelu(_p(x), _p(out), _i64(x.size), st)
    return out


def gelu_exact(x, st=None):
    st = _st_of(x, st)
    x = np.ascontiguousarray(x); out = np.empty_like(x)
    lib().ref_gelu_exact(_p(x), _p(out), _i64(x.size), st)
    return out


def add_bias(x, bias, st=None):
    st = _st_of(x, st)
    x = np.ascontiguousarray(x); out = np.empty_like(x)
    stride = int(np.prod(x.shape[2:], dtype=np.int64))
    lib().ref_add_bias(_p(x), _p(np.ascontiguousarray(bias)), _p(out), _i64(x.size), _i64(stride), _i64(x.shape[1]), st)
    return out


def binary(a, b, op, st=None):
    st = _st_of(a, st)
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b); out = np.empty_like(a)
    lib().ref_binary(_p(a), _p(b), _p(out), _i64(a.size), {"add": 0, "sub": 1, "mul": 2, "div": 3}[op], st)
    return out


def scalar_mul(x, scale, st=None):
    st = _st_of(x, st)
    x = np.ascontiguousarray(x); out = np.empty_like(x)
    lib().ref_scalar_mul(_p(x), _p(out), _i64(x.size), ctypes.c_float(scale), st)
    return out


def embedding(w, idx):
    w = np.ascontiguousarray(w); idx = np.ascontiguousarray(idx, dtype=np.int32)
    out = np.empty(idx.shape + (w.shape[1],), w.dtype)
    lib().ref_embedding(_p(w), _p(idx), _p(out), _i64(idx.size), _i64(w.shape[1]), _i64(w.dtype.itemsize))
    return out


def gather(x, dim, idx):
    x = np.ascontiguousarray(x); idx = np.ascontiguousarray(idx, dtype=np.int32)
    assert x.dtype.itemsize == 4
    out = np.empty(idx.shape, x.dtype)
    lib().ref_gather(_p(x), _p(idx), _p(out), _i64(idx.shape[0]), _i64(idx.shape[1]), _i64(x.shape[1]), int(dim))
    return out


def index_select(x, dim, idx):
    x = np.ascontiguousarray(x); idx = np.ascontiguousarray(idx, dtype=np.int32)
    assert x.dtype.itemsize == 4
    shape = (idx.shape[0], x.shape[1]) if dim == 0 else (x.shape[0], idx.shape[0])
    out = np.empty(shape, x.dtype)
    lib().ref_index_select(_p(x), _p(idx), _p(out), _i64(shape[0]), _i64(shape[1]), _i64(x.shape[1]), int(dim))
    return out


def argmax(x, st=None):
    st = _st_of(x, st)
    x = np.ascontiguousarray(x)
    cols = x.shape[-1]
    out = np.empty(x.shape[:-1] if x.ndim > 1 else (1,), np.int32)
    lib().ref_argmax(_p(x), _p(out), _i64(x.size // cols), _i64(cols), st)
    return out


def quantize(x, dtype, scale, zero_point=0, st=None):
    st = _st_of(x, st)
    x = np.ascontiguousarray(x)
    signed = dtype in ("int8", "i8")
    out = np.empty(x.shape, np.int8 if signed else np.uint8)
    lib().ref_quantize(_p(x), _p(out), _i64(x.size), ctypes.c_float(scale), ctypes.c_int32(zero_point), int(signed), st)
    return out


def dequantize(q, dtype, scale, zero_point=0):
    q = np.ascontiguousarray(q)
    st = ST[dtype]
    out = np.empty(q.shape, _NP[st])
    lib().ref_dequantize(_p(q), _p(out), _i64(q.size), ctypes.c_float(scale), ctypes.c_int32(zero_point), int(q.dtype == np.int8), st)
    return out


def attention(q, k, v, causal, st=None):
    st = _st_of(q, st)
    q = np.ascontiguousarray(q); k = np.ascontiguousarray(k); v = np.ascontiguousarray(v)
    tq, d = q.shape[-2:]; tk = k.shape[-2]; dv = v.shape[-1]
    bh = q.size // (tq * d)
    out = np.empty(q.shape[:-1] + (dv,), q.dtype)
    scratch = np.empty(tq * tk, q.dtype)
    lib().ref_attention(_p(q), _p(k), _p(v), _p(out), _p(scratch), _i64(bh), _i64(tq), _i64(tk), _i64(d), _i64(dv), int(bool(causal)), st)
    return out


def quantize_rows(w, st=None):
    st = _st_of(w, st)
    w = np.ascontiguousarray(w)
    q = np.empty(w.shape, np.int8); s = np.empty(w.shape[0], np.float32)
    lib().ref_quantize_rows(_p(w), _p(q), _p(s), _i64(w.shape[0]), _i64(w.shape[1]), st)
    return q, s


def matmul_int8(x, q, scales, st=None):
    st = _st_of(x, st)
    x = np.ascontiguousarray(x); q = np.ascontiguousarray(q, dtype=np.int8); scales = np.ascontiguousarray(scales, dtype=np.float32)
    k = x.shape[-1]; m = x.size // k; n = q.shape[0]
    out = np.empty(x.shape[:-1] + (n,), x.dtype)
    lib().ref_matmul_int8(_p(x), _p(q), _p(scales), _p(out), _i64(m), _i64(n), _i64(k), st)
    return out
