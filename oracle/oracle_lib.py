"""TEST INFRASTRUCTURE — ctypes loader of the CPU restatement (liboracle_linear.so) and of the
reference's own CUDA kernels (_ref/libref_mlp.so). Imported only by tests/, by
__graft_entry__.smoke() and by bench.py's CPU-baseline legs; the product never imports it."""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle_linear.so")
REF_SO = os.path.join(HERE, "_ref", "libref_mlp.so")
REF_TRAIN_SO = os.path.join(HERE, "_ref", "libref_train.so")
REF_TRAIN_B200_SO = os.path.join(HERE, "_ref", "libref_train_b200.so")


def build(reference_root=None):
    """make the CPU oracle; make the reference-kernel libraries too when a reference checkout is named
    (argument, or the environment variable GPT2CU_REFERENCE) and exists."""
    subprocess.run(["make", "-C", HERE], check=True, capture_output=True)
    reference_root = reference_root or os.environ.get("GPT2CU_REFERENCE")
    if reference_root and os.path.exists(os.path.join(reference_root, "include", "gpt2", "layers", "mlp.h")):
        res = subprocess.run(["make", "-C", HERE, "ref", f"REF={reference_root}"], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("make ref failed:\n" + res.stdout[-2000:] + res.stderr[-4000:])


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build()
        L = ctypes.CDLL(ORACLE_SO)
        F = ctypes.POINTER(ctypes.c_float)
        D = ctypes.POINTER(ctypes.c_double)
        I = ctypes.c_int
        L.oracle_linear_forward_f32.argtypes = [F, F, F, F, I, I, I, I]
        L.oracle_linear_forward_f64.argtypes = [D, F, F, F, I, I, I, I]
        L.oracle_linear_backward_input_f32.argtypes = [F, F, F, I, I, I, I]
        L.oracle_linear_backward_input_f64.argtypes = [D, F, F, I, I, I, I]
        L.oracle_linear_backward_weight_f32.argtypes = [F, F, F, F, I, I, I, I]
        L.oracle_linear_backward_weight_f64.argtypes = [D, D, F, F, I, I, I, I]
        L.oracle_gelu_f32.argtypes = [F, F, ctypes.c_long]
        L.oracle_gelu_grad_mul_f64.argtypes = [D, F, D, ctypes.c_long]
        L.oracle_set_threads.argtypes = [I]
        L.oracle_get_threads.restype = I
        _lib = L
    return _lib


def _f(a):
    return None if a is None else a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _d(a):
    return None if a is None else a.ctypes.data_as(ctypes.POINTER(ctypes.c_double))


def _c(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def set_threads(n):
    lib().oracle_set_threads(n)


def get_threads():
    return lib().oracle_get_threads()


def forward(x, w, b=None, f64=False):
    """x [M,K], w [K,N], b [N] or None -> y [M,N] (float32 reference order, or float64 truth)"""
    x, w, b = _c(x), _c(w), _c(b)
    M, K = x.shape
    N = w.shape[1]
    if f64:
        out = np.empty((M, N), np.float64)
        rc = lib().oracle_linear_forward_f64(_d(out), _f(x), _f(w), _f(b), M, 1, K, N)
    else:
        out = np.empty((M, N), np.float32)
        rc = lib().oracle_linear_forward_f32(_f(out), _f(x), _f(w), _f(b), M, 1, K, N)
    assert rc == 0
    return out


def backward_input(dy, w, f64=False):
    """dy [M,N], w [K,N] -> dx [M,K]"""
    dy, w = _c(dy), _c(w)
    M, N = dy.shape
    K = w.shape[0]
    if f64:
        out = np.empty((M, K), np.float64)
        rc = lib().oracle_linear_backward_input_f64(_d(out), _f(dy), _f(w), M, 1, K, N)
    else:
        out = np.empty((M, K), np.float32)
        rc = lib().oracle_linear_backward_input_f32(_f(out), _f(dy), _f(w), M, 1, K, N)
    assert rc == 0
    return out


def backward_weight(dy, x, want_bias=True, f64=False):
    """dy [M,N], x [M,K] -> (dw [K,N], db [N] or None)"""
    dy, x = _c(dy), _c(x)
    M, N = dy.shape
    K = x.shape[1]
    if f64:
        dw = np.empty((K, N), np.float64)
        db = np.empty((N,), np.float64) if want_bias else None
        rc = lib().oracle_linear_backward_weight_f64(_d(dw), _d(db), _f(dy), _f(x), M, 1, K, N)
    else:
        dw = np.empty((K, N), np.float32)
        db = np.empty((N,), np.float32) if want_bias else None
        rc = lib().oracle_linear_backward_weight_f32(_f(dw), _f(db), _f(dy), _f(x), M, 1, K, N)
    assert rc == 0
    return dw, db


def gelu(x):
    x = _c(x)
    out = np.empty_like(x)
    lib().oracle_gelu_f32(_f(out), _f(x), x.size)
    return out


def gelu_grad_mul(x, g):
    """g * gelu'(x) in float64 (the reference's GELU backward without its accumulate)"""
    x = _c(x)
    g = np.ascontiguousarray(g, np.float64)
    out = np.empty(x.shape, np.float64)
    lib().oracle_gelu_grad_mul_f64(_d(out), _f(x), _d(g), x.size)
    return out


def max_rel_err(got, truth):
    """max_i |got_i - truth_i| / max_i |truth_i| — the error metric of the parity thresholds"""
    truth = np.asarray(truth, np.float64)
    got = np.asarray(got, np.float64)
    denom = np.max(np.abs(truth))
    if denom == 0:
        return float(np.max(np.abs(got)))
    return float(np.max(np.abs(got - truth)) / denom)


# ---- the reference's own CUDA kernels (GPU box only) ----
_ref = None


def ref_lib():
    """Returns the library of reference kernels, or None when it was not built."""
    global _ref
    if _ref is None and os.path.exists(REF_SO):
        L = ctypes.CDLL(REF_SO)
        P, I = ctypes.c_void_p, ctypes.c_int
        L.ref_mlp_forward.argtypes = [P, P, P, P, I, I, I, I, P]
        L.ref_mlp_backward_input.argtypes = [P, P, P, I, I, I, I, P]
        L.ref_mlp_backward_weight.argtypes = [P, P, P, P, I, I, I, I, P]
        _ref = L
    return _ref


_ref_train = None


def ref_train_lib():
    """The reference's own training step (src/train.cu and its layer kernels, unmodified, behind
    oracle/ref_train_shim.cu), or None when it was not built. One model per process."""
    global _ref_train
    if _ref_train is None and os.path.exists(REF_TRAIN_SO):
        L = ctypes.CDLL(REF_TRAIN_SO)
        L.ref_train_create.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_uint]
        L.ref_train_create.restype = ctypes.c_int
        L.ref_train_num_params.restype = ctypes.c_longlong
        L.ref_train_set_params.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        L.ref_train_set_params.restype = ctypes.c_int
        L.ref_train_step.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        L.ref_train_step.restype = ctypes.c_float
        L.ref_train_sync.restype = ctypes.c_int
        _bind_train(L)
        _ref_train = L
    return _ref_train


def _bind_train(L):
    P, I = ctypes.c_void_p, ctypes.c_int
    L.ref_train_forward_backward.argtypes = [P, P]
    L.ref_train_forward_backward.restype = ctypes.c_float
    L.ref_train_get_grads.argtypes = [P, ctypes.c_longlong]
    L.ref_train_get_grads.restype = I
    L.ref_attention_forward.argtypes = [P, P, P, P, I, I, I, I]
    L.ref_attention_forward.restype = I
    L.ref_attention_backward.argtypes = [P, P, P, P, P, P, I, I, I, I]
    L.ref_attention_backward.restype = I


_ref_train_b200 = None


def ref_train_b200_lib():
    """The same training step with its 15 linear-layer launch sites rewritten to this library's launchers
    (oracle/Makefile target _ref/libref_train_b200.so), or None when it was not built. One model per process."""
    global _ref_train_b200
    if _ref_train_b200 is None and os.path.exists(REF_TRAIN_B200_SO):
        L = ctypes.CDLL(REF_TRAIN_B200_SO)
        L.ref_train_create.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_uint]
        L.ref_train_create.restype = ctypes.c_int
        L.ref_train_num_params.restype = ctypes.c_longlong
        L.ref_train_set_params.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        L.ref_train_set_params.restype = ctypes.c_int
        L.ref_train_step.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        L.ref_train_step.restype = ctypes.c_float
        L.ref_train_sync.restype = ctypes.c_int
        _bind_train(L)
        _ref_train_b200 = L
    return _ref_train_b200
