"""ctypes front end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the bench's CPU-baseline legs may import this
module; the runtime itself never does.  `Oracle` wraps liboracle.so (the C
restatement in builtins_oracle.c); `RefOcl` wraps _ref/libref_ocl.so (the
reference's own OpenCL C kernel bodies compiled as C), when that file exists.
Both expose the builtins under the reference's native kernel names
(`ffill`, `fadd`, ..., `fmatmul`), on contiguous float32 numpy arrays.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_F = ctypes.POINTER(ctypes.c_float)
_D = ctypes.POINTER(ctypes.c_double)
_U = ctypes.POINTER(ctypes.c_uint64)


def build(quiet=True):
    """Run oracle/Makefile (gcc only; builds _ref when the reference tree is there)."""
    out = subprocess.run(["make", "-C", _HERE], capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if not quiet:
        print(out.stdout)


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def _p(a):
    return a.ctypes.data_as(_F)


class Oracle:
    """The C restatement (oracle/builtins_oracle.c)."""

    kind = "port"

    def __init__(self, threads=1):
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        self.lib = ctypes.CDLL(path)
        L = self.lib
        L.oracle_set_threads.argtypes = [ctypes.c_int]
        L.oracle_max_threads.restype = ctypes.c_int
        L.oracle_ffill.argtypes = [ctypes.c_float, _F, ctypes.c_uint64]
        L.oracle_fcopy.argtypes = [_F, _F, ctypes.c_uint64]
        L.oracle_fadd.argtypes = [_F, ctypes.c_float, _F, ctypes.c_float, _F, ctypes.c_uint64]
        L.oracle_fmul.argtypes = [_F, _F, _F, ctypes.c_uint64]
        L.oracle_fdivide.argtypes = [_F, _F, _F, ctypes.c_uint64]
        L.oracle_fsigmoid.argtypes = [_F, _F, ctypes.c_uint64, ctypes.c_int]
        L.oracle_flogloss.argtypes = [_F, _F, _F, ctypes.c_uint64]
        L.oracle_fmulconcat.argtypes = [_F, _F, _F, ctypes.c_uint64]
        u = ctypes.c_uint64
        L.oracle_frelu.argtypes = [_F, _F, u]
        L.oracle_fsoftmax.argtypes = [_F, _F, u]
        L.oracle_fpool.argtypes = [_F, u, u, u, u, u, u, _F]
        L.oracle_fconv2d.argtypes = [_F, u, u, _F, u, u, _F]
        L.oracle_ftranspose.argtypes = [_F, u, u, _F]
        L.oracle_fslice.argtypes = [_F, u, u, _F]
        L.oracle_fmatmul.argtypes = [ctypes.c_int, ctypes.c_int, u, u, u, _F, _F, _F]
        L.oracle_fmatmul_f64.argtypes = [ctypes.c_int, ctypes.c_int, u, u, u, _F, _F, _D, _D]
        L.oracle_fmatmul_entries_f64.argtypes = [ctypes.c_int, ctypes.c_int, u, u, u, _F, _F,
                                                 _U, _U, u, _D, _D]
        self.set_threads(threads)

    def set_threads(self, n):
        self.threads = max(1, int(n))
        self.lib.oracle_set_threads(self.threads)

    def max_threads(self):
        return int(self.lib.oracle_max_threads())

    def ffill(self, pattern, n):
        out = np.empty(n, np.float32)
        self.lib.oracle_ffill(ctypes.c_float(pattern), _p(out), n)
        return out

    def fcopy(self, a):
        a = _f32(a)
        out = np.empty_like(a)
        self.lib.oracle_fcopy(_p(a), _p(out), a.size)
        return out

    def fadd(self, a, sa, b, sb):
        a, b = _f32(a), _f32(b)
        out = np.empty_like(a)
        self.lib.oracle_fadd(_p(a), ctypes.c_float(sa), _p(b), ctypes.c_float(sb), _p(out), a.size)
        return out

    def fmul(self, a, b):
        a, b = _f32(a), _f32(b)
        out = np.empty_like(a)
        self.lib.oracle_fmul(_p(a), _p(b), _p(out), a.size)
        return out

    def fdivide(self, a, b):
        a, b = _f32(a), _f32(b)
        out = np.empty_like(a)
        self.lib.oracle_fdivide(_p(a), _p(b), _p(out), a.size)
        return out

    def fsigmoid(self, a, clamp=True):
        a = _f32(a)
        out = np.empty_like(a)
        self.lib.oracle_fsigmoid(_p(a), _p(out), a.size, 1 if clamp else 0)
        return out

    def flogloss(self, predicted, ground_truth):
        p, y = _f32(predicted), _f32(ground_truth)
        out = np.empty_like(p)
        self.lib.oracle_flogloss(_p(p), _p(y), _p(out), p.size)
        return out

    def fmulconcat(self, gradient, local):
        g, l = _f32(gradient), _f32(local)
        out = np.empty_like(l)
        self.lib.oracle_fmulconcat(_p(g), _p(l), _p(out), l.size)
        return out

    def frelu(self, a):
        a = _f32(a)
        out = np.empty_like(a)
        self.lib.oracle_frelu(_p(a), _p(out), a.size)
        return out

    def fsoftmax(self, a):
        a = _f32(a)
        out = np.empty_like(a)
        self.lib.oracle_fsoftmax(_p(a), _p(out), a.size)
        return out

    def fpool(self, a, window, stride):
        a = _f32(a)
        h, w = a.shape
        out = np.empty(((h - window[0]) // stride[0] + 1, (w - window[1]) // stride[1] + 1), np.float32)
        self.lib.oracle_fpool(_p(a), h, w, window[0], window[1], stride[0], stride[1], _p(out))
        return out

    def ftranspose(self, a):
        a = _f32(a)
        rows, cols = a.shape
        out = np.empty((cols, rows), np.float32)
        self.lib.oracle_ftranspose(_p(a), rows, cols, _p(out))
        return out

    def fslice(self, a, index):
        a = _f32(a)
        out = np.empty(a.shape[1:], np.float32)
        self.lib.oracle_fslice(_p(a), out.size, int(index), _p(out))
        return out

    def fconv2d(self, a, kernel):
        a, kernel = _f32(a), _f32(kernel)
        h, w = a.shape
        kh, kw = kernel.shape
        out = np.empty((h - kh + 1, w - kw + 1), np.float32)
        self.lib.oracle_fconv2d(_p(a), h, w, _p(kernel), kh, kw, _p(out))
        return out

    def fmatmul(self, tl, tr, left, right):
        left, right = _f32(left), _f32(right)
        m, n, k = matmul_dims(tl, tr, left.shape, right.shape)
        out = np.empty((m, n), np.float32)
        self.lib.oracle_fmatmul(int(tl), int(tr), m, n, k, _p(left), _p(right), _p(out))
        return out

    def fmatmul_f64(self, tl, tr, left, right):
        """(double-accumulated product, sum_k |a||b|) as float64 arrays."""
        left, right = _f32(left), _f32(right)
        m, n, k = matmul_dims(tl, tr, left.shape, right.shape)
        out = np.empty((m, n), np.float64)
        mag = np.empty((m, n), np.float64)
        self.lib.oracle_fmatmul_f64(int(tl), int(tr), m, n, k, _p(left), _p(right),
                                    out.ctypes.data_as(_D), mag.ctypes.data_as(_D))
        return out, mag

    def fmatmul_entries_f64(self, tl, tr, left, right, rows, cols):
        left, right = _f32(left), _f32(right)
        m, n, k = matmul_dims(tl, tr, left.shape, right.shape)
        rows = np.ascontiguousarray(rows, np.uint64)
        cols = np.ascontiguousarray(cols, np.uint64)
        out = np.empty(rows.size, np.float64)
        mag = np.empty(rows.size, np.float64)
        self.lib.oracle_fmatmul_entries_f64(int(tl), int(tr), m, n, k, _p(left), _p(right),
                                            rows.ctypes.data_as(_U), cols.ctypes.data_as(_U),
                                            rows.size, out.ctypes.data_as(_D),
                                            mag.ctypes.data_as(_D))
        return out, mag


def matmul_dims(tl, tr, lshape, rshape):
    """m, n, k from the stored shapes, as MatMulOperationInternal.cpp:39-40 does:
    m = tl ? left.shape[1] : left.shape[0]; n = tr ? right.shape[0] : right.shape[1]."""
    m = lshape[1] if tl else lshape[0]
    k = lshape[0] if tl else lshape[1]
    n = rshape[0] if tr else rshape[1]
    k2 = rshape[1] if tr else rshape[0]
    if k != k2:
        raise ValueError(f"inner dimensions differ: {k} vs {k2}")
    return int(m), int(n), int(k)


class RefOcl:
    """The reference's OpenCL C kernels compiled as C (oracle/_ref/libref_ocl.so)."""

    kind = "reference"

    @staticmethod
    def available():
        return os.path.exists(os.path.join(_HERE, "_ref", "libref_ocl.so"))

    def __init__(self, threads=1):
        path = os.path.join(_HERE, "_ref", "libref_ocl.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = ctypes.CDLL(path)
        L = self.lib
        u = ctypes.c_uint64
        L.ref_set_threads.argtypes = [ctypes.c_int]
        L.ref_max_threads.restype = ctypes.c_int
        L.ref_ffill.argtypes = [ctypes.c_float, _F, u]
        L.ref_fcopy.argtypes = [_F, _F, u]
        L.ref_fadd.argtypes = [_F, ctypes.c_float, _F, ctypes.c_float, _F, u]
        L.ref_fmul.argtypes = [_F, _F, _F, u]
        L.ref_fdivide.argtypes = [_F, _F, _F, u]
        L.ref_fsigmoid.argtypes = [_F, _F, u]
        L.ref_flogloss.argtypes = [_F, _F, _F, u]
        L.ref_fmulconcat.argtypes = [_F, _F, _F, u]
        L.ref_fmatmul.argtypes = [ctypes.c_int, ctypes.c_int, u, u, u, _F, _F, _F]
        self.set_threads(threads)

    def set_threads(self, n):
        self.threads = max(1, int(n))
        self.lib.ref_set_threads(self.threads)

    def max_threads(self):
        return int(self.lib.ref_max_threads())

    def ffill(self, pattern, n):
        out = np.empty(n, np.float32)
        self.lib.ref_ffill(ctypes.c_float(pattern), _p(out), n)
        return out

    def fcopy(self, a):
        a = _f32(a)
        out = np.empty_like(a)
        self.lib.ref_fcopy(_p(a), _p(out), a.size)
        return out

    def fadd(self, a, sa, b, sb):
        a, b = _f32(a), _f32(b)
        out = np.empty_like(a)
        self.lib.ref_fadd(_p(a), ctypes.c_float(sa), _p(b), ctypes.c_float(sb), _p(out), a.size)
        return out

    def fmul(self, a, b):
        a, b = _f32(a), _f32(b)
        out = np.empty_like(a)
        self.lib.ref_fmul(_p(a), _p(b), _p(out), a.size)
        return out

    def fdivide(self, a, b):
        a, b = _f32(a), _f32(b)
        out = np.empty_like(a)
        self.lib.ref_fdivide(_p(a), _p(b), _p(out), a.size)
        return out

    def fsigmoid(self, a, clamp=True):
        if not clamp:
            raise ValueError("the reference's OpenCL C sigmoid always clamps")
        a = _f32(a)
        out = np.empty_like(a)
        self.lib.ref_fsigmoid(_p(a), _p(out), a.size)
        return out

    def flogloss(self, predicted, ground_truth):
        p, y = _f32(predicted), _f32(ground_truth)
        out = np.empty_like(p)
        self.lib.ref_flogloss(_p(p), _p(y), _p(out), p.size)
        return out

    def fmulconcat(self, gradient, local):
        g, l = _f32(gradient), _f32(local)
        out = np.empty_like(l)
        self.lib.ref_fmulconcat(_p(g), _p(l), _p(out), l.size)
        return out

    def fmatmul(self, tl, tr, left, right):
        left, right = _f32(left), _f32(right)
        m, n, k = matmul_dims(tl, tr, left.shape, right.shape)
        out = np.empty((m, n), np.float32)
        self.lib.ref_fmatmul(int(tl), int(tr), m, n, k, _p(left), _p(right), _p(out))
        return out
