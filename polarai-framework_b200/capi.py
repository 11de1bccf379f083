"""ctypes binding of libpolar_b200.so (include/polar_b200.h).

There is no fallback: if the library has not been built, or a call returns a
non-zero status, an exception is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libpolar_b200.so")

_u64 = ctypes.c_uint64
_f = ctypes.c_float
_p = ctypes.c_void_p
_i = ctypes.c_int


class PolarB200Error(RuntimeError):
    def __init__(self, status, text):
        super().__init__(f"polar_b200 status {status}: {text}")
        self.status = status


class Tensor(ctypes.Structure):
    _fields_ = [("data", _p), ("dims", _u64), ("shape", ctypes.POINTER(_u64))]


class Arg(ctypes.Structure):
    _fields_ = [("is_tensor", _i), ("tensor", Tensor), ("scalar", _f), ("integer", ctypes.c_int64)]


SIGNATURES = {
    "polar_b200_last_error": (ctypes.c_char_p, []),
    "polar_b200_version": (_i, []),
    "polar_b200_built_for_sm": (_i, []),
    "polar_b200_ffill": (_i, [_f, _p, _u64, _p]),
    "polar_b200_fcopy": (_i, [_p, _p, _u64, _p]),
    "polar_b200_fadd": (_i, [_p, _f, _p, _f, _p, _u64, _p]),
    "polar_b200_fmul": (_i, [_p, _p, _p, _u64, _p]),
    "polar_b200_fdivide": (_i, [_p, _p, _p, _u64, _p]),
    "polar_b200_fsigmoid": (_i, [_p, _p, _u64, _p]),
    "polar_b200_fsigmoid_unclamped": (_i, [_p, _p, _u64, _p]),
    "polar_b200_flogloss": (_i, [_p, _p, _p, _u64, _p]),
    "polar_b200_fsigmoid_grad": (_i, [_p, _p, _p, _u64, _p]),
    "polar_b200_fsigmoid_logloss_grad": (_i, [_p, _p, _p, _u64, _p]),
    "polar_b200_fmulconcat": (_i, [_p, _p, _p, _u64, _p]),
    "polar_b200_frelu": (_i, [_p, _p, _u64, _p]),
    "polar_b200_fsoftmax": (_i, [_p, _p, _u64, _p, _u64, _p]),
    "polar_b200_fpool": (_i, [_p, _u64, _u64, _u64, _u64, _u64, _u64, _p, _p]),
    "polar_b200_fconv2d": (_i, [_p, _u64, _u64, _p, _u64, _u64, _p, _p]),
    "polar_b200_ftranspose": (_i, [_p, _u64, _u64, _p, _p]),
    "polar_b200_fslice": (_i, [_p, _u64, _u64, _u64, _p, _p]),
    "polar_b200_fmatmul": (_i, [_i, _i, _u64, _u64, _u64, _p, _p, _p, _p, _u64, _p]),
    "polar_b200_fmatmul_sigmoid": (_i, [_i, _i, _u64, _u64, _u64, _p, _p, _p, _p, _u64, _p]),
    "polar_b200_fmatmul_sigmoid_grad": (_i, [_i, _i, _u64, _u64, _u64, _p, _p, _p, _p, _p, _u64, _p]),
    "polar_b200_fmatmul_t_f_rows": (_i, [_u64, _u64, _u64, _u64, _u64, _p, _p, _p, _p, _u64, _p]),
    "polar_b200_fmatmul_t_f_rows_workspace_bytes": (_u64, [_u64, _u64, _u64]),
    "polar_b200_fdense_grad": (_i, [_u64, _u64, _u64, _p, _p, _p, _p, _p, _p, _u64, _p]),
    "polar_b200_fdense_grad_workspace_bytes": (_u64, [_u64, _u64, _u64]),
    "polar_b200_fmatmul_workspace_bytes": (_u64, [_i, _i, _u64, _u64, _u64]),
    "polar_b200_fmatmul_ffma": (_i, [_i, _i, _u64, _u64, _u64, _p, _p, _p, _p]),
    "polar_b200_fmatmul_tc": (_i, [_i, _i, _u64, _u64, _u64, _p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "polar_b200_fmatmul_tn_small_n_static": (_i, [_i, _u64, _u64, _u64, _p, _p, _p, _p]),
    "polar_b200_static_scratch_bytes": (_u64, []),
    "polar_b200_fmatmul_path": (_i, [_i, _i, _u64, _u64, _u64]),
    "polar_b200_fmatmul_tc_plan": (None, [_i, _i, _u64, _u64, _u64, _p, _p, _p]),
    "polar_b200_device_status": (_i, []),
    "polar_b200_device_status_clear": (None, []),
    "polar_b200_device_status_of": (_i, [_i]),
    "polar_b200_check_device_status": (_i, []),
    "polar_b200_set_wait_limit_ns": (None, [_u64]),
    "polar_b200_wait_limit_ns": (_u64, []),
    "polar_b200_fsum": (_i, [_p, _p, _u64, _p]),
    "polar_b200_fsum_f32": (_i, [_p, _p, _u64, _p, _u64, _p]),
    "polar_b200_fsum_f32_workspace_bytes": (_u64, [_u64]),
    "polar_b200_peer_alloc": (_i, [_u64, ctypes.POINTER(_p)]),
    "polar_b200_peer_free": (_i, [_p]),
    "polar_b200_peer_export": (_i, [_p, ctypes.POINTER(ctypes.c_ubyte)]),
    "polar_b200_peer_open": (_i, [ctypes.POINTER(ctypes.c_ubyte), ctypes.POINTER(_p)]),
    "polar_b200_peer_close": (_i, [_p]),
    "polar_b200_allreduce_fadd": (_i, [ctypes.POINTER(_p), ctypes.c_uint32, ctypes.c_uint32, _u64, _p,
                                       ctypes.c_uint32, _f, _f, _p]),
    "polar_b200_allreduce_fadd_range": (_i, [ctypes.POINTER(_p), ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
                                             _u64, _u64, _p, ctypes.c_uint32, _f, _f, _p]),
    "polar_b200_allreduce_fadd_multicast": (_i, [ctypes.POINTER(_p), _p, ctypes.c_uint32, ctypes.c_uint32,
                                                 ctypes.c_uint32, _u64, _u64, _p, ctypes.c_uint32, _f, _f, _p]),
    "polar_b200_launch_by_name": (_i, [ctypes.c_char_p, ctypes.POINTER(Arg), _u64, _p, _u64, _p]),
    "polar_b200_launch_workspace_bytes": (_u64, [ctypes.c_char_p, ctypes.POINTER(Arg), _u64]),
    "polar_b200_launch_count": (_u64, []),
    "polar_b200_result_count": (_i, [ctypes.c_char_p]),
}


class Library:
    """The loaded shared library with typed entry points and status checking."""

    def __init__(self, path=LIB_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(
                f"{path} is not built; run `python polarai-framework_b200/build.py` (needs nvcc)")
        self.path = path
        self.cdll = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(self.cdll, name)  # AttributeError if the symbol is missing
            fn.restype = res
            fn.argtypes = args

    def last_error(self):
        return self.cdll.polar_b200_last_error().decode()

    def check(self, status):
        if status != 0:
            raise PolarB200Error(status, self.last_error())

    def call(self, name, *args):
        """Calls an int-returning entry point and raises on a non-zero status."""
        self.check(getattr(self.cdll, name)(*args))

    def launch_count(self):
        return int(self.cdll.polar_b200_launch_count())


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = Library()
    return _lib
