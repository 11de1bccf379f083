"""ctypes binding of libpolar_rt_cuda.so (include/polar_b200_rt.h): the device
runtime plugin seen through its flat C view.

`Runtime` mirrors what a PolarAI executor does with a device runtime: records are
identified by virtual address, data enters through a host write (ath_load),
builtins are launched by native kernel name with LaunchCommand/ArgDesc/TensorInfo
structs laid out as in the reference
(include/polarai/backend/generic/runtime/LaunchCommand.h:19-31, TensorInfo.h:17-22),
results leave through a host read (OutputNodeAccessor).
"""
import ctypes
import os

import numpy as np

from .capi import PolarB200Error

_HERE = os.path.dirname(os.path.abspath(__file__))
RT_LIB_PATH = os.path.join(_HERE, "lib", "libpolar_rt_cuda.so")

_u64 = ctypes.c_uint64
_p = ctypes.c_void_p
_i = ctypes.c_int


class TensorInfo(ctypes.Structure):
    _fields_ = [("virtAddr", _u64), ("dataType", _i), ("dims", _u64), ("shape", ctypes.POINTER(_u64))]


class ArgDesc(ctypes.Structure):
    TENSOR, DATA = 0, 1
    _fields_ = [("size", _u64), ("arg", _p), ("type", _i)]


class LaunchCommand(ctypes.Structure):
    _fields_ = [("kernelName", ctypes.c_char_p), ("argsCount", _u64), ("args", ctypes.POINTER(ArgDesc)),
                ("nativeKernelName", ctypes.c_char_p)]


class RtUpdate(ctypes.Structure):
    _fields_ = [("weight_va", _u64), ("weight_bytes", _u64), ("weight_offset", _u64), ("grad_offset", _u64),
                ("count", _u64)]


RT_SIGNATURES = {
    "polar_b200_rt_open": (_p, []),
    "polar_b200_rt_close": (None, [_p]),
    "polar_b200_rt_device_count": (_i, [_p]),
    "polar_b200_rt_device_name": (ctypes.c_char_p, [_p, _i]),
    "polar_b200_rt_allocate": (_i, [_p, _i, _u64, _u64]),
    "polar_b200_rt_deallocate": (_i, [_p, _u64, _u64]),
    "polar_b200_rt_write": (_i, [_p, _u64, _u64, _p]),
    "polar_b200_rt_host_begin_write": (_i, [_p, _u64, _u64, ctypes.POINTER(_p)]),
    "polar_b200_rt_host_end_write": (_i, [_p, _u64, _u64]),
    "polar_b200_rt_read": (_i, [_p, _u64, _u64, _p]),
    "polar_b200_rt_launch": (_i, [_p, _i, ctypes.POINTER(LaunchCommand)]),
    "polar_b200_rt_adopt": (_i, [_p, _i, _u64, _u64, _p]),
    "polar_b200_rt_allreduce_fadd": (_i, [_p, _i, ctypes.POINTER(_p), _p, ctypes.c_uint32, ctypes.c_uint32,
                                          ctypes.c_uint32, _u64, _u64, ctypes.POINTER(RtUpdate), ctypes.c_uint32,
                                          ctypes.c_float, ctypes.c_float]),
    "polar_b200_rt_barrier": (_i, [_p, _i]),
    "polar_b200_rt_device_ptr": (_p, [_p, _i, _u64, _u64]),
    "polar_b200_rt_stream": (_p, [_p, _i]),
    "polar_b200_rt_bytes_in_use": (_u64, [_p, _i]),
    "polar_b200_rt_set_memory_limit": (_i, [_p, _i, _u64]),
    "polar_b200_rt_last_error": (ctypes.c_char_p, [_p]),
}

DATATYPE_FLOAT = 2  # polarai::core::DataType::FLOAT


def load_rt_library(path=RT_LIB_PATH):
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path} is not built; run `python polarai-framework_b200/build.py`")
    cdll = ctypes.CDLL(path)
    for name, (res, args) in RT_SIGNATURES.items():
        fn = getattr(cdll, name)
        fn.restype = res
        fn.argtypes = args
    for name in ("initContext", "closeContext"):
        getattr(cdll, name)  # the two symbols RuntimeDriver looks up
    return cdll


class Tensor:
    """A record of the runtime: virtual address + shape (float32)."""

    def __init__(self, virt_addr, shape):
        self.virt_addr = int(virt_addr)
        self.shape = tuple(int(s) for s in shape)
        self.numel = int(np.prod(self.shape)) if self.shape else 1
        self.bytes = 4 * self.numel
        self._shape_arr = (_u64 * max(1, len(self.shape)))(*self.shape)
        self.info = TensorInfo(self.virt_addr, DATATYPE_FLOAT, len(self.shape), self._shape_arr)


class Runtime:
    def __init__(self):
        self.cdll = load_rt_library()
        self.h = self.cdll.polar_b200_rt_open()
        if not self.h:
            raise RuntimeError("polar_b200_rt_open failed")
        self._next_va = 1   # the reference's virtual addresses start at 1 and are byte-granular

    def close(self):
        if self.h:
            self.cdll.polar_b200_rt_close(self.h)
            self.h = None

    def _check(self, status):
        if status != 0:
            raise PolarB200Error(status, self.cdll.polar_b200_rt_last_error(self.h).decode())

    def device_count(self):
        return self.cdll.polar_b200_rt_device_count(self.h)

    def device_name(self, i):
        return self.cdll.polar_b200_rt_device_name(self.h, i).decode()

    def tensor(self, shape, device=0):
        t = Tensor(self._next_va, shape)
        self._next_va += t.bytes
        self._check(self.cdll.polar_b200_rt_allocate(self.h, device, t.virt_addr, t.bytes))
        return t

    def adopt(self, shape, device_ptr, device=0):
        """A record whose device copy is memory the caller owns (never freed by the runtime)."""
        t = Tensor(self._next_va, shape)
        self._next_va += t.bytes
        self._check(self.cdll.polar_b200_rt_adopt(self.h, device, t.virt_addr, t.bytes, device_ptr))
        return t

    def free(self, t):
        self._check(self.cdll.polar_b200_rt_deallocate(self.h, t.virt_addr, t.bytes))

    def write(self, t, array):
        a = np.ascontiguousarray(array, np.float32)
        if a.size != t.numel:
            raise ValueError("size mismatch")
        self._check(self.cdll.polar_b200_rt_write(self.h, t.virt_addr, t.bytes, a.ctypes.data))

    def write_ptr(self, t, host_ptr):
        self._check(self.cdll.polar_b200_rt_write(self.h, t.virt_addr, t.bytes, host_ptr))

    def host_buffer(self, t):
        """Begins an in-place write: returns the record's pinned host buffer as a numpy array to
        fill (the old contents are not preserved); publish() ends the write and starts the upload."""
        h = _p()
        self._check(self.cdll.polar_b200_rt_host_begin_write(self.h, t.virt_addr, t.bytes, ctypes.byref(h)))
        return np.ctypeslib.as_array(ctypes.cast(h, ctypes.POINTER(ctypes.c_float)), (t.numel,)).reshape(t.shape)

    def publish(self, t):
        self._check(self.cdll.polar_b200_rt_host_end_write(self.h, t.virt_addr, t.bytes))

    def read(self, t, out=None):
        if out is None:
            out = np.empty(t.shape, np.float32)
        self._check(self.cdll.polar_b200_rt_read(self.h, t.virt_addr, t.bytes, out.ctypes.data))
        return out

    def command(self, native_name, args, kernel_name=None):
        """A LaunchCommand built once and launched many times (launch_command): the structs a
        compiled graph would keep on its stack.  Returns (command, objects to keep alive)."""
        n = len(args)
        descs = (ArgDesc * max(1, n))()
        keep = [descs]
        for i, a in enumerate(args):
            if isinstance(a, Tensor):
                keep.append(a)
                descs[i] = ArgDesc(0, ctypes.cast(ctypes.pointer(a.info), _p), ArgDesc.TENSOR)
            else:
                f = ctypes.c_float(float(a))
                keep.append(f)
                descs[i] = ArgDesc(4, ctypes.cast(ctypes.pointer(f), _p), ArgDesc.DATA)
        cmd = LaunchCommand((kernel_name or ("node_" + native_name)).encode(), n, descs, native_name.encode())
        return cmd, keep

    def launch_command(self, cmd, device=0):
        rc = self.cdll.polar_b200_rt_launch(self.h, device, ctypes.byref(cmd))
        if rc != 0:
            self._check(rc)

    def launch(self, native_name, args, device=0, kernel_name=None):
        """args: Tensor objects and Python floats, in LaunchCommand order."""
        n = len(args)
        descs = (ArgDesc * max(1, n))()
        keep = []
        for i, a in enumerate(args):
            if isinstance(a, Tensor):
                descs[i] = ArgDesc(0, ctypes.cast(ctypes.pointer(a.info), _p), ArgDesc.TENSOR)
            else:
                f = ctypes.c_float(float(a))
                keep.append(f)
                descs[i] = ArgDesc(4, ctypes.cast(ctypes.pointer(f), _p), ArgDesc.DATA)
        name = native_name.encode()
        cmd = LaunchCommand((kernel_name or ("node_" + native_name)).encode(), n, descs, name)
        self._check(self.cdll.polar_b200_rt_launch(self.h, device, ctypes.byref(cmd)))

    def barrier(self, device=0):
        self._check(self.cdll.polar_b200_rt_barrier(self.h, device))

    def device_ptr(self, t, device=0):
        return self.cdll.polar_b200_rt_device_ptr(self.h, device, t.virt_addr, t.bytes)

    def stream(self, device=0):
        return self.cdll.polar_b200_rt_stream(self.h, device)

    def bytes_in_use(self, device=0):
        return int(self.cdll.polar_b200_rt_bytes_in_use(self.h, device))

    def set_memory_limit(self, nbytes, device=0):
        self._check(self.cdll.polar_b200_rt_set_memory_limit(self.h, device, int(nbytes)))


class RuntimeBuiltins:
    """The oracle's call signatures, every call through Device::launch with host
    buffers on both sides (the path an executor takes)."""

    def __init__(self, rt=None, device=0):
        self.rt = rt or Runtime()
        self.device = device

    def _run(self, name, ins, out_shape, scalars_at=()):
        rt = self.rt
        args, temps = [], []
        for x in ins:
            if isinstance(x, np.ndarray):
                t = rt.tensor(x.shape, self.device)
                rt.write(t, x)
                temps.append(t)
                args.append(t)
            else:
                args.append(x)
        out = rt.tensor(out_shape, self.device)
        args.append(out)
        rt.launch(name, args, self.device)
        res = rt.read(out)
        for t in temps + [out]:
            rt.free(t)
        return res

    def ffill(self, pattern, n):
        return self._run("ffill", [float(pattern)], (n,))

    def fcopy(self, a):
        a = np.asarray(a, np.float32)
        return self._run("fcopy", [a], a.shape)

    def fadd(self, a, sa, b, sb):
        a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
        return self._run("fadd", [a, float(sa), b, float(sb)], a.shape)

    def fmul(self, a, b):
        a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
        return self._run("fmul", [a, b], a.shape)

    def fdivide(self, a, b):
        a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
        return self._run("fdivide", [a, b], a.shape)

    def fsigmoid(self, a):
        a = np.asarray(a, np.float32)
        return self._run("fsigmoid", [a], a.shape)

    def flogloss(self, p, y):
        p, y = np.asarray(p, np.float32), np.asarray(y, np.float32)
        return self._run("flogloss", [p, y], p.shape)

    def fmulconcat(self, g, l):
        g, l = np.asarray(g, np.float32), np.asarray(l, np.float32)
        return self._run("fmulconcat", [g, l], l.shape)

    def fmatmul(self, tl, tr, left, right):
        left, right = np.asarray(left, np.float32), np.asarray(right, np.float32)
        m = left.shape[1] if tl else left.shape[0]
        n = right.shape[0] if tr else right.shape[1]
        name = f"fmatmul_{'t' if tl else 'f'}_{'t' if tr else 'f'}"
        return self._run(name, [left, right], (m, n))


class RuntimeProgramExecutor:
    """Runs a builtin Program (program.py) through the device-runtime plugin, the way a PolarAI
    executor drives a runtime: one record per tensor, inputs written from host buffers
    (ath_load's role: host copy into the record's pinned memory, upload started at once on the
    device's upload stream), one Device::launch per builtin by native name, outputs read back to
    the host.  The launch commands are built once.

    A program with an ALLREDUCE_FADD op (program.fuse_gradient_exchange) needs `peers`, a
    PeerGradients built for program.exchanged(): those gradients are adopted as records whose
    device memory is the rank's NVLink peer buffer, and the op becomes
    polar_b200_rt_allreduce_fadd (an exchange the program marks "overlapped" runs in order here:
    the plugin drives one stream per device).  Plain ALLREDUCE ops are no-ops here (single rank)."""

    def __init__(self, program, rt=None, device=0, peers=None):
        self.program = program
        self.rt = rt or Runtime()
        self.device = device
        exchanged = program.exchanged()
        if exchanged and (peers is None or sorted(peers.tensors) != sorted(exchanged)):
            raise ValueError(f"the program exchanges gradients over peer memory: pass `peers` built for {exchanged}")
        self.peers = peers if exchanged else None
        self.t = {}
        for name, shape in program.tensors.items():
            if name in exchanged:
                self.t[name] = self.rt.adopt(shape, peers.tensors[name].data_ptr(), device)
            else:
                self.t[name] = self.rt.tensor(shape, device)
        for name, value in program.constants.items():
            self.rt.launch("ffill", [float(value), self.t[name]], device)
        self._steps = []
        self._keep = []
        for kernel, args in program.ops:
            if kernel == "ALLREDUCE":
                continue
            if kernel in ("ALLREDUCE_FADD", "ALLREDUCE_FADD_PART"):
                if kernel == "ALLREDUCE_FADD":
                    pieces, channel = [(args[i], args[i + 1], 0, -1) for i in range(2, len(args), 2)], 0
                else:
                    from .program import exchange_pieces
                    pieces, channel = exchange_pieces(args), int(args[2])
                upd = (RtUpdate * len(pieces))()
                spans = []
                for u, (w, g, r0, rows) in zip(upd, pieces):
                    off, count = peers.offsets[g]
                    wt = self.t[w]
                    woff = 0
                    if rows >= 0:
                        cols = count // wt.shape[0]
                        off, count, woff = off + r0 * cols, rows * cols, r0 * cols
                    u.weight_va, u.weight_bytes, u.weight_offset = wt.virt_addr, wt.bytes, woff
                    u.grad_offset, u.count = off, count
                    spans.append((off, off + (count + 3) // 4 * 4))
                spans.sort()
                first, total = spans[0][0], spans[-1][1] - spans[0][0]
                if kernel == "ALLREDUCE_FADD":
                    first, total = 0, peers.n
                self._steps.append(("exchange", (upd, len(pieces), float(args[0]), float(args[1]), channel, first,
                                                 total)))
                continue
            cmd, keep = self.rt.command(kernel, [self.t[a] if isinstance(a, str) else a for a in args])
            self._keep.append(keep)
            self._steps.append(("launch", cmd))

    def set_inputs(self, **arrays):
        for name, a in arrays.items():
            self.rt.write(self.t[name], a)

    def run(self):
        rt, dev = self.rt, self.device
        for kind, what in self._steps:
            if kind == "launch":
                rt.launch_command(what, dev)
            else:
                upd, n, sw, sg, channel, first, total = what
                p = self.peers
                rt._check(rt.cdll.polar_b200_rt_allreduce_fadd(rt.h, dev, p.buffers, p.multicast, p.rank, p.world, channel, first,
                                                               total, upd, n, sw, sg))

    def output(self, name, out=None):
        return self.rt.read(self.t[name], out)

    def close(self):
        for t in self.t.values():
            self.rt.free(t)
        self.t = {}
