"""The builtins on torch CUDA tensors, under the reference's native kernel names.

`DeviceBuiltins` launches on torch's current stream with device tensors (what
the benchmark times); `HostBuiltins` has the oracle's call signatures - numpy in,
numpy out - and moves the data through the device, for the parity tests.
torch is used for device memory and streams only.
"""
import numpy as np
import torch

from .capi import lib


def _ptr(t):
    return t.data_ptr() if t is not None else None


def _stream(t):
    """torch's current stream ON THE TENSOR'S DEVICE (not on whatever device is current)."""
    return torch.cuda.current_stream(t.device).cuda_stream


def _chk(*ts):
    for t in ts:
        if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
            raise ValueError("builtins take contiguous float32 CUDA tensors")


class DeviceBuiltins:
    def __init__(self):
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: the PolarAI B200 builtins have no CPU path")
        self.lib = lib()

    def ffill(self, pattern, out):
        _chk(out)
        self.lib.call("polar_b200_ffill", float(pattern), _ptr(out), out.numel(), _stream(out))
        return out

    def fcopy(self, a, out):
        _chk(a, out)
        self.lib.call("polar_b200_fcopy", _ptr(a), _ptr(out), out.numel(), _stream(out))
        return out

    def fadd(self, a, sa, b, sb, out):
        _chk(a, b, out)
        self.lib.call("polar_b200_fadd", _ptr(a), float(sa), _ptr(b), float(sb), _ptr(out), out.numel(),
                      _stream(out))
        return out

    def fmul(self, a, b, out):
        _chk(a, b, out)
        self.lib.call("polar_b200_fmul", _ptr(a), _ptr(b), _ptr(out), out.numel(), _stream(out))
        return out

    def fdivide(self, a, b, out):
        _chk(a, b, out)
        self.lib.call("polar_b200_fdivide", _ptr(a), _ptr(b), _ptr(out), out.numel(), _stream(out))
        return out

    def fsigmoid(self, a, out, clamp=True):
        _chk(a, out)
        name = "polar_b200_fsigmoid" if clamp else "polar_b200_fsigmoid_unclamped"
        self.lib.call(name, _ptr(a), _ptr(out), out.numel(), _stream(out))
        return out

    def flogloss(self, predicted, ground_truth, out):
        _chk(predicted, ground_truth, out)
        self.lib.call("polar_b200_flogloss", _ptr(predicted), _ptr(ground_truth), _ptr(out), out.numel(),
                      _stream(out))
        return out

    def fmulconcat(self, gradient, local, out):
        _chk(gradient, local, out)
        self.lib.call("polar_b200_fmulconcat", _ptr(gradient), _ptr(local), _ptr(out), out.numel(), _stream(out))
        return out

    def frelu(self, a, out):
        _chk(a, out)
        self.lib.call("polar_b200_frelu", _ptr(a), _ptr(out), out.numel(), _stream(out))
        return out

    def fsoftmax(self, a, out):
        _chk(a, out)
        self.lib.call("polar_b200_fsoftmax", _ptr(a), _ptr(out), out.numel(), None, 0, _stream(out))
        return out

    def fpool(self, a, window, stride, out):
        _chk(a, out)
        h, w = a.shape
        self.lib.call("polar_b200_fpool", _ptr(a), h, w, window[0], window[1], stride[0], stride[1], _ptr(out),
                      _stream(out))
        return out

    def fconv2d(self, a, kernel, out):
        _chk(a, kernel, out)
        h, w = a.shape
        kh, kw = kernel.shape
        self.lib.call("polar_b200_fconv2d", _ptr(a), h, w, _ptr(kernel), kh, kw, _ptr(out), _stream(out))
        return out

    def ftranspose(self, a, out):
        _chk(a, out)
        rows, cols = a.shape
        self.lib.call("polar_b200_ftranspose", _ptr(a), rows, cols, _ptr(out), _stream(out))
        return out

    def fslice(self, a, index, out):
        _chk(a, out)
        self.lib.call("polar_b200_fslice", _ptr(a), a.shape[0], out.numel(), int(index), _ptr(out), _stream(out))
        return out

    def fsum(self, a, acc):
        """Adds sum(a) to the float64 one-element tensor `acc`."""
        _chk(a)
        self.lib.call("polar_b200_fsum", _ptr(a), _ptr(acc), a.numel(), _stream(a))
        return acc

    def fmatmul(self, tl, tr, left, right, out):
        _chk(left, right, out)
        m, n, k = matmul_dims(tl, tr, left.shape, right.shape)
        if tuple(out.shape) != (m, n):
            raise ValueError(f"out must be [{m},{n}]")
        self.lib.call("polar_b200_fmatmul", int(tl), int(tr), m, n, k, _ptr(left), _ptr(right), _ptr(out),
                      None, 0, _stream(out))
        return out

    def fmatmul_ffma(self, tl, tr, left, right, out):
        _chk(left, right, out)
        m, n, k = matmul_dims(tl, tr, left.shape, right.shape)
        self.lib.call("polar_b200_fmatmul_ffma", int(tl), int(tr), m, n, k, _ptr(left), _ptr(right),
                      _ptr(out), _stream(out))
        return out

    def fmatmul_tc(self, tl, tr, left, right, out, tile_n=256, slab_k=16, passes=3, write_hi=0, splits=1):
        _chk(left, right, out)
        m, n, k = matmul_dims(tl, tr, left.shape, right.shape)
        self.lib.call("polar_b200_fmatmul_tc", int(tl), int(tr), m, n, k, _ptr(left), _ptr(right),
                      _ptr(out), tile_n, slab_k, passes, write_hi, splits, _stream(out))
        return out

    def device_status(self):
        return int(self.lib.cdll.polar_b200_device_status())


def matmul_dims(tl, tr, lshape, rshape):
    m = lshape[1] if tl else lshape[0]
    k = lshape[0] if tl else lshape[1]
    n = rshape[0] if tr else rshape[1]
    k2 = rshape[1] if tr else rshape[0]
    if k != k2:
        raise ValueError(f"inner dimensions differ: {k} vs {k2}")
    return int(m), int(n), int(k)


class HostBuiltins:
    """numpy in / numpy out, every call through the device."""

    def __init__(self, device="cuda:0"):
        self.dev = torch.device(device)
        self.d = DeviceBuiltins()

    def _up(self, a):
        return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(self.dev)

    def _down(self, t):
        torch.cuda.synchronize(self.dev)
        return t.cpu().numpy()

    def ffill(self, pattern, n):
        return self._down(self.d.ffill(pattern, torch.empty(n, device=self.dev)))

    def fcopy(self, a):
        a = self._up(a)
        return self._down(self.d.fcopy(a, torch.empty_like(a)))

    def fadd(self, a, sa, b, sb):
        a, b = self._up(a), self._up(b)
        return self._down(self.d.fadd(a, sa, b, sb, torch.empty_like(a)))

    def fmul(self, a, b):
        a, b = self._up(a), self._up(b)
        return self._down(self.d.fmul(a, b, torch.empty_like(a)))

    def fdivide(self, a, b):
        a, b = self._up(a), self._up(b)
        return self._down(self.d.fdivide(a, b, torch.empty_like(a)))

    def fsigmoid(self, a, clamp=True):
        a = self._up(a)
        return self._down(self.d.fsigmoid(a, torch.empty_like(a), clamp))

    def flogloss(self, p, y):
        p, y = self._up(p), self._up(y)
        return self._down(self.d.flogloss(p, y, torch.empty_like(p)))

    def fmulconcat(self, g, l):
        g, l = self._up(g), self._up(l)
        return self._down(self.d.fmulconcat(g, l, torch.empty_like(l)))

    def frelu(self, a):
        a = self._up(a)
        return self._down(self.d.frelu(a, torch.empty_like(a)))

    def fsoftmax(self, a):
        a = self._up(a)
        return self._down(self.d.fsoftmax(a, torch.empty_like(a)))

    def fpool(self, a, window, stride):
        a = self._up(a)
        h, w = a.shape
        out = torch.empty(((h - window[0]) // stride[0] + 1, (w - window[1]) // stride[1] + 1), device=self.dev)
        return self._down(self.d.fpool(a, window, stride, out))

    def fconv2d(self, a, kernel):
        a, kernel = self._up(a), self._up(kernel)
        out = torch.empty((a.shape[0] - kernel.shape[0] + 1, a.shape[1] - kernel.shape[1] + 1), device=self.dev)
        return self._down(self.d.fconv2d(a, kernel, out))

    def ftranspose(self, a):
        a = self._up(a)
        return self._down(self.d.ftranspose(a, torch.empty((a.shape[1], a.shape[0]), device=self.dev)))

    def fslice(self, a, index):
        a = self._up(a)
        return self._down(self.d.fslice(a, index, torch.empty(tuple(a.shape[1:]), device=self.dev)))

    def fmatmul(self, tl, tr, left, right, which="auto", **kw):
        l, r = self._up(left), self._up(right)
        m, n, k = matmul_dims(tl, tr, l.shape, r.shape)
        out = torch.empty((m, n), device=self.dev)
        fn = {"auto": self.d.fmatmul, "ffma": self.d.fmatmul_ffma, "tc": self.d.fmatmul_tc}[which]
        return self._down(fn(tl, tr, l, r, out, **kw))
