"""The weight gradients of a data-parallel step, held in NVLink peer memory.

Each rank allocates one peer buffer (polar_b200_peer_alloc), exports it as a CUDA IPC
handle, gathers every rank's handle over the process group and maps the others.  The
gradients of the program are views into the rank's own buffer, so the matmuls that
produce them write straight into memory the peers can read; `launch` then issues
polar_b200_allreduce_fadd - sum over ranks and weight update in one kernel per rank.
The reference has no counterpart (one device, no collective: ExecutorImpl.cpp:71-75).
"""
import ctypes

import torch

from .capi import lib

HANDLE_BYTES = 64
CONTROL_BYTES = 1024     # POLAR_B200_PEER_CONTROL_BYTES: four channels of 256 bytes


class UpdateSegment(ctypes.Structure):
    _fields_ = [("weights", ctypes.c_void_p), ("offset", ctypes.c_uint64), ("count", ctypes.c_uint64)]


class _DeviceSpan:
    """Lets torch wrap device memory it did not allocate (CUDA array interface)."""

    def __init__(self, ptr, count):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False),
                                         "version": 2, "strides": None}


def payload_layout(shapes):
    """Offsets (in floats, each a multiple of 4) of the gradients in the payload, and its
    total length."""
    offsets, at = {}, 0
    for name, shape in shapes.items():
        count = 1
        for d in shape:
            count *= int(d)
        offsets[name] = (at, count)
        at += (count + 3) // 4 * 4
    return offsets, at


def slice_bounds(n_floats, rank, world):
    """The part of the payload (in float4 units) that `rank` sums and distributes: the
    same split the kernel computes."""
    n4 = (n_floats + 3) // 4
    per = (n4 + world - 1) // world
    lo = min(rank * per, n4)
    return lo, min(lo + per, n4)


def _gather_over_process_group(handle, world):
    import torch.distributed as dist
    out = [None] * world
    dist.all_gather_object(out, handle)
    return out


class PeerGradients:
    def __init__(self, shapes, rank=0, world=1, device="cuda:0", all_gather=None):
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: peer memory has no CPU path in this package")
        if not 0 <= rank < world <= 16:
            raise ValueError(f"rank {rank} of {world}: at most 16 ranks")
        self.lib = lib()
        self.rank, self.world = rank, world
        self.device = torch.device(device)
        self.offsets, self.n = payload_layout(shapes)
        c = self.lib.cdll
        with torch.cuda.device(self.device):
            own = ctypes.c_void_p()
            self.lib.check(c.polar_b200_peer_alloc(self.n * 4, ctypes.byref(own)))
            self.own = own.value
            handle = (ctypes.c_ubyte * HANDLE_BYTES)()
            self.lib.check(c.polar_b200_peer_export(self.own, handle))
            if world > 1:
                handles = (all_gather or _gather_over_process_group)(bytes(handle), world)
            else:
                handles = [bytes(handle)]
            self.buffers = (ctypes.c_void_p * world)()
            self._opened = []
            for r in range(world):
                if r == rank:
                    self.buffers[r] = self.own
                    continue
                h = (ctypes.c_ubyte * HANDLE_BYTES).from_buffer_copy(handles[r])
                p = ctypes.c_void_p()
                self.lib.check(c.polar_b200_peer_open(h, ctypes.byref(p)))
                self.buffers[r] = p.value
                self._opened.append(p.value)
            flat = torch.as_tensor(_DeviceSpan(self.own + CONTROL_BYTES, self.n), device=self.device)
        self.flat = flat
        self.tensors = {name: flat[off:off + count].view(*shapes[name])
                        for name, (off, count) in self.offsets.items()}

    def segments(self, pairs):
        """ctypes segment table for (weight tensor, gradient name) pairs."""
        seg = (UpdateSegment * len(pairs))()
        for i, (w, g) in enumerate(pairs):
            off, count = self.offsets[g]
            if w.numel() != count or not w.is_contiguous():
                raise ValueError(f"weight of {g}: {tuple(w.shape)} does not match the gradient")
            seg[i].weights, seg[i].offset, seg[i].count = w.data_ptr(), off, count
        return seg

    def piece_segments(self, pieces):
        """Segment table and payload range [first, first + count) for (weight tensor, gradient name,
        first row, rows) pieces - rows < 0 = the whole tensor - which must be adjacent in the payload."""
        seg = (UpdateSegment * len(pieces))()
        spans = []
        for i, (w, g, r0, rows) in enumerate(pieces):
            off, count = self.offsets[g]
            if w.numel() != count or not w.is_contiguous():
                raise ValueError(f"weight of {g}: {tuple(w.shape)} does not match the gradient")
            if rows >= 0:
                cols = count // w.shape[0]
                off, count = off + r0 * cols, rows * cols
                ptr = w.data_ptr() + 4 * r0 * cols
            else:
                ptr = w.data_ptr()
            seg[i].weights, seg[i].offset, seg[i].count = ptr, off, count
            spans.append((off, off + (count + 3) // 4 * 4))
        spans.sort()
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            if a1 != b0:
                raise ValueError("the pieces of one exchange must be adjacent in the payload")
        return seg, spans[0][0], spans[-1][1] - spans[0][0]

    def launch_range(self, channel, first, count, seg, scale_w, scale_g, stream):
        rc = self.lib.cdll.polar_b200_allreduce_fadd_range(self.buffers, self.rank, self.world, channel, first, count,
                                                           seg, len(seg), scale_w, scale_g, stream)
        if rc != 0:
            self.lib.check(rc)

    def launch(self, seg, scale_w, scale_g, stream):
        rc = self.lib.cdll.polar_b200_allreduce_fadd(self.buffers, self.rank, self.world, self.n, seg, len(seg),
                                                     scale_w, scale_g, stream)
        if rc != 0:
            self.lib.check(rc)

    def phase_times_us(self, channel=0):
        """Durations of the last launch's phases on this rank and channel, from the control
        block's timestamps (CTA 0): wait for all ranks' gradients, sum + distribute the slice,
        wait for all slices, update."""
        torch.cuda.synchronize(self.device)
        ctl = torch.as_tensor(_DeviceSpan(self.own, CONTROL_BYTES // 4), device=self.device)
        base = channel * 64
        t = ctl[base + 40:base + 50].view(torch.int64).cpu().tolist()
        return {"ready_wait": (t[1] - t[0]) / 1e3, "sum_slice": (t[2] - t[1]) / 1e3,
                "done_wait": (t[3] - t[2]) / 1e3, "update": (t[4] - t[3]) / 1e3}

    def close(self):
        """Unmaps the peers' buffers and frees this rank's.  Every rank must have finished
        its last step (a barrier on the host) before any rank calls this."""
        c = self.lib.cdll
        torch.cuda.synchronize(self.device)
        self.tensors, self.flat = {}, None
        with torch.cuda.device(self.device):
            for p in self._opened:
                c.polar_b200_peer_close(p)
            self._opened = []
            if self.own:
                c.polar_b200_peer_free(self.own)
                self.own = None
