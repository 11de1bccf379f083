"""The weight gradients of a data-parallel step, held in NVLink peer memory.

Two ways to get memory that every rank can reach:
 - "multicast": torch's symmetric memory (one allocation per rank, mapped into every rank, and
   bound to an NVLink multicast object).  The exchange kernel then sums a slice inside the
   switch with one load and delivers it to all ranks with one store
   (polar_b200_allreduce_fadd_multicast).
 - "ipc": each rank allocates one peer buffer (polar_b200_peer_alloc), exports it as a CUDA IPC
   handle, gathers every rank's handle over the process group and maps the others; the kernel
   reads its slice from every peer and writes the sum to every peer with plain loads and stores.
"auto" is the second unless POLAR_B200_PEER_MULTICAST=1 is set, in which case it takes the first
from eight ranks up when every rank can (a vote over the process group): through the switch a
rank's links carry its whole gradient vector once in each direction (its own copy out to the
switch, the sums back), peer to peer (world - 1) / world of it twice - a third less at eight
ranks, but more at two.  Measured (slice phase): two ranks 40 us in the switch against 26 us peer to
peer, four ranks 36.2 against 35.4 us, eight ranks 35.3 against 40.2 us.
Use "ipc" wherever a rank may leave while the others still run (failure tests): memory bound
to a multicast object must not lose a participant in mid-run.

The gradients of the program are views into the rank's own buffer, so the matmuls that
produce them write straight into memory the peers can read; `launch` then issues the exchange
- sum over ranks and weight update in one kernel per rank.
The reference has no counterpart (one device, no collective: ExecutorImpl.cpp:71-75).
"""
import os
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
    def __init__(self, shapes, rank=0, world=1, device="cuda:0", all_gather=None, transport="auto"):
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: peer memory has no CPU path in this package")
        if not 0 <= rank < world <= 16:
            raise ValueError(f"rank {rank} of {world}: at most 16 ranks")
        if transport not in ("auto", "ipc", "multicast"):
            raise ValueError(f"transport {transport!r}: auto, ipc or multicast")
        if transport == "auto":
            # the in-switch form is opt-in: POLAR_B200_PEER_MULTICAST=1 lets "auto" take it from
            # eight ranks up (measured equal to peer to peer at four ranks, slower at two)
            transport = "auto" if os.environ.get("POLAR_B200_PEER_MULTICAST", "0") == "1" else "ipc"
        self.lib = lib()
        self.rank, self.world = rank, world
        self.device = torch.device(device)
        self.offsets, self.n = payload_layout(shapes)
        self.multicast = None        # multicast address of the buffers, when the transport is "multicast"
        self.transport = "ipc"
        self.why_not_multicast = ""
        self._symm = None
        self._opened = []
        self.own = None
        self._owns_buffer = False
        with torch.cuda.device(self.device):
            if all_gather is None and ((transport == "auto" and world >= 8) or (transport == "multicast" and world > 1)):
                self._try_multicast()
                if self.multicast is None and transport == "multicast":
                    raise RuntimeError("no NVLink multicast for the gradient buffers: " + self.why_not_multicast)
            if self.multicast is None:
                self._map_over_ipc(all_gather)
            flat = torch.as_tensor(_DeviceSpan(self.own + CONTROL_BYTES, self.n), device=self.device)
        self.flat = flat
        self.tensors = {name: flat[off:off + count].view(*shapes[name])
                        for name, (off, count) in self.offsets.items()}

    def _try_multicast(self):
        """Symmetric memory with a multicast address, agreed by all ranks (a vote: either every
        rank takes it or none does)."""
        import torch.distributed as dist
        symm, err = None, ""
        try:
            import torch.distributed._symmetric_memory as symm_mem
            floats = CONTROL_BYTES // 4 + (self.n + 3) // 4 * 4
            t = symm_mem.empty(floats, dtype=torch.float32, device=self.device)
            t.zero_()
            torch.cuda.synchronize(self.device)
            h = symm_mem.rendezvous(t, dist.group.WORLD)
            ptrs = [int(p) for p in h.buffer_ptrs]
            mc = int(h.multicast_ptr)
            if len(ptrs) != self.world or ptrs[self.rank] != t.data_ptr():
                err = "symmetric memory gave an unexpected pointer table"
            elif mc == 0:
                err = "symmetric memory has no multicast address on this machine"
            else:
                symm = (t, h, ptrs, mc)
        except Exception as exc:                               # noqa: BLE001 - any failure means "not available here"
            err = f"{type(exc).__name__}: {exc}"
        ok = torch.tensor([1 if symm else 0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) != 1:
            self.why_not_multicast = err or "another rank could not"
            return
        t, h, ptrs, mc = symm
        self._symm = (t, h)
        self.own = ptrs[self.rank]
        self.buffers = (ctypes.c_void_p * self.world)(*ptrs)
        self.multicast = mc
        self.transport = "multicast"
        dist.barrier()      # every rank's control block is zero before anyone launches

    def _map_over_ipc(self, all_gather):
        c = self.lib.cdll
        own = ctypes.c_void_p()
        self.lib.check(c.polar_b200_peer_alloc(self.n * 4, ctypes.byref(own)))
        self.own = own.value
        self._owns_buffer = True
        handle = (ctypes.c_ubyte * HANDLE_BYTES)()
        self.lib.check(c.polar_b200_peer_export(self.own, handle))
        if self.world > 1:
            handles = (all_gather or _gather_over_process_group)(bytes(handle), self.world)
        else:
            handles = [bytes(handle)]
        self.buffers = (ctypes.c_void_p * self.world)()
        for r in range(self.world):
            if r == self.rank:
                self.buffers[r] = self.own
                continue
            h = (ctypes.c_ubyte * HANDLE_BYTES).from_buffer_copy(handles[r])
            p = ctypes.c_void_p()
            self.lib.check(c.polar_b200_peer_open(h, ctypes.byref(p)))
            self.buffers[r] = p.value
            self._opened.append(p.value)

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
        rc = self.lib.cdll.polar_b200_allreduce_fadd_multicast(self.buffers, self.multicast, self.rank, self.world,
                                                               channel, first, count, seg, len(seg), scale_w, scale_g,
                                                               stream)
        if rc != 0:
            self.lib.check(rc)

    def launch(self, seg, scale_w, scale_g, stream):
        rc = self.lib.cdll.polar_b200_allreduce_fadd_multicast(self.buffers, self.multicast, self.rank, self.world, 0, 0,
                                                               self.n, seg, len(seg), scale_w, scale_g, stream)
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
        if self._symm is not None:
            # symmetric memory: no rank lets go of its part while another may still be inside a kernel
            import torch.distributed as dist
            dist.barrier()
            self._symm = None
            self.multicast = None
            self.own = None
            return
        with torch.cuda.device(self.device):
            for p in self._opened:
                c.polar_b200_peer_close(p)
            self._opened = []
            if self.own and self._owns_buffer:
                c.polar_b200_peer_free(self.own)
            self.own = None
