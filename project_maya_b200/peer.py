"""Set-up of the peer-memory all-reduce transport (the host side of maya_peer_ar; startup only, it allocates).

Two ways to build a group:
  PeerGroup.over_processes(rank, world, stride)  one process per GPU (torch.distributed initialised): every rank creates
      its receive and flag buffers, the IPC handles travel through all_gather_object, each rank maps the others' buffers.
  PeerGroup.on_one_device(nm, stride)            all nm "ranks" on the current GPU with plain device pointers: for tests
      of the protocol's arithmetic, flags and time-out without a second GPU (ranks then run one after another).
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import PeerArDesc, PeerArFailure
from .api import MayaError, _check, _ptr, _stream


class PeerRank:
    """One rank's view: its maya_peer_ar descriptor plus the tensors that keep the device arrays alive."""

    def __init__(self, mi: int, nm: int, stride: int, recv_ptr: int, flags_ptr: int, peer_recv: list[int],
                 peer_flags: list[int], timeout_ms: float, keep=None):
        self.mi, self.nm, self.stride = mi, nm, stride
        self.error = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.failure = torch.zeros(C.sizeof(PeerArFailure), dtype=torch.uint8, device="cuda")
        self.recv_tab = torch.tensor(peer_recv, dtype=torch.int64, device="cuda")
        self.flag_tab = torch.tensor(peer_flags, dtype=torch.int64, device="cuda")
        self.seq_counter = torch.zeros(2, dtype=torch.int32, device="cuda")   # [0] the count, [1] scratch of the launches
        self.desc = PeerArDesc(recv_ptr, self.recv_tab.data_ptr(), flags_ptr, self.flag_tab.data_ptr(),
                               self.error.data_ptr(), self.failure.data_ptr(), stride, int(timeout_ms * 1e6), nm,
                               self.seq_counter.data_ptr())
        self.device_seq = False     # True: layer and prompt-path calls take their sequence number from seq_counter
        self.seq = 0
        self.keep = keep

    def next_seq(self) -> int:
        """The next sequence number: modulo 2^32, never 0 (0xffffffff is followed by 2, which keeps the two receive
        slots alternating), as the device-side count does."""
        self.seq = 2 if self.seq == 0xFFFFFFFF else self.seq + 1
        return self.seq

    def set_device_seq(self, on: bool) -> None:
        """Hand the count to the device (calls then pass seq 0 and can be captured in a CUDA graph) or take it back."""
        if on:
            self.seq_counter[0] = int(np.array(self.seq, np.uint32).view(np.int32))
            self.seq_counter[1] = 0
        else:
            torch.cuda.synchronize()
            self.seq = int(np.array(int(self.seq_counter[0].item()), np.int32).view(np.uint32))
        self.device_seq = on

    def allreduce(self, x, seq: int | None = None, stream=None):
        """allreduce_peer: x (f32, numel % 4 == 0) becomes the rank-ordered sum over the group, in place."""
        seq = self.next_seq() if seq is None else seq
        _check("allreduce_peer", _lib.load().maya_allreduce_peer(_ptr(x), x.numel(), C.byref(self.desc), self.mi, seq,
                                                                _stream(stream)))
        return x

    def poisoned(self) -> bool:
        torch.cuda.synchronize()
        return bool(self.error.item() & 1)

    def failure_record(self) -> PeerArFailure:
        torch.cuda.synchronize()
        return PeerArFailure.from_buffer_copy(bytes(self.failure.cpu().numpy()))


class PeerGroup:
    @staticmethod
    def on_one_device(nm: int, stride: int, timeout_ms: float = 50.0) -> list[PeerRank]:
        lib = _lib.load()
        rb, fb = lib.maya_peer_ar_recv_bytes(nm, stride), lib.maya_peer_ar_flag_bytes(nm)
        if rb == 0 or fb == 0:
            raise MayaError("peer_ar sizes", -1)
        recv = [torch.zeros(rb, dtype=torch.uint8, device="cuda") for _ in range(nm)]
        flags = [torch.zeros(fb, dtype=torch.uint8, device="cuda") for _ in range(nm)]
        rp, fp = [t.data_ptr() for t in recv], [t.data_ptr() for t in flags]
        return [PeerRank(m, nm, stride, rp[m], fp[m], rp, fp, timeout_ms, keep=(recv, flags)) for m in range(nm)]

    @staticmethod
    def over_processes(rank: int, world: int, stride: int, timeout_ms: float = 2000.0) -> PeerRank:
        import torch.distributed as dist
        lib = _lib.load()
        rb, fb = lib.maya_peer_ar_recv_bytes(world, stride), lib.maya_peer_ar_flag_bytes(world)
        handles, mine = [], []
        for nbytes in (rb, fb):
            ptr = C.c_void_p()
            h = C.create_string_buffer(64)
            _check("peer_buffer_create", lib.maya_peer_buffer_create(nbytes, C.byref(ptr), h))
            mine.append(ptr.value)
            handles.append(h.raw)
        gathered: list = [None] * world
        dist.all_gather_object(gathered, handles)
        peer_recv, peer_flags = [0] * world, [0] * world
        for m in range(world):
            if m == rank:
                peer_recv[m], peer_flags[m] = mine
                continue
            for j, table in enumerate((peer_recv, peer_flags)):
                ptr = C.c_void_p()
                _check("peer_buffer_open", lib.maya_peer_buffer_open(gathered[m][j], C.byref(ptr)))
                table[m] = ptr.value
        _check("peer_ar_preload", lib.maya_peer_ar_preload(_stream()))
        torch.cuda.synchronize()
        dist.barrier()
        return PeerRank(rank, world, stride, mine[0], mine[1], peer_recv, peer_flags, timeout_ms)
