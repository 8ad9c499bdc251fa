"""Exchange buffers of a tensor-parallel group for sums through peer memory (``skv_comm`` of the C ABI).

Every rank allocates one buffer with ``cudaMalloc``, hands its 64-byte IPC handle to the other ranks over
``torch.distributed`` and maps theirs; the row-parallel products of a decode step (``skv_gemv_tp``) then store
their partial sums - each value paired with an epoch in one 8-byte store - straight into every GPU's buffer over
NVLink, and the next product polls for the epoch and adds them up, in place of an all-reduce launch.  ``PeerExchange.emulated`` builds the same views for several "ranks" on one device inside one
process: kernels of different ranks then run one after the other on a stream, which is how the single-GPU tests
drive the protocol (no kernel ever waits for one that has not been launched).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ._lib import SkvComm, check, lib


class PeerExchange:
    def __init__(self, group, cap_elems: int, device: torch.device, wait_kpolls: int = 0):
        L = lib()
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.cap_elems = -(-int(cap_elems) // 8) * 8
        self.device = device
        torch.cuda.set_device(device)
        nbytes = L.skv_comm_bytes(self.world, self.cap_elems)
        own = ctypes.c_void_p()
        check(L.skv_comm_alloc(nbytes, ctypes.byref(own)), "skv_comm_alloc")
        self._own = own.value
        handle = ctypes.create_string_buffer(64)
        check(L.skv_comm_export(self._own, handle), "skv_comm_export")
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        bases = (ctypes.c_void_p * self.world)()
        self._opened = []
        for r, h in enumerate(handles):
            if r == self.rank:
                bases[r] = self._own
                continue
            peer = ctypes.c_void_p()
            check(L.skv_comm_open(ctypes.create_string_buffer(h, 64), ctypes.byref(peer)), "skv_comm_open")
            self._opened.append(peer.value)
            bases[r] = peer.value
        self.view = SkvComm()
        check(L.skv_comm_view(ctypes.byref(self.view), bases, self.world, self.rank, self.cap_elems), "skv_comm_view")
        self.view.wait_kpolls = wait_kpolls                # 0: the library's default, about five seconds
        dist.barrier(group=group)                      # every rank has mapped every buffer before any use

    @classmethod
    def emulated(cls, world: int, cap_elems: int, device: torch.device, wait_kpolls: int = 0) -> list["PeerExchange"]:
        """``world`` views over buffers that all live on ``device`` (one process, for tests)."""
        L = lib()
        cap = -(-int(cap_elems) // 8) * 8
        nbytes = L.skv_comm_bytes(world, cap)
        torch.cuda.set_device(device)
        bases = (ctypes.c_void_p * world)()
        for r in range(world):
            p = ctypes.c_void_p()
            check(L.skv_comm_alloc(nbytes, ctypes.byref(p)), "skv_comm_alloc")
            bases[r] = p.value
        out = []
        for r in range(world):
            x = cls.__new__(cls)
            x.world, x.rank, x.cap_elems, x.device = world, r, cap, device
            x._own, x._opened = bases[r], []
            x.view = SkvComm()
            check(L.skv_comm_view(ctypes.byref(x.view), bases, world, r, cap), "skv_comm_view")
            x.view.wait_kpolls = wait_kpolls
            out.append(x)
        return out

    def ref(self):
        return ctypes.byref(self.view)

    def tick(self, stream: int | None) -> None:
        """Advance the step counter that stamps this step's exchanges (once per decode step, on every rank)."""
        check(lib().skv_comm_tick(ctypes.byref(self.view), stream), "skv_comm_tick")

    def status(self) -> int:
        """The buffer's status word (``ST_WAIT_TIMEOUT`` when a wait for another GPU gave up); synchronises."""
        rc = lib().skv_comm_status(ctypes.byref(self.view))
        if rc < 0:
            check(rc, "skv_comm_status")
        return rc

    def __del__(self):
        try:                                               # unmap and free if the owner forgot to
            self.close()
        except Exception:
            pass

    def close(self) -> None:
        """Unmap the other ranks' buffers and free this rank's (idempotent).  Call it once no kernel that uses the
        exchange is in flight on any rank."""
        L = lib()
        for p in self._opened:
            L.skv_comm_close(p)
        self._opened = []
        if self._own:
            L.skv_comm_free(self._own)
            self._own = None
