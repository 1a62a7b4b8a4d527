"""``SymmetricHeap``: one block of device memory per rank, mapped into every rank of the node at known addresses, plus
(where the GPUs support it) an NVSwitch multicast view of the same memory.

The native part (``csrc/comm/symm_heap.cu``) allocates with the driver's virtual-memory API and exports the block as a
POSIX file descriptor; this module moves the descriptors between the processes -- over Unix-domain sockets with
``SCM_RIGHTS`` (``socket.send_fds``), the socket paths being exchanged through the ``torch.distributed`` group -- and
drives the collective steps in the right order with barriers in between:

    allocate + map locally -> exchange fds -> map every peer's block
    rank 0 creates the multicast object -> everyone imports it, adds its device -> barrier -> binds its block ->
    barrier -> maps the multicast view

``heap.peer_ptrs[r]`` is the address of rank r's block in this process (``peer_ptrs[rank]`` is the local block),
``heap.mc_ptr`` the address of the multicast view (0 without multicast support): a ``multimem.st`` to ``mc_ptr + off``
writes offset ``off`` of every rank's block, a ``multimem.ld_reduce`` from it returns the sum over the ranks.

``close()`` releases in the reverse order, again with barriers, because a rank must not free memory that is still
bound to a multicast object its peers use.  The reference has no peer memory (its device-memory FFI is declared but
never implemented, ``crates/kv/src/gpu_memory.rs:479-501``).
"""
from __future__ import annotations

import ctypes as C
import os
import socket
import tempfile
import threading
import uuid
from typing import List, Optional

import torch

from ..ops import _native as N


def _lib():
    lib = N.cuda_lib()
    if not getattr(lib, "_ub_symm_ready", False):
        u64p, ip, vpp = C.POINTER(C.c_ulonglong), C.POINTER(C.c_int), C.POINTER(C.c_void_p)
        lib.ub_symm_error.restype = C.c_char_p
        lib.ub_symm_supported.argtypes = [C.c_int, ip, ip]
        lib.ub_symm_round_size.argtypes = [C.c_ulonglong, C.c_int, C.c_int, u64p]
        lib.ub_symm_alloc.argtypes = [C.c_ulonglong, C.c_int, u64p, ip, vpp]
        lib.ub_symm_map_peer.argtypes = [C.c_int, C.c_ulonglong, C.c_int, u64p, vpp]
        lib.ub_symm_unmap.argtypes = [C.c_void_p, C.c_ulonglong, C.c_ulonglong]
        lib.ub_symm_mc_create.argtypes = [C.c_ulonglong, C.c_int, u64p, ip]
        lib.ub_symm_mc_import.argtypes = [C.c_int, u64p]
        lib.ub_symm_mc_add_device.argtypes = [C.c_ulonglong, C.c_int]
        lib.ub_symm_mc_bind.argtypes = [C.c_ulonglong, C.c_ulonglong, C.c_ulonglong]
        lib.ub_symm_mc_map.argtypes = [C.c_ulonglong, C.c_ulonglong, C.c_int, vpp]
        lib.ub_symm_mc_release.argtypes = [C.c_ulonglong, C.c_void_p, C.c_ulonglong, C.c_int]
        lib.ub_symm_probe.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_void_p]
        for n in ("ub_symm_supported", "ub_symm_round_size", "ub_symm_alloc", "ub_symm_map_peer", "ub_symm_unmap",
                  "ub_symm_mc_create", "ub_symm_mc_import", "ub_symm_mc_add_device", "ub_symm_mc_bind", "ub_symm_mc_map",
                  "ub_symm_mc_release", "ub_symm_probe"):
            getattr(lib, n).restype = C.c_int
        lib._ub_symm_ready = True
    return lib


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: {_lib().ub_symm_error().decode() or rc}")


def supported(device_index: int):
    """(can export allocations as file descriptors, supports NVSwitch multicast) for a CUDA device ordinal."""
    a, b = C.c_int(0), C.c_int(0)
    _check(_lib().ub_symm_supported(device_index, C.byref(a), C.byref(b)), "ub_symm_supported")
    return bool(a.value), bool(b.value)


class _Raw:
    """Device memory described through the CUDA array interface, so that ``torch.as_tensor`` can view it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class _FdServer:
    """Hands this rank's descriptors to each peer that connects (one message per peer)."""

    def __init__(self, fds: List[int], n_peers: int):
        self.path = os.path.join(tempfile.gettempdir(), f"ub_symm_{uuid.uuid4().hex}.sock")
        self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self.sock.bind(self.path)
        self.sock.listen(max(n_peers, 1))
        self.fds, self.n, self.error = fds, n_peers, None
        self.thread = threading.Thread(target=self._serve, daemon=True)
        self.thread.start()

    def _serve(self):
        try:
            for _ in range(self.n):
                conn, _ = self.sock.accept()
                with conn:
                    socket.send_fds(conn, [b"fd"], self.fds)
        except Exception as e:          # noqa: BLE001 - reported by close()
            self.error = e

    def close(self):
        self.thread.join(timeout=60)
        self.sock.close()
        try:
            os.unlink(self.path)
        except OSError:
            pass
        if self.error is not None:
            raise self.error


def _fetch_fds(path: str, n: int) -> List[int]:
    with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as s:
        s.connect(path)
        _, fds, _, _ = socket.recv_fds(s, 16, n)
    if len(fds) != n:
        raise RuntimeError(f"expected {n} descriptors from {path}, got {len(fds)}")
    return list(fds)


class SymmetricHeap:
    def __init__(self):
        self.rank = self.world = 0
        self.device = None
        self.nbytes = 0
        self.local_ptr = 0
        self.peer_ptrs: List[int] = []
        self.mc_ptr = 0
        self._handles: List[int] = []
        self._mc = 0
        self._group = None
        self._closed = False

    @classmethod
    def create(cls, nbytes: int, rank: int, world: int, group, device, multicast: Optional[bool] = None) -> "SymmetricHeap":
        """Collective over ``group`` (all ``world`` ranks on one node).  ``multicast``: None = use it when every device
        supports it, False = peer mappings only, True = required."""
        import torch.distributed as dist

        lib = _lib()
        dev = torch.device(device)
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        h = cls()
        h.rank, h.world, h.device, h._group = rank, world, torch.device("cuda", idx), group
        vmm, mc_ok = supported(idx)
        if not vmm:
            raise RuntimeError("this device cannot export allocations as POSIX file descriptors")
        flags = [None] * world
        dist.all_gather_object(flags, bool(mc_ok), group=group)
        use_mc = all(flags) and world > 1 if multicast is None else bool(multicast)
        if multicast and not all(flags):
            raise RuntimeError("NVSwitch multicast is not supported on every rank's device")
        size = C.c_ulonglong(0)
        _check(lib.ub_symm_round_size(nbytes, idx, world if use_mc else 0, C.byref(size)), "ub_symm_round_size")
        h.nbytes = int(size.value)
        handle, fd, va = C.c_ulonglong(0), C.c_int(-1), C.c_void_p(0)
        _check(lib.ub_symm_alloc(h.nbytes, idx, C.byref(handle), C.byref(fd), C.byref(va)), "ub_symm_alloc")
        h.local_ptr = int(va.value)
        h._handles = [0] * world
        h._handles[rank] = int(handle.value)
        h.peer_ptrs = [0] * world
        h.peer_ptrs[rank] = h.local_ptr
        my_fds = [fd.value]
        mc_fd = -1
        if use_mc and rank == 0:
            mc, mfd = C.c_ulonglong(0), C.c_int(-1)
            _check(lib.ub_symm_mc_create(h.nbytes, world, C.byref(mc), C.byref(mfd)), "ub_symm_mc_create")
            h._mc, mc_fd = int(mc.value), mfd.value
            my_fds.append(mc_fd)
        server = _FdServer(my_fds, world - 1)
        paths = [None] * world
        dist.all_gather_object(paths, server.path, group=group)
        for r in range(world):
            if r == rank:
                continue
            got = _fetch_fds(paths[r], 2 if (use_mc and r == 0) else 1)
            ph, pva = C.c_ulonglong(0), C.c_void_p(0)
            _check(lib.ub_symm_map_peer(got[0], h.nbytes, idx, C.byref(ph), C.byref(pva)), f"ub_symm_map_peer({r})")
            h._handles[r], h.peer_ptrs[r] = int(ph.value), int(pva.value)
            os.close(got[0])
            if use_mc and r == 0:
                mc = C.c_ulonglong(0)
                _check(lib.ub_symm_mc_import(got[1], C.byref(mc)), "ub_symm_mc_import")
                h._mc = int(mc.value)
                os.close(got[1])
        dist.barrier(group)
        server.close()
        os.close(fd.value)
        if mc_fd >= 0:
            os.close(mc_fd)
        if use_mc:
            _check(lib.ub_symm_mc_add_device(h._mc, idx), "ub_symm_mc_add_device")
            dist.barrier(group)
            _check(lib.ub_symm_mc_bind(h._mc, h._handles[rank], h.nbytes), "ub_symm_mc_bind")
            dist.barrier(group)
            mva = C.c_void_p(0)
            _check(lib.ub_symm_mc_map(h._mc, h.nbytes, idx, C.byref(mva)), "ub_symm_mc_map")
            h.mc_ptr = int(mva.value)
        h.tensor().zero_()
        torch.cuda.synchronize(h.device)
        dist.barrier(group)
        return h

    def tensor(self) -> torch.Tensor:
        """The local block as a uint8 tensor (a view: it does not own the memory)."""
        return torch.as_tensor(_Raw(self.local_ptr, self.nbytes), device=self.device)

    def close(self) -> None:
        """Collective: every rank calls it, with none of its kernels on this memory still running."""
        if self._closed:
            return
        import torch.distributed as dist

        self._closed = True
        lib = _lib()
        torch.cuda.synchronize(self.device)
        dist.barrier(self._group)
        if self._mc:
            lib.ub_symm_mc_release(self._mc, C.c_void_p(self.mc_ptr), self.nbytes, self.device.index)
            self._mc, self.mc_ptr = 0, 0
        dist.barrier(self._group)
        for r in range(self.world):
            if r != self.rank and self.peer_ptrs[r]:
                lib.ub_symm_unmap(C.c_void_p(self.peer_ptrs[r]), self.nbytes, self._handles[r])
        dist.barrier(self._group)
        lib.ub_symm_unmap(C.c_void_p(self.local_ptr), self.nbytes, self._handles[self.rank])
        self.peer_ptrs, self.local_ptr = [], 0


def probe(kind: int, src_ptr: int, dst_ptr: int, nbytes: int, device, iters: int = 10, ctas: int = 0) -> float:
    """GB/s of one copy kernel between two addresses of a symmetric heap (CUDA events, best of ``iters`` after a
    warm-up): kind 0 plain copy (peer store when dst is a peer mapping, peer load when src is), 1 ``multimem.st`` of
    local data to a multicast address, 2 ``multimem.ld_reduce`` from a multicast address into local memory."""
    lib = _lib()
    st = torch.cuda.current_stream(device).cuda_stream
    best = None
    for i in range(iters + 2):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        _check(lib.ub_symm_probe(kind, C.c_void_p(src_ptr), C.c_void_p(dst_ptr), nbytes, ctas, C.c_void_p(st)), "ub_symm_probe")
        b.record()
        torch.cuda.synchronize(device)
        ms = a.elapsed_time(b)
        if i >= 2:
            best = ms if best is None else min(best, ms)
    return nbytes / best / 1e6
