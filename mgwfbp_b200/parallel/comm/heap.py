# -*- coding: utf-8 -*-
"""Symmetric memory for the NVLink data plane: heaps (one region per rank, every peer's region mapped
locally) and the arena that hands out blocks of them.

Three heap flavours with one interface (``base``, ``peer_base[r]``, ``mc_base``, ``nbytes``, ``close()``):

``VmmHeap``        the default.  ``cuMemCreate`` memory exported as POSIX file descriptors and mapped by
                   every peer with ``cuMemMap`` (``csrc/symm_heap.cu``).  When the GPUs sit behind an
                   NVSwitch the region is also bound to a **multicast object**; ``mc_base + off`` then
                   addresses offset ``off`` of every rank's region at once, which the NVLS all-reduce
                   (``multimem.ld_reduce`` / ``multimem.st``) needs.  Descriptors travel between the
                   processes over Unix datagram sockets (``SCM_RIGHTS``); everything else (sizes, success
                   flags) over the gloo control plane.
``IpcHeap``        ``cudaMalloc`` + CUDA IPC handles.  No multicast.  Fallback when VMM sharing is not
                   possible, and the flavour the failure tests ask for (``MGWFBP_HEAP=ipc``): a rank that
                   dies while its memory is bound to a multicast object can disturb the other GPUs.
``TorchSymmHeap``  ``torch.distributed._symmetric_memory`` (``MGWFBP_HEAP=torch``), kept for comparison.

``SymmArena`` is a first-fit allocator over a list of such heaps.  Every rank performs the same
sequence of ``alloc`` / ``free`` calls, so offsets agree without communication; a new heap is added
(collectively) only when no existing one has room.  This replaces Horovod's fusion buffer
(reference ``distributed_optimizer.py:21-26`` delegates it to the C++ core).
"""
from __future__ import annotations

import array
import ctypes as C
import os
import socket
import struct
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ...ops import _lib
from ...settings import logger
from .. import runtime

_ALIGN = 256
_nonce: Optional[str] = None
_exchange_seq = 0


def _round_up(n: int, a: int) -> int:
    return (int(n) + a - 1) // a * a


def _agree(ok: bool) -> bool:
    """True only when every rank says so."""
    return all(runtime.allgather_object(bool(ok)))


# ---------------------------------------------------------------------------------------------------
# file-descriptor exchange
# ---------------------------------------------------------------------------------------------------
def _socket_name(seq: int, rank: int) -> bytes:
    return ('\0mgwfbp-%s-%d-%d' % (_nonce, seq, rank)).encode()


def exchange_fds(my_fd: Optional[int], senders: Sequence[int], timeout_s: float = 60.0) -> Dict[int, int]:
    """Every rank listed in ``senders`` hands ``my_fd`` to every other rank; returns ``{sender: descriptor}`` with the
    descriptors as they arrived in this process.  Collective over the whole job."""
    global _nonce, _exchange_seq
    rank, world = runtime.rank(), runtime.size()
    if _nonce is None:
        _nonce = runtime.broadcast_object(os.urandom(8).hex(), 0)
    _exchange_seq += 1
    seq = _exchange_seq
    sock = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
    got: Dict[int, int] = {}
    try:
        sock.bind(_socket_name(seq, rank))
        sock.settimeout(timeout_s)
        runtime.barrier()                                   # every receiver is bound
        if rank in senders:
            for r in range(world):
                if r != rank:
                    sock.sendmsg([struct.pack('i', rank)],
                                 [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array('i', [int(my_fd)]))], 0,
                                 _socket_name(seq, r))
        expect = [s for s in senders if s != rank]
        while len(got) < len(expect):
            fds = array.array('i')
            msg, ancdata, _flags, _addr = sock.recvmsg(16, socket.CMSG_LEN(fds.itemsize))
            for level, kind, data in ancdata:
                if level == socket.SOL_SOCKET and kind == socket.SCM_RIGHTS:
                    fds.frombytes(data[:len(data) - (len(data) % fds.itemsize)])
            if len(fds) != 1:
                raise OSError('message without a file descriptor')
            got[struct.unpack('i', msg[:4])[0]] = fds[0]
        runtime.barrier()
    finally:
        sock.close()
    return got


# ---------------------------------------------------------------------------------------------------
# heaps
# ---------------------------------------------------------------------------------------------------
class IpcHeap:
    """One symmetric region: same size and layout on every rank, all peers mapped locally (CUDA IPC)."""
    kind = 'ipc'

    def __init__(self, lib, nbytes: int):
        self.lib = lib
        self.nbytes = _round_up(nbytes, _ALIGN)
        self.rank, self.world = runtime.rank(), runtime.size()
        base = C.c_void_p()
        _lib.check(lib.mgw_heap_create(self.nbytes, C.byref(base)), 'heap_create')
        self.base = int(base.value)
        handle = C.create_string_buffer(64)
        _lib.check(lib.mgw_heap_export(self.base, handle), 'heap_export')
        handles = runtime.allgather_object(bytes(handle.raw))
        self.peer_base: List[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.peer_base.append(self.base)
                continue
            p = C.c_void_p()
            _lib.check(lib.mgw_heap_open(C.create_string_buffer(h, 64), C.byref(p)), 'heap_open(rank %d)' % r)
            self.peer_base.append(int(p.value))
        self.mc_base = 0
        runtime.barrier()

    def close(self) -> None:
        if self.base:
            runtime.barrier()
            for r, p in enumerate(self.peer_base):
                if r != self.rank:
                    self.lib.mgw_heap_close(p)
            self.lib.mgw_heap_destroy(self.base)
            self.base = 0


class TorchSymmHeap:
    """Same interface on top of ``torch.distributed._symmetric_memory`` (adds a multicast address)."""
    kind = 'torch'

    def __init__(self, lib, nbytes: int):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.lib = lib
        self.nbytes = _round_up(nbytes, _ALIGN)
        self.rank, self.world = runtime.rank(), runtime.size()
        dev = torch.device('cuda', torch.cuda.current_device())
        self._tensor = symm.empty(self.nbytes, dtype=torch.uint8, device=dev)
        self._handle = symm.rendezvous(self._tensor, dist.group.WORLD.group_name)
        self._tensor.zero_()
        torch.cuda.synchronize()
        self.peer_base = [int(p) for p in self._handle.buffer_ptrs]
        self.base = self.peer_base[self.rank]
        self.mc_base = int(getattr(self._handle, 'multicast_ptr', 0) or 0)
        runtime.barrier()

    def close(self) -> None:
        self._tensor = None
        self._handle = None
        self.base = 0


class VmmUnavailable(RuntimeError):
    pass


class VmmHeap:
    """``cuMemCreate`` region per rank, shared through file descriptors, bound to an NVSwitch multicast object when
    the devices support it and ``multicast`` is asked for.  Construction is collective; if ANY rank fails at a step,
    every rank undoes the step together (multicast: continue without; sharing itself: raise ``VmmUnavailable``)."""
    kind = 'vmm'

    def __init__(self, lib, nbytes: int, multicast: bool = True):
        self.lib = lib
        self.rank, self.world = runtime.rank(), runtime.size()
        self._h = None
        self.base = 0
        self.mc_base = 0
        self.peer_base: List[int] = []
        sup = (C.c_int * 2)()
        rc = lib.mgw_vmm_supported(sup)
        flags = runtime.allgather_object((rc == 0 and bool(sup[0]), rc == 0 and bool(sup[1])))
        if not all(f[0] for f in flags):
            raise VmmUnavailable('VMM allocations with file-descriptor handles are not available on every rank: %s'
                                 % (lib.mgw_last_error() or b'').decode(errors='replace'))
        want_mc = bool(multicast and self.world > 1 and all(f[1] for f in flags))
        heap, base, got = C.c_void_p(), C.c_void_p(), C.c_size_t()
        rc = lib.mgw_vmm_create(C.c_size_t(int(nbytes)), self.world, int(want_mc), C.byref(heap), C.byref(base), C.byref(got))
        err = (lib.mgw_last_error() or b'').decode(errors='replace') if rc != 0 else ''
        sizes = runtime.allgather_object(int(got.value) if rc == 0 else -1)
        if rc == 0:
            self._h, self.base, self.nbytes = heap, int(base.value), int(got.value)
        if any(s < 0 for s in sizes) or len(set(sizes)) != 1:
            self._destroy()
            raise VmmUnavailable('cuMemCreate region could not be set up on every rank (%s; sizes %s)' % (err, sizes))
        # ---- map every peer's region
        ok, err = True, ''
        fd = C.c_int(-1)
        if self.world > 1:
            if lib.mgw_vmm_export_fd(self._h, C.byref(fd)) != 0:
                ok, err = False, (lib.mgw_last_error() or b'').decode(errors='replace')
            if not _agree(ok):
                self._close_fd(fd.value)
                self._destroy()
                raise VmmUnavailable('export of the region as a file descriptor failed (%s)' % err)
            try:
                incoming = exchange_fds(fd.value, list(range(self.world)))
            except OSError as e:
                ok, err, incoming = False, 'descriptor exchange: %s' % e, {}
            self._close_fd(fd.value)
            peers: Dict[int, int] = {}
            for r, pfd in sorted(incoming.items()):
                p = C.c_void_p()
                if ok and lib.mgw_vmm_import_peer(self._h, r, pfd, C.byref(p)) == 0:
                    peers[r] = int(p.value)
                else:
                    if ok:
                        err = (lib.mgw_last_error() or b'').decode(errors='replace')
                    ok = False
            if not _agree(ok and len(peers) == self.world - 1):
                self._destroy()
                raise VmmUnavailable('mapping the peers\' regions failed (%s)' % err)
            self.peer_base = [self.base if r == self.rank else peers[r] for r in range(self.world)]
        else:
            self.peer_base = [self.base]
        # ---- multicast binding (optional)
        if want_mc:
            self._bind_multicast()
        runtime.barrier()

    @staticmethod
    def _close_fd(fd: int) -> None:
        if fd is not None and fd >= 0:
            try:
                os.close(fd)
            except OSError:
                pass

    def _bind_multicast(self) -> None:
        lib = self.lib
        ok, err = True, ''

        def fail(step):
            nonlocal ok, err
            ok, err = False, '%s: %s' % (step, (lib.mgw_last_error() or b'').decode(errors='replace'))
        fd = C.c_int(-1)
        if self.rank == 0 and lib.mgw_vmm_mc_create(self._h, self.world, C.byref(fd)) != 0:
            fail('cuMulticastCreate')
        created = runtime.broadcast_object(ok, 0)
        if not created:
            if self.rank == 0:
                logger.warning('NVSwitch multicast object could not be created (%s); NVLS all-reduce is off', err)
            lib.mgw_vmm_destroy(self._h, 1)
            return
        try:
            incoming = exchange_fds(fd.value if self.rank == 0 else None, [0])
        except OSError as e:
            ok, err, incoming = False, 'descriptor exchange: %s' % e, {}
        if self.rank == 0:
            self._close_fd(fd.value)
        elif ok and lib.mgw_vmm_mc_import(self._h, incoming[0]) != 0:
            fail('import of the multicast object')
        if ok and lib.mgw_vmm_mc_add_device(self._h) != 0:
            fail('cuMulticastAddDevice')
        if _agree(ok):                                       # every device has joined: binding may start
            mc = C.c_void_p()
            if lib.mgw_vmm_mc_bind(self._h, C.byref(mc)) != 0:
                fail('cuMulticastBindMem')
            if _agree(ok):
                self.mc_base = int(mc.value)
                return
        errs = [e for e in runtime.allgather_object(err) if e]
        if self.rank == 0:
            logger.warning('binding the symmetric heap to an NVSwitch multicast object failed (%s); NVLS all-reduce is off',
                           errs[:1])
        lib.mgw_vmm_destroy(self._h, 1)

    def _destroy(self) -> None:
        if self._h is not None:
            self.lib.mgw_vmm_destroy(self._h, 0)
            self._h = None
        self.base = 0
        self.mc_base = 0

    def close(self) -> None:
        if self._h is not None:
            torch.cuda.synchronize()
            runtime.barrier()                 # nobody still reads or writes this rank's region
            self._destroy()
            runtime.barrier()


def heap_kind() -> str:
    return os.environ.get('MGWFBP_HEAP', 'auto').lower()


def make_heap(lib, nbytes: int):
    """A new symmetric heap of at least ``nbytes`` (collective).  ``MGWFBP_HEAP`` = ``auto`` (VMM heap with multicast
    when possible, else CUDA IPC), ``vmm``, ``ipc`` or ``torch``; ``MGWFBP_NVLS=0`` keeps the VMM heap but does not
    bind it to a multicast object."""
    kind = heap_kind()
    if kind == 'torch':
        return TorchSymmHeap(lib, nbytes)
    if kind in ('auto', 'vmm'):
        want_mc = os.environ.get('MGWFBP_NVLS', '1').strip().lower() not in ('0', 'false', 'no', 'off')
        try:
            return VmmHeap(lib, nbytes, multicast=want_mc)
        except VmmUnavailable as e:
            if kind == 'vmm':
                raise
            if runtime.rank() == 0:
                logger.warning('%s; using the CUDA IPC heap', e)
    return IpcHeap(lib, nbytes)


# ---------------------------------------------------------------------------------------------------
# arena
# ---------------------------------------------------------------------------------------------------
class Block:
    """``nbytes`` of symmetric memory at the same offset of every rank's heap."""
    __slots__ = ('heap', 'off', 'nbytes', 'seg')

    def __init__(self, heap, off: int, nbytes: int, seg: int):
        self.heap, self.off, self.nbytes, self.seg = heap, off, nbytes, seg

    @property
    def base(self) -> int:
        return self.heap.base + self.off

    def peer(self, r: int) -> int:
        return self.heap.peer_base[r] + self.off

    @property
    def mc(self) -> int:
        return (self.heap.mc_base + self.off) if self.heap.mc_base else 0


class FreeList:
    """First-fit free list with coalescing over ``[0, size)`` (pure bookkeeping, also used without a GPU)."""

    def __init__(self, size: int):
        self.size = int(size)
        self.free: List[Tuple[int, int]] = [(0, int(size))]        # (offset, length), sorted by offset

    def take(self, nbytes: int) -> Optional[int]:
        n = _round_up(max(int(nbytes), 1), _ALIGN)
        for i, (off, length) in enumerate(self.free):
            if length >= n:
                if length == n:
                    del self.free[i]
                else:
                    self.free[i] = (off + n, length - n)
                return off
        return None

    def give(self, off: int, nbytes: int) -> None:
        n = _round_up(max(int(nbytes), 1), _ALIGN)
        items = sorted(self.free + [(int(off), n)])
        merged: List[Tuple[int, int]] = []
        for o, l in items:
            if merged and merged[-1][0] + merged[-1][1] > o:
                raise ValueError('double free or overlap at offset %d' % o)
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + l)
            else:
                merged.append((o, l))
        self.free = merged

    def used(self) -> int:
        return self.size - sum(l for _, l in self.free)


class SymmArena:
    """Blocks of symmetric memory for everything the data plane needs (flags, staging areas, gathered rows, scratch)."""

    def __init__(self, lib, segment_bytes: Optional[int] = None):
        self.lib = lib
        if segment_bytes is None:
            segment_bytes = int(os.environ.get('MGWFBP_ARENA_MB', '1024')) << 20
        self.segment_bytes = int(segment_bytes)
        self.heaps: List[object] = []
        self.lists: List[FreeList] = []

    @property
    def has_multicast(self) -> bool:
        return bool(self.heaps) and all(h.mc_base for h in self.heaps)

    def alloc(self, nbytes: int) -> Block:
        for i, fl in enumerate(self.lists):
            off = fl.take(nbytes)
            if off is not None:
                return Block(self.heaps[i], off, _round_up(max(int(nbytes), 1), _ALIGN), i)
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError('the symmetric arena must grow outside CUDA graph capture (run eager steps first)')
        heap = make_heap(self.lib, max(self.segment_bytes, _round_up(nbytes, 1 << 21)))
        self.heaps.append(heap)
        self.lists.append(FreeList(heap.nbytes))
        if runtime.rank() == 0:
            logger.info('symmetric arena: segment %d, %s heap, %.0f MB%s', len(self.heaps) - 1, heap.kind, heap.nbytes / 2 ** 20,
                        ', NVSwitch multicast bound' if heap.mc_base else '')
        return self.alloc(nbytes)

    def free(self, block: Optional[Block]) -> None:
        """Return a block.  The caller guarantees (device synchronisation + host barrier) that no rank still uses it."""
        if block is not None and block.seg < len(self.lists):
            self.lists[block.seg].give(block.off, block.nbytes)

    def zero(self, block: Block) -> None:
        holder = _RawMemory(block.base, block.nbytes)
        torch.as_tensor(holder, device=torch.device('cuda', torch.cuda.current_device())).zero_()

    def close(self) -> None:
        for h in self.heaps:
            h.close()
        self.heaps, self.lists = [], []


class _RawMemory:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {'shape': (int(nbytes),), 'typestr': '|u1', 'data': (int(ptr), False), 'version': 2}
