"""Symmetric memory: one peer-mapped heap per process group, plus flag words for kernel-level
signalling between GPUs of one node.

Every rank ``cudaMalloc``s a heap of the same size, exports a CUDA IPC handle, and maps every
peer's heap; the 64-byte handles travel over the host process group.  Allocation is a bump
allocator that all ranks call in the same order, so a tensor has the same offset on every rank
and ``peer_ptrs(t)`` is ``base[p] + offset``.  The first 64 KiB of each heap hold 8192 uint64
flag words; ``signal`` stores a value into one word on every peer (release), ``wait`` spins on the
local words with a wall-clock bound and reports a timeout through the kernel error word instead
of hanging.

The kernels that use these pointers issue plain peer loads and stores; nothing here binds memory
to a switch-side reduction object, so a rank that exits between steps leaves its peers' memory mappings valid.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

FLAG_WORDS = 8192
FLAG_BYTES = FLAG_WORDS * 8
ALIGN = 1024
DEFAULT_TIMEOUT_NS = 30_000_000_000


class _RawCudaArray:
    """Adapter that lets ``torch.as_tensor`` alias raw device memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _declare(L: ctypes.CDLL) -> None:
    vp, i32, u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong
    L.cm_symm_alloc.argtypes = [ctypes.POINTER(vp), ctypes.c_size_t]
    L.cm_symm_free.argtypes = [vp]
    L.cm_ipc_get_handle.argtypes = [vp, ctypes.c_char_p]
    L.cm_ipc_open_handle.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    L.cm_ipc_close_handle.argtypes = [vp]
    L.cm_can_access_peer.argtypes = [i32, i32]
    L.cm_signal_peers.argtypes = [vp, i32, i32, u64, vp]
    L.cm_wait_flags.argtypes = [vp, i32, i32, u64, u64, vp, vp]
    L.cm_put_words.argtypes = [vp, vp, i32, ctypes.c_longlong, i32, vp]
    for n in ("cm_symm_alloc", "cm_symm_free", "cm_ipc_get_handle", "cm_ipc_open_handle", "cm_ipc_close_handle",
              "cm_can_access_peer", "cm_signal_peers", "cm_wait_flags", "cm_put_words"):
        getattr(L, n).restype = i32


class SymmetricHeap:
    def __init__(self, group, ranks: Sequence[int], nbytes: int, device: torch.device):
        from ..ops import cuda as cu
        self.L = cu.lib()
        _declare(self.L)
        self.group, self.ranks = group, list(ranks)
        self.world = len(self.ranks)
        self.me = self.ranks.index(dist.get_rank()) if dist.is_initialized() else 0
        self.device = device
        self.nbytes = (nbytes + FLAG_BYTES + ALIGN - 1) // ALIGN * ALIGN
        base = ctypes.c_void_p()
        rc = self.L.cm_symm_alloc(ctypes.byref(base), self.nbytes)
        if rc:
            raise RuntimeError(f"symmetric heap allocation of {self.nbytes} bytes failed (cuda error {rc})")
        self.base = base.value
        handle = ctypes.create_string_buffer(64)
        rc = self.L.cm_ipc_get_handle(self.base, handle)
        if rc:
            raise RuntimeError(f"cudaIpcGetMemHandle failed ({rc})")
        handles: List[Optional[bytes]] = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, handle.raw, group=group)
        else:
            handles[0] = handle.raw
        self.peer_base: List[int] = []
        for i, h in enumerate(handles):
            if i == self.me:
                self.peer_base.append(self.base)
                continue
            p = ctypes.c_void_p()
            rc = self.L.cm_ipc_open_handle(h, ctypes.byref(p))
            if rc:
                raise RuntimeError(f"cudaIpcOpenMemHandle for peer {i} failed ({rc}); peer access is required")
            self.peer_base.append(p.value)
        self._bytes = torch.as_tensor(_RawCudaArray(self.base, self.nbytes), device=device)
        self.flags = self._bytes[:FLAG_BYTES].view(torch.int64)
        self._top = FLAG_BYTES
        self._flag_ptrs = torch.tensor(self.peer_base, dtype=torch.int64, device=device)
        self._offsets: Dict[int, int] = {}
        self.timeout_ns = DEFAULT_TIMEOUT_NS

    # ---- allocation ----------------------------------------------------------------------
    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """Same call order on every rank.  Returns a zero-initialised tensor in the heap."""
        n = 1
        for s in (shape if isinstance(shape, (tuple, list)) else (shape,)):
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        off = (self._top + ALIGN - 1) // ALIGN * ALIGN
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {nbytes} bytes at {off}, heap is {self.nbytes}")
        self._top = off + nbytes
        t = self._bytes[off:off + nbytes].view(dtype).view(shape)
        self._offsets[t.data_ptr()] = off
        return t

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base
        if not (0 <= off < self.nbytes):
            raise ValueError("tensor is not in this symmetric heap")
        return off

    def peer_ptrs(self, t: torch.Tensor) -> List[int]:
        off = self.offset_of(t)
        return [b + off for b in self.peer_base]

    def peer_tensor(self, t: torch.Tensor, peer: int) -> torch.Tensor:
        """Tensor view of peer ``peer``'s copy of the symmetric tensor ``t`` (same shape and dtype), usable as the
        destination of this package's own copy / GEMM-epilogue stores.  Never hand it to a library kernel."""
        if peer == self.me:
            return t
        nbytes = t.numel() * t.element_size()
        raw = torch.as_tensor(_RawCudaArray(self.peer_base[peer] + self.offset_of(t), nbytes), device=self.device)
        return raw.view(t.dtype).view(t.shape)

    def wait_one(self, index: int, rank: int, value: int, timeout_ns: Optional[int] = None) -> None:
        """Bounded device-side wait until rank ``rank`` (position in the group) has signalled ``value`` on ``index``."""
        from ..ops.cuda import err_word, stream_ptr
        rc = self.L.cm_wait_flags(self.flags.data_ptr(), index * self.world + rank, 1, value,
                                  self.timeout_ns if timeout_ns is None else timeout_ns,
                                  err_word(self.device).data_ptr(), stream_ptr())
        if rc:
            raise RuntimeError(f"cm_wait_flags failed ({rc})")

    def peer_ptr_array(self, t: torch.Tensor):
        ptrs = self.peer_ptrs(t)
        return (ctypes.c_void_p * self.world)(*ptrs)

    # ---- signalling ------------------------------------------------------------------------
    def signal(self, index: int, value: int) -> None:
        """After all work queued so far on the current stream, store ``value`` into flag word
        ``index * world + me`` of every peer."""
        from ..ops.cuda import stream_ptr
        if not 0 <= (index + 1) * self.world <= FLAG_WORDS:
            raise IndexError(f"flag index {index} out of range for {self.world} ranks ({FLAG_WORDS} words)")
        rc = self.L.cm_signal_peers(self._flag_ptrs.data_ptr(), self.world, index * self.world + self.me, value,
                                    stream_ptr())
        if rc:
            raise RuntimeError(f"cm_signal_peers failed ({rc})")

    def wait(self, index: int, value: int, timeout_ns: Optional[int] = None) -> None:
        """Queue a bounded device-side wait until every rank has signalled ``value`` on ``index``."""
        from ..ops.cuda import err_word, stream_ptr
        if not 0 <= (index + 1) * self.world <= FLAG_WORDS:
            raise IndexError(f"flag index {index} out of range for {self.world} ranks ({FLAG_WORDS} words)")
        rc = self.L.cm_wait_flags(self.flags.data_ptr(), index * self.world, self.world, value,
                                  self.timeout_ns if timeout_ns is None else timeout_ns,
                                  err_word(self.device).data_ptr(), stream_ptr())
        if rc:
            raise RuntimeError(f"cm_wait_flags failed ({rc})")

    def barrier(self, index: int, value: int) -> None:
        self.signal(index, value)
        self.wait(index, value)

    def all_gather_words(self, src: torch.Tensor, buf: torch.Tensor, index: int, value: int) -> torch.Tensor:
        """All-gather of a small int64 vector without a library collective: every rank stores ``src`` [n] into row ``me``
        of the symmetric tensor ``buf`` [world, n] on every peer, then the group meets on flag ``index``.  Returns the
        local ``buf``.  The caller must not reuse ``buf`` before every rank has consumed the previous contents (one
        later barrier of the same group is enough)."""
        from ..ops.cuda import stream_ptr
        n = src.numel()
        assert src.dtype == torch.int64 and src.is_contiguous() and buf.dtype == torch.int64 and tuple(buf.shape) == (self.world, n)
        ptrs = getattr(buf, "_peer_ptr_tensor", None)
        if ptrs is None:
            ptrs = torch.tensor(self.peer_ptrs(buf), dtype=torch.int64, device=self.device)
            buf._peer_ptr_tensor = ptrs
        rc = self.L.cm_put_words(src.data_ptr(), ptrs.data_ptr(), self.world, self.me * n, n, stream_ptr())
        if rc:
            raise RuntimeError(f"cm_put_words failed ({rc})")
        self.barrier(index, value)
        return buf

    def close(self) -> None:
        for i, p in enumerate(self.peer_base):
            if i != self.me and p:
                self.L.cm_ipc_close_handle(p)
        self.peer_base = []
        if self.base:
            self._bytes = None
            self.flags = None
            self.L.cm_symm_free(self.base)
            self.base = 0


def peer_access_available(pc) -> bool:
    """True when every GPU of this node-local group can map the others' memory."""
    if not torch.cuda.is_available() or pc.world_size <= 1:
        return False
    from ..ops import cuda as cu
    L = cu.lib()
    _declare(L)
    me = torch.cuda.current_device()
    return all(L.cm_can_access_peer(me, d) for d in range(torch.cuda.device_count()) if d != me)
