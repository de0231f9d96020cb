"""Symmetric device memory: every rank allocates the same-sized buffer, exports it with CUDA IPC
and maps every peer's buffer, so kernels can load from / store to peer memory over NVLink directly.

``SymmetricHeap`` is a bump allocator over one such buffer; ``SymmetricTensor`` bundles a local
torch view with the peers' raw pointers. A small symmetric flag region carries the epoch words
of the in-kernel barriers. Handles are exchanged with ``torch.distributed`` (plumbing only).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _native as N

MAX_WORLD = 16
FLAG_CHANNELS = 8


class CommCtx(C.Structure):
    _fields_ = [("flags_local", C.c_void_p), ("flags_peer", C.c_void_p * MAX_WORLD),
                ("rank", C.c_int), ("world", C.c_int), ("epoch", C.c_uint),
                ("wait_ns", C.c_ulonglong), ("err", C.c_void_p)]


class FusedDpArgs(C.Structure):
    _fields_ = [("grads", C.c_void_p * MAX_WORLD), ("params", C.c_void_p * MAX_WORLD),
                ("sumsq_slots", C.c_void_p * MAX_WORLD), ("reduced", C.c_void_p),
                ("sumsq_local", C.c_void_p), ("mq", C.c_void_p), ("vq", C.c_void_p),
                ("m_absmax", C.c_void_p), ("v_absmax", C.c_void_p), ("grad_norm_out", C.c_void_p),
                ("shard_elems", C.c_longlong), ("lr", C.c_float), ("beta1", C.c_float),
                ("beta2", C.c_float), ("eps", C.c_float), ("weight_decay", C.c_float),
                ("max_grad_norm", C.c_float), ("step", C.c_int), ("seed", C.c_uint),
                ("stochastic", C.c_int), ("stamps", C.c_void_p)]


class CollArgs(C.Structure):
    _fields_ = [("src", C.c_void_p * MAX_WORLD), ("dst_peers", C.c_void_p * MAX_WORLD),
                ("dst", C.c_void_p), ("count", C.c_longlong), ("op", C.c_int), ("dtype", C.c_int),
                ("root", C.c_int), ("avg", C.c_int)]


def _bind(lib):
    P, I, L = C.c_void_p, C.c_int, C.c_longlong
    sigs = {"eri_symm_malloc": [L, C.POINTER(P)], "eri_symm_free": [P],
            "eri_ipc_get_handle": [P, P], "eri_ipc_open_handle": [P, C.POINTER(P)],
            "eri_ipc_close_handle": [P], "eri_ipc_handle_size": [],
            "eri_fused_dp_step": [C.POINTER(CommCtx), C.POINTER(FusedDpArgs), P],
            "eri_collective": [C.POINTER(CommCtx), C.POINTER(CollArgs), P]}
    for n, a in sigs.items():
        fn = getattr(lib, n)
        fn.argtypes, fn.restype = a, C.c_int


class _RawCudaBuffer:
    """Exposes a raw device pointer through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class SymmetricHeap:
    def __init__(self, nbytes: int, group=None):
        self.lib = N.require()
        _bind(self.lib)
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.world > MAX_WORLD:
            raise ValueError(f"world size {self.world} > {MAX_WORLD}")
        self.nbytes = (nbytes + 4095) // 4096 * 4096
        p = C.c_void_p()
        N.check(self.lib.eri_symm_malloc(self.nbytes, C.byref(p)), "symm_malloc")
        self.local_ptr = p.value
        self._raw = _RawCudaBuffer(self.local_ptr, self.nbytes)
        self.bytes_view = torch.as_tensor(self._raw, device=torch.device("cuda", torch.cuda.current_device()))
        self.bytes_view.zero_()
        torch.cuda.synchronize()
        self.peer_ptrs = [self.local_ptr]
        self._opened = []
        if self.world > 1:
            hs = self.lib.eri_ipc_handle_size()
            buf = (C.c_char * hs)()
            N.check(self.lib.eri_ipc_get_handle(self.local_ptr, buf), "ipc_get_handle")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(buf), group=group)
            self.peer_ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.peer_ptrs.append(self.local_ptr)
                    continue
                q = C.c_void_p()
                hb = (C.c_char * hs).from_buffer_copy(h)
                N.check(self.lib.eri_ipc_open_handle(hb, C.byref(q)), "ipc_open_handle")
                self.peer_ptrs.append(q.value)
                self._opened.append(q.value)
            dist.barrier(group=group)
        self._off = 0

    def alloc(self, nbytes: int, align: int = 256) -> int:
        off = (self._off + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted ({off + nbytes} > {self.nbytes})")
        self._off = off + nbytes
        return off

    def tensor(self, shape, dtype):
        n = 1
        for s in (shape if isinstance(shape, (tuple, list)) else (shape,)):
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        off = self.alloc(nb)
        t = self.bytes_view[off:off + nb].view(dtype).view(shape)
        return SymmetricTensor(t, [p + off for p in self.peer_ptrs])

    def close(self):
        for p in self._opened:
            self.lib.eri_ipc_close_handle(p)
        self._opened = []


class SymmetricTensor:
    def __init__(self, local: torch.Tensor, peer_ptrs):
        self.local = local
        self.peer_ptrs = peer_ptrs

    def ptr_array(self):
        arr = (C.c_void_p * MAX_WORLD)()
        for i, p in enumerate(self.peer_ptrs):
            arr[i] = p
        return arr


class Communicator:
    """Flag region + status word + epoch counter shared by the in-kernel barriers, and the
    pull-based collectives built on them."""

    OPS = {"all_gather": 0, "reduce_scatter": 1, "all_reduce": 2, "all_to_all": 3, "broadcast": 4,
           "barrier": 5}

    def __init__(self, heap: SymmetricHeap, wait_ms: float = 2000.0):
        self.heap = heap
        self.lib = heap.lib
        self.rank, self.world = heap.rank, heap.world
        self.flags = heap.tensor((FLAG_CHANNELS, MAX_WORLD), torch.int32)
        self.flags.local.zero_()
        self.err = torch.zeros(1, dtype=torch.int32, device=self.flags.local.device)
        self.epoch = 0
        self.wait_ns = int(wait_ms * 1e6)
        torch.cuda.synchronize()
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=heap.group)

    def ctx(self) -> CommCtx:
        self.epoch += 1
        c = CommCtx()
        c.flags_local = self.flags.local.data_ptr()
        for i, p in enumerate(self.flags.peer_ptrs):
            c.flags_peer[i] = p
        c.rank, c.world, c.epoch, c.wait_ns = self.rank, self.world, self.epoch, self.wait_ns
        c.err = self.err.data_ptr()
        return c

    def status(self) -> int:
        """Synchronise and read the status word: 0, or ((phase) << 8) | peer of a wait that ran
        out. The word is cleared after reading."""
        v = int(self.err.item())
        if v:
            self.err.zero_()
        return v

    def collective(self, op: str, src: SymmetricTensor, dst: torch.Tensor | None = None,
                   dst_sym: SymmetricTensor | None = None, count: int | None = None, root=0, avg=False):
        a = CollArgs()
        for i, p in enumerate(src.peer_ptrs):
            a.src[i] = p
        if dst_sym is not None:
            for i, p in enumerate(dst_sym.peer_ptrs):
                a.dst_peers[i] = p
            a.dst = dst_sym.local.data_ptr()
        elif dst is not None:
            a.dst = dst.data_ptr()
        a.count = count if count is not None else src.local.numel() // (self.world if op in ("reduce_scatter", "all_reduce", "all_to_all") else 1)
        a.op = self.OPS[op]
        a.dtype = 0 if src.local.dtype == torch.bfloat16 else 1
        a.root, a.avg = root, int(avg)
        c = self.ctx()
        N.check(self.lib.eri_collective(C.byref(c), C.byref(a), N.stream_ptr()), f"collective:{op}")
