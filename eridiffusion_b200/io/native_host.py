"""ctypes binding of ``lib/liberi_b200_host.so`` (mmap safetensors reader with pinned
double-buffered host->device streaming, pinned pool, SHA-256, xorshift permutation)."""
from __future__ import annotations

import ctypes as C
import json
from pathlib import Path

import torch

_PATH = Path(__file__).resolve().parent.parent / "lib" / "liberi_b200_host.so"
_lib = None


def lib():
    global _lib
    if _lib is None:
        try:
            h = C.CDLL(str(_PATH))
        except OSError:
            return None
        P, L, I = C.c_void_p, C.c_longlong, C.c_int
        h.eri_pinned_alloc.restype, h.eri_pinned_alloc.argtypes = P, [L]
        h.eri_pinned_free.argtypes = [P]
        h.eri_pinned_stats.argtypes = [C.POINTER(L)] * 3
        h.eri_st_open.restype, h.eri_st_open.argtypes = P, [C.c_char_p]
        h.eri_st_header.restype, h.eri_st_header.argtypes = C.c_char_p, [P]
        h.eri_st_data_offset.restype, h.eri_st_data_offset.argtypes = L, [P]
        h.eri_st_close.argtypes = [P]
        h.eri_st_read_host.restype, h.eri_st_read_host.argtypes = I, [P, L, L, P]
        h.eri_st_read_device.restype, h.eri_st_read_device.argtypes = I, [P, L, L, P, P]
        h.eri_sha256_file.restype, h.eri_sha256_file.argtypes = I, [C.c_char_p, C.c_char_p]
        h.eri_sha256_bytes.restype, h.eri_sha256_bytes.argtypes = I, [C.c_char_p, L, C.c_char_p]
        h.eri_xorshift_permutation.argtypes = [L, C.c_ulonglong, C.POINTER(L)]
        if hasattr(h, "eri_prefetch_create"):
            h.eri_prefetch_create.restype, h.eri_prefetch_create.argtypes = P, [I, I]
            h.eri_prefetch_submit.restype, h.eri_prefetch_submit.argtypes = L, [P, C.c_char_p, L, L]
            h.eri_prefetch_wait.restype, h.eri_prefetch_wait.argtypes = I, [P, L, C.POINTER(P), C.POINTER(L)]
            h.eri_prefetch_release.restype, h.eri_prefetch_release.argtypes = I, [P, L]
            h.eri_prefetch_bytes_read.restype, h.eri_prefetch_bytes_read.argtypes = L, [P]
            h.eri_prefetch_destroy.argtypes = [P]
        _lib = h
    return _lib


def sha256_file(path) -> str:
    out = C.create_string_buffer(65)
    if lib().eri_sha256_file(str(path).encode(), out) != 0:
        raise FileNotFoundError(path)
    return out.value.decode()


def sha256_bytes(b: bytes) -> str:
    out = C.create_string_buffer(65)
    lib().eri_sha256_bytes(b, len(b), out)
    return out.value.decode()


def xorshift_permutation(n, seed):
    arr = (C.c_longlong * n)()
    lib().eri_xorshift_permutation(n, seed, arr)
    return list(arr)


_DT = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
       "I8": torch.int8, "U8": torch.uint8, "F64": torch.float64, "I16": torch.int16, "BOOL": torch.bool}


class NativeSafeFile:
    """mmap-backed safetensors file; ``get`` streams a tensor to the device through pinned staging."""

    def __init__(self, path):
        self.h = lib().eri_st_open(str(path).encode())
        if not self.h:
            raise OSError(f"cannot open {path}")
        self.header = json.loads(lib().eri_st_header(self.h).decode())
        self.metadata = self.header.pop("__metadata__", {})

    def keys(self):
        return list(self.header)

    def get(self, name, device="cpu", dtype=None):
        e = self.header[name]
        b, en = e["data_offsets"]
        dt = _DT[e["dtype"]]
        t = torch.empty(e["shape"], dtype=dt, device=device)
        if t.numel():
            if t.is_cuda:
                rc = lib().eri_st_read_device(self.h, b, en - b, t.data_ptr(), torch.cuda.current_stream().cuda_stream)
            else:
                rc = lib().eri_st_read_host(self.h, b, en - b, t.data_ptr())
            if rc != 0:
                raise IOError(f"{name}: read failed ({rc})")
        return t.to(dtype) if dtype is not None else t

    def close(self):
        if self.h:
            lib().eri_st_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


class Prefetcher:
    """Read-ahead of file byte ranges on native worker threads into pinned buffers
    (``csrc/host/prefetch.cpp``). ``submit`` returns a ticket at once (it blocks only while
    ``max_inflight`` tickets are outstanding), ``wait`` returns the bytes as a uint8 tensor that
    aliases the pinned buffer, ``release`` hands the buffer back to the pool."""

    _ERR = {-1: "unknown ticket", -2: "cannot open the file", -3: "short read", -4: "out of memory"}

    def __init__(self, threads: int = 4, max_inflight: int = 16):
        h = lib()
        if h is None or not hasattr(h, "eri_prefetch_create"):
            raise RuntimeError("native host library without the prefetcher; run python -m eridiffusion_b200.csrc.build")
        self.max_inflight = max(1, int(max_inflight))
        self._h, self._p = h, h.eri_prefetch_create(threads, max_inflight)

    def submit(self, path, offset: int, nbytes: int) -> int:
        t = self._h.eri_prefetch_submit(self._p, str(path).encode(), int(offset), int(nbytes))
        if t < 0:
            raise ValueError(f"prefetch submit rejected ({path}, {offset}, {nbytes})")
        return t

    def submit_tensor(self, safe_file, name: str) -> int:
        """Queue the payload of tensor ``name`` of an ``io.safetensors.SafeFile``."""
        b, e = safe_file.header[name]["data_offsets"]
        return self.submit(safe_file.path, safe_file._base + b, e - b)

    def wait(self, ticket: int):
        ptr, n = C.c_void_p(), C.c_longlong()
        code = self._h.eri_prefetch_wait(self._p, ticket, C.byref(ptr), C.byref(n))
        if code != 0:
            raise OSError(f"prefetch ticket {ticket}: {self._ERR.get(code, code)}")
        if n.value == 0:
            return torch.empty(0, dtype=torch.uint8)
        buf = (C.c_ubyte * n.value).from_address(ptr.value)
        return torch.frombuffer(buf, dtype=torch.uint8)

    def release(self, ticket: int) -> None:
        self._h.eri_prefetch_release(self._p, ticket)

    def bytes_read(self) -> int:
        return self._h.eri_prefetch_bytes_read(self._p)

    def close(self):
        if self._p:
            self._h.eri_prefetch_destroy(self._p)
            self._p = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()
