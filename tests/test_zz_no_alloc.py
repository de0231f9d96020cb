"""The allocation-free attention backward, called through its exported C symbol.

Some users of this library cannot allocate device memory when they call it (a host application
with a fixed memory budget, a plug-in inside another framework's allocator, a latency-critical
loop). For them `eri_flash_attn_bwd_noalloc` keeps its scratch in a static device array. This test
loads the shared object directly with ctypes, runs the entry point twice in a row on different
inputs (the second call sees the first call's leftovers in the shared scratch) and compares each
result with the regular entry point, which uses caller-provided scratch.

The file name sorts last on purpose: if this test fails, a run that stops at the first failure has
already executed every other test.
"""
import ctypes as C
import math
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = Path(__file__).resolve().parents[1] / "eridiffusion_b200" / "lib" / "liberi_b200_kernels.so"


def _lib():
    lib = C.CDLL(str(LIB))
    P, I, F = C.c_void_p, C.c_int, C.c_float
    lib.eri_flash_attn_bwd_noalloc.argtypes = [P] * 9 + [I] * 5 + [F, P]
    lib.eri_flash_attn_bwd_noalloc.restype = I
    lib.eri_flash_attn_bwd_noalloc_strerror.argtypes = [I]
    lib.eri_flash_attn_bwd_noalloc_strerror.restype = C.c_char_p
    lib.eri_flash_attn_bwd_noalloc_max_rows.restype = I
    lib.eri_flash_attn_bwd_noalloc_status.restype = I
    return lib


def _mk(B, L, H, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(B, L, H, D, device="cuda", generator=g).bfloat16()


def _run_noalloc(lib, do, q, k, v, out, lse):
    B, Lq, H, D = q.shape
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    rc = lib.eri_flash_attn_bwd_noalloc(
        do.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
        dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, H, Lq, k.shape[1], D,
        1.0 / math.sqrt(D), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.eri_flash_attn_bwd_noalloc_strerror(rc)
    return dq, dk, dv


def test_noalloc_backward_matches_regular_entry_point_twice():
    from eridiffusion_b200.ops import flash_attn as FA
    lib = _lib()
    # The third call has a query length that is not a multiple of 128 and follows larger calls: its
    # padded rows of the shared scratch still hold the earlier calls' values unless the kernel
    # rewrites them, which is the one place where leftovers could leak into a result.
    for call, (B, H, Lq, Lk, D) in enumerate([(1, 2, 384, 256, 128), (2, 3, 256, 320, 64), (1, 2, 200, 256, 128)]):
        q, k, v = _mk(B, Lq, H, D, 10 + call), _mk(B, Lk, H, D, 20 + call), _mk(B, Lk, H, D, 30 + call)
        do = _mk(B, Lq, H, D, 40 + call)
        out, lse = FA.fwd(q, k, v)
        ref = FA.bwd(do, q, k, v, out, lse)
        got = _run_noalloc(lib, do, q, k, v, out, lse)
        torch.cuda.synchronize()
        assert lib.eri_flash_attn_bwd_noalloc_status() == 0
        for a, b in zip(got, ref):
            # the same kernels on the same inputs, only the scratch lives elsewhere: bit-equal
            assert torch.equal(a, b), (call, (a.float() - b.float()).abs().max().item())


def test_noalloc_rejects_oversized_problem():
    lib = _lib()
    cap = lib.eri_flash_attn_bwd_noalloc_max_rows()
    B, H, Lq, D = 1, 64, 8192, 128          # 64 * 8192 rows > cap
    assert B * H * Lq > cap
    rc = lib.eri_flash_attn_bwd_noalloc(None, None, None, None, None, None, None, None, None,
                                        B, H, Lq, 128, D, 0.1, None)
    assert rc == -6
    assert b"TOO_LARGE" in lib.eri_flash_attn_bwd_noalloc_strerror(rc)
