"""ctypes binding of the in-tree CUDA library.

The kernels are exported as plain C functions taking raw device pointers and a CUDA stream, so the
binding layer is a table of argument types. ``lib()`` loads ``lib/liberi_b200_kernels.so`` (building
it when the sources are newer and a compiler is present). On a machine with a GPU a missing
library is an error, never a silent fallback: ``require()`` raises ``NativeLibraryError``.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent.parent
# ERI_B200_DEBUG_BOUNDS=1 loads the bounds-checked debug variant (csrc/build.py builds it on demand)
DEBUG_BOUNDS = os.environ.get("ERI_B200_DEBUG_BOUNDS") == "1"
_LIB_PATH = _PKG / "lib" / ("liberi_b200_kernels_debug.so" if DEBUG_BOUNDS else "liberi_b200_kernels.so")
_lock = threading.Lock()
_lib = None
_launches = 0  # number of kernel launches issued through this module (for bench accounting)


class NativeLibraryError(RuntimeError):
    pass


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("b", C.c_void_p), ("lora_h", C.c_void_p), ("lora_b", C.c_void_p),
        ("bias", C.c_void_p), ("residual", C.c_void_p), ("gate", C.c_void_p),
        ("pre_in", C.c_void_p), ("out", C.c_void_p), ("out2", C.c_void_p),
        ("pre_out", C.c_void_p),
        ("lda", C.c_longlong), ("ldb", C.c_longlong), ("ld_h", C.c_longlong),
        ("ld_lb", C.c_longlong),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("lora_r", C.c_int),
        ("act", C.c_int), ("n_split", C.c_int),
        ("ldc", C.c_int), ("ldc2", C.c_int), ("ld_pre", C.c_int), ("ldr", C.c_int),
        ("rows_per_batch", C.c_int), ("gate_stride", C.c_int),
        ("force_bn", C.c_int), ("alpha", C.c_float), ("b_mn", C.c_int),
        ("n_copy", C.c_int), ("n_jobs", C.c_int),
        ("jobs", C.c_void_p), ("flags", C.c_void_p), ("flag_target", C.c_void_p),
        ("b_flag_rows", C.c_int), ("a_flag_cols", C.c_int), ("rot_n_rows", C.c_int),
        ("rot_k_cols", C.c_int), ("a_flag_rows", C.c_int),
        ("scatter_world", C.c_int), ("scatter_rank", C.c_int), ("scatter_part_cols", C.c_int),
        ("scatter_group_cols", C.c_int), ("scatter_local_rows", C.c_int),
        ("scatter_out", C.c_void_p * 16), ("rowsq", C.c_void_p), ("rowsq_parts", C.c_int),
        ("pdl", C.c_int),
        ("b_local", C.c_void_p), ("ldb_local", C.c_longlong),
        ("loc_mode", C.c_int), ("loc_lo", C.c_int), ("loc_hi", C.c_int), ("n_jobs_nl", C.c_int),
        ("jobs_nl", C.c_void_p), ("flag_target_nl", C.c_void_p),
        ("a_mn", C.c_int), ("glu", C.c_int),
        ("dbg_out_bytes", C.c_longlong), ("dbg_out2_bytes", C.c_longlong), ("dbg_pre_bytes", C.c_longlong),
        ("dbg_res_bytes", C.c_longlong), ("scatter_mode", C.c_int), ("stamps", C.c_void_p), ("join_round", C.c_int), ("all_flag", C.c_int),
    ]


class GatherJob(C.Structure):
    """One copy job of the gather-fused GEMM (mirrors ``GatherJob`` in csrc/gemm.cu)."""
    _fields_ = [("src", C.c_void_p), ("dst", C.c_void_p), ("rows", C.c_int), ("row_bytes", C.c_int),
                ("src_stride", C.c_longlong), ("dst_stride", C.c_longlong), ("flag", C.c_int),
                ("pad", C.c_int)]


_P, _I, _L, _F, _U64, _U32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_ulonglong, C.c_uint

_SIGNATURES = {
    "eri_norm_modulate_fwd": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P],
    "eri_norm_modulate_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "eri_norm_modulate_fwd_warp": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P],
    "eri_norm_modulate_bwd_warp": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "eri_norm_modulate_bwd_warp_add": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "eri_norm_check_error": [],
    "eri_norm_set_smem_variant": [C.c_int],
    "eri_adamw8bit_set_pair_variant": [C.c_int],
    "eri_qknorm_rope_fwd": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "eri_qknorm_rope_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F,
                            _I, _I, _I, _P],
    "eri_gate_residual": [_P, _P, _P, _P, _L, _I, _I, _I, _P],
    "eri_gate_grad": [_P, _P, _P, _I, _I, _I, _P],
    "eri_slot_reduce": [_P, _P, _I, _L, _F, _I, _P],
    "eri_act_fwd": [_P, _P, _L, _I, _P],
    "eri_act_bwd": [_P, _P, _P, _L, _I, _P],
    "eri_act_bwd_rows": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _P],
    "eri_act_fwd_rows": [_P, _L, _P, _L, _I, _I, _I, _P],
    "eri_glu_fwd": [_P, _P, _I, _I, _I, _I, _P],
    "eri_glu_bwd": [_P, _P, _P, _I, _I, _I, _I, _P],
    "eri_noise_mix": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _U64, _U64, _P],
    "eri_randn_bf16": [_P, _L, _U64, _U64, _F, _F, _P],
    "eri_mse_fwd_bwd": [_P, _P, _P, _P, _P, _L, _L, _F, _P],
    "eri_sumsq_bf16": [_P, _L, _P, _P],
    "eri_post_clamp_u8": [_P, _P, _L, _P],
    "eri_poison_fill": [_P, _L, _U32, _P],
    "eri_adamw8bit_step": [_P, _P, _P, _P, _P, _P, _P, _L, _F, _F, _F, _F, _F, _I, _F, _F, _U32, _I, _P],
    "eri_adamw8bit_step_scaled": [_P, _P, _P, _P, _P, _P, _P, _L, _F, _F, _F, _F, _F, _I, _F, _F, _U32, _I, _P, _P],
    "eri_adamw32_step": [_P, _P, _P, _P, _P, _L, _I, _F, _F, _F, _F, _F, _I, _F, _F, _U32, _I, _P],
    "eri_ema_update": [_P, _P, _L, _F, _P],
    "eri_scale_bf16": [_P, _L, _P, _F, _F, _P],
    "eri_gn_stats_fwd": [_P, _P, _I, _I, _I, _P],
    "eri_gn_apply_fwd": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "eri_gn_stats_bwd": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "eri_gn_apply_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "eri_row_l2norm": [_P, _P, _L, _I, _P],
    "eri_topk_desc": [_P, _P, _I, _I, _I, _P],
    "eri_build_inverse": [_P, _P, _I, _I, _I, _P],
    "eri_gather_rows": [_P, _P, _P, _I, _I, _I, _I, _P],
    "eri_reinject_rows": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
    "eri_dequant_int8": [_P, _P, _P, _L, _I, _P],
    "eri_dequant_4bit": [_P, _P, _P, _L, _I, _I, _P],
    "eri_gemm_skinny": [_P, _L, _P, _L, _P, _I, _I, _I, _I, _F, _P],
    "eri_gemm_skinny_check_error": [],
    "eri_gemm_rank_stream": [_P, _L, _P, _L, _P, _I, _I, _I, _I, _F, _P],
    "eri_gemm_rank_stream2": [_P, _L, _P, _L, _P, _I, _I, _F, _P, _L, _P, _L, _P, _I, _I, _F, _I, _I, _P],
    "eri_gemm_tokred": [_P, _L, _P, _L, _P, _I, _I, _I, _I, _F, _I, _I, _L, _P],
    "eri_gemm_tokred_check_error": [],
    "eri_gemm_tokred_set_target": [_I],
    "eri_gemm_init": [],
    "eri_gemm_check_error": [],
    "eri_gemm_bf16": [C.POINTER(GemmArgs), _P],
    "eri_gemm2_bf16": [C.POINTER(GemmArgs), _P],
    "eri_gemm2_bf16_group2": [C.POINTER(GemmArgs), C.POINTER(GemmArgs), _P],
    "eri_gemm2_check_error": [],
    "eri_gemm2_gather_count": [],
    "eri_rows_wgrad": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _F, _P],
    "eri_rows_dgrad": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P],
    "eri_gemv_bf16": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
}


def _maybe_build() -> None:
    if os.environ.get("ERI_B200_NO_BUILD") == "1":
        return
    try:
        from ..csrc import build as _b
        _b.build_kernels(debug_bounds=DEBUG_BOUNDS)
    except Exception:
        if not _LIB_PATH.exists():
            raise


def lib():
    """Return the loaded kernel library, or ``None`` when it cannot be loaded here (CPU-only box
    without the CUDA runtime)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            if not _LIB_PATH.exists():
                _maybe_build()
            handle = C.CDLL(str(_LIB_PATH))
        except Exception:
            return None
        for name, argtypes in _SIGNATURES.items():
            try:
                fn = getattr(handle, name)
            except AttributeError:
                continue
            fn.argtypes = argtypes
            fn.restype = C.c_int
        _lib = handle
    return _lib


def extent_bytes(t) -> int:
    """Bytes from ``t``'s first element to the end of its storage (what a kernel may touch through a
    pointer to ``t``); passed to the kernels for the bounds-checked debug build."""
    if t is None:
        return 0
    return t.untyped_storage().nbytes() - t.storage_offset() * t.element_size()


def debug_bounds_report() -> dict:
    """Violations recorded by the bounds-checked debug build since the last call, per kernel file:
    ``{file: {"code", "count", "line", "value"}}`` (empty: clean, or not the debug build). Reading
    synchronises the device and clears the records."""
    h = lib()
    out = {}
    if h is None:
        return out
    buf = (C.c_int * 4)()
    for tag in ("gemm", "gemm2", "tokred", "fa", "route"):
        fn = getattr(h, f"eri_{tag}_debug_bounds", None)
        if fn is None:
            if DEBUG_BOUNDS:
                raise NativeLibraryError(f"the debug library does not export eri_{tag}_debug_bounds")
            continue
        fn.argtypes, fn.restype = [C.POINTER(C.c_int)], C.c_int
        if fn(buf) > 0:
            out[tag] = {"code": buf[0], "count": buf[1], "line": buf[2], "value": buf[3]}
    return out


def available() -> bool:
    return torch.cuda.is_available() and lib() is not None


def require():
    h = lib()
    if h is None:
        raise NativeLibraryError(
            f"native kernel library {_LIB_PATH} is missing or failed to load; run "
            "`python -m eridiffusion_b200.csrc.build` (needs nvcc) before using CUDA tensors")
    return h


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def stream_ptr() -> int:
    """Handle of the current CUDA stream of the current device. Every kernel call asks for it (thousands
    of times per training step), so the two direct runtime queries are used when this torch build has
    them: ``torch.cuda.current_stream()`` builds a Python Stream object per call (~15 us)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def check(code: int, what: str) -> None:
    global _launches
    _launches += 1
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code}")


def launch_count() -> int:
    return _launches
