"""Materialised slices and slice-gradient accumulation (``csrc/narrow.cu``).

``narrow_copy(x, dim, start, length)`` returns a dense copy of ``x.narrow(dim, start, length)``
for tensors of rank <= 8 with any strides and any dtype; its gradient is added into a zero buffer of
``x``'s shape. ``narrow_backward_add(grad_out, grad_in, dim, start)`` adds a slice gradient into an
existing, larger gradient buffer in place (no temporary of the full shape).

Reference: ``eri_narrow_strided_kernel`` (crates/core/cuda/narrow_strided.cu:18-99) and
``narrow_backward_scatter_add_kernel_v2`` (crates/core/cuda/narrow_strided_backward.cu:88-214),
bound in crates/core/src/tensor_narrow.rs. A slice is one-to-one, so the accumulation here uses
no atomics. Inside the framework plain slices stay views; use these when a kernel needs a dense
operand or when many slice gradients accumulate into one buffer.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _native as N

_P, _I, _L = C.c_void_p, C.c_int, C.c_longlong
_LP = C.POINTER(C.c_longlong)
N._SIGNATURES.update({
    "eri_narrow_copy": [_P, _P, _L, _L, _L, _L, _L, _I, _P],
    "eri_narrow_backward_add": [_P, _P, _L, _L, _L, _L, _L, _I, _P],
    "eri_narrow_strided": [_P, _P, _I, _LP, _LP, _L, _I, _P],
    "eri_narrow_backward_add_strided": [_P, _P, _I, _LP, _LP, _L, _I, _P],
})
_DTYPE_TAG = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
MAX_RANK = 8


def _fn(name):
    lib = N.require()
    fn = getattr(lib, name)
    fn.argtypes = N._SIGNATURES[name]
    fn.restype = C.c_int
    return fn


def _split(shape, dim):
    outer = 1
    for s in shape[:dim]:
        outer *= s
    inner = 1
    for s in shape[dim + 1:]:
        inner *= s
    return outer, inner


def _check(x, dim, start, length):
    if x.dim() < 1 or x.dim() > MAX_RANK:
        raise ValueError(f"narrow: rank {x.dim()} not in 1..{MAX_RANK}")
    dim = dim % x.dim()
    if start < 0 or length < 0 or start + length > x.shape[dim]:
        raise IndexError(f"narrow: [{start}, {start + length}) outside dimension of size {x.shape[dim]}")
    return dim


def _arr(vals):
    return (C.c_longlong * len(vals))(*vals)


@torch.no_grad()
def narrow_copy_raw(x: torch.Tensor, dim: int, start: int, length: int) -> torch.Tensor:
    dim = _check(x, dim, start, length)
    if not x.is_cuda:
        return x.narrow(dim, start, length).contiguous()
    shape = list(x.shape)
    shape[dim] = length
    out = torch.empty(shape, dtype=x.dtype, device=x.device)
    if out.numel() == 0:
        return out
    if x.is_contiguous():
        outer, inner = _split(x.shape, dim)
        N.check(_fn("eri_narrow_copy")(x.data_ptr(), out.data_ptr(), outer, x.shape[dim], inner, start,
                                       length, x.element_size(), N.stream_ptr()), "narrow_copy")
    else:
        N.check(_fn("eri_narrow_strided")(x.data_ptr(), out.data_ptr(), x.dim(), _arr(shape),
                                          _arr(list(x.stride())), start * x.stride(dim), x.element_size(),
                                          N.stream_ptr()), "narrow_strided")
    return out


@torch.no_grad()
def narrow_backward_add(grad_out: torch.Tensor, grad_in: torch.Tensor, dim: int, start: int) -> torch.Tensor:
    """``grad_in.narrow(dim, start, grad_out.shape[dim]) += grad_out`` in place; returns ``grad_in``.
    ``grad_in`` may be strided but must not alias itself (no expanded dimensions)."""
    dim = _check(grad_in, dim, start, grad_out.shape[dim % grad_in.dim()])
    length = grad_out.shape[dim]
    want = list(grad_in.shape)
    want[dim] = length
    if list(grad_out.shape) != want or grad_out.dtype != grad_in.dtype:
        raise ValueError(f"narrow_backward_add: gradient {tuple(grad_out.shape)} {grad_out.dtype} does not "
                         f"match the slice {tuple(want)} {grad_in.dtype}")
    if any(st == 0 and sz > 1 for st, sz in zip(grad_in.stride(), grad_in.shape)):
        raise ValueError("narrow_backward_add: destination has an expanded (stride 0) dimension")
    if not grad_in.is_cuda or grad_in.dtype not in _DTYPE_TAG:
        grad_in.narrow(dim, start, length).add_(grad_out)
        return grad_in
    if grad_out.numel() == 0:
        return grad_in
    go = grad_out.contiguous()
    tag = _DTYPE_TAG[grad_in.dtype]
    if grad_in.is_contiguous():
        outer, inner = _split(grad_in.shape, dim)
        N.check(_fn("eri_narrow_backward_add")(go.data_ptr(), grad_in.data_ptr(), outer, grad_in.shape[dim],
                                               inner, start, length, tag, N.stream_ptr()), "narrow_backward_add")
    else:
        N.check(_fn("eri_narrow_backward_add_strided")(go.data_ptr(), grad_in.data_ptr(), grad_in.dim(),
                                                       _arr(want), _arr(list(grad_in.stride())),
                                                       start * grad_in.stride(dim), tag, N.stream_ptr()),
                "narrow_backward_add_strided")
    return grad_in


class _NarrowCopy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, start, length):
        ctx.meta = (x.shape, x.dtype, x.device, dim, start)
        return narrow_copy_raw(x, dim, start, length)

    @staticmethod
    def backward(ctx, g):
        shape, dtype, device, dim, start = ctx.meta
        gi = torch.zeros(shape, dtype=dtype, device=device)
        narrow_backward_add(g.to(dtype), gi, dim, start)
        return gi, None, None, None


def narrow_copy(x: torch.Tensor, dim: int, start: int, length: int) -> torch.Tensor:
    """Dense, differentiable copy of ``x.narrow(dim, start, length)``."""
    return _NarrowCopy.apply(x, dim, start, length)
