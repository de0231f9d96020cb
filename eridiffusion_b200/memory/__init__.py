"""Memory subsystems: block swap / layer streaming, quantised base weights, pinned staging pool,
workspace arena with debug poison, memory profiler, batch-size pressure policy.

Reference parts covered: ``BlockSwapManager`` (GPU <-> pinned host, LRU, prefetch;
src/memory/block_swapping.rs:19-489, defaults 20 GB budget / 8 active blocks / prefetch 4 at
:113-145; crates/common/blockswap/src/manager.rs:12-51), ``FluxLayerStreamer``
(src/trainers/flux_layer_streaming.rs:65-131: persistent layers, per-layer LR multipliers),
``QuantoManager`` (INT8 absmax / INT4 / NF4; src/memory/quanto.rs:168-426), ``MemoryPool`` with
size classes (src/memory/pool.rs:64-395), poison fill 0xCD / 0xDD / bf16 NaN
(crates/core/src/cuda_memory.rs:42-94), ``MemoryProfiler`` (src/memory/profiler.rs:13-75),
``MemoryStrategy`` / ``MemoryPressure`` (src/trainers/memory_optimizer.rs).

On a 180 GB part the training configurations of this repository keep every block resident; block
swap exists for models or batch sizes that exceed that, and for parity of the config surface
(``use_layer_streaming``, ``streaming_memory_limit_gb``, ``low_vram``, ``quantize``).
"""
from __future__ import annotations

import time
from collections import OrderedDict
from dataclasses import dataclass, field

import torch
import torch.nn as nn


# ------------------------------------------------------------------------- block swap
@dataclass
class BlockSwapConfig:
    gpu_budget_gb: float = 20.0
    max_active_blocks: int = 8
    prefetch: int = 4
    persistent: tuple = ()          # indices that never leave the GPU


class BlockSwapManager:
    """Keeps a window of transformer blocks on the GPU; the rest lives in pinned host memory.
    ``run(i, fn)`` makes block i resident (prefetching the next ones on a copy stream), runs
    ``fn(block)`` and evicts least-recently-used blocks beyond the window."""

    def __init__(self, blocks, cfg: BlockSwapConfig | None = None, device=None, frozen_only=False):
        self.blocks = list(blocks)
        self.cfg = cfg or BlockSwapConfig()
        self.frozen_only = frozen_only
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.cuda = self.device.type == "cuda"
        self.copy_stream = torch.cuda.Stream() if self.cuda else None
        self.resident = OrderedDict()                # index -> event (copy finished)
        self.host = {}
        self.stats = {"loads": 0, "evictions": 0, "prefetch_hits": 0, "bytes_h2d": 0}
        per_block = max(1, self._block_bytes(self.blocks[0]))
        by_budget = int(self.cfg.gpu_budget_gb * 2 ** 30 // per_block)
        self.window = max(1, min(self.cfg.max_active_blocks, by_budget, len(self.blocks)))
        for i, b in enumerate(self.blocks):
            self.host[i] = {n: (p.detach().cpu().pin_memory() if self.cuda else p.detach().cpu())
                            for n, p in self._swappable(b)}
            if self.cuda and i not in self.cfg.persistent:
                self._drop(i)
            else:
                self.resident[i] = None

    @staticmethod
    def _block_bytes(b):
        return sum(p.numel() * p.element_size() for p in b.parameters())

    def _swappable(self, b):
        """Tensors that move between host and device. With ``frozen_only`` (training with adapters)
        trainable tensors stay where they are: they live in the optimizer's flat arena."""
        return [(n, p) for n, p in b.named_parameters() if not (self.frozen_only and p.requires_grad)]

    def _drop(self, i):
        for n, p in self._swappable(self.blocks[i]):
            p.data = torch.empty(0, dtype=p.dtype, device=self.device)

    def _load(self, i, sync=False):
        if i in self.resident:
            self.resident.move_to_end(i)
            return
        ev = None
        if self.cuda:
            with torch.cuda.stream(self.copy_stream):
                for n, p in self._swappable(self.blocks[i]):
                    src = self.host[i][n]
                    p.data = src.to(self.device, non_blocking=True)
                    self.stats["bytes_h2d"] += src.numel() * src.element_size()
                ev = torch.cuda.Event()
                ev.record(self.copy_stream)
        else:
            for n, p in self._swappable(self.blocks[i]):
                p.data = self.host[i][n]
        self.resident[i] = ev
        self.stats["loads"] += 1

    def plan(self, i, direction=1):
        """Indices that should be resident while block i runs (``direction`` -1: the backward pass
        walks the stack from the last block to the first)."""
        if direction < 0:
            return [j for j in range(i, max(-1, i - 1 - self.cfg.prefetch), -1)]
        return [j for j in range(i, min(len(self.blocks), i + 1 + self.cfg.prefetch))]

    def prefetch_next(self, i, direction=1):
        for j in self.plan(i, direction)[1:]:
            if len(self.resident) < self.window + len(self.cfg.persistent):
                self._load(j)

    def release_previous(self, i):
        while len(self.resident) > self.window + len(self.cfg.persistent):
            victim = next((j for j in self.resident if j != i and j not in self.cfg.persistent), None)
            if victim is None:
                break
            # trainable tensors are written back before eviction
            if any(p.requires_grad for _, p in self._swappable(self.blocks[victim])):
                for n, p in self._swappable(self.blocks[victim]):
                    self.host[victim][n].copy_(p.detach(), non_blocking=True)
            self.resident.pop(victim)
            self._drop(victim)
            self.stats["evictions"] += 1

    def run(self, i, fn, direction=1):
        hit = i in self.resident
        self._load(i)
        if hit:
            self.stats["prefetch_hits"] += 1
        ev = self.resident[i]
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        self.prefetch_next(i, direction)
        out = fn(self.blocks[i])
        self.release_previous(i)
        return out


def forward_with_swap(blocks, x, step, cfg: BlockSwapConfig | None = None):
    """Block-swap driver (crates/models/qwen_image/src/block_swap.rs:16-32): ``step(block, x) -> x``."""
    mgr = BlockSwapManager(blocks, cfg)
    for i in range(len(mgr.blocks)):
        x = mgr.run(i, lambda b: step(b, x))
    return x, mgr.stats


# ------------------------------------------------------------------------- quantised base weights
NF4_LEVELS = torch.tensor([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
                           -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
                           0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
                           0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0])


@dataclass
class QuantizedTensor:
    kind: str
    data: torch.Tensor
    scale: torch.Tensor
    shape: tuple
    block: int

    def dequantize(self, dtype=torch.bfloat16):
        return dequantize(self, dtype)

    def nbytes(self):
        return self.data.numel() * self.data.element_size() + self.scale.numel() * self.scale.element_size()


def quantize(w: torch.Tensor, kind="int8", block=64) -> QuantizedTensor:
    """int8: per-output-row absmax; int4 / nf4: per-``block`` absmax, two codes per byte."""
    shape = tuple(w.shape)
    wf = w.detach().float()
    if kind == "int8":
        s = wf.abs().amax(dim=-1, keepdim=True).clamp_min(1e-12) / 127.0
        q = torch.round(wf / s).clamp(-127, 127).to(torch.int8)
        return QuantizedTensor(kind, q, s.squeeze(-1), shape, 0)
    flat = wf.reshape(-1, block)
    s = flat.abs().amax(dim=1, keepdim=True).clamp_min(1e-12)
    if kind == "int4":
        q = (torch.round(flat / s * 7.0).clamp(-8, 7) + 8).to(torch.uint8)
    elif kind == "nf4":
        q = (flat / s).unsqueeze(-1).sub(NF4_LEVELS.to(wf.device)).abs().argmin(-1).to(torch.uint8)
    else:
        raise ValueError(kind)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()
    return QuantizedTensor(kind, packed, s.squeeze(1), shape, block)


def _dequantize_native(q: QuantizedTensor, out=None):
    """CUDA path: one kernel expands the codes into a bf16 operand (csrc/dequant.cu)."""
    from ..ops import _native as N
    lib = N.require()
    n = 1
    for s in q.shape:
        n *= s
    if out is None:
        out = torch.empty(q.shape, dtype=torch.bfloat16, device=q.data.device)
    scale = q.scale.float().contiguous()
    if q.kind == "int8":
        cols = q.shape[-1]
        N.check(lib.eri_dequant_int8(q.data.data_ptr(), scale.data_ptr(), out.data_ptr(), n // cols, cols,
                                     N.stream_ptr()), "dequant_int8")
    else:
        N.check(lib.eri_dequant_4bit(q.data.data_ptr(), scale.data_ptr(), out.data_ptr(), n, q.block,
                                     1 if q.kind == "nf4" else 0, N.stream_ptr()), "dequant_4bit")
    return out


def dequantize(q: QuantizedTensor, dtype=torch.bfloat16, out=None):
    if q.data.is_cuda and dtype == torch.bfloat16 and q.data.is_contiguous():
        from ..ops import functional as F
        ok = (q.shape[-1] % 16 == 0) if q.kind == "int8" else (q.block % 32 == 0)
        if ok and F.get_backend() == "fused":
            return _dequantize_native(q, out)
    if q.kind == "int8":
        return (q.data.float() * q.scale.unsqueeze(-1)).to(dtype).view(q.shape)
    lo, hi = (q.data & 0xF).long(), (q.data >> 4).long()
    codes = torch.stack([lo, hi], dim=-1).flatten(1)
    if q.kind == "int4":
        vals = (codes.float() - 8.0) / 7.0
    else:
        vals = NF4_LEVELS.to(q.data.device)[codes]
    return (vals * q.scale.unsqueeze(1)).to(dtype).view(q.shape)


class QuantizedLinear(nn.Module):
    """Frozen base weight stored quantised; dequantised per call into a scratch tensor and fed to
    the fused linear (adapters attach as usual)."""

    def __init__(self, linear, kind="int8", block=64):
        super().__init__()
        self.q = quantize(linear.weight, kind, block)
        self.bias = linear.bias
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.adapter = getattr(linear, "adapter", None)
        self.weight_dtype = linear.weight.dtype

    @property
    def weight(self):
        return self.q.dequantize(self.weight_dtype)

    def frozen_transpose(self):
        return None

    def forward(self, x, act=None, residual=None, gate=None):
        from ..ops import functional as F
        if self.adapter is not None:
            return self.adapter(self, x, act=act, residual=residual, gate=gate)
        return F.linear(x, self.weight, self.bias, act=act, residual=residual, gate=gate)


def quantize_model(model: nn.Module, kind="int8", min_numel=1 << 16):
    from ..models.layers import Linear
    n = 0
    for mod in list(model.modules()):
        for cname, child in list(mod.named_children()):
            if type(child) is Linear and child.weight.numel() >= min_numel and not child.weight.requires_grad:
                setattr(mod, cname, QuantizedLinear(child, kind))
                n += 1
    return n


# ------------------------------------------------------------------------- pinned pool / workspace
class PinnedPool:
    """Size-classed pool of pinned host buffers (powers of two) for staging copies."""

    def __init__(self, max_bytes=4 << 30):
        self.free = {}
        self.max_bytes, self.held = max_bytes, 0

    def get(self, nbytes):
        cls = 1 << max(12, (nbytes - 1).bit_length())
        lst = self.free.get(cls)
        if lst:
            return lst.pop()
        self.held += cls
        pin = torch.cuda.is_available()
        return torch.empty(cls, dtype=torch.uint8, pin_memory=pin)

    def put(self, buf):
        if self.held > self.max_bytes:
            self.held -= buf.numel()
            return
        self.free.setdefault(buf.numel(), []).append(buf)


POISON_ALLOC, POISON_FREE, POISON_BF16_NAN = 0xCDCDCDCD, 0xDDDDDDDD, 0x7FC17FC1


class WorkspaceArena:
    """Bump allocator over one device buffer with an optional poison fill on take / reset, so a
    kernel that reads scratch it never wrote shows up as NaNs (debug aid; compute-sanitizer is not
    available on the GPU pool this project is developed on)."""

    def __init__(self, nbytes, device="cuda", debug=False):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.off, self.debug, self.peak = 0, debug, 0

    def _poison(self, view, pattern):
        from ..ops import _native as N
        if view.is_cuda and N.lib() is not None:
            N.check(N.require().eri_poison_fill(view.data_ptr(), view.numel(), pattern, N.stream_ptr()), "poison")
        else:
            view.view(torch.int32).fill_(pattern - (1 << 32) if pattern >= (1 << 31) else pattern)

    def take(self, shape, dtype):
        n = 1
        for s in shape:
            n *= s
        nb = (n * torch.empty((), dtype=dtype).element_size() + 255) // 256 * 256
        if self.off + nb > self.buf.numel():
            raise MemoryError(f"workspace cap exceeded: {self.off + nb} > {self.buf.numel()}")
        view = self.buf[self.off:self.off + nb]
        if self.debug:
            self._poison(view, POISON_BF16_NAN if dtype == torch.bfloat16 else POISON_ALLOC)
        self.off += nb
        self.peak = max(self.peak, self.off)
        return view[: n * torch.empty((), dtype=dtype).element_size()].view(dtype).view(shape)

    def reset(self):
        if self.debug and self.off:
            self._poison(self.buf[: self.off], POISON_FREE)
        self.off = 0


# ------------------------------------------------------------------------- profiler / pressure
@dataclass
class MemoryEvent:
    kind: str          # allocation | deallocation | peak | oom | checkpoint
    bytes: int
    tag: str
    t: float = field(default_factory=time.time)


class MemoryProfiler:
    def __init__(self):
        self.events: list[MemoryEvent] = []

    def record(self, kind, nbytes, tag=""):
        self.events.append(MemoryEvent(kind, int(nbytes), tag))

    def snapshot(self, tag=""):
        if torch.cuda.is_available():
            self.record("peak", torch.cuda.max_memory_allocated(), tag)
            return torch.cuda.memory_allocated()
        return 0

    def summary(self):
        peak = max((e.bytes for e in self.events if e.kind == "peak"), default=0)
        return {"events": len(self.events), "peak_gb": peak / 2 ** 30,
                "ooms": sum(1 for e in self.events if e.kind == "oom")}


def memory_pressure(device=None) -> str:
    """low | medium | high | critical from the free fraction of device memory."""
    if not torch.cuda.is_available():
        return "low"
    free, total = torch.cuda.mem_get_info(device)
    used = 1 - free / total
    return "critical" if used > 0.95 else "high" if used > 0.85 else "medium" if used > 0.6 else "low"


def suggest_batch_size(current, pressure):
    return {"critical": max(1, current // 2), "high": max(1, current - 1)}.get(pressure, current)


def is_oom_error(e: BaseException) -> bool:
    """CUDA OOM string -> typed check (crates/core/src/cuda/mod.rs:69-96)."""
    return isinstance(e, torch.cuda.OutOfMemoryError) or "out of memory" in str(e).lower()
