"""Fake fabric: an in-process, CPU-only model of the peer-memory communication layer.

The device code in ``csrc/comm.cu`` talks to its peers through three things only: a symmetric
heap every rank can address, a matrix of epoch flags written with release stores and read with
acquire loads, and bounded spin waits that record ``((channel + 1) << 8) | peer`` in a status word
when they run out. This module restates exactly that protocol with threads standing in for GPUs
and host tensors for device memory, so the host-side logic that surrounds the kernels (shard maps,
epoch accounting, status decoding, recovery after a time-out) and the protocol itself can be
tested without a GPU, and so failures can be injected on the host: a dropped flag write, a rank
that is late or never arrives.

It also carries a small explicit-state model checker for the flag barrier (``check_flag_barrier``):
it enumerates every interleaving of the ranks' signal / wait steps over several epochs and checks
that no rank leaves barrier ``e`` before every rank has entered it and that no interleaving
deadlocks, with epochs compared by signed difference as the kernel does.

The reference has no communication layer to test (its gradient synchronisation is a stub,
crates/training/src/distributed.rs:284-319) and no fake backend (its test suite has no
distributed test at all).
"""
from __future__ import annotations

import threading
import time
from collections import deque

import torch

from ..optim.adamw8bit import BLOCK, dequantize_m, dequantize_v, quantize_m, quantize_v

MAX_WORLD = 16
FLAG_CHANNELS = 8


class CommTimeout(RuntimeError):
    """A bounded wait ran out. ``channel`` is the barrier phase, ``peer`` the rank whose flag never
    arrived, ``rank`` the rank that gave up."""

    def __init__(self, rank, status):
        self.rank, self.status = rank, status
        self.channel, self.peer = (status >> 8) - 1, status & 0xFF
        super().__init__(f"rank {rank}: wait on channel {self.channel} for peer {self.peer} timed out")


def decode_status(status: int):
    """Status word of the device kernels -> ``None`` or ``(channel, peer)``."""
    return None if status == 0 else ((status >> 8) - 1, status & 0xFF)


class FakeFabric:
    """``world`` ranks with a symmetric heap each, a flag matrix each and a status word each."""

    def __init__(self, world: int, heap_bytes: int = 1 << 20, wait_s: float = 1.0):
        if not 1 <= world <= MAX_WORLD:
            raise ValueError(f"world must be in 1..{MAX_WORLD}")
        self.world, self.wait_s = world, wait_s
        self.heaps = [torch.zeros(heap_bytes, dtype=torch.uint8) for _ in range(world)]
        self.flags = [[[0] * MAX_WORLD for _ in range(FLAG_CHANNELS)] for _ in range(world)]
        self.status = [0] * world
        self.epoch = [0] * world
        self._off = 0
        self._cv = threading.Condition()
        self._drop = set()       # (src, dst, channel, epoch) flag writes to lose
        self._delay = {}         # rank -> seconds slept before each signal
        self.log = []            # (rank, event, channel, epoch) in observed order

    # ---------------------------------------------------------------- symmetric allocation
    def alloc(self, shape, dtype):
        """One tensor per rank at the same heap offset (what ``SymmetricHeap.tensor`` returns on
        each rank); every rank may read and write every entry."""
        n = 1
        for s in (shape if isinstance(shape, (tuple, list)) else (shape,)):
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        off = (self._off + 255) // 256 * 256
        if off + nb > self.heaps[0].numel():
            raise MemoryError("fake symmetric heap exhausted")
        self._off = off + nb
        return [h[off:off + nb].view(dtype).view(shape) for h in self.heaps]

    # ---------------------------------------------------------------- fault injection (host side)
    def drop_flag(self, src, dst, channel, epoch):
        self._drop.add((src, dst, channel, epoch))

    def delay_rank(self, rank, seconds):
        self._delay[rank] = seconds

    # ---------------------------------------------------------------- the protocol
    def signal(self, rank, channel, epoch):
        d = self._delay.get(rank)
        if d:
            time.sleep(d)
        with self._cv:
            for p in range(self.world):
                if (rank, p, channel, epoch) in self._drop:
                    continue
                self.flags[p][channel][rank] = epoch
            self.log.append((rank, "signal", channel, epoch))
            self._cv.notify_all()

    def wait(self, rank, channel, epoch) -> bool:
        deadline = time.monotonic() + self.wait_s
        with self._cv:
            for p in range(self.world):
                while _sdiff(self.flags[rank][channel][p], epoch) < 0:
                    left = deadline - time.monotonic()
                    if left <= 0:
                        if self.status[rank] == 0:
                            self.status[rank] = ((channel + 1) << 8) | p
                        self.log.append((rank, "timeout", channel, epoch))
                        return False
                    self._cv.wait(left)
            self.log.append((rank, "pass", channel, epoch))
        return True

    def barrier(self, rank, channel, epoch) -> bool:
        self.signal(rank, channel, epoch)
        return self.wait(rank, channel, epoch)

    def read_status(self, rank) -> int:
        v, self.status[rank] = self.status[rank], 0
        return v

    # ---------------------------------------------------------------- running ranks
    def run(self, fn, ranks=None):
        """Run ``fn(FabricRank)`` on one thread per rank; return the list of results. A rank whose
        function raises has its exception returned in its slot (the others keep running, as other
        GPUs would)."""
        ranks = list(range(self.world)) if ranks is None else list(ranks)
        out = [None] * self.world

        def body(r):
            try:
                out[r] = fn(FabricRank(self, r))
            except BaseException as e:      # noqa: BLE001 - surfaced to the caller
                out[r] = e

        ts = [threading.Thread(target=body, args=(r,), daemon=True) for r in ranks]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return out


def _sdiff(a: int, b: int) -> int:
    """Signed 32-bit difference, the comparison the kernels use so epochs may wrap."""
    d = (a - b) & 0xFFFFFFFF
    return d - (1 << 32) if d & 0x80000000 else d


class FabricRank:
    """One rank's view: the pull collectives and the fused data-parallel step, phase by phase as
    the kernels run them."""

    def __init__(self, fabric: FakeFabric, rank: int):
        self.f, self.rank, self.world = fabric, rank, fabric.world

    def _next_epoch(self):
        self.f.epoch[self.rank] += 1
        return self.f.epoch[self.rank]

    def _bar(self, channel, epoch):
        if not self.f.barrier(self.rank, channel, epoch):
            raise CommTimeout(self.rank, self.f.read_status(self.rank))

    # every collective: barrier (inputs ready) -> pull from peers -> barrier (peers done reading)
    def all_gather(self, src, dst):
        e = self._next_epoch()
        self._bar(0, e)
        n = src[self.rank].numel()
        for i in range(self.world):
            p = (self.rank + i) % self.world
            dst.view(-1)[p * n:(p + 1) * n] = src[p].view(-1)
        self._bar(1, e)
        return dst

    def reduce_scatter(self, src, dst, avg=False):
        e = self._next_epoch()
        self._bar(0, e)
        n = src[self.rank].numel() // self.world
        acc = torch.zeros(n, dtype=torch.float32)
        for i in range(self.world):
            p = (self.rank + i) % self.world
            acc += src[p].view(-1)[self.rank * n:(self.rank + 1) * n].float()
        if avg:
            acc /= self.world
        dst.view(-1)[:n] = acc.to(dst.dtype)
        self._bar(1, e)
        return dst

    def all_reduce(self, src, dst, avg=False):
        e = self._next_epoch()
        self._bar(0, e)
        acc = torch.zeros(src[self.rank].numel(), dtype=torch.float32)
        for i in range(self.world):
            acc += src[(self.rank + i) % self.world].view(-1).float()
        if avg:
            acc /= self.world
        dst.view(-1)[:] = acc.to(dst.dtype)
        self._bar(1, e)
        return dst

    def all_to_all(self, src, dst):
        e = self._next_epoch()
        self._bar(0, e)
        n = src[self.rank].numel() // self.world
        for i in range(self.world):
            p = (self.rank + i) % self.world
            dst.view(-1)[p * n:(p + 1) * n] = src[p].view(-1)[self.rank * n:(self.rank + 1) * n]
        self._bar(1, e)
        return dst

    def broadcast(self, src, dst, root=0):
        e = self._next_epoch()
        self._bar(0, e)
        dst.view(-1)[:] = src[root].view(-1)
        self._bar(1, e)
        return dst

    def barrier(self):
        self._bar(0, self._next_epoch())

    # ------------------------------------------------------------ fused data-parallel step
    def fused_dp_step(self, grads, params, sumsq_slots, state, lr, betas=(0.9, 0.999), eps=1e-8,
                      weight_decay=0.01, max_grad_norm=0.0, step=1):
        """The phases of ``fused_dp_step_kernel``: pull-reduce this rank's gradient shard,
        exchange squared norms, clip, 8-bit AdamW on the shard, push the new parameters to every
        rank. ``state`` is a dict with ``m_q, v_q, m_absmax, v_absmax`` for this rank's shard.
        Returns the global gradient norm; a non-finite norm skips the update on every rank."""
        e = self._next_epoch()
        W, r = self.world, self.rank
        n = grads[r].numel() // W
        if n % BLOCK:
            raise ValueError("shard must be a multiple of the quantisation block")
        lo, hi = r * n, (r + 1) * n
        self._bar(0, e)                                  # every rank's gradients are final
        red = torch.zeros(n, dtype=torch.float32)
        for i in range(W):
            red += grads[(r + i) % W].view(-1)[lo:hi].float()
        red /= W
        ss = float((red * red).sum())
        for p in range(W):                               # push my partial norm into every slot table
            sumsq_slots[p].view(-1)[r] = ss
        self._bar(1, e)
        total = float(sumsq_slots[r].view(-1)[:W].sum())
        norm = total ** 0.5
        if total == total and total not in (float("inf"), float("-inf")):
            gs = min(1.0, max_grad_norm / (norm + 1e-6)) if max_grad_norm > 0 else 1.0
            b1, b2 = betas
            g = red * gs
            m = b1 * dequantize_m(state["m_q"], state["m_absmax"]) + (1 - b1) * g
            v = b2 * dequantize_v(state["v_q"], state["v_absmax"]) + (1 - b2) * g * g
            upd = (m / (1 - b1 ** step)) / ((v / (1 - b2 ** step)).sqrt() + eps)
            own = params[r].view(-1)[lo:hi]
            new = (own.float() * (1 - lr * weight_decay) - lr * upd).to(own.dtype)
            state["m_q"], state["m_absmax"] = quantize_m(m)
            state["v_q"], state["v_absmax"] = quantize_v(v)
            for p in range(W):                           # all-gather by push
                params[p].view(-1)[lo:hi] = new
        self._bar(2, e)                                  # every rank's pushes have landed
        return norm


# --------------------------------------------------------------------------------------------
# explicit-state model checker for the flag barrier
# --------------------------------------------------------------------------------------------
def check_flag_barrier(world: int = 2, epochs: int = 2, channels: int = 2, drop=None):
    """Enumerate every interleaving of the barrier protocol and return a report.

    Each rank runs, for epoch 1..epochs and channel 0..channels-1: ``world`` flag stores (one per
    peer, in any order relative to the other ranks' steps) and then a wait for all ``world`` flags
    of that channel to reach the epoch. ``drop`` is an optional set of ``(src, dst, channel, epoch)``
    stores that are lost. Checked: (safety) a rank passes the wait of (epoch, channel) only after
    every rank has begun signalling it; (liveness) every maximal interleaving ends with all ranks
    finished, unless a store was dropped, in which case the ranks that can never pass are
    reported as ``stuck`` (the kernel turns that into a time-out status).
    """
    drop = drop or set()
    prog = [(e, c) for e in range(1, epochs + 1) for c in range(channels)]
    # per-rank program counter: (phase index, stores done 0..world); stores done == world -> waiting
    init = (tuple((0, 0) for _ in range(world)),
            tuple(0 for _ in range(world * channels * world)))     # flags[dst][channel][src]

    def fidx(dst, ch, src):
        return (dst * channels + ch) * world + src

    seen, todo = {init}, deque([init])
    violations, stuck_states, finals = [], set(), 0
    while todo:
        pcs, flags = todo.popleft()
        moved = False
        for r in range(world):
            ph, k = pcs[r]
            if ph == len(prog):
                continue
            e, ch = prog[ph]
            if k < world:                                          # store my epoch into peer k
                nf = list(flags)
                if (r, k, ch, e) not in drop:
                    nf[fidx(k, ch, r)] = e
                nxt = (pcs[:r] + ((ph, k + 1),) + pcs[r + 1:], tuple(nf))
            else:                                                  # wait
                if any(flags[fidx(r, ch, s)] < e for s in range(world)):
                    continue
                for s in range(world):                             # safety: peers have entered (e, ch)
                    if pcs[s][0] < ph:
                        violations.append((r, s, e, ch))
                nxt = (pcs[:r] + ((ph + 1, 0),) + pcs[r + 1:], flags)
            moved = True
            if nxt not in seen:
                seen.add(nxt)
                todo.append(nxt)
        if not moved:
            if all(pc[0] == len(prog) for pc in pcs):
                finals += 1
            else:
                stuck_states.add(tuple(r for r in range(world) if pcs[r][0] < len(prog)))
    return {"states": len(seen), "finals": finals, "violations": violations,
            "stuck": sorted(stuck_states)}
