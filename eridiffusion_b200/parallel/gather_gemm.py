"""Operand gathers fused into the GEMM launch.

``GatherPlan`` describes how an operand is assembled in a local landing buffer from slabs that
live on peer GPUs: a device array of copy jobs (source pointer, destination pointer, rows, row
bytes, strides, slab id) plus one counter per slab. The GEMM launch (``csrc/gemm.cu``) reserves
its first ``n_copy`` CTAs to execute the jobs with bulk copies through shared memory; compute CTAs wait on
the counter of the slab they are about to read and start with this rank's own slab, so the tensor
cores work on data that has landed while the remaining slabs are still crossing NVLink.

Two layouts are provided:
  * ``rows``  — the operand's rows are sharded (ZeRO-3 weight [N, K] sharded along N): slab p =
    rows [p*N/W, (p+1)*N/W). Used as B ([N, K], y = x W^T; waits per output-column tile) or,
    with ``along_k=True``, as the MN-major B of dX = dY W (waits per K block).
  * ``cols``  — the operand's columns come from different peers (Ulysses reverse all-to-all: the
    out-projection input [L_local, H*Dh] takes column block p from peer p's attention output);
    waits per K block.
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import _native as N


class GatherOrder:
    """Order of a step's weight gathers, recorded in one step and followed in the next (ZeRO-3 next-layer
    prefetch). ``begin`` closes a step: what was recorded becomes the expected order. ``advance(key)``
    takes the gather that is about to run and returns the key of the one expected AFTER it, or None when
    the step has left the recorded order, the order ends here, or nothing has been recorded yet."""

    def __init__(self):
        self.seq, self.rec, self.pos, self.follow = [], [], 0, False

    def begin(self, enabled=True):
        if self.rec:
            self.seq = self.rec
        self.rec, self.pos = [], 0
        self.follow = bool(enabled) and bool(self.seq)

    def advance(self, key):
        if self.follow and (self.pos >= len(self.seq) or self.seq[self.pos] != key):
            self.follow = False                       # this step leaves the recorded order
        self.rec.append(key)
        self.pos += 1
        return self.seq[self.pos] if (self.follow and self.pos < len(self.seq)) else None


class GatherPlan:
    def __init__(self, rank: int, world: int, n_copy: int = 16, device=None, n_flags: int | None = None):
        self.rank, self.world, self.n_copy = rank, world, n_copy
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.jobs = []
        self.jobs_nl = []                 # the same jobs without this rank's own slab
        n_flags = n_flags or world
        self.n_slab_flags = n_flags
        # one more counter after the slab counters: every finished job bumps it, so a producer reads
        # "everything has landed" with one load per tile and then skips the per-slab checks
        n_flags += 1
        self.targets = [0] * n_flags
        self.targets_nl = [0] * n_flags
        self.local = None                 # dict(ptr, ld, mode, lo, hi): own slab readable in place
        self.slabs = None                 # [(src, dst, bytes, first counter, counters)] per peer, own first
        self._dev_jobs = None
        self.flags = torch.zeros(n_flags, dtype=torch.int32, device=self.device)
        self._targets_dev = None
        self.kw = {}
        self.remote_bytes = 0

    def _add(self, src, dst, rows, row_bytes, src_stride, dst_stride, flag, remote=True):
        assert row_bytes % 16 == 0 and src % 16 == 0 and dst % 16 == 0
        assert src_stride == row_bytes or row_bytes <= 32 * 1024, "a strided row must fit one copy stage"
        if remote:
            self.remote_bytes += rows * row_bytes
        j = N.GatherJob()
        j.src, j.dst, j.rows, j.row_bytes = src, dst, rows, row_bytes
        j.src_stride, j.dst_stride, j.flag = src_stride, dst_stride, flag
        self.jobs.append(j)
        self.targets[flag] += 1
        self.targets[-1] += 1
        if remote:
            self.jobs_nl.append(j)
            self.targets_nl[flag] += 1
            self.targets_nl[-1] += 1

    @classmethod
    def rows(cls, rank, world, shard_ptrs, landing: torch.Tensor, along_k=False, n_copy=16,
             rows_per_job=64, flag_rows=256, slab_flags=False):
        """landing [N, K]; shard_ptrs[p] -> peer p's [N/W, K] contiguous shard. One counter per
        ``flag_rows`` landing rows, so a tile (or K range) starts as soon as its own rows are
        there instead of waiting for a peer's whole slab."""
        Nn, K = landing.shape
        assert Nn % world == 0
        per = Nn // world
        # (For dX = dY W, where every output tile needs every slab, moving W by 256-wide column blocks in
        # tile order was tried: the 512-byte row pieces copy at a third of the rate of whole slabs, and
        # the emulated 8-rank launch took 511 us against ~360 us. Whole slabs in ring order it is.)
        # A slab that is not a multiple of 256 rows (9216 / 8 = 1152, 3072 / 8 = 384) keeps counters
        # INSIDE the slab at the largest granule that divides it; one counter per whole slab would
        # hold every tile of a slab back until its last byte has landed.
        # Along K (dX = dY W) every tile walks all slabs, and each new counter costs its producer a
        # global load in the middle of the K loop: one counter per whole slab there.
        # ``slab_flags``: one counter per slab in every case (copy-engine prefetch: a whole slab is one copy
        # and every counter costs the host one stream memory write).
        for cand in ((per,) if (along_k or slab_flags) else ()) + (flag_rows, 128, 64):
            if per % cand == 0 and cand % rows_per_job == 0:
                flag_rows = cand
                break
        else:
            if per % rows_per_job == 0 and per >= rows_per_job:
                flag_rows = rows_per_job
            else:
                flag_rows = per
        pl = cls(rank, world, n_copy, landing.device, n_flags=Nn // flag_rows)
        rb = K * landing.element_size()
        # Slab after slab in ring order from this rank's own: the GEMM walks its tiles (or its K ranges)
        # in the same order, so the copy CTAs fill the slab that is needed next instead of all slabs a
        # little. (Interleaving the peers row group by row group made the LAST rows of the next slab land
        # at the very end of the gather: every producer then waited ~70 % of the copy time in total.)
        order = [(rank + i) % world for i in range(world)]
        for p in order:
            r0 = 0
            while r0 < per:
                nr = min(rows_per_job, per - r0)
                pl._add(shard_ptrs[p] + r0 * rb, landing.data_ptr() + (p * per + r0) * landing.stride(0) * landing.element_size(),
                        nr, rb, rb, landing.stride(0) * landing.element_size(), (p * per + r0) // flag_rows, remote=p != rank)
                r0 += nr
        # The rotation only says where the tile / K order starts; it is a whole number of 256-column
        # pair tiles / 64-wide K blocks so that the two-CTA kernel accepts the plan on every rank,
        # whatever the slab size. It is rounded UP into this rank's own slab: rounded down, the first
        # tile would begin in the previous rank's slab, which is the LAST one the copy CTAs fill, and
        # every producer would sit out the whole gather before its first load.
        if along_k:
            pl.kw = dict(a_flag_cols=flag_rows, rot_k_cols=(-(-(rank * per) // 64) * 64) % Nn)
        else:
            pl.kw = dict(b_flag_rows=flag_rows, rot_n_rows=(-(-(rank * per) // 256) * 256) % Nn)
        # whole slabs in the same order, for the copy-engine variant of the gather
        sb = per * rb
        pl.slabs = [(shard_ptrs[p], landing.data_ptr() + p * per * landing.stride(0) * landing.element_size(), sb,
                     p * per // flag_rows, per // flag_rows) for p in order] \
            if landing.stride(0) == K else None
        # the own shard can feed the GEMM in place (second tensor map) when the kernel supports it
        pl.local = dict(ptr=shard_ptrs[rank], ld=K, mode=2 if along_k else 1, lo=rank * per, hi=(rank + 1) * per)
        return pl._finish()

    @classmethod
    def cols(cls, rank, world, src_ptrs, src_row_offset, src_stride_bytes, landing: torch.Tensor,
             n_copy=16, rows_per_job=128):
        """landing [L, W*C]: column block p <- peer p's rows [src_row_offset, +L) of a [*, C]
        matrix with row stride ``src_stride_bytes``."""
        L, WC = landing.shape
        Cc = WC // world
        es = landing.element_size()
        groups = (L + rows_per_job - 1) // rows_per_job
        pl = cls(rank, world, n_copy, landing.device, n_flags=world * groups)
        order = [(rank + i) % world for i in range(world)]
        r0 = 0
        while r0 < L:
            nr = min(rows_per_job, L - r0)
            for p in order:
                pl._add(src_ptrs[p] + (src_row_offset + r0) * src_stride_bytes,
                        landing.data_ptr() + (r0 * landing.stride(0) + p * Cc) * es,
                        nr, Cc * es, src_stride_bytes, landing.stride(0) * es, p * groups + r0 // rows_per_job, remote=p != rank)
            r0 += nr
        # one counter per (column block, 128-row group): a tile waits for its own rows only
        pl.kw = dict(a_flag_cols=Cc, rot_k_cols=rank * Cc, a_flag_rows=rows_per_job)
        # this rank's own column block can be read where it lives (mode 3: K range of the A operand)
        pl.local = dict(ptr=src_ptrs[rank] + src_row_offset * src_stride_bytes, ld=src_stride_bytes // es,
                        mode=3, lo=rank * Cc, hi=(rank + 1) * Cc)
        return pl._finish()

    def _finish(self):
        arr = (N.GatherJob * len(self.jobs))(*self.jobs)
        raw = bytes(arr)
        self._dev_jobs = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(self.device)
        self._targets_dev = torch.tensor(self.targets, dtype=torch.int32, device=self.device)
        if self.local is not None and self.jobs_nl:
            arr = (N.GatherJob * len(self.jobs_nl))(*self.jobs_nl)
            self._dev_jobs_nl = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(self.device)
            self._targets_nl_dev = torch.tensor(self.targets_nl, dtype=torch.int32, device=self.device)
        else:
            self.local = None
        return self

    def launch_args(self):
        """Zero the slab counters (stream-ordered) and return the ``gather=`` dict for
        ``ops.functional.gemm_native``."""
        self.flags.zero_()
        d = dict(n_copy=self.n_copy, n_jobs=len(self.jobs), jobs=self._dev_jobs.data_ptr(),
                 flags=self.flags.data_ptr(), flag_target=self._targets_dev.data_ptr(),
                 copy_bytes=self.remote_bytes, all_flag=self.n_slab_flags + 1, **self.kw)
        if self.local is not None:
            d["local"] = dict(self.local, n_jobs=len(self.jobs_nl), jobs=self._dev_jobs_nl.data_ptr(),
                              flag_target=self._targets_nl_dev.data_ptr())
        return d

    def launch_args_engine(self, side_stream):
        """Copy-engine variant: every slab is one asynchronous device-to-device copy on
        ``side_stream`` followed by stream memory writes that set the slab's counters to their
        targets; the GEMM launch then has no copy CTAs (``n_copy`` 0) and only waits on the counters.
        Peer reads by the copy engines run at link rate, where copy CTAs pulling with bulk copies
        saturate near 200 GB/s per GPU however many CTAs pull."""
        if self.slabs is None:
            return self.launch_args()
        lib = N.require()
        if not hasattr(lib.eri_peer_copy_flags, "_bound"):
            lib.eri_peer_copy_flags.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_int,
                                                C.c_uint, C.c_void_p]
            lib.eri_peer_copy_flags.restype = C.c_int
            lib.eri_peer_copy_flags._bound = True
        self.flags.zero_()
        ev = torch.cuda.Event()
        ev.record()                       # counters are zero and the landing buffer's last reader is done
        side_stream.wait_event(ev)
        for src, dst, nbytes, f0, nfl in self.slabs:
            code = lib.eri_peer_copy_flags(dst, src, nbytes, self.flags.data_ptr() + 4 * f0, nfl,
                                           self.targets[f0], side_stream.cuda_stream)
            if code:
                raise RuntimeError(f"copy-engine gather failed with code {code}")
        return dict(n_copy=0, n_jobs=0, jobs=0, flags=self.flags.data_ptr(),
                    flag_target=self._targets_dev.data_ptr(), **self.kw)

    def issue_engine(self, side_stream):
        """Copy-engine gather on ``side_stream``: counters zeroed, one asynchronous copy per slab in ring
        order followed by stream memory writes that set the slab's counters, then the "everything has
        landed" counter. The caller orders ``side_stream`` behind the landing buffer's last reader."""
        lib = N.require()
        if not hasattr(lib.eri_peer_copy_flags, "_bound"):
            lib.eri_peer_copy_flags.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_int,
                                                C.c_uint, C.c_void_p]
            lib.eri_peer_copy_flags.restype = C.c_int
            lib.eri_peer_copy_flags._bound = True
        with torch.cuda.stream(side_stream):
            self.flags.zero_()
        jobs = list(self.slabs) + [(0, 0, 0, self.n_slab_flags, 1)]
        for src, dst, nbytes, f0, nfl in jobs:
            code = lib.eri_peer_copy_flags(dst, src, nbytes, self.flags.data_ptr() + 4 * f0, nfl,
                                           self.targets[f0], side_stream.cuda_stream)
            if code:
                raise RuntimeError(f"copy-engine gather failed with code {code}")

    def engine_args(self):
        """``gather=`` dict of a launch whose slabs were (or are being) delivered by ``issue_engine``: no
        copy CTAs, the tiles only look at the counters."""
        return dict(n_copy=0, n_jobs=0, jobs=0, flags=self.flags.data_ptr(),
                    flag_target=self._targets_dev.data_ptr(), all_flag=self.n_slab_flags + 1, **self.kw)

    def bytes_from_peers(self):
        return self.remote_bytes
