"""ZeRO-3 style parameter sharding with the all-gather fused into the consuming GEMM.

Every large ``Linear`` keeps only rows ``[rank*N/W, (rank+1)*N/W)`` of its weight, stored in
symmetric (peer-mapped) memory. Nothing is gathered ahead of time:

* forward  ``y = x W^T``: one launch of the tcgen05 GEMM whose first CTAs pull the peers' row
  slabs into a local landing buffer while the compute CTAs start on this rank's own slab and wait
  per output-column tile on the slab counters (``GatherPlan.rows``);
* backward ``dX = dY W``: the same landing data is the MN-major B operand, gathered again along
  the reduction dimension (``along_k=True``), no transposed copy;
* ``dW``: the weight-gradient GEMM (tcgen05, both activations token-major) pushes every row slab of
  its result straight into the owning rank's receive buffer from its epilogue (row-slab peer
  scatter: the reduce-scatter's transfer runs tile by tile under the GEMM), one in-kernel barrier
  later the owner adds the ``world`` slots (``eri_slot_reduce``); no NCCL, no staging pass.
  ``ERI_B200_ZERO3_FUSED_RS=0`` restores the staged form (local GEMM, then a pull-based
  reduce-scatter kernel);
* conditioning-vector linears (adaLN modulation) are sharded too: every rank applies its row
  slab to the vectors of all ranks (tiny all-gather in, all-to-all out), so a third of a
  Qwen-Image block's weights never crosses NVLink at all.

The single-GPU analogue in the reference is weight streaming
(``WeightProvider::{load_block_to_gpu, prefetch_block, release_block}``,
crates/training/src/streaming.rs:12-17): materialise -> run -> release per block.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.layers import Linear, SmallLinear
from ..ops import functional as F
from ..ops import reference as R
from .dist import ProcessGroup, ReduceOp
from .gather_gemm import GatherOrder, GatherPlan
from .symm import Communicator, SymmetricHeap


class Zero3Context:
    def __init__(self, pg: ProcessGroup | None = None, heap_bytes: int = 1 << 30,
                 max_weight_elems: int = 64 << 20, n_copy: int = 16, wait_ms: float = 2000.0):
        self.pg = pg or ProcessGroup()
        self.rank, self.world = self.pg.rank, self.pg.world_size
        # symmetric memory: parameter shards (heap_bytes), the dW staging buffer and two receive
        # buffers of the fused weight-gradient reduce-scatter (alternating by layer)
        self.stamps = None
        self.fused_rs = os.environ.get("ERI_B200_ZERO3_FUSED_RS", "1") == "1"
        self.heap = SymmetricHeap(heap_bytes + max_weight_elems * 2 * (3 if self.fused_rs else 1) + (4 << 20),
                                  group=self.pg.group)
        self.comm = Communicator(self.heap, wait_ms)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.landing = [torch.empty(max_weight_elems, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.stage = self.heap.tensor((max_weight_elems,), torch.bfloat16)
        # scratch of the conditioning-vector collectives (modulation linears): 256 K elements each
        self.native_small = os.environ.get("ERI_B200_ZERO3_MOD", "native") != "nccl"
        self.small_bf16 = self.heap.tensor((1 << 18,), torch.bfloat16)
        self.small_f32 = self.heap.tensor((1 << 18,), torch.float32)
        self.recv = [self.heap.tensor((max_weight_elems,), torch.bfloat16) for _ in range(2)] if self.fused_rs else []
        self._recv_flip = 0
        self.n_copy = n_copy
        # "sm": copy CTAs inside the GEMM launch pull the slabs; "ce": the copy engines do, on a side
        # stream, and the GEMM only waits on the landing counters (ERI_B200_ZERO3_GATHER overrides)
        self.gather_engine = os.environ.get("ERI_B200_ZERO3_GATHER", "sm")
        self.copy_stream = torch.cuda.Stream(device=dev) if self.gather_engine == "ce" else None
        self._flip = 0
        self._plans = {}
        self.gathered_bytes = 0
        # Next-layer prefetch: the order of the gathers of a step is recorded; from the second step on,
        # while layer i's GEMM runs, the copy engines pull layer i + 1's slabs into the other landing
        # buffer on a side stream, so that launch i + 1 has no copy CTAs and finds its counters set.
        self.prefetch = os.environ.get("ERI_B200_ZERO3_PREFETCH", "1") == "1" and self.world > 1
        self.prefetch_stream = torch.cuda.Stream(device=dev) if self.prefetch else None
        self._order = GatherOrder()
        self._pf = self._pf_done = None
        self.prefetched_launches = 0

    # allocator handed to ParamArena so that the shards live in peer-mapped memory
    def arena_alloc(self, n, dtype, device):
        return self.heap.tensor((n,), dtype).local

    def peer_ptrs_of(self, t: torch.Tensor):
        off = t.data_ptr() - self.heap.local_ptr
        assert 0 <= off < self.heap.nbytes, "tensor is not inside the symmetric heap"
        return [p + off for p in self.heap.peer_ptrs]

    def next_landing(self, n, k):
        if n * k > self.landing[0].numel():
            raise ValueError(f"a [{n}, {k}] weight does not fit the landing buffers "
                             f"(max_weight_elems={self.landing[0].numel()}): raise it in Zero3Context")
        i = self._flip
        self._flip ^= 1
        return self.landing[i][: n * k].view(n, k), i

    def begin_step(self):
        """Marks the start of a step (forward + backward between two optimizer updates). The gathers of
        the step that just ended become the order that the next one is expected to follow; nothing is
        ever prefetched across this call, because the shards change under the optimizer."""
        self._drain_prefetch()
        self._flip = 0
        self._order.begin(self.prefetch)

    def _drain_prefetch(self):
        if self._pf is not None:
            # a prefetch nobody consumed still writes a landing buffer: the current stream waits for it
            torch.cuda.current_stream().wait_event(self._pf_done)
            self._pf = None

    def _issue_prefetch(self, key, li):
        ptr, n, k, along_k = key
        pk = (key, li, "engine")
        pl = self._plans.get(pk)
        if pl is None:
            off = ptr - self.heap.local_ptr
            landing = self.landing[li][: n * k].view(n, k)
            pl = GatherPlan.rows(self.rank, self.world, [p + off for p in self.heap.peer_ptrs], landing,
                                 along_k=along_k, n_copy=self.n_copy, slab_flags=True)
            self._plans[pk] = pl
        # the other landing buffer's last reader is the GEMM launched before the current one: both are
        # already on this stream, the copies start behind the earlier one
        ev = torch.cuda.Event()
        ev.record()
        self.prefetch_stream.wait_event(ev)
        pl.issue_engine(self.prefetch_stream)
        self._pf_done = torch.cuda.Event()
        self._pf_done.record(self.prefetch_stream)
        self._pf = (key, li, pl)

    def plan(self, shard: torch.Tensor, n, k, along_k: bool):
        landing, li = self.next_landing(n, k)
        skey = (shard.data_ptr(), n, k, along_k)
        ready = None
        if self._pf is not None:
            if self._pf[0] == skey and self._pf[1] == li:
                ready, self._pf = self._pf[2], None
            else:
                self._drain_prefetch()
        nxt = self._order.advance(skey)
        if nxt is not None:
            self._issue_prefetch(nxt, li ^ 1)
        if ready is not None:
            self.gathered_bytes += ready.bytes_from_peers()
            self.prefetched_launches += 1
            ready.prefetched = True
            return ready, landing
        key = (shard.data_ptr(), n, k, along_k, li)
        pl = self._plans.get(key)
        if pl is None:
            # A weight with few output tiles (N <= 4096: at most 16 column tiles) is needed almost
            # whole by the first wave of tiles, so the gather has to finish early: twice the copy CTAs
            # (emulated 8-rank launch of [4608 x 12288] x [3072 x 12288]^T: compute done at 317 us
            # against 360 us).
            # The input-gradient GEMM (along_k) needs every slab in each tile, so its first wave runs at
            # the speed of the gather: twice the copy CTAs there as well (316 against 355 us emulated).
            n_copy = self.n_copy * 2 if ((along_k or n <= 4096) and self.n_copy <= 16) else self.n_copy
            pl = GatherPlan.rows(self.rank, self.world, self.peer_ptrs_of(shard), landing,
                                 along_k=along_k, n_copy=n_copy)
            self._plans[key] = pl
        self.gathered_bytes += pl.bytes_from_peers()
        return pl, landing

    def next_recv(self):
        """Receive buffer of the next fused weight-gradient reduce-scatter. Two alternate: a fast
        peer may already push layer l + 1's slabs while this rank still adds up layer l's (it cannot
        be two layers ahead: it has to pass layer l + 1's barrier, which this rank enters only after
        its reduction of layer l)."""
        r = self.recv[self._recv_flip]
        self._recv_flip ^= 1
        return r

    def gather_args(self, pl):
        if getattr(pl, "prefetched", False):
            return pl.engine_args()
        if self.copy_stream is not None:
            return pl.launch_args_engine(self.copy_stream)
        args = pl.launch_args()
        if self.stamps is not None:
            # phase record of the next gather launch: [0] is a minimum, so it starts at all ones
            self.stamps.zero_()
            self.stamps[0] = -1
            args = dict(args, stamps=self.stamps)
        return args

    def phase_times_us(self):
        """Phases of the last gather-fused launch recorded with ``stamps`` (a device int64[8] tensor
        assigned by the caller), in microseconds from the first CTA's start."""
        s = self.stamps.tolist()
        t0 = s[0]
        return {"all_slabs_landed": (s[1] - t0) / 1e3, "last_compute_cta_done": (s[2] - t0) / 1e3,
                "producers_that_waited": s[5], "mean_wait_of_those": (s[3] / s[5] / 1e3) if s[5] else 0.0,
                "longest_wait": s[4] / 1e3}

    def small_collective(self, op: str, src: torch.Tensor, dst: torch.Tensor, count: int) -> bool:
        """``op`` (all_gather / all_to_all / reduce_scatter) on a conditioning-vector sized bf16 / fp32
        tensor through the symmetric heap's collective kernel (flag barrier, peer loads, flag barrier:
        one launch, no NCCL). Returns False when the tensor does not fit the scratch buffer or the
        native path is switched off (``ERI_B200_ZERO3_MOD=nccl``); the caller then uses NCCL."""
        if not self.native_small or src.dtype not in (torch.bfloat16, torch.float32):
            return False
        buf = self.small_bf16 if src.dtype == torch.bfloat16 else self.small_f32
        n = src.numel()
        if n > buf.local.numel() or not dst.is_contiguous() or dst.dtype != src.dtype or \
                (count * src.element_size()) % 16 or dst.data_ptr() % 16:
            return False
        buf.local[:n].copy_(src.reshape(-1))
        self.comm.collective(op, buf, dst=dst, count=count)
        return True

    def barrier(self):
        """Cross-GPU barrier on the current stream (a kernel; no host synchronisation)."""
        if self.world > 1:
            self.comm.collective("barrier", self.stage, count=0)


class _Zero3LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shard, bias, z3, n_out, act, residual, gate):
        shp = x.shape
        K = shp[-1]
        x2 = x.contiguous().view(-1, K)
        M = x2.shape[0]
        L = shp[-2]
        pl, landing = z3.plan(shard, n_out, K, along_k=False)
        pre = torch.empty(M, n_out, dtype=x.dtype, device=x.device) if act is not None else None
        res2 = None if residual is None else residual.contiguous().view(-1, n_out)
        gate_v = None
        if gate is not None:
            gate_v, _ = F._mod_view(gate, n_out)
        y = F.gemm_native(x2, landing, bias=bias, act=act, pre_out=pre, residual=res2, gate=gate_v,
                          rows_per_batch=L, gather=z3.gather_args(pl))
        ctx.save_for_backward(x2, shard, pre, gate_v)
        ctx.meta = (shp, n_out, L, act, residual is not None, bias is not None)
        ctx.z3 = z3
        return y.view(*shp[:-1], n_out)

    @staticmethod
    def backward(ctx, dy):
        x2, shard, pre, gate_v = ctx.saved_tensors
        shp, n_out, L, act, has_res, has_bias = ctx.meta
        z3 = ctx.z3
        M, K = x2.shape
        dy2 = dy.contiguous().view(M, n_out)
        d_res = dy.reshape(*shp[:-1], n_out) if has_res else None
        if gate_v is not None:
            dy2 = F.gate_residual(None, dy2.view(-1, L, n_out), gate_v).view(M, n_out)
        if act is not None:
            g = torch.empty_like(dy2)
            F.N.check(F.N.require().eri_act_bwd(dy2.data_ptr(), pre.data_ptr(), g.data_ptr(),
                                                dy2.numel(), 0 if act == "gelu" else 1,
                                                F.N.stream_ptr()), "act_bwd")
            dy2 = g
        dx = None
        if ctx.needs_input_grad[0]:
            pl, landing = z3.plan(shard, n_out, K, along_k=True)
            dx = F.gemm_native(dy2, landing, b_mn=True, gather=z3.gather_args(pl)).view(shp)
        dshard = None
        if ctx.needs_input_grad[1]:
            per = n_out // z3.world
            fused = (z3.world > 1 and z3.fused_rs and n_out >= 256 and K >= 256 and M >= 64 and K % 8 == 0
                     and n_out % 8 == 0 and F._wgrad_ok(dy2, x2))
            if fused:
                # every rank's partial slab for rank d lands in slot `rank` of d's receive buffer while
                # the GEMM is still running; one barrier, then the owner adds the slots
                recv = z3.next_recv()
                F.gemm_native(dy2, x2, a_mn=True, b_mn=True, out=recv.local[: n_out * K].view(n_out, K),
                              scatter=dict(world=z3.world, rank=z3.rank, mode=1, local_rows=per, part_cols=0,
                                           group_cols=0, ptrs=recv.peer_ptrs))
                z3.barrier()
                dshard = torch.empty(per, K, dtype=dy2.dtype, device=dy2.device)
                F.N.check(F.N.require().eri_slot_reduce(recv.local.data_ptr(), dshard.data_ptr(), z3.world, per * K,
                                                        1.0 / z3.world, 0, F.N.stream_ptr()), "slot_reduce")
            else:
                stage = z3.stage.local[: n_out * K].view(n_out, K)
                F.wgrad(dy2, x2, out=stage)
                if z3.world > 1:
                    dshard = torch.empty(per, K, dtype=dy2.dtype, device=dy2.device)
                    z3.comm.collective("reduce_scatter", z3.stage, dst=dshard, count=per * K, avg=True)
                else:
                    dshard = stage.clone()
        dbias = dy2.sum(0) if (has_bias and ctx.needs_input_grad[2]) else None
        return dx, dshard, dbias, None, None, None, d_res, None


class Zero3Linear(nn.Module):
    def __init__(self, lin: Linear, z3: Zero3Context):
        super().__init__()
        self.in_features, self.out_features = lin.in_features, lin.out_features
        per = lin.out_features // z3.world
        self.weight = nn.Parameter(lin.weight.detach()[z3.rank * per:(z3.rank + 1) * per].clone())
        self.bias = lin.bias
        self.z3 = z3
        self.adapter = None

    def forward(self, x, act=None, residual=None, gate=None):
        if gate is not None and gate.requires_grad:
            y = _Zero3LinearFn.apply(x, self.weight, self.bias, self.z3, self.out_features, act, None, None)
            return F.gate_residual(residual, y, gate)
        return _Zero3LinearFn.apply(x, self.weight, self.bias, self.z3, self.out_features, act,
                                    residual, gate)


class _Zero3SmallFn(torch.autograd.Function):
    """Row-sharded linear on conditioning vectors: all ranks' vectors visit every shard."""

    @staticmethod
    def forward(ctx, x, shard, bias_shard, z3, silu_in):
        W = z3.world
        B, K = x.shape
        xs = torch.empty(W * B, K, dtype=x.dtype, device=x.device)
        if W > 1:
            if not z3.small_collective("all_gather", x, xs, B * K):
                dist.all_gather_into_tensor(xs, x.contiguous(), group=z3.pg.group)
        else:
            xs.copy_(x)
        ys = F.small_linear(xs, shard, bias_shard, silu_in=silu_in) if W * B <= 8 else \
            torch.nn.functional.linear(torch.nn.functional.silu(xs) if silu_in else xs, shard, bias_shard)
        per = shard.shape[0]
        out = torch.empty(W, B, per, dtype=x.dtype, device=x.device)
        if W > 1:
            if not z3.small_collective("all_to_all", ys, out, B * per):
                dist.all_to_all_single(out, ys.view(W, B, per).contiguous(), group=z3.pg.group)
        else:
            out.copy_(ys.view(W, B, per))
        ctx.save_for_backward(xs, shard)
        ctx.meta = (W, B, K, per, silu_in, bias_shard is not None)
        ctx.z3 = z3
        return out.permute(1, 0, 2).reshape(B, W * per)

    @staticmethod
    def backward(ctx, dy):
        xs, shard = ctx.saved_tensors
        W, B, K, per, silu_in, has_bias = ctx.meta
        z3 = ctx.z3
        dyw = dy.reshape(B, W, per).permute(1, 0, 2).contiguous()
        dys = torch.empty_like(dyw)
        if W > 1:
            if not z3.small_collective("all_to_all", dyw, dys, B * per):
                dist.all_to_all_single(dys, dyw, group=z3.pg.group)
        else:
            dys.copy_(dyw)
        dys = dys.view(W * B, per)
        xin = torch.nn.functional.silu(xs.float()).to(xs.dtype) if silu_in else xs
        dshard = F.small_wgrad(dys, xin, 1.0 / W) if ctx.needs_input_grad[1] else None   # already summed over ranks
        dbias = dys.sum(0) / W if (has_bias and ctx.needs_input_grad[2]) else None
        dx = None
        if ctx.needs_input_grad[0]:
            dxs = F.small_dgrad(dys, shard)
            if silu_in:
                xf = xs.float()
                sg = torch.sigmoid(xf)
                dxs = (dxs.float() * (sg * (1 + xf * (1 - sg)))).to(xs.dtype)
            dx = torch.empty(B, K, dtype=dxs.dtype, device=dxs.device)
            if W > 1:
                if not z3.small_collective("reduce_scatter", dxs, dx, B * K):
                    dist.reduce_scatter_tensor(dx, dxs.contiguous(), group=z3.pg.group)
            else:
                dx.copy_(dxs)
        return dx, dshard, dbias, None, None


class Zero3SmallLinear(nn.Module):
    def __init__(self, lin: SmallLinear, z3: Zero3Context):
        super().__init__()
        per = lin.out_features // z3.world
        sl = slice(z3.rank * per, (z3.rank + 1) * per)
        self.weight = nn.Parameter(lin.weight.detach()[sl].clone())
        self.bias = nn.Parameter(lin.bias.detach()[sl].clone()) if lin.bias is not None else None
        self.z3 = z3
        self.in_features, self.out_features = lin.in_features, lin.out_features

    def forward(self, x, silu_in=False):
        shp = x.shape
        y = _Zero3SmallFn.apply(x.reshape(-1, shp[-1]), self.weight, self.bias, self.z3, silu_in)
        return y.view(*shp[:-1], self.out_features)


def shard_model(model: nn.Module, z3: Zero3Context, min_numel: int = 1 << 16):
    """Replace every large Linear / SmallLinear of ``model`` by its row-sharded version.
    Returns (sharded parameter list, replicated parameter list), shards first."""
    W = z3.world
    for name, mod in list(model.named_modules()):
        for cname, child in list(mod.named_children()):
            if isinstance(child, SmallLinear):
                if child.weight.numel() >= min_numel and child.out_features % W == 0:
                    setattr(mod, cname, Zero3SmallLinear(child, z3))
            elif isinstance(child, Linear):
                if (child.weight.numel() >= min_numel and child.out_features % (W * 64) == 0
                        and child.in_features % 64 == 0 and child.adapter is None):
                    setattr(mod, cname, Zero3Linear(child, z3))
    sharded, replicated = [], []
    for mod in model.modules():
        if isinstance(mod, (Zero3Linear, Zero3SmallLinear)):
            sharded.append(mod.weight)
            if isinstance(mod, Zero3SmallLinear) and mod.bias is not None:
                sharded.append(mod.bias)
    ids = {id(p) for p in sharded}
    replicated = [p for p in model.parameters() if id(p) not in ids and p.requires_grad]
    return sharded, replicated


class Zero3Sync:
    """``grad_sync`` object for ``Trainer`` in ZeRO-3 mode: shards are updated locally, replicated
    parameters (norm scales, biases, small embedders) get an averaged gradient."""

    fused_optimizer = False
    mode = "zero3"

    def __init__(self, z3: Zero3Context, sharded, replicated):
        self.z3, self.pg = z3, z3.pg
        self.rank, self.world_size = z3.rank, z3.world
        self.sharded, self.replicated = sharded, replicated
        self.arena = self.optimizer = None
        self.n_shard = 0

    arena_alloc = property(lambda self: self.z3.arena_alloc)

    def ordered_params(self):
        return list(self.sharded) + list(self.replicated)

    def optimizer_shard(self):
        return None

    def attach(self, arena, optimizer):
        self.arena, self.optimizer = arena, optimizer
        k = len(self.sharded)
        self.n_shard = arena.offsets[k] if k < len(arena.offsets) else arena.numel
        if self.world_size > 1 and self.n_shard < arena.numel:
            self.pg.broadcast(arena.data[self.n_shard:], 0)
        self.z3.barrier()
        self.z3.begin_step()

    def reduce_grads(self):
        if self.world_size > 1 and self.n_shard < self.arena.numel:
            self.pg.all_reduce(self.arena.grad[self.n_shard:], ReduceOp.AVG)
        self.z3.barrier()          # every rank has finished gathering for its backward

    def grad_sumsq(self, out=None):
        g = self.arena.grad
        ss = F.sumsq(g[: self.n_shard]) if self.n_shard else torch.zeros((), device=g.device)
        if self.world_size > 1:
            self.pg.all_reduce(ss, ReduceOp.SUM)
        if self.n_shard < g.numel():
            ss = ss + F.sumsq(g[self.n_shard:])
        if out is not None:
            out.copy_(ss)
            return out
        return ss

    def gather_params(self):
        self.z3.barrier()          # all shards updated before anyone gathers for the next forward
        self.z3.begin_step()
