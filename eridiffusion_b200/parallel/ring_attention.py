"""Context parallelism: ring attention over the ranks of a process group.

Every rank holds a contiguous slice of the sequence for Q, K and V (``[B, L/P, H, Dh]``). The
key / value slices travel once around the ring; at each of the ``P`` steps a rank attends its own
queries to the slice it currently holds and folds the partial result into a running
``(out, lse)`` pair with the log-sum-exp merge

    lse' = logaddexp(lse_a, lse_b);   out' = out_a * exp(lse_a - lse') + out_b * exp(lse_b - lse')

which is the same online-softmax recurrence the reference runs over key chunks on ONE device
(``sdpa_chunked_bf16``, crates/training/src/sdxl/runtime.rs:2814-3025, running max / sum /
rescale at :2958-2997; ``streaming_attn_bf16_fp32``, crates/training/src/flux/runtime.rs:707-745).
The reference has no cross-device form of it; this module is the multi-GPU extension of that
mechanism for sequences that do not fit one GPU even with Ulysses (whose degree is bounded by the
number of heads).

The per-slice products run on the tcgen05 flash-attention kernels when they apply (bf16, head size
64 / 128, slices of at least 128 tokens): the forward kernel already returns the log-sum-exp, and
the backward kernels take the FINAL ``out`` / ``lse`` so that each slice's call yields exactly its
share of ``dQ`` and the complete ``dK`` / ``dV`` of that slice. Otherwise the same statements run
in fp32 PyTorch (CPU ranks under gloo, odd shapes).

The transfer of step ``s + 1``'s slice is posted (``batch_isend_irecv``) before step ``s``'s
product is launched, so on NCCL it overlaps the kernels. In the backward the keys / values are
forwarded the same way (in their own dtype) and the slice's fp32 gradient accumulator follows after
the step's products; it is home again after ``P`` hops. Non-causal attention has equal work
per slice, so no zig-zag reordering is needed.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist


# ---------------------------------------------------------------------------- one slice
def _use_native(q, k, v):
    if not q.is_cuda or q.dtype != torch.bfloat16:
        return False
    from ..ops import flash_attn as FA
    return FA.supported(q, k, v) and FA.has_backward()


def block_forward(q, k, v, scale):
    """Attention of ``q`` against one key / value slice. Returns (out fp32 ``[B, Lq, H, Dh]``,
    lse fp32 ``[B, H, Lq]``)."""
    if _use_native(q, k, v):
        from ..ops import flash_attn as FA
        o, lse = FA.fwd(q, k, v, scale)
        return o.float(), lse
    s = torch.einsum("blhd,bmhd->bhlm", q.float(), k.float()) * scale
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    return torch.einsum("bhlm,bmhd->blhd", p, v.float()), lse


def block_backward(do, q, k, v, out, lse, scale):
    """Gradient share of one slice given the final ``out`` / ``lse`` of the whole sequence:
    ``P = exp(S - lse)``, ``dV = P^T dO``, ``dS = P * (dO V^T - rowsum(dO * out))``,
    ``dQ = dS K * scale``, ``dK = dS^T Q * scale``. Returns fp32 tensors."""
    if _use_native(q, k, v):
        from ..ops import flash_attn as FA
        dq, dk, dv = FA.bwd(do.to(q.dtype).contiguous(), q, k, v, out.to(q.dtype).contiguous(),
                            lse.contiguous(), scale)
        return dq.float(), dk.float(), dv.float()
    qf, kf, vf, dof = q.float(), k.float(), v.float(), do.float()
    s = torch.einsum("blhd,bmhd->bhlm", qf, kf) * scale
    p = torch.exp(s - lse.unsqueeze(-1))
    dv = torch.einsum("bhlm,blhd->bmhd", p, dof)
    dp = torch.einsum("blhd,bmhd->bhlm", dof, vf)
    delta = (dof * out.float()).sum(-1).permute(0, 2, 1)                  # [B, H, Lq]
    ds = p * (dp - delta.unsqueeze(-1)) * scale
    return torch.einsum("bhlm,bmhd->blhd", ds, kf), torch.einsum("bhlm,blhd->bmhd", ds, qf), dv


def merge(out_a, lse_a, out_b, lse_b):
    """Fold two partial attention results over disjoint key sets into one."""
    lse = torch.logaddexp(lse_a, lse_b)
    wa = torch.exp(lse_a - lse).permute(0, 2, 1).unsqueeze(-1)            # [B, Lq, H, 1]
    wb = torch.exp(lse_b - lse).permute(0, 2, 1).unsqueeze(-1)
    return out_a * wa + out_b * wb, lse


# ---------------------------------------------------------------------------- the ring
def _rotate(buf, group, rank, world):
    """Post send-to-next / receive-from-previous of ``buf``; returns (requests, landing buffer)."""
    nxt = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
    prv = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
    land = torch.empty_like(buf)
    ops = [dist.P2POp(dist.isend, buf, nxt, group), dist.P2POp(dist.irecv, land, prv, group)]
    return dist.batch_isend_irecv(ops), land


def _wait(reqs):
    for r in reqs:
        r.wait()


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, group):
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        kv = torch.stack((k, v))                                          # one message per hop
        out = lse = None
        for s in range(world):
            reqs = land = None
            if s + 1 < world:
                reqs, land = _rotate(kv, group, rank, world)
            o_s, lse_s = block_forward(q, kv[0], kv[1], scale)
            out, lse = (o_s, lse_s) if out is None else merge(out, lse, o_s, lse_s)
            if reqs is not None:
                _wait(reqs)
                kv = land
        out_t = out.to(q.dtype).contiguous()
        ctx.save_for_backward(q, k, v, out_t, lse)
        ctx.scale, ctx.group = scale, group
        return out_t

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        group, scale = ctx.group, ctx.scale
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        do = do.contiguous()
        dq = torch.zeros_like(q, dtype=torch.float32)
        # keys / values travel in their own dtype and are forwarded BEFORE this step's products (the
        # next rank needs them one step later), so that transfer overlaps the kernels; the fp32
        # gradient accumulator of the slice follows after the products and is home after P hops
        kv = torch.stack((k, v))
        dkv = torch.zeros_like(kv, dtype=torch.float32)
        for s in range(world):
            kv_reqs = kv_land = None
            if s + 1 < world:
                kv_reqs, kv_land = _rotate(kv, group, rank, world)
            dq_s, dk_s, dv_s = block_backward(do, q, kv[0], kv[1], out, lse, scale)
            dq += dq_s
            dkv[0] += dk_s
            dkv[1] += dv_s
            reqs, land = _rotate(dkv, group, rank, world)
            _wait(reqs)
            dkv = land
            if kv_reqs is not None:
                _wait(kv_reqs)
                kv = kv_land
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None


def ring_attention(q, k, v, scale=None, group=None):
    """Non-causal attention of the full sequence whose slices live on the ranks of ``group``
    (default: the world group). ``q, k, v``: this rank's ``[B, L_local, H, Dh]`` slices; every
    rank must hold a slice of the same length. Returns this rank's ``[B, L_local, H, Dh]``
    output slice; differentiable."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        from ..ops import functional as F
        return F.attention(q, k, v, scale)
    return _RingAttention.apply(q, k, v, scale, group)


def shard_sequence(x, group=None, dim=1):
    """This rank's contiguous slice of ``x`` along ``dim`` (length must divide by the group size)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if x.shape[dim] % world:
        raise ValueError(f"sequence length {x.shape[dim]} is not a multiple of the group size {world}")
    n = x.shape[dim] // world
    return x.narrow(dim, rank * n, n).contiguous()
