"""Quantised expert bank and expert selection.

Reference: ``QuantKind{None, Q8, NF4}``, ``QWeight``, ``quantize_weight`` / ``dequantize_to_bf16``,
``ExpertBank{insert, fetch_topk_bf16}`` and ``select_topk_global`` (crates/models/wan22/src/
moe_quant.rs:6-48). In the reference the quantiser is a pass-through and the selection returns the
first k ids. Here the bank stores real int8 / NF4 codes (``memory.quantize``; expanded by the
dequantisation kernel on the GPU) and the selection is a top-k over router scores.

Wan 2.2 itself is not token-routed: its two "experts" are two whole transformers chosen by the
timestep (``models/nextdit.py``: ``WanDualExpert``); the bank serves that case too (two entries,
one resident in bf16 at a time) and token-routed feed-forward experts.
"""
from __future__ import annotations

import enum

import torch

from ..memory import QuantizedTensor, dequantize, quantize


class QuantKind(str, enum.Enum):
    NONE = "none"
    Q8 = "q8"
    NF4 = "nf4"


def quantize_weight(w: torch.Tensor, kind: QuantKind | str):
    kind = QuantKind(kind)
    if kind == QuantKind.NONE:
        return w.detach().to(torch.bfloat16)
    return quantize(w, "int8" if kind == QuantKind.Q8 else "nf4")


def dequantize_to_bf16(qw) -> torch.Tensor:
    return dequantize(qw, torch.bfloat16) if isinstance(qw, QuantizedTensor) else qw.to(torch.bfloat16)


class ExpertBank:
    def __init__(self, kind: QuantKind | str = QuantKind.Q8):
        self.kind = QuantKind(kind)
        self.experts: dict[int, object] = {}

    def insert(self, expert_id: int, weight):
        """``weight``: a tensor (quantised on insertion) or an already quantised weight."""
        self.experts[expert_id] = weight if isinstance(weight, QuantizedTensor) else quantize_weight(weight, self.kind)

    def __len__(self):
        return len(self.experts)

    def nbytes(self) -> int:
        return sum(q.nbytes() if isinstance(q, QuantizedTensor) else q.numel() * q.element_size()
                   for q in self.experts.values())

    def fetch_topk_bf16(self, ids):
        """[(id, bf16 weight)] for the ids that are present, in the order asked."""
        return [(int(i), dequantize_to_bf16(self.experts[int(i)])) for i in ids if int(i) in self.experts]


def select_topk_global(scores_or_total, k: int):
    """With an int: the first ``k`` ids (the reference's behaviour). With router scores
    ``[tokens, experts]``: the ``k`` experts with the largest total probability mass over all
    tokens, i.e. the set worth keeping resident for this batch."""
    if isinstance(scores_or_total, int):
        return list(range(min(k, scores_or_total)))
    s = scores_or_total.float().softmax(-1).sum(0)
    return torch.topk(s, min(k, s.numel())).indices.tolist()


def route_tokens(scores: torch.Tensor, k: int, allowed=None):
    """Per-token top-k routing: returns (expert ids [tokens, k], normalised weights [tokens, k]).
    ``allowed``: restrict the choice to these expert ids (the resident set)."""
    s = scores.float()
    if allowed is not None:
        mask = torch.full_like(s, float("-inf"))
        mask[:, list(allowed)] = 0
        s = s + mask
    w, idx = torch.topk(s.softmax(-1), k, dim=-1)
    return idx, w / w.sum(-1, keepdim=True).clamp_min(1e-12)


def moe_linear(x: torch.Tensor, scores: torch.Tensor, bank: ExpertBank, k: int = 2, resident: int | None = None):
    """y[t] = sum_j w[t, j] * x[t] @ W[e(t, j)]^T over the top-k experts of each token, expanding only
    the experts some token uses (at most ``resident`` of them, chosen by ``select_topk_global``)."""
    allowed = select_topk_global(scores, resident) if resident else None
    idx, w = route_tokens(scores, k, allowed)
    out = None
    for e, We in bank.fetch_topk_bf16(sorted(set(idx.flatten().tolist()))):
        hit = idx == e                                              # [T, k]
        rows = hit.any(-1)
        y = x[rows].to(We.dtype) @ We.t()
        if out is None:
            out = torch.zeros(x.shape[0], We.shape[0], dtype=torch.float32, device=x.device)
        out[rows] += y.float() * (w * hit)[rows].sum(-1, keepdim=True)
    return out.to(x.dtype)
