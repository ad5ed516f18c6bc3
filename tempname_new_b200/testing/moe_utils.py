"""MoE routing tensors for tests and examples (reference: ``python/flux/testing/moe_utils.py``).

``splits = bincount(experts)``; ``scatter_index = argsort(argsort(experts, stable))`` gives the
row of every (token, k) entry in the expert-sorted order; ``gather_index`` is its inverse divided
by top-k (the token of each sorted row)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class moe_gating_args:
    choosed_experts: torch.Tensor   # [tokens, topk] int32
    scatter_index: torch.Tensor     # [tokens, topk] int32
    gather_index: torch.Tensor      # [tokens * topk] int32: token of sorted row
    topk_index: torch.Tensor        # [tokens * topk] int32: k of sorted row
    splits_gpu: torch.Tensor        # [E] int32
    splits_cpu: torch.Tensor
    gate_weight: Optional[torch.Tensor] = None   # [tokens, topk] float32


def calc_scatter_index_stable(choosed_experts: torch.Tensor) -> torch.Tensor:
    flat = choosed_experts.reshape(-1)
    order = torch.argsort(flat, stable=True)
    scatter = torch.empty_like(order)
    scatter[order] = torch.arange(order.numel(), device=flat.device)
    return scatter.view(choosed_experts.shape).to(torch.int32)


def calc_gather_index_stable(choosed_experts: torch.Tensor):
    order = torch.argsort(choosed_experts.reshape(-1), stable=True)
    topk = choosed_experts.shape[1]
    return (order // topk).to(torch.int32), (order % topk).to(torch.int32)


def is_gather_index_stable(gather_index: torch.Tensor, splits: torch.Tensor) -> bool:
    """Inside every expert the token ids must not decrease."""
    start = 0
    for n in splits.tolist():
        seg = gather_index[start:start + n]
        if n > 1 and bool((seg[1:] < seg[:-1]).any()):
            return False
        start += n
    return True


def gen_moe_gating_args(E: int, topk: int, ntokens: int, drop_ratio: float = 0.0, weights: Optional[torch.Tensor] = None,
                        device=None, seed: int = 0, round_robin: bool = False) -> moe_gating_args:
    """Routing for ``ntokens`` tokens: round-robin (perfectly balanced) or sampled without
    replacement from ``weights`` (uniform by default)."""
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    g = torch.Generator().manual_seed(seed)
    if round_robin:
        base = torch.arange(ntokens * topk) % E
        chosen = base.view(ntokens, topk)
    else:
        w = torch.ones(E) if weights is None else weights.float().cpu()
        chosen = torch.multinomial(w.expand(ntokens, E), topk, replacement=False, generator=g)
    chosen = chosen.to(torch.int32).to(device)
    gate = torch.rand(ntokens, topk, generator=g)
    gate = (gate / gate.sum(1, keepdim=True)).to(device)
    splits = torch.bincount(chosen.reshape(-1).long(), minlength=E).to(torch.int32)
    gi, ti = calc_gather_index_stable(chosen)
    return moe_gating_args(chosen, calc_scatter_index_stable(chosen), gi, ti, splits, splits.cpu(), gate)


def gate_func(hidden: torch.Tensor, gate_weight: torch.Tensor, topk: int):
    """Softmax router: returns (choosed_experts [tokens, topk], normalised gate weights)."""
    logits = hidden.float() @ gate_weight.float().t()
    probs = torch.softmax(logits, dim=-1)
    w, idx = probs.topk(topk, dim=-1)
    return idx.to(torch.int32), w / w.sum(-1, keepdim=True)
