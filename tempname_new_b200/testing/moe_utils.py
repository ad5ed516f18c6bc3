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


def calc_gather_index(scatter_index: torch.Tensor, row_start: int, row_end: int, BLOCK_SIZE: int = 1024):
    """(token, k) of the sorted rows [row_start, row_end): the inverse of ``scatter_index`` on that
    range (reference: ``calc_gather_index``, python/flux/testing/moe_utils.py:96-138, a Triton
    kernel there; ``BLOCK_SIZE`` is accepted for the signature)."""
    ntokens, topk = scatter_index.shape
    flat = scatter_index.reshape(-1).long()
    pos = torch.arange(flat.numel(), device=flat.device)
    sel = (flat >= row_start) & (flat < row_end)
    gather = torch.zeros(row_end - row_start, dtype=torch.int32, device=flat.device)
    topk_index = torch.zeros_like(gather)
    gather[flat[sel] - row_start] = (pos[sel] // topk).to(torch.int32)
    topk_index[flat[sel] - row_start] = (pos[sel] % topk).to(torch.int32)
    return gather, topk_index


def calc_scatter_index_stable_sync(choosed_experts: torch.Tensor, splits_gpu: torch.Tensor) -> torch.Tensor:
    """The stable scatter index built expert by expert from the split counts (one device sync per
    expert; reference: python/flux/testing/moe_utils.py:147-155)."""
    scatter = torch.full_like(choosed_experts, -1, dtype=torch.int32)
    start = (splits_gpu.cumsum(0) - splits_gpu).tolist()
    for e, n in enumerate(splits_gpu.tolist()):
        scatter[choosed_experts == e] = torch.arange(start[e], start[e] + n, dtype=torch.int32,
                                                     device=choosed_experts.device)
    return scatter


def moe_gather_rs_forward_torch(TP_GROUP, M: int, eid_start: int, ep_rank_m_start: int, ep_rank_m_end: int,
                                inputs, weights, split_cpu: torch.Tensor, token_index: torch.Tensor,
                                topk_index: torch.Tensor, topk: int, input_scales, weight_scales, output_vec_scales,
                                do_all_reduce: bool = False, fast_acc: bool = False) -> torch.Tensor:
    """PyTorch statement of MoE layer 1 (reference: python/flux/testing/moe_gather_rs_utils.py:26-120):
    per expert ``x_e @ W_e^T`` times ``weight_scale[e] * input_scale``, times the row's gate weight,
    placed at row ``topk * token + k`` of an [M, N] matrix, summed over the top-k entries of every
    token and over the weight groups, then reduce-scattered (or all-reduced) over ``TP_GROUP``.
    ``M`` = tokens * topk of the whole job; rows [ep_rank_m_start, ep_rank_m_end) of the sorted
    order are this rank's."""
    import torch.distributed as dist
    if isinstance(inputs, torch.Tensor):
        inputs, weights = [inputs], [weights]
        input_scales, weight_scales, output_vec_scales = [input_scales], [weight_scales], [output_vec_scales]
    x0 = inputs[0]
    out_dtype = torch.bfloat16 if x0.dtype.itemsize == 1 else x0.dtype
    N = weights[0].shape[1]
    full = torch.zeros(M, N, dtype=torch.float32, device=x0.device)
    rows = (topk * token_index[ep_rank_m_start:ep_rank_m_end].long() + topk_index[ep_rank_m_start:ep_rank_m_end].long())
    for x, w, isc, wsc, ovs in zip(inputs, weights, input_scales, weight_scales, output_vec_scales):
        outs, acc = [], 0
        for e in range(w.shape[0]):
            n = int(split_cpu[e + eid_start])
            y = x[acc:acc + n].float() @ w[e].float().t()
            if wsc is not None:
                y = y * wsc.reshape(-1)[e].float()
            if isc is not None:
                y = y * isc.reshape(-1)[0].float()
            outs.append(y)
            acc += n
        y = torch.cat(outs)
        if ovs is not None:
            y = y * ovs.float().reshape(-1, 1)
        part = torch.zeros_like(full)
        part[rows] = y.to(out_dtype).float()
        full += part
    reduced = full.view(M // topk, topk, N).sum(1).to(out_dtype)
    W = dist.get_world_size(TP_GROUP)
    if do_all_reduce:
        dist.all_reduce(reduced, group=TP_GROUP)
        return reduced
    out = torch.empty(M // topk // W, N, dtype=out_dtype, device=x0.device)
    if W > 1:
        dist.reduce_scatter(out, [c.contiguous() for c in reduced.chunk(W)], group=TP_GROUP)
    else:
        out.copy_(reduced)
    return out
