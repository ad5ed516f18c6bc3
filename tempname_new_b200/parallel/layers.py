"""Megatron-style tensor-parallel linear layers with sequence-parallel activations, built on
the fused ops.

* ``ColumnParallelLinear``: weight ``[out/W, in]``; forward = all-gather(tokens) fused into the
  GEMM (``AGKernel``); backward dgrad = GEMM fused with reduce-scatter (``GemmRS``).
* ``RowParallelLinear``: weight ``[out, in/W]``; forward = ``GemmRS``; backward dgrad =
  ``AGKernel`` on the gathered output gradient.
Weight gradients are plain library GEMMs on the gathered activations.

Reference: the fork patches Megatron's ``RowParallelLinear.forward`` with ``GemmRS`` and keeps
Megatron's own backward (``tools/a800/e2e/adapter.py:14-116``); here both directions of both
layers run on the fused kernels, and ``patch_megatron_linears`` applies the same idea to a live
Megatron model when Megatron-LM is importable.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
from torch import nn

from ..ops.ag_gemm import AGKernel
from ..ops.gemm_rs import GemmRS


class _OpCache:
    """Fused-op objects keyed by shape: they own symmetric buffers (an all-gather landing buffer, the
    reduce-scatter staging slabs: hundreds of MB at transformer shapes), so one set per process group
    serves every layer of a model: layers run one after the other on a stream, and the ops' call
    numbers keep consecutive uses apart. ``_OpCache.shared(group)`` returns that per-group instance
    (the reference's Megatron adapter likewise keeps one op per shape)."""

    _per_group = {}

    def __init__(self, group):
        self.group = group
        self.ops = {}

    @classmethod
    def shared(cls, group) -> "_OpCache":
        key = id(group)
        c = cls._per_group.get(key)
        if c is None or c.group is not group:
            c = cls._per_group[key] = cls(group)
        return c

    def ag(self, full_m, n, k, dtype) -> AGKernel:
        key = ("ag", full_m, n, k, dtype)
        if key not in self.ops:
            self.ops[key] = AGKernel(self.group, 1, full_m, n, k, dtype)
        return self.ops[key]

    def rs(self, max_m, n, dtype) -> GemmRS:
        key = ("rs", max_m, n, dtype)
        if key not in self.ops:
            self.ops[key] = GemmRS(self.group, 1, max_m, n, dtype)
        return self.ops[key]


class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, cache: _OpCache, act, need_gathered=True):
        W = dist.get_world_size(cache.group)
        seg, K = x.shape
        M = seg * W
        op = cache.ag(M, weight.shape[0], K, x.dtype)
        # the gathered activations are only needed for the weight gradient
        gathered = torch.empty((M, K), dtype=x.dtype, device=x.device) if need_gathered else None
        out = op.forward(x, weight, bias=bias, gathered_input=gathered, act=act)
        ctx.save_for_backward(gathered, weight)
        ctx.cache, ctx.has_bias, ctx.act = cache, bias is not None, act
        return out

    @staticmethod
    def backward(ctx, grad_out):
        if ctx.act not in (None, "none"):
            raise RuntimeError("fused activation is forward-only; use act=None when training")
        gathered, weight = ctx.saved_tensors
        cache = ctx.cache
        g = grad_out.contiguous()
        # dgrad: [M, out/W] @ [out/W, in] summed over ranks and scattered over M
        op = cache.rs(g.shape[0], weight.shape[1], g.dtype)
        grad_x = op.forward(g, weight, None, transpose_weight_override=True)
        grad_w = g.t().matmul(gathered) if gathered is not None else None
        grad_b = g.sum(0) if ctx.has_bias else None
        return grad_x, grad_w, grad_b, None, None, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, cache: _OpCache):
        op = cache.rs(x.shape[0], weight.shape[0], x.dtype)
        out = op.forward(x, weight)
        ctx.save_for_backward(x, weight)
        ctx.cache = cache
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, weight = ctx.saved_tensors
        cache = ctx.cache
        W = dist.get_world_size(cache.group)
        g = grad_out.contiguous()
        M = g.shape[0] * W
        # dgrad: all_gather(grad)[M, out] @ weight[out, in/W]
        op = cache.ag(M, weight.shape[1], weight.shape[0], g.dtype)
        gathered = torch.empty((M, g.shape[1]), dtype=g.dtype, device=g.device)
        grad_x = op.forward(g, weight, transpose_weight=True, gathered_input=gathered)
        grad_w = gathered.t().matmul(x)
        return grad_x, grad_w, None


class ColumnParallelLinear(nn.Module):
    """y[tokens, out/W] = all_gather(x[tokens/W, in]) @ W[out/W, in]^T + b."""

    def __init__(self, in_features: int, out_features: int, tp_group=None, bias: bool = True,
                 dtype: torch.dtype = torch.bfloat16, device=None, init_std: float = 0.02):
        super().__init__()
        self.group = tp_group if tp_group is not None else dist.group.WORLD
        W = dist.get_world_size(self.group)
        if out_features % W:
            raise ValueError("out_features must divide over the TP group")
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features // W, in_features, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=init_std)
        self.bias = nn.Parameter(torch.zeros(out_features // W, dtype=dtype, device=device)) if bias else None
        self._cache = _OpCache.shared(self.group)

    def forward(self, x: torch.Tensor, act: Optional[str] = None) -> torch.Tensor:
        need = torch.is_grad_enabled() and self.weight.requires_grad
        return _ColumnParallelFn.apply(x, self.weight, self.bias, self._cache, act, need)


class RowParallelLinear(nn.Module):
    """y[tokens/W, out] = reduce_scatter(x[tokens, in/W] @ W[out, in/W]^T) + b."""

    def __init__(self, in_features: int, out_features: int, tp_group=None, bias: bool = True,
                 dtype: torch.dtype = torch.bfloat16, device=None, init_std: float = 0.02):
        super().__init__()
        self.group = tp_group if tp_group is not None else dist.group.WORLD
        W = dist.get_world_size(self.group)
        if in_features % W:
            raise ValueError("in_features must divide over the TP group")
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features // W, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=init_std)
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        self._cache = _OpCache.shared(self.group)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = _RowParallelFn.apply(x, self.weight, self._cache)
        return y + self.bias if self.bias is not None else y


def patch_megatron_linears(model, tp_group=None, row: bool = True, column: bool = True) -> int:
    """Route the forward of Megatron-LM ``RowParallelLinear`` / ``ColumnParallelLinear`` modules
    of ``model`` (sequence-parallel, no gradient-accumulation fusion) through the fused ops.
    Returns the number of patched modules. Needs Megatron-LM to be importable."""
    try:
        from megatron.core.tensor_parallel import layers as mlayers  # type: ignore
        from megatron.core import parallel_state  # type: ignore
    except Exception as e:  # pragma: no cover - Megatron is not part of this image
        raise RuntimeError("Megatron-LM is not importable in this environment") from e
    group = tp_group if tp_group is not None else parallel_state.get_tensor_model_parallel_group()
    cache = _OpCache.shared(group)
    n = 0
    for _, mod in model.named_modules():
        if row and isinstance(mod, mlayers.RowParallelLinear) and mod.sequence_parallel and mod.input_is_parallel:
            def fwd(self, input_, _cache=cache):
                s = input_.shape
                y = _RowParallelFn.apply(input_.reshape(-1, s[-1]).contiguous(), self.weight, _cache)
                y = y.reshape(s[0] // dist.get_world_size(_cache.group), *s[1:-1], self.weight.shape[0])
                if self.skip_bias_add:
                    return y, self.bias
                return (y + self.bias if self.bias is not None else y), None
            mod.forward = fwd.__get__(mod)
            n += 1
        elif column and isinstance(mod, mlayers.ColumnParallelLinear) and mod.sequence_parallel:
            def fwd(self, input_, _cache=cache, **_):
                s = input_.shape
                b = None if self.skip_bias_add else self.bias
                y = _ColumnParallelFn.apply(input_.reshape(-1, s[-1]).contiguous(), self.weight, b, _cache, None,
                                            torch.is_grad_enabled() and self.weight.requires_grad)
                y = y.reshape(s[0] * dist.get_world_size(_cache.group), *s[1:-1], self.weight.shape[0])
                return y, (self.bias if self.skip_bias_add else None)
            mod.forward = fwd.__get__(mod)
            n += 1
    return n
