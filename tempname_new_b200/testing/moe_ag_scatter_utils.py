"""A test context for MoE layer 0 and its step-by-step PyTorch statement (reference:
``python/flux/testing/moe_ag_scatter_utils.py``: ``MoeMlp1Ctx`` :26-192, ``MoeAgScatterWithTorch``
:195-262). The context owns every tensor of one layer-0 problem on this rank: the token shard,
the all-gather target, the expert weights of this rank (``weight_groups`` of them), routing
tensors, and output buffers. ``MoeAgScatterWithTorch`` runs the layer in three visible steps
(all-gather, row gather, per-expert GEMM) so that a fused op can be checked stage by stage."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .moe_utils import gen_moe_gating_args
from .utils import all_gather_into_tensor_with_fp8


class MoeMlp1Ctx:
    def __init__(self, TP_GROUP, EP_GROUP, b: int, s: int, h: int, ffn_size: int, nexperts: int, topk: int,
                 input_dtype: torch.dtype, output_dtype: Optional[torch.dtype], dist: str = "uniform",
                 fast_accum: bool = False, weight_groups: int = 1, drop_token: bool = False, debug: bool = False,
                 generator: Optional[torch.Generator] = None, stable: bool = True):
        import torch.distributed as tdist
        self.b, self.s, self.h, self.ffn_size = b, s, h, ffn_size
        self.nexperts, self.topk, self.ntokens = nexperts, topk, b * s
        self.fast_accum, self.weight_groups, self.drop_token = fast_accum, weight_groups, drop_token
        self.tp_rank, self.tp_size = tdist.get_rank(TP_GROUP), tdist.get_world_size(TP_GROUP)
        self.ep_rank, self.ep_size = tdist.get_rank(EP_GROUP), tdist.get_world_size(EP_GROUP)
        if nexperts % self.ep_size or self.tp_size % self.ep_size:
            raise ValueError("experts and ranks must divide over the expert-parallel size")
        self.ffn_tp_size = self.tp_size // self.ep_size
        self.nexperts_ep = nexperts // self.ep_size
        if ffn_size % self.ffn_tp_size or self.ntokens % self.tp_size:
            raise ValueError("ffn_size / tokens must divide over the ranks")
        self.ffn_size_shard = ffn_size // self.ffn_tp_size
        self.ntokens_shard = self.ntokens // self.tp_size
        self.is_s8 = input_dtype == torch.int8
        self.input_scale = None
        out_dtype = output_dtype or (torch.bfloat16 if input_dtype.itemsize == 1 else input_dtype)
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        seed = 17 if generator is None else int(generator.initial_seed())
        weights = None if dist in ("uniform", "random_uniform") else torch.rand(
            nexperts, generator=torch.Generator().manual_seed(seed))
        g = gen_moe_gating_args(nexperts, topk, self.ntokens, 0.0, weights, device=dev, seed=seed)
        self.choosed_experts, self.scatter_index = g.choosed_experts, g.scatter_index
        self.gather_index, self.topk_index = g.gather_index.long(), g.topk_index
        self.splits_gpu, self.splits_cpu = g.splits_gpu, g.splits_cpu
        e0 = self.nexperts_ep * self.ep_rank
        self.nrows_ep = int(self.splits_cpu[e0:e0 + self.nexperts_ep].sum())
        gen = torch.Generator().manual_seed(seed + 1 + self.tp_rank)
        wgen = torch.Generator().manual_seed(seed + 1000 + self.ep_rank * 31 + self.tp_rank % self.ffn_tp_size)

        def make(shape, scale, gg):
            return (torch.randn(*shape, generator=gg) * scale).to(input_dtype).to(dev)

        self.inputs_shard = make((self.ntokens_shard, h), 0.5, gen)
        self.inputs = torch.zeros(self.ntokens, h, dtype=input_dtype, device=dev)
        self.scatter_inputs = torch.zeros(self.ntokens * topk, h, dtype=input_dtype, device=dev)
        self.weights: List[torch.Tensor] = [make((self.nexperts_ep, self.ffn_size_shard, h), 0.1, wgen)
                                            for _ in range(weight_groups)]
        self.output_scale = [torch.ones(self.nexperts_ep, dtype=torch.float32, device=dev)
                             for _ in range(weight_groups)]
        self.bias = None
        self.outputs = [torch.zeros(self.nrows_ep, self.ffn_size_shard, dtype=out_dtype, device=dev)
                        for _ in range(weight_groups)]

    def clear_outputs(self) -> None:
        for o in self.outputs:
            o.zero_()
        self.inputs.zero_()
        self.scatter_inputs.zero_()

    def get_outputs_clone(self):
        return [o.clone() for o in self.outputs]


class MoeAgScatterWithTorch:
    @staticmethod
    def comm_impl(ctx: MoeMlp1Ctx, TP_GROUP) -> None:
        if dist.get_world_size(TP_GROUP) > 1:
            all_gather_into_tensor_with_fp8(ctx.inputs, ctx.inputs_shard, group=TP_GROUP)
        else:
            ctx.inputs.copy_(ctx.inputs_shard)

    @staticmethod
    def scatter_impl(ctx: MoeMlp1Ctx) -> None:
        fp8 = ctx.inputs.dtype.itemsize == 1 and ctx.inputs.dtype.is_floating_point
        src = ctx.inputs.view(torch.uint8) if fp8 else ctx.inputs
        rows = torch.index_select(src, 0, ctx.gather_index.to(src.device))
        ctx.scatter_inputs.view(rows.dtype).copy_(rows)

    @staticmethod
    def gemm_impl(ctx: MoeMlp1Ctx, gemm_only_op=None) -> None:
        e0 = ctx.nexperts_ep * ctx.ep_rank
        base = int(ctx.splits_cpu[:e0].sum())
        off = 0
        for e in range(ctx.nexperts_ep):
            n = int(ctx.splits_cpu[e0 + e])
            if n == 0:
                continue
            x = ctx.scatter_inputs[base + off:base + off + n]
            for i in range(ctx.weight_groups):
                y = x.float() @ ctx.weights[i][e].float().t()
                if ctx.bias is not None:
                    y = y + ctx.bias[i][e].float()
                y = y * ctx.output_scale[i][e]
                ctx.outputs[i][off:off + n] = y.to(ctx.outputs[i].dtype)
            off += n

    @staticmethod
    def forward(ctx: MoeMlp1Ctx, TP_GROUP, gemm_only_op=None):
        MoeAgScatterWithTorch.comm_impl(ctx, TP_GROUP)
        MoeAgScatterWithTorch.scatter_impl(ctx)
        MoeAgScatterWithTorch.gemm_impl(ctx, gemm_only_op)
        return ctx.outputs
