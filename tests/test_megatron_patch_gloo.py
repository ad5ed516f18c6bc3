"""`patch_megatron_linears` against a stand-in for Megatron-LM's tensor-parallel layers: two CPU
ranks, sequence-parallel Column -> Row block in Megatron's [seq, batch, hidden] layout, compared
with the all-gather / matmul / reduce-scatter statement (reference: the fork's Megatron adapter,
tools/a800/e2e/adapter.py:14-116)."""
import sys
import types

import torch
import torch.distributed as dist
from torch import nn

from conftest import run_gloo


def _install_stub_megatron(group):
    """Modules named like Megatron-LM's, with just the attributes the patch looks at."""
    layers = types.ModuleType("megatron.core.tensor_parallel.layers")

    class ColumnParallelLinear(nn.Module):
        def __init__(self, in_f, out_f, world, skip_bias_add=False):
            super().__init__()
            self.weight = nn.Parameter(torch.randn(out_f // world, in_f) * 0.1)
            self.bias = nn.Parameter(torch.randn(out_f // world) * 0.1)
            self.sequence_parallel, self.skip_bias_add = True, skip_bias_add

        def forward(self, x):
            raise AssertionError("the unpatched Megatron forward ran")

    class RowParallelLinear(nn.Module):
        def __init__(self, in_f, out_f, world, skip_bias_add=True):
            super().__init__()
            self.weight = nn.Parameter(torch.randn(out_f, in_f // world) * 0.1)
            self.bias = nn.Parameter(torch.randn(out_f) * 0.1)
            self.sequence_parallel, self.input_is_parallel, self.skip_bias_add = True, True, skip_bias_add

        def forward(self, x):
            raise AssertionError("the unpatched Megatron forward ran")

    layers.ColumnParallelLinear, layers.RowParallelLinear = ColumnParallelLinear, RowParallelLinear
    ps = types.ModuleType("megatron.core.parallel_state")
    ps.get_tensor_model_parallel_group = lambda: group
    tp = types.ModuleType("megatron.core.tensor_parallel")
    tp.layers = layers
    core = types.ModuleType("megatron.core")
    core.tensor_parallel, core.parallel_state = tp, ps
    meg = types.ModuleType("megatron")
    meg.core = core
    sys.modules.update({"megatron": meg, "megatron.core": core, "megatron.core.tensor_parallel": tp,
                        "megatron.core.tensor_parallel.layers": layers, "megatron.core.parallel_state": ps})
    return layers


def _patched_block_matches_torch(rank, world):
    from tempname_new_b200.parallel.layers import patch_megatron_linears
    group = dist.group.WORLD
    layers = _install_stub_megatron(group)
    torch.manual_seed(10 + rank)
    S, B, Hd, F = 8 * world, 2, 16, 32 * world
    model = nn.Sequential()
    model.add_module("fc1", layers.ColumnParallelLinear(Hd, F, world))
    model.add_module("fc2", layers.RowParallelLinear(F, Hd, world))
    assert patch_megatron_linears(model) == 2
    x = torch.randn(S // world, B, Hd, requires_grad=True)          # this rank's sequence shard
    h, b1 = model.fc1(x)
    assert b1 is None and h.shape == (S, B, F // world)
    y, b2 = model.fc2(h)
    assert y.shape == (S // world, B, Hd) and b2 is model.fc2.bias  # skip_bias_add hands the bias back

    # the same block written with collectives
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x.detach())
    full = torch.cat(parts)                                           # [S, B, Hd]
    h_ref = full @ model.fc1.weight.detach().t() + model.fc1.bias.detach()
    assert torch.allclose(h, h_ref, atol=1e-4)
    part = h_ref @ model.fc2.weight.detach().t()
    dist.all_reduce(part)
    y_ref = part[rank * (S // world):(rank + 1) * (S // world)]
    assert torch.allclose(y, y_ref, atol=1e-3)

    # gradients flow through both patched layers (dgrad on the fused ops, wgrad on matmul)
    y.square().sum().backward()
    assert x.grad is not None and x.grad.shape == x.shape and torch.isfinite(x.grad).all()
    assert model.fc1.weight.grad is not None and model.fc2.weight.grad is not None
    # dgrad of the block, stated with collectives: dY -> gather over sequence -> fc2^T -> fc1^T -> reduce-scatter
    gy = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(gy, (2 * y).detach())
    gh = torch.cat(gy) @ model.fc2.weight.detach()
    gx = gh @ model.fc1.weight.detach()
    dist.all_reduce(gx)
    assert torch.allclose(x.grad, gx[rank * (S // world):(rank + 1) * (S // world)], atol=1e-3)


def test_patch_megatron_linears_on_stub_megatron():
    run_gloo(_patched_block_matches_torch, 2)
