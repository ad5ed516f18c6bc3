"""MoE layers on one GPU (world size 1): grouped GEMM with gathered rows, gate-weighted epilogue
and the top-k combine kernel, against a dense PyTorch statement."""
import os

import pytest
import torch
import torch.distributed as dist

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    d = torch.device("cuda", 0)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29543")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=d)
    return d


@pytest.mark.parametrize("tpr,H,ffn,E,topk", [(256, 512, 768, 8, 2), (1000, 256, 384, 16, 4), (64, 128, 256, 4, 1)])
def test_moe_layers_single_gpu(dev, tpr, H, ffn, E, topk):
    from moe_common import run_moe_layer
    run_moe_layer(0, 1, 1, torch.bfloat16, dev, tpr=tpr, H=H, ffn=ffn, E=E, topk=topk, tol=3e-2)


def test_grouped_gemm_plain(dev):
    import tempname_new_b200 as flux
    E, N, K = 6, 384, 256
    splits = torch.tensor([100, 0, 257, 128, 1, 300])
    w = (torch.randn(E, N, K, device=dev) * 0.1).bfloat16()
    x = torch.randn(int(splits.sum()), K, device=dev).bfloat16()
    out = flux.GemmGroupedV3(w, E).forward(x, splits)
    row = 0
    for e, n in enumerate(splits.tolist()):
        ref = x[row:row + n].float() @ w[e].float().t()
        if n:
            assert (out[row:row + n].float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
        row += n


def test_grouped_gemm_fp8_with_scales(dev):
    """e4m3 operands, per-expert weight scale and a scalar input scale applied in the epilogue,
    bf16 output (reference: GemmGroupedV2.forward on 8-bit inputs, src/pybind/gemm_only.cc:171-190)."""
    import tempname_new_b200 as flux
    E, N, K = 5, 512, 384
    splits = torch.tensor([130, 0, 300, 64, 77])
    w = (torch.randn(E, N, K, device=dev) * 0.5).to(torch.float8_e4m3fn)
    x = torch.randn(int(splits.sum()), K, device=dev).to(torch.float8_e4m3fn)
    ws = torch.rand(E, device=dev) + 0.5
    xs = torch.tensor([0.25], device=dev)
    out = flux.GemmGroupedV3(w, E).forward(x, splits, input_scale=xs, weight_scale=ws)
    assert out.dtype == torch.bfloat16
    row = 0
    for e, n in enumerate(splits.tolist()):
        ref = (x[row:row + n].float() @ w[e].float().t()) * ws[e] * 0.25
        if n:
            assert (out[row:row + n].float() - ref).abs().max().item() <= 3e-2 * max(1.0, ref.abs().max().item())
        row += n


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float8_e4m3fn])
def test_moe_layer0_two_weight_groups_share_one_gather(dev, dtype):
    """forward_multiple_weights: gate and up projections on the same gathered rows (the second group
    reads the sorted buffer that the first launch filled)."""
    from moe_common import routed_problem
    import tempname_new_b200 as flux
    tokens, H, ffn, E, topk = 512, 256, 384, 8, 2
    experts, gate, scatter, splits, order = routed_problem(tokens, topk, E, seed=5, device=dev)
    x = (torch.randn(tokens, H, device=dev) * 0.5).to(dtype)
    wg = (torch.randn(E, ffn, H, device=dev) * 0.2).to(dtype)
    wu = (torch.randn(E, ffn, H, device=dev) * 0.2).to(dtype)
    env = flux.DistEnvTPWithEP(dist.group.WORLD, 1, None, ep_size=1)
    op = flux.GemmGroupedV3AGScatter(env, flux.MoeArguments(tokens, H, ffn, E, topk, dtype, torch.bfloat16))
    for _ in range(2):
        og, ou = op.forward_multiple_weights(x, [wg, wu], splits, scatter)
        rows = x[order // topk].float()
        offs = [0] + splits.cumsum(0).tolist()
        for e in range(E):
            lo, hi = offs[e], offs[e + 1]
            if hi > lo:
                for o, w in ((og, wg), (ou, wu)):
                    ref = rows[lo:hi] @ w[e].float().t()
                    assert (o[lo:hi].float() - ref).abs().max().item() <= 3e-2 * max(1.0, ref.abs().max().item())
    op.check_status()


def test_moe_layer1_fused_fp8(dev):
    """The fused combine on e4m3 operands: per-expert weight scales, gate weights per row."""
    from moe_common import routed_problem
    import tempname_new_b200 as flux
    tokens, H, ffn, E, topk = 384, 512, 256, 8, 2
    experts, gate, scatter, splits, order = routed_problem(tokens, topk, E, seed=6, device=dev)
    act = torch.randn(tokens * topk, ffn, device=dev).to(torch.float8_e4m3fn)     # expert-sorted rows
    w2 = (torch.randn(E, H, ffn, device=dev) * 0.3).to(torch.float8_e4m3fn)
    ws = torch.rand(E, device=dev) + 0.5
    row_gate = gate.reshape(-1)[order].contiguous()
    op = flux.GemmGroupedV3GatherRS(E, tokens * topk, H, topk, 0, 1, 1, 1, tp_group=dist.group.WORLD)
    for _ in range(2):
        out = op.forward_gather_rs(act, w2, splits.cpu(), scatter.reshape(-1), weight_scale=ws,
                                   output_vec_scale=row_gate)
        assert out.dtype == torch.bfloat16
        offs = [0] + splits.cumsum(0).tolist()
        y = torch.empty(tokens * topk, H, device=dev)
        for e in range(E):
            lo, hi = offs[e], offs[e + 1]
            y[lo:hi] = (act[lo:hi].float() @ w2[e].float().t()) * ws[e]
        y = (y * row_gate[:, None]).bfloat16().float()
        ref = y[scatter.reshape(-1).long()].view(tokens, topk, H).sum(1)
        assert (out.float() - ref).abs().max().item() <= 3e-2 * max(1.0, ref.abs().max().item())
    op.check_status()
