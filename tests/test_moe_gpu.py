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
