"""Tensor-parallel layers on 2 CPU ranks: forward and backward against a single-process
statement of the same math."""
import torch
import torch.distributed as dist

from conftest import run_gloo


def _tp_mlp(rank, world):
    from tempname_new_b200.models.tp_mlp import TPMLP
    torch.manual_seed(0)
    hidden, ffn, tokens = 64, 256, 32 * world
    # full (unsharded) parameters, identical on every rank
    w1 = torch.randn(ffn, hidden) * 0.1
    b1 = torch.randn(ffn) * 0.1
    w2 = torch.randn(hidden, ffn) * 0.1
    b2 = torch.randn(hidden) * 0.1
    x_full = torch.randn(tokens, hidden)
    mlp = TPMLP(hidden, ffn, dtype=torch.float32)
    fs, hs = ffn // world, tokens // world
    with torch.no_grad():
        mlp.fc1.weight.copy_(w1[rank * fs:(rank + 1) * fs])
        mlp.fc1.bias.copy_(b1[rank * fs:(rank + 1) * fs])
        mlp.fc2.weight.copy_(w2[:, rank * fs:(rank + 1) * fs])
        mlp.fc2.bias.copy_(b2)
    x = x_full[rank * hs:(rank + 1) * hs].clone().requires_grad_(True)
    y = mlp(x)
    # reference
    xr = x_full.clone().requires_grad_(True)
    w1r, w2r = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    yr = torch.nn.functional.gelu(xr @ w1r.t() + b1, approximate="tanh") @ w2r.t() + b2
    torch.testing.assert_close(y, yr[rank * hs:(rank + 1) * hs], rtol=1e-4, atol=1e-4)
    g_full = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(5))
    y.backward(g_full[rank * hs:(rank + 1) * hs])
    yr.backward(g_full)
    torch.testing.assert_close(x.grad, xr.grad[rank * hs:(rank + 1) * hs], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(mlp.fc1.weight.grad, w1r.grad[rank * fs:(rank + 1) * fs], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(mlp.fc2.weight.grad, w2r.grad[:, rank * fs:(rank + 1) * fs], rtol=1e-4, atol=1e-4)
    # inference path with the activation fused into the first GEMM
    with torch.no_grad():
        y2 = mlp(x.detach())
    torch.testing.assert_close(y2, y.detach(), rtol=1e-5, atol=1e-5)


def test_tp_mlp_forward_backward_gloo_w2():
    run_gloo(_tp_mlp, 2)
