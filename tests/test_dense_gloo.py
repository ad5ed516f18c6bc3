"""CPU/gloo world_size=2 plumbing: GEMM-RS and AG-GEMM through the public ops on shared host
memory, checked against torch.matmul + dist.reduce_scatter / all_gather."""
import torch
import torch.distributed as dist

from conftest import run_gloo


def _data(rows, cols, k, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(rows, cols, generator=g) / (k ** 0.5)


def _gemm_rs(rank, world):
    import tempname_new_b200 as flux
    flux.init_flux_shm()
    M, Kl, N = 256, 256, 384
    a = _data(M, Kl, Kl * world, 0 + rank)
    w = _data(N, Kl, Kl * world, 100 + rank)
    op = flux.GemmRS(dist.group.WORLD, 1, M, N, torch.float32)
    for _ in range(3):  # repeated calls exercise the call-number flags
        out = op.forward(a, w)
        full = a @ w.t()
        ref = torch.empty(M // world, N)
        dist.reduce_scatter(ref, list(full.chunk(world)))
        assert out.shape == ref.shape
        torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
    bias = _data(M, N, 1, 7)
    out = op.forward(a, w, bias=bias)  # bias is added on every rank, i.e. W times after the sum
    full = a @ w.t() + bias
    dist.reduce_scatter(ref, list(full.chunk(world)))
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)


def _ag_gemm(rank, world):
    import tempname_new_b200 as flux
    flux.init_flux_shm()
    seg, K, Nl = 128, 512, 192
    a = _data(seg, K, K, 0 + rank)
    w = _data(Nl, K, K, 100 + rank)
    op = flux.AGKernel(dist.group.WORLD, 1, seg * world, Nl, K, torch.float32)
    for _ in range(3):
        gathered = torch.empty(seg * world, K)
        out = op.forward(a, w, gathered_input=gathered)
        parts = [torch.empty_like(a) for _ in range(world)]
        dist.all_gather(parts, a)
        full = torch.cat(parts)
        torch.testing.assert_close(gathered, full, rtol=0, atol=0)
        torch.testing.assert_close(out, full @ w.t(), rtol=1e-5, atol=1e-5)
    wt = w.t().contiguous()
    out_t = op.forward(a, wt, transpose_weight=True)
    torch.testing.assert_close(out_t, out, rtol=1e-6, atol=1e-6)


def _int8(rank, world):
    """Signed 8-bit operands with two per-tensor scales through both fused ops (CPU statement of
    what the kind::i8 kernels compute: exact integer products, scaled, rounded to bf16)."""
    import tempname_new_b200 as flux
    flux.init_flux_shm()
    M, Kl, N = 64, 32, 48
    g = torch.Generator().manual_seed(3 + rank)
    a = torch.randint(-127, 128, (M, Kl), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (N, Kl), generator=g, dtype=torch.int8)
    sa, sb = torch.tensor([0.02]), torch.tensor([0.01])
    op = flux.GemmRS(dist.group.WORLD, 1, M, N, torch.int8, output_dtype=torch.bfloat16)
    out = op.forward(a, w, input_scale=sa, weight_scale=sb)
    full = (a.float() @ w.float().t()) * 2e-4
    ref = torch.empty(M // world, N)
    dist.reduce_scatter(ref, list(full.chunk(world)))
    assert out.dtype == torch.bfloat16
    assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max()     # bf16 rounding of the result
    seg = M // world
    w2 = torch.randint(-127, 128, (N, Kl * 2), generator=torch.Generator().manual_seed(11), dtype=torch.int8)
    a2 = torch.randint(-127, 128, (seg, Kl * 2), generator=g, dtype=torch.int8)
    ag = flux.AGKernel(dist.group.WORLD, 1, M, N, Kl * 2, torch.int8, output_dtype=torch.bfloat16)
    out = ag.forward(a2, w2, input_scale=sa, weight_scale=sb)
    parts = [torch.empty_like(a2) for _ in range(world)]
    dist.all_gather(parts, a2)
    ref = (torch.cat(parts).float() @ w2.float().t()) * 2e-4
    assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max()


def _varying_shapes(rank, world):
    """One op object, calls with different row counts in a row (the call-number flags must not
    depend on the shape of the previous call), ranks entering the calls at different times."""
    import time
    import tempname_new_b200 as flux
    flux.init_flux_shm()
    N, Kl = 48, 32
    rs = flux.GemmRS(dist.group.WORLD, 1, 256, N, torch.float32)
    ag = flux.AGKernel(dist.group.WORLD, 1, 256, N, Kl, torch.float32)
    for i, M in enumerate([256, 64, 128, 32, 256, 64]):
        if (i + rank) % 2:
            time.sleep(0.02)                      # skew the ranks
        a = _data(M, Kl, Kl * world, 10 * i + rank)
        w = _data(N, Kl, Kl * world, 100 + rank)
        out = rs.forward(a, w)
        ref = torch.empty(M // world, N)
        dist.reduce_scatter(ref, list((a @ w.t()).chunk(world)))
        torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
        seg = M // world
        a2 = _data(seg, Kl, Kl, 20 * i + rank)
        out2 = ag.forward(a2, w)
        parts = [torch.empty_like(a2) for _ in range(world)]
        dist.all_gather(parts, a2)
        torch.testing.assert_close(out2, torch.cat(parts) @ w.t(), rtol=1e-5, atol=1e-5)


def _symm(rank, world):
    import tempname_new_b200 as flux
    ts = flux.create_tensor_list((4, 8), torch.float32)
    assert len(ts) == world
    ts[rank].fill_(rank + 1)
    gb = flux.GroupBarrier()
    gb.barrier_all()
    for r in range(world):
        assert float(ts[r].sum()) == (r + 1) * 32
    gb.barrier_all()
    ts[(rank + 1) % world][0, 0] = -5.0  # write into the neighbour's block
    gb.barrier_all()
    assert float(ts[rank][0, 0]) == -5.0


def test_gemm_rs_gloo_w2():
    run_gloo(_gemm_rs, 2)


def test_ag_gemm_gloo_w2():
    run_gloo(_ag_gemm, 2)


def test_gemm_rs_gloo_w4():
    run_gloo(_gemm_rs, 4)


def test_symmetric_memory_and_barrier_gloo():
    run_gloo(_symm, 3)


def test_int8_operands_gloo():
    run_gloo(_int8, 2)


def test_calls_with_varying_shapes_gloo():
    run_gloo(_varying_shapes, 2)

