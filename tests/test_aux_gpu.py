"""GPU tests of the auxiliary kernels against plain PyTorch statements of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda", 0)


def _dequant_1x128(q, sinv, M, K):
    MB, KB = sinv.shape[0], sinv.shape[1]
    full = sinv.permute(0, 2, 1).reshape(MB * 128, KB)[:M]            # [M, KB]
    return q.float() * full.repeat_interleave(128, dim=1)[:, :K]


@pytest.mark.parametrize("M,K", [(256, 384), (1000, 520), (128, 128), (4096, 2048)])
@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float32])
def test_quantize_vector_blockwise(dev, M, K, in_dtype):
    from tempname_new_b200.ops.quantization import Quantization, quantize_vector_blockwise_torch
    x = (torch.randn(M, K, device=dev) * 3).to(in_dtype)
    x[0, :128] = 0  # an all-zero block
    op = Quantization(in_dtype, torch.float8_e4m3fn)
    q, s, qt, st = op.quantize_vector_blockwise(x, True)
    q_ref, s_ref = quantize_vector_blockwise_torch(x)
    qt_ref, st_ref = quantize_vector_blockwise_torch(x.t().contiguous())
    torch.testing.assert_close(s[..., :], s_ref, rtol=1e-6, atol=0) if M % 128 == 0 else None
    # scales of rows that exist must match; compare dequantised values, allowing one fp8 step
    d, d_ref = _dequant_1x128(q, s, M, K), _dequant_1x128(q_ref, s_ref, M, K)
    assert (d - d_ref).abs().max().item() <= 0.07 * x.float().abs().max().item()
    assert (d - x.float()).abs().max().item() <= 0.07 * x.float().abs().max().item()
    mism = (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean().item()
    assert mism < 1e-4, mism
    dt, dt_ref = _dequant_1x128(qt, st, K, M), _dequant_1x128(qt_ref, st_ref, K, M)
    assert (dt - dt_ref).abs().max().item() <= 0.07 * x.float().abs().max().item()
    assert (dt - x.float().t()).abs().max().item() <= 0.07 * x.float().abs().max().item()
    q2, s2, none_q, none_s = op.quantize_vector_blockwise(x, False)
    assert none_q is None and none_s is None and torch.equal(q2.view(torch.uint8), q.view(torch.uint8))


@pytest.mark.parametrize("M,K", [(256, 384), (1000, 520), (2048, 4096)])
def test_quantize_square_blockwise(dev, M, K):
    from tempname_new_b200.ops.quantization import Quantization, quantize_square_blockwise_torch
    x = (torch.randn(M, K, device=dev) * 2).bfloat16()
    op = Quantization(torch.bfloat16, torch.float8_e4m3fn)
    q, s, qt, st = op.quantize_square_blockwise(x, True)
    q_ref, s_ref = quantize_square_blockwise_torch(x)
    torch.testing.assert_close(s, s_ref, rtol=1e-6, atol=0)
    mism = (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean().item()
    assert mism < 1e-4, mism
    assert torch.equal(qt.view(torch.uint8), q.t().contiguous().view(torch.uint8))
    torch.testing.assert_close(st, s.t().contiguous(), rtol=0, atol=0)
    xb = torch.stack([x, -x * 0.5])
    qb, sb, qtb, stb = op.batch_quantize_square_blockwise(xb, True)
    assert torch.equal(qb[0].view(torch.uint8), q.view(torch.uint8))
    torch.testing.assert_close(sb[1], s * 0.5, rtol=1e-6, atol=0)
    assert qtb.shape == (2, K, M) and stb.shape[0] == 2


@pytest.mark.parametrize("n", [1, 2047, 2048, 4097, 1048580, 1048573, 8388603])
def test_inplace_cast(dev, n):
    from tempname_new_b200.ops.misc import InplaceCast, inplace_cast_fp32_to_bf16
    op = InplaceCast(8388608, dev)
    for _ in range(2):
        t = torch.rand(n, device=dev)
        ref = t.to(torch.bfloat16)
        op.from_fp32_to_bf16(t)
        assert torch.equal(t.view(torch.bfloat16)[:n], ref)
    op.check_status()
    t = torch.randn(n, device=dev)
    ref = t.to(torch.bfloat16)
    inplace_cast_fp32_to_bf16(t)
    assert torch.equal(t.view(torch.bfloat16)[:n], ref)


def test_bitwise_check_and_uniform(dev):
    from tempname_new_b200.ops.misc import bitwise_check, uniform_initialize
    a = torch.randn(1000, 333, device=dev).bfloat16()
    b = a.clone()
    assert bitwise_check(a, b)
    b[999, 332] += 1
    assert not bitwise_check(a, b)
    t = torch.empty(1 << 20, device=dev)
    uniform_initialize(t, 7, -0.5, 1.5)
    assert t.min().item() >= -0.5 and t.max().item() < 1.5
    assert abs(t.mean().item() - 0.5) < 0.01
    t2 = torch.empty_like(t)
    uniform_initialize(t2, 7, -0.5, 1.5)
    assert bitwise_check(t, t2)
    h = torch.empty(4096, device=dev, dtype=torch.bfloat16)
    uniform_initialize(h, 1, 0.0, 1.0)
    assert 0.4 < h.float().mean().item() < 0.6


@pytest.mark.parametrize("tokens,topk,E", [(64, 2, 8), (5000, 8, 64), (8192, 4, 32), (1, 1, 1)])
def test_moe_index_build(dev, tokens, topk, E):
    from tempname_new_b200.ops.misc import calc_scatter_index, moe_index_build
    g = torch.Generator(device=dev).manual_seed(3)
    ce = torch.randint(0, E, (tokens, topk), device=dev, generator=g, dtype=torch.int32)
    splits, offsets, scatter, gather, tki = moe_index_build(ce, E)
    flat = ce.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    ref_scatter = torch.empty_like(order)
    ref_scatter[order] = torch.arange(order.numel(), device=dev)
    assert torch.equal(splits.long(), torch.bincount(flat, minlength=E))
    assert torch.equal(offsets[1:].long(), torch.bincount(flat, minlength=E).cumsum(0))
    assert torch.equal(scatter.reshape(-1).long(), ref_scatter)
    assert torch.equal(gather.long(), order // topk)
    assert torch.equal(tki.long(), order % topk)
    assert torch.equal(calc_scatter_index(ce, splits).reshape(-1).long(), ref_scatter)


def test_rows_sum_kernels(dev):
    """topk_scatter_reduce and bsr_reduce on the row-sum kernel against fp32 statements."""
    import tempname_new_b200 as flux
    g = torch.Generator(device=dev).manual_seed(4)
    rows, topk, H = 1000, 4, 384
    x = torch.randn(rows * topk, H, device=dev, generator=g).bfloat16()
    idx = torch.randperm(rows * topk, device=dev, generator=g).to(torch.int32)
    out = flux.topk_scatter_reduce(x, idx, topk)
    ref = x[idx.long().view(rows, topk)].float().sum(1)
    assert out.shape == (rows, H)
    assert (out.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    slabs = torch.randn(6, 300, 256, device=dev, generator=g).half()
    o2 = torch.empty(300, 256, device=dev, dtype=torch.float16)
    flux.bsr_reduce(slabs, o2, 128, 128)
    ref2 = slabs.float().sum(0)
    assert (o2.float() - ref2).abs().max().item() <= 1e-2 * max(1.0, ref2.abs().max().item())
