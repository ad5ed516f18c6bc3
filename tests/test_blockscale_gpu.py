"""Block-scaled fp8 GEMM on the GPU against the PyTorch statement of the op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda", 0)


def _quantized(M, N, K, dev, seed=0):
    import tempname_new_b200 as flux
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(M, K, device=dev, generator=g).bfloat16()
    w = (torch.randn(N, K, device=dev, generator=g) * 0.05).bfloat16()
    # make block scales differ a lot so that a wrong scale index shows
    x[: M // 2] *= 8
    w[:, K // 2:] *= 0.1
    qz = flux.Quantization(torch.bfloat16, torch.float8_e4m3fn)
    xq, sx, _, _ = qz.quantize_vector_blockwise(x, False)
    wq, sw, _, _ = qz.quantize_square_blockwise(w, False)
    return x, w, xq, sx, wq, sw


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (512, 1024, 2048), (1024, 3584, 8192),
                                   (384, 2176, 640)])   # 128 x 256 tiles with a half-empty last column tile
def test_blockscale_gemm(dev, M, N, K):
    import tempname_new_b200 as flux
    x, w, xq, sx, wq, sw = _quantized(M, N, K, dev)
    op = flux.BlockScaleGemm(torch.float8_e4m3fn, torch.float8_e4m3fn, torch.bfloat16)
    out = op.forward(xq, wq, input_scale=sx, weight_scale=sw)
    ref = flux.blockscale_gemm_torch(xq, wq, sx, sw, torch.float32)
    full = x.float() @ w.float().t()
    tol = 2e-2 * max(1.0, ref.abs().max().item())
    assert (out.float() - ref).abs().max().item() <= tol
    # and the quantised product tracks the unquantised one
    rel = (out.float() - full).norm() / full.norm()
    assert rel.item() < 0.06


def test_blockscale_bias_and_grouped(dev):
    import tempname_new_b200 as flux
    M, N, K, E = 512, 256, 512, 2
    x, w, xq, sx, wq, sw = _quantized(M, N * E, K, dev, seed=1)
    op = flux.BlockScaleGemm()
    bias = torch.randn(N * E, device=dev).bfloat16()
    out = op.forward(xq, wq, bias=bias, input_scale=sx, weight_scale=sw)
    ref = flux.blockscale_gemm_torch(xq, wq, sx, sw, torch.float32, bias)
    assert (out.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    wq3, sw3 = wq.view(E, N, K), sw.view(E, N // 128, K // 128)
    outg = op.forward_grouped(xq, torch.tensor([256, 256]), wq3, input_scale=sx, weight_scale=sw3)
    # the same on one stream must give the same bits
    one = flux.BlockScaleGemm(num_streams=1).forward_multi_stream(xq, [256, 256], wq3, input_scale=sx, weight_scale=sw3)
    assert torch.equal(outg, one)
    for e in range(E):
        r = flux.blockscale_gemm_torch(xq[e * 256:(e + 1) * 256], wq3[e], sx[e * 2:(e + 1) * 2], sw3[e], torch.float32)
        assert (outg[e * 256:(e + 1) * 256].float() - r).abs().max().item() <= 2e-2 * max(1.0, r.abs().max().item())


def test_blockscale_per_expert_forms_on_side_streams(dev):
    """Experts of different sizes (one empty) dealt over three side streams, called twice in a row and
    followed at once by work on the caller's stream: the join must order it after every expert."""
    import tempname_new_b200 as flux
    N, K, E = 256, 512, 5
    splits = [128, 384, 0, 256, 640]
    M = sum(splits)
    x, w, xq, sx, wq, sw = _quantized(M, N * E, K, dev, seed=3)
    wq3, sw3 = wq.view(E, N, K), sw.view(E, N // 128, K // 128)
    op = flux.BlockScaleGemm(num_streams=3)
    for _ in range(2):
        out = op.forward_multi_stream(xq, splits, wq3, input_scale=sx, weight_scale=sw3)
        total = out.float().sum()                       # the caller's stream reads the result right away
    row = 0
    ref_total = 0.0
    for e, cnt in enumerate(splits):
        if cnt:
            r = flux.blockscale_gemm_torch(xq[row:row + cnt], wq3[e], sx[row // 128:(row + cnt) // 128], sw3[e],
                                           torch.float32)
            assert (out[row:row + cnt].float() - r).abs().max().item() <= 2e-2 * max(1.0, r.abs().max().item())
            ref_total += out[row:row + cnt].float().sum().item()
        row += cnt
    assert abs(total.item() - ref_total) <= 1e-3 * max(1.0, abs(ref_total))


@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (1024, 1024, 1024)])
def test_blockscale_wgrad_form_per_column_weight_scales(dev, M, N, K):
    """Both operands carry 1x128 scales (weight_scale [N/128, K/128, 128]): the weight-gradient form,
    on the kernel, against the PyTorch statement."""
    import tempname_new_b200 as flux
    x, w, xq, sx, _, _ = _quantized(M, N, K, dev, seed=2)
    qz = flux.Quantization(torch.bfloat16, torch.float8_e4m3fn)
    wq, sw, _, _ = qz.quantize_vector_blockwise(w, False)           # 1x128 scales for the weight rows too
    assert tuple(sw.shape) == (N // 128, K // 128, 128)
    op = flux.BlockScaleGemm()
    out = op.wgrad(xq, wq, input_scale=sx, weight_scale=sw)
    ref = flux.blockscale_gemm_torch(xq, wq, sx, sw, torch.float32)
    assert (out.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())


def test_blockscale_ragged_rows(dev):
    """M that is not a multiple of 128: the last row block is partial (its scales exist, rows clipped)."""
    import tempname_new_b200 as flux
    M, N, K = 300, 256, 512
    x, w, xq, sx, wq, sw = _quantized(M, N, K, dev, seed=3)
    assert sx.shape[0] == 3
    out = flux.BlockScaleGemm().forward(xq, wq, input_scale=sx, weight_scale=sw)
    ref = flux.blockscale_gemm_torch(xq, wq, sx, sw, torch.float32)
    assert out.shape == (M, N)
    assert (out.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
