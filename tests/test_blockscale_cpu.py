"""The PyTorch statement of the block-scaled GEMM agrees with dequantise-then-matmul."""
import torch


def test_blockscale_oracle_matches_dequantised_matmul():
    import tempname_new_b200 as flux
    from tempname_new_b200.ops.quantization import (quantize_square_blockwise_torch,
                                                    quantize_vector_blockwise_torch)
    torch.manual_seed(0)
    M, N, K = 256, 384, 512
    x, w = torch.randn(M, K), torch.randn(N, K) * 0.1
    xq, sx = quantize_vector_blockwise_torch(x)
    wq, sw = quantize_square_blockwise_torch(w)
    out = flux.blockscale_gemm_torch(xq, wq, sx, sw, torch.float32)
    xd = xq.float() * sx.permute(0, 2, 1).reshape(M, K // 128).repeat_interleave(128, dim=1)
    wd = wq.float() * sw.repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)
    torch.testing.assert_close(out, xd @ wd.t(), rtol=1e-4, atol=1e-3)
    assert ((out - x @ w.t()).norm() / (x @ w.t()).norm()).item() < 0.05
    # per-column ("groupwise") weight scales
    wq2, sw2 = quantize_vector_blockwise_torch(w)
    out2 = flux.BlockScaleGemm().wgrad(xq, wq2, input_scale=sx, weight_scale=sw2)
    wd2 = wq2.float() * sw2.permute(0, 2, 1).reshape(N, K // 128).repeat_interleave(128, dim=1)
    torch.testing.assert_close(out2.float(), (xd @ wd2.t()).bfloat16().float(), rtol=2e-2, atol=2e-2)
