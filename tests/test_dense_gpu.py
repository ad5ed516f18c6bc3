"""GPU numerics of the tcgen05 dense kernel against a plain fp32 PyTorch statement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda", 0)


def _ab(M, N, K, dev, dtype=torch.bfloat16, seed=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    a = (torch.randn(M, K, device=dev, generator=g) * (2.0 / K ** 0.5)).to(dtype)
    b = (torch.randn(N, K, device=dev, generator=g)).to(dtype)
    return a, b


def _tol(ref):
    return 2e-2 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("M,N,K,tile_n", [
    (128, 256, 64, 256), (128, 128, 64, 128), (256, 512, 512, 256), (384, 640, 1024, 128),
    (200, 264, 72, 256), (200, 264, 72, 128), (1000, 1000, 1000, 0), (4096, 2048, 4096, 0),
])
def test_gemm_only_bf16(dev, M, N, K, tile_n):
    from tempname_new_b200.ops import _dense
    a, b = _ab(M, N, K, dev)
    out = torch.full((M, N), float("nan"), device=dev, dtype=torch.bfloat16)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    _dense.plain_gemm(a, b, out, tile_n=tile_n, status=status)
    ref = a.float() @ b.float().t()
    assert status.tolist()[0] == 0
    assert not torch.isnan(out).any()
    assert (out.float() - ref).abs().max().item() <= _tol(ref)


@pytest.mark.parametrize("act", [None, "gelu", "relu", "silu"])
def test_gemm_only_bias_act(dev, act):
    import tempname_new_b200 as flux
    from tempname_new_b200.ops import _dense
    from tempname_new_b200.ops.gemm_only import apply_act
    a, b = _ab(512, 768, 512, dev)
    bias = torch.randn(768, device=dev).bfloat16()
    out = torch.empty(512, 768, device=dev, dtype=torch.bfloat16)
    _dense.plain_gemm(a, b, out, bias, act=act)
    ref = apply_act(a.float() @ b.float().t() + bias.float(), act)
    assert (out.float() - ref).abs().max().item() <= _tol(ref)
    bias2 = torch.randn(512, 768, device=dev).bfloat16()   # full [M, N] bias
    op = flux.GemmOnly(torch.bfloat16)
    out2 = op.forward(a, b, bias=bias2)
    ref2 = a.float() @ b.float().t() + bias2.float()
    assert (out2.float() - ref2).abs().max().item() <= _tol(ref2)


def test_gemm_only_fp16_and_transpose_weight(dev):
    import tempname_new_b200 as flux
    a, b = _ab(256, 384, 256, dev, torch.float16)
    op = flux.GemmOnly(torch.float16, transpose_weight=True)
    out = op.forward(a, b.t().contiguous())
    ref = a.float() @ b.float().t()
    assert out.dtype == torch.float16
    assert (out.float() - ref).abs().max().item() <= 1e-2 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("M,N,K,knobs", [
    (512, 384, 320, {}),                                            # 128-wide single-CTA tiles, ragged K
    (1024, 512, 1024, {"cta_group": 2, "tile_n": 256}),             # CTA pairs, 256 x 256
    (2048, 1024, 512, {"cta_group": 2, "tile_n": 256, "tile_m": 512}),   # CTA pairs, 512 x 256
    (1000, 520, 264, {"cta_group": 1, "tile_n": 256}),              # ragged everywhere
])
def test_weight_held_as_kn_is_read_in_place(dev, M, N, K, knobs, monkeypatch):
    """A [K, N] weight (``transpose_weight``) goes to the kernel as it is: MN-major operand tiles.
    The result must equal both the fp32 statement and the kernel's result on a re-laid-out copy."""
    import tempname_new_b200 as flux
    from tempname_new_b200.ops import _dense
    torch.manual_seed(M + N)
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w_kn = torch.randn(K, N, device=dev, dtype=torch.bfloat16)     # [K, N], N contiguous
    assert _dense.kn_in_place(w_kn.t())
    out = _dense.plain_gemm(a, w_kn.t(), torch.empty(M, N, device=dev, dtype=torch.bfloat16), **knobs)
    ref = a.float() @ w_kn.float()
    assert (out.float() - ref).abs().max().item() <= _tol(ref)
    out_copy = _dense.plain_gemm(a, w_kn.t().contiguous(), torch.empty_like(out), **knobs)
    assert torch.equal(out, out_copy)
    # the public op takes the same route
    op = flux.GemmOnly(torch.bfloat16, transpose_weight=True)
    assert (op.forward(a, w_kn).float() - ref).abs().max().item() <= _tol(ref)
    # and the copy is still there for whoever switches the in-place read off
    monkeypatch.setenv("FLUXB_KN_IN_PLACE", "0")
    assert (op.forward(a, w_kn).float() - ref).abs().max().item() <= _tol(ref)


@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_gemm_only_fp8_per_tensor_scale(dev, dtype):
    import tempname_new_b200 as flux
    a, b = _ab(256, 512, 1024, dev)
    a8, b8 = a.to(dtype), (b * 0.25).to(dtype)
    sa = torch.tensor([0.5], device=dev)
    sb = torch.tensor([4.0], device=dev)
    op = flux.GemmOnly(dtype, output_dtype=torch.bfloat16, use_fp8_gemm=True)
    out = op.forward(a8, b8, input_scale=sa, weight_scale=sb)
    ref = (a8.float() @ b8.float().t()) * 2.0
    assert (out.float() - ref).abs().max().item() <= 3e-2 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("M,N,K", [(256, 512, 1024), (1024, 768, 512)])
def test_gemm_only_int8(dev, M, N, K):
    """Signed 8-bit operands, s32 accumulation, dequantised by the two per-tensor scales."""
    import tempname_new_b200 as flux
    g = torch.Generator(device="cpu").manual_seed(5)
    a8 = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).to(dev)
    b8 = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).to(dev)
    sa = torch.tensor([0.01], device=dev)
    sb = torch.tensor([0.02], device=dev)
    op = flux.GemmOnly(torch.int8, output_dtype=torch.bfloat16)
    out = op.forward(a8, b8, input_scale=sa, weight_scale=sb)
    ref = (a8.double() @ b8.double().t()).float() * 2e-4
    assert (out.float() - ref).abs().max().item() <= 1e-2 * max(1.0, ref.abs().max().item())


def test_single_rank_fused_ops_match_matmul(dev):
    """World size 1: AGKernel and GemmRS reduce to the plain kernel and must agree with it."""
    import os
    import torch.distributed as dist
    import tempname_new_b200 as flux
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    a, b = _ab(512, 256, 384, dev)
    ref = a.float() @ b.float().t()
    ag = flux.AGKernel(dist.group.WORLD, 1, 512, 256, 384, torch.bfloat16)
    rs = flux.GemmRS(dist.group.WORLD, 1, 512, 256, torch.bfloat16)
    gathered = torch.empty_like(a)
    o1 = ag.forward(a, b, gathered_input=gathered)
    o2 = rs.forward(a, b)
    assert torch.equal(gathered, a)
    assert (o1.float() - ref).abs().max().item() <= _tol(ref)
    assert (o2.float() - ref).abs().max().item() <= _tol(ref)
    ag.check_status()
    rs.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("a2a_only", [False, True])
def test_single_rank_ulysses_projections(dev, a2a_only):
    """World size 1: the pre-attention epilogue store and the post-attention input read (in place,
    and through the landing buffer when the re-laid-out input is asked for) against fp32 matmul."""
    import os
    import torch.distributed as dist
    import tempname_new_b200 as flux
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    pg = dist.group.WORLD
    bs, seq, nh, hd = 2, 384, 4, 128
    hidden = nh * hd
    x = (torch.randn(bs, seq, hidden, device=dev) * 0.5).bfloat16()
    w = (torch.randn(hidden, hidden, device=dev) * 0.05).bfloat16()
    y = (x.reshape(-1, hidden).float() @ w.float().t())
    pre = flux.GemmAllToAllTranspose(pg, 1, 1, bs, seq, hidden, hd, hidden, torch.bfloat16)
    (q,) = pre.forward(x, w)
    ref_q = y.reshape(bs, seq, nh, hd).permute(0, 2, 1, 3)
    assert (q.float() - ref_q).abs().max().item() <= _tol(ref_q)
    pre.check_status()
    attn = (torch.randn(bs, nh, seq, hd, device=dev) * 0.5).bfloat16()
    inp = attn.permute(0, 2, 1, 3).contiguous() if a2a_only else attn
    gi_ref = attn.permute(0, 2, 1, 3).reshape(bs, seq, hidden)
    ref = gi_ref.reshape(-1, hidden).float() @ w.float().t()
    post = flux.AllToAllTransposeGemm(pg, 1, 1, bs, nh, seq, hd, torch.bfloat16, a2a_only=a2a_only)
    for _ in range(2):
        out = post.forward(inp, w)
        assert (out.reshape(-1, hidden).float() - ref).abs().max().item() <= _tol(ref)
    gi = torch.empty(bs, seq, hidden, device=dev, dtype=torch.bfloat16)
    out = post.forward(inp, w, a2a_transpose_output=gi)
    assert torch.equal(gi, gi_ref)
    assert (out.reshape(-1, hidden).float() - ref).abs().max().item() <= _tol(ref)
    post.check_status()


def test_bounded_wait_reports_timeout(dev):
    """A device wait on a flag that nothing sets gives up after its limit and reports it in the
    status record; the context stays usable."""
    import ctypes
    from tempname_new_b200 import _native
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    rc = _native.lib().fluxb_wait_flag(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint32(1),
                                       ctypes.c_uint64(200_000_000), ctypes.c_void_p(status.data_ptr()),
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    st = status.tolist()
    assert st[0] == 12 and st[2] == 0 and st[3] == 1
    # a satisfied wait leaves the status clean, and the device still works
    flag.fill_(3)
    status.zero_()
    _native.lib().fluxb_wait_flag(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint32(2),
                                  ctypes.c_uint64(200_000_000), ctypes.c_void_p(status.data_ptr()),
                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0


def test_smoke_entry(dev):
    import __graft_entry__ as g
    g.smoke()


@pytest.mark.gpu
def test_kernel_timeline_records_stamps(dev):
    """The optional per-CTA timeline: stamps are ordered and cover every CTA that ran."""
    import tempname_new_b200 as flux
    a, b = _ab(1024, 1024, 512, dev)
    op = flux.GemmOnly(torch.bfloat16)
    with flux.KernelTimeline(dev) as tl:
        out = op.forward(a, b)
        torch.cuda.synchronize()
    ref = a.float() @ b.float().t()
    assert (out.float() - ref).abs().max().item() <= _tol(ref)
    s = tl.summary()
    assert s["entry_us"]["min"] == 0.0
    assert s["first_tile_loads_us"]["min"] > 0.0
    assert s["epilogue_done_us"]["max"] >= s["last_tile_loads_us"]["max"]
    # off again: the buffer stays as it is
    before = tl.buf.clone()
    op.forward(a, b)
    torch.cuda.synchronize()
    assert torch.equal(before, tl.buf)



def test_sm_margin_leaves_sms_to_a_second_stream(dev):
    """``sm_margin`` shrinks the grid of a fused op (reference: the ``sm_margin`` arguments of the
    Ulysses and MoE ops, src/gemm_a2a_transpose/ths_op/gemm_all2all_transpose.cc:559-560). With 16
    SMs left free the op runs beside a stream of elementwise kernels, uses at most 148 - 16 CTAs
    and still completes with the right result."""
    import os
    import torch.distributed as dist
    import tempname_new_b200 as flux
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    a, b = _ab(8192, 4096, 1024, dev)                  # more tiles than CTAs at any tile shape
    ref = a.float() @ b.float().t()
    rs = flux.GemmRS(dist.group.WORLD, 1, 8192, 4096, torch.bfloat16)
    rs.sm_margin = 16
    side = torch.cuda.Stream(dev)
    busy = torch.ones(64 << 20, device=dev)
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        for _ in range(40):
            busy.mul_(1.0001)
    with flux.KernelTimeline(dev) as tl:
        out = rs.forward(a, b)
        torch.cuda.synchronize()
    rs.check_status()
    assert (out.float() - ref).abs().max().item() <= _tol(ref)
    ctas = int((tl.buf[:, 6] > 0).sum().item())        # CTAs that stamped the end of their epilogue
    assert 0 < ctas <= sms - 16


def test_int8_per_row_and_per_column_scales(dev):
    """The reference's int8 convention: input_scale [M, 1], weight_scale [1, N] - honoured element by
    element on the GPU, and any other shape is refused instead of being cut to its first element."""
    import tempname_new_b200 as flux
    M, N, K = 384, 640, 512
    g = torch.Generator(device="cpu").manual_seed(9)
    a8 = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).to(dev)
    b8 = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).to(dev)
    sa = (torch.rand(M, 1, device=dev) * 0.02 + 0.001)
    sb = (torch.rand(1, N, device=dev) * 0.02 + 0.001)
    op = flux.GemmOnly(torch.int8, output_dtype=torch.bfloat16)
    out = op.forward(a8, b8, input_scale=sa, weight_scale=sb)
    ref = (a8.double() @ b8.double().t()).float() * sa * sb
    assert (out.float() - ref).abs().max().item() <= 1e-2 * max(1.0, ref.abs().max().item())
    # per-row scale with a per-tensor weight scale
    out2 = op.forward(a8, b8, input_scale=sa, weight_scale=torch.tensor([0.01], device=dev))
    ref2 = (a8.double() @ b8.double().t()).float() * sa * 0.01
    assert (out2.float() - ref2).abs().max().item() <= 1e-2 * max(1.0, ref2.abs().max().item())
    with pytest.raises(ValueError):
        op.forward(a8, b8, input_scale=sa[:7], weight_scale=sb)
