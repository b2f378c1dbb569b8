"""tcgen05 GEMM (through the C ABI) against a plain fp32 torch matmul of the same bf16 inputs."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def ref_epilogue(acc, bias, act):
    if bias is not None:
        acc = acc + bias
    if act == 1:
        acc = acc * torch.sigmoid(acc)
    elif act == 2:
        acc = torch.relu(acc)
    return acc


@pytest.fixture(params=["single", "pair"])
def tile_mode(request, ctx):
    """Large products run either on one CTA per 128 x 256 tile or on a two-CTA cluster per 256 x 256 tile."""
    ctx.set_option("gemm_pair_tiles", 2 if request.param == "pair" else 0)
    yield request.param
    ctx.set_option("gemm_pair_tiles", 1)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 128), (200, 256, 256), (4032, 1024, 1024),
                                   (4032, 4096, 1024), (4032, 1024, 4096), (37, 640, 1024), (20000, 256, 256),
                                   (1, 128, 64), (9500, 2048, 1024), (19000 + 77, 1024, 256)])
def test_bf16_store_modes(ctx, tile_mode, M, N, K):
    import scriptrs_b200 as sb

    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda", generator=g) * 0.1
    acc = a.float() @ w.float().t()
    # f32 store, no activation: only the accumulation order differs
    out = torch.full((M, N), float("nan"), device="cuda")
    torch.cuda.synchronize()  # the context launches on its own stream
    sb.gemm(ctx, a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, d_bias=bias.data_ptr(), out_mode=1)
    ctx.synchronize()
    ref = ref_epilogue(acc, bias, 0)
    err = (out - ref).norm() / ref.norm()
    assert torch.isfinite(out).all()
    assert err < 1e-5, float(err)
    # bf16 store with SiLU
    outb = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    sb.gemm(ctx, a.data_ptr(), w.data_ptr(), outb.data_ptr(), M, N, K, d_bias=bias.data_ptr(), act=1, out_mode=0)
    ctx.synchronize()
    ref = ref_epilogue(acc, bias, 1)
    err = (outb.float() - ref).norm() / ref.norm()
    assert err < 4e-3, float(err)
    # residual accumulate with ReLU and alpha = 0.5
    res0 = torch.randn(M, N, device="cuda", generator=g)
    res = res0.clone()
    torch.cuda.synchronize()
    sb.gemm(ctx, a.data_ptr(), w.data_ptr(), res.data_ptr(), M, N, K, d_bias=bias.data_ptr(), act=2, out_mode=2,
            alpha=0.5)
    ctx.synchronize()
    ref = res0 + 0.5 * ref_epilogue(acc, bias, 2)
    err = (res - ref).norm() / ref.norm()
    assert err < 1e-5, float(err)


def test_rows_beyond_m_are_untouched(ctx):
    import scriptrs_b200 as sb

    M, N, K = 130, 128, 64
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    out = torch.full((M + 126, N), 7.0, device="cuda")
    torch.cuda.synchronize()
    sb.gemm(ctx, a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, out_mode=1)
    ctx.synchronize()
    assert (out[M:] == 7.0).all()
    ref = a.float() @ w.float().t()
    assert (out[:M] - ref).norm() / ref.norm() < 1e-5


def test_unsupported_shapes_are_rejected(ctx):
    import scriptrs_b200 as sb

    a = torch.zeros(128, 96, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(128, 96, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(128, 128, device="cuda")
    with pytest.raises(sb.ScriptrsError) as e:
        sb.gemm(ctx, a.data_ptr(), w.data_ptr(), out.data_ptr(), 128, 128, 96, out_mode=1)
    assert e.value.status == 11


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 256, 1024), (4032, 4096, 1024), (4032, 1024, 4096),
                                   (9500 + 3, 2048, 1024)])
def test_fp8_e4m3_with_row_and_channel_scales(ctx, tile_mode, M, N, K):
    """e4m3 operands, fp32 accumulation, per-row and per-output-channel scales applied in the epilogue."""
    import scriptrs_b200 as sb

    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    rs = a.abs().amax(dim=1) / 448.0
    cs = w.abs().amax(dim=1) / 448.0
    aq = (a / rs[:, None]).to(torch.float8_e4m3fn)
    wq = (w / cs[:, None]).to(torch.float8_e4m3fn)
    bias = torch.randn(N, device="cuda", generator=g) * 0.1
    ref = (aq.float() @ wq.float().t()) * rs[:, None] * cs[None, :] + bias
    out = torch.full((M, N), float("nan"), device="cuda")
    torch.cuda.synchronize()
    sb.gemm(ctx, aq.data_ptr(), wq.data_ptr(), out.data_ptr(), M, N, K, d_bias=bias.data_ptr(), out_mode=1, fp8=True,
            d_row_scale=rs.data_ptr(), d_col_scale=cs.data_ptr())
    ctx.synchronize()
    assert torch.isfinite(out).all()
    err = (out - ref).norm() / ref.norm()
    assert err < 1e-5, float(err)   # same quantised operands on both sides: only the summation order differs
