"""GPU parity of the activation quantiser (fp16 / bf16 -> NVFP4) against the CPU
restatement in oracle/, byte for byte, and its use as the GEMM's A operand."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _unpermute(oracle, sf_perm, rows, k):
    return oracle.unpermute_sf(sf_perm.cpu(), rows, k // 16)[:, :, 0]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,k", [(128, 256), (200, 512), (1, 64), (1000, 1792), (4096, 7168)])
def test_matches_oracle_bit_for_bit(pkg, oracle, dtype, rows, k):
    g = torch.Generator().manual_seed(rows * 31 + k)
    x = (torch.randn(rows, k, generator=g) * torch.rand(rows, 1, generator=g) * 8).to(dtype)
    q, sf_perm = pkg.quantize.quantize_nvfp4(x.cuda())
    torch.cuda.synchronize()
    want_q, want_sf = oracle.quantize_nvfp4(x)
    assert torch.equal(q.view(torch.uint8).cpu()[:, :, 0], want_q)
    assert torch.equal(_unpermute(oracle, sf_perm, rows, k), want_sf)
    assert pkg.formats.is_kernel_sf_layout(sf_perm, rows, k, 1)


def test_edge_values(pkg, oracle):
    # zeros, negative zero, exact rounding ties, values that saturate the scale factor, tiny blocks
    rows, k = 128, 256
    x = torch.zeros(rows, k, dtype=torch.float16)
    x[0, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    x[1, :16] = 65504.0                      # amax / 6 > 448: the scale saturates, codes saturate at 6
    x[2, :16] = -0.0
    x[3, :16] = 6.0e-8                       # subnormal fp16: the scale rounds to zero, codes are zero
    x[4, 16:32] = torch.linspace(-3, 3, 16)
    x[5, :] = torch.arange(k, dtype=torch.float32).half() / 7
    for dtype in (torch.float16, torch.bfloat16):
        xd = x.to(dtype)
        q, sf_perm = pkg.quantize.quantize_nvfp4(xd.cuda())
        torch.cuda.synchronize()
        want_q, want_sf = oracle.quantize_nvfp4(xd)
        assert torch.equal(q.view(torch.uint8).cpu()[:, :, 0], want_q), dtype
        assert torch.equal(_unpermute(oracle, sf_perm, rows, k), want_sf), dtype


def test_padding_rows_get_zero_scale_factors(pkg):
    rows, k = 72, 256
    x = torch.randn(rows, k).half().cuda()
    _q, sf_perm = pkg.quantize.quantize_nvfp4(x)
    torch.cuda.synchronize()
    raw = sf_perm.view(torch.uint8).cpu()        # (32, 4, 1, 4, 4, 1): row = a + 32 * b
    row = torch.arange(32).view(32, 1) + 32 * torch.arange(4).view(1, 4)
    assert torch.all(raw[:, :, 0, :, :, 0][row >= rows] == 0)
    assert torch.any(raw[:, :, 0, :, :, 0][row < rows] != 0)


def test_row_pitch_and_rejections(pkg, oracle):
    big = torch.randn(64, 1024).half().cuda()
    view = big[:, :512]                           # pitch 1024, k 512
    q, sf_perm = pkg.quantize.quantize_nvfp4(view)
    torch.cuda.synchronize()
    want_q, want_sf = oracle.quantize_nvfp4(view.cpu())
    assert torch.equal(q.view(torch.uint8).cpu()[:, :, 0], want_q)
    assert torch.equal(_unpermute(oracle, sf_perm, 64, 512), want_sf)
    # a view that is only 16-byte aligned with a pitch that is not a multiple of 32 bytes
    odd = torch.randn(40, 520).half().cuda()[:, 8:8 + 256]
    q, sf_perm = pkg.quantize.quantize_nvfp4(odd)
    torch.cuda.synchronize()
    want_q, want_sf = oracle.quantize_nvfp4(odd.cpu())
    assert torch.equal(q.view(torch.uint8).cpu()[:, :, 0], want_q)
    assert torch.equal(_unpermute(oracle, sf_perm, 40, 256), want_sf)
    with pytest.raises(ValueError, match="64"):
        pkg.quantize.quantize_nvfp4(torch.zeros(8, 48, dtype=torch.float16, device="cuda"))
    with pytest.raises(ValueError):
        pkg.quantize.quantize_nvfp4(torch.zeros(8, 64, dtype=torch.float32, device="cuda"))
    with pytest.raises(ValueError):
        pkg.quantize.quantize_nvfp4(torch.zeros(8, 64, dtype=torch.float16))


def test_quantised_activations_feed_the_dual_gemm(pkg, oracle):
    # quantise A on the GPU, keep the generator's B1/B2: the GEMM must agree with the oracle run on
    # the oracle-quantised A (same bytes), i.e. the quantiser's output is a valid `a` / `sfa_perm`
    m, n, k = 256, 256, 512
    data = list(pkg.inputs.generate_input(m, n, k, 1, 5, dist="reference", device="cuda"))
    x = (torch.randn(m, k, generator=torch.Generator().manual_seed(9)) * 0.5).half()
    q, sf_perm = pkg.quantize.quantize_nvfp4(x.cuda())
    data[0], data[6] = q, sf_perm
    out = pkg.dual_gemm.custom_kernel(tuple(data))
    torch.cuda.synchronize()
    want_q, want_sf = oracle.quantize_nvfp4(x)
    cpu = [t.cpu() if t is not None else None for t in data]
    fp32 = oracle.dual_gemm_fp32(want_q.view(m, k // 2, 1), cpu[1], cpu[2], want_sf.view(m, k // 16, 1), cpu[4], cpu[5])
    assert oracle.compare(out, fp32.to(torch.float16), 1e-3, 1e-3, expected_fp32=fp32) == []


@pytest.mark.parametrize("m,n,k", [(256, 128, 256), (512, 384, 1024), (2048, 1024, 512)])
@pytest.mark.parametrize("dist", ["reference", "uniform16"])
def test_dual_gemm_with_quantised_output_equals_quantising_its_fp16_result(pkg, oracle, m, n, k, dist):
    data = pkg.inputs.generate_input(m, n, k, 1, 21, dist=dist, device="cuda")
    a, b1, b2, _, _, _, sfa, sfb1, sfb2, c = data
    q, sf_perm = pkg.dual_gemm.dual_gemm_quantized(a, b1, b2, sfa, sfb1, sfb2)
    c.fill_(float("nan"))
    plain = pkg.dual_gemm.custom_kernel(data, variant=5)      # same kernel, fp16 output
    torch.cuda.synchronize()
    assert pkg._lib.read_status(0) == 0
    want_q, want_sf = oracle.quantize_nvfp4(plain[:, :, 0].cpu())
    assert torch.equal(q.view(torch.uint8).cpu()[:, :, 0], want_q)
    assert torch.equal(_unpermute(oracle, sf_perm, m, n), want_sf)
    assert pkg.formats.is_kernel_sf_layout(sf_perm, m, n, 1)


def test_quantised_output_feeds_a_second_gemm(pkg, oracle):
    # SwiGLU FFN: h = silu(x W1^T) * (x W2^T) quantised in the epilogue, then y = h W3^T as a one-group GEMM
    m, n, k = 256, 512, 256
    data = pkg.inputs.generate_input(m, n, k, 1, 4, dist="reference", device="cuda")
    a, b1, b2, _, _, _, sfa, sfb1, sfb2, _c = data
    hq, hsf = pkg.dual_gemm.dual_gemm_quantized(a, b1, b2, sfa, sfb1, sfb2)
    down = pkg.inputs.generate_grouped_input([m], [256], [n], 1, 8, dist="reference", device="cuda")
    (_a3, w3, y), (_sfa3, sfw3), (_sfa3p, sfw3p) = down[0][0], down[1][0], down[2][0]
    down[0][0] = (hq, w3, y)
    down[2][0] = (hsf, sfw3p)
    out = pkg.group_gemm.custom_kernel(down)[0]
    torch.cuda.synchronize()
    h_bytes = hq.view(torch.uint8).cpu()
    h_sf = oracle.unpermute_sf(hsf.cpu(), m, n // 16)
    want = oracle.gemm_fp32(h_bytes, h_sf, w3.cpu(), sfw3.cpu()).to(torch.float16)
    assert oracle.compare(out, want, 1e-3, 1e-3) == []


def test_quantised_output_needs_m_multiple_of_256(pkg):
    data = pkg.inputs.generate_input(128, 128, 256, 1, 0, device="cuda")
    a, b1, b2, _, _, _, sfa, sfb1, sfb2, _c = data
    with pytest.raises(ValueError, match="256"):
        pkg.dual_gemm.dual_gemm_quantized(a, b1, b2, sfa, sfb1, sfb2)


def test_benchmark_size_fused_output_equals_the_quantiser(pkg, oracle):
    # M=8192, N=14336, K=4096: 48 tiles per CTA pair, both accumulator buffers in rotation.  The fused epilogue
    # and the stand-alone quantiser applied to the plain kernel's C must give the same bytes everywhere; a window
    # of both is checked against the oracle.
    m, n, k = 8192, 14336, 4096
    d = pkg.inputs.generate_input(m, n, k, 1, 0, dist="reference", device="cuda")
    a, b1, b2, _, _, _, sfa, sfb1, sfb2, _c = d
    q, sf_perm = pkg.dual_gemm.dual_gemm_quantized(a, b1, b2, sfa, sfb1, sfb2)
    plain = pkg.dual_gemm.custom_kernel(d)
    q2, sf_perm2 = pkg.quantize.quantize_nvfp4(plain[:, :, 0])
    torch.cuda.synchronize()
    assert pkg._lib.read_status(0) == 0
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8))
    assert torch.equal(sf_perm.view(torch.uint8), sf_perm2.view(torch.uint8))
    want_q, want_sf = oracle.quantize_nvfp4(plain[:512, :, 0].cpu())
    assert torch.equal(q.view(torch.uint8).cpu()[:512, :, 0], want_q)
    assert torch.equal(_unpermute(oracle, sf_perm, m, n)[:512], want_sf)
