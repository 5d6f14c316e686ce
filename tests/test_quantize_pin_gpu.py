"""Pin of the activation quantiser's recipe and byte layout to a third-party NVFP4 quantiser.

The reference generates pre-quantised operands and has no quantiser of its own, so the recipe of
``b200_quantize_nvfp4`` (scale factor = e4m3(amax / 6) per 16 values, value = e2m1(x / scale factor),
round to nearest even, low nibble = even k, scale factors in 128 x 4 tiles) has nothing in the reference
to be compared with.  vLLM ships a CUDA NVFP4 quantiser (``vllm._custom_ops.scaled_fp4_quant``) that
writes the same two buffers for the same consumer, cuBLASLt's block-scaled GEMM: packed e2m1 [rows, k/2]
and e4m3 scale factors in the swizzled 128 x 4 layout.  With a global scale of 1 the two recipes are the
same arithmetic; vLLM evaluates the two divisions with approximate reciprocals, so a quotient that is an
exact rounding tie in real arithmetic (common for fp16 / bf16 inputs with their few mantissa bits: about
0.3 % of the values of the test data) may land on the other side, one e2m1 step away.  The test therefore
asks for the same layout, the same scale-factor bytes and the same value bytes except for that fraction.  It skips where vLLM or its compiled
op is not usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_DIFFERENT_SCALE_BYTES = 5e-4
MAX_DIFFERENT_VALUE_BYTES = 2e-2


def _vllm_quantiser():
    try:
        from vllm import _custom_ops as ops
    except Exception as exc:                       # noqa: BLE001 - any import problem means "not usable here"
        pytest.skip(f"vLLM is not importable here: {str(exc)[:200]}")
    if not hasattr(ops, "scaled_fp4_quant"):
        pytest.skip("this vLLM has no scaled_fp4_quant")
    return ops.scaled_fp4_quant


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,k", [(128, 256), (1024, 1792), (4096, 7168)])
def test_same_bytes_as_vllm_up_to_reciprocal_ties(pkg, dtype, rows, k):
    quant = _vllm_quantiser()
    g = torch.Generator().manual_seed(rows + k)
    x = (torch.randn(rows, k, generator=g) * torch.rand(rows, 1, generator=g) * 8).to(dtype).cuda()
    try:
        their_q, their_sf = quant(x, torch.ones(1, dtype=torch.float32, device="cuda"))
        torch.cuda.synchronize()
    except Exception as exc:                       # noqa: BLE001
        pytest.skip(f"vLLM's quantiser does not run here: {str(exc)[:200]}")
    q, sf_perm = pkg.quantize.quantize_nvfp4(x)
    torch.cuda.synchronize()
    assert pkg._lib.read_status(0) == 0
    ours_q = q.view(torch.uint8)[:, :, 0]
    assert their_q.shape == ours_q.shape
    # the buffer behind sf_perm is [row tile][k tile][32][4][4], the swizzled layout itself
    ours_sf = sf_perm.view(torch.uint8).permute(5, 2, 4, 0, 1, 3).contiguous().view(-1)
    their_sf = their_sf.contiguous().view(torch.uint8).view(-1)
    assert their_sf.numel() == ours_sf.numel()
    sf_diff = (their_sf != ours_sf).float().mean().item()
    q_diff = (their_q.view(torch.uint8) != ours_q).float().mean().item()
    assert sf_diff <= MAX_DIFFERENT_SCALE_BYTES, sf_diff
    assert q_diff <= MAX_DIFFERENT_VALUE_BYTES, q_diff
    # a differing value is one e2m1 step away (further only inside a block whose scale factor differs)
    lo_a, lo_b = their_q.view(torch.uint8) & 0xF, ours_q & 0xF
    step = ((lo_a & 7).int() - (lo_b & 7).int()).abs()
    assert (step > 1).float().mean().item() <= MAX_DIFFERENT_SCALE_BYTES
