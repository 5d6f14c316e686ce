"""Pin of the grouped GEMM to a third-party kernel on the GPU.

The grouped problem's ``reference.py`` (the ``torch._scaled_mm`` loop its checker would call) is not part of
the reference checkout, and the reference's own grouped kernels do not run under the installed DSL.  vLLM ships
the CUTLASS grouped block-scaled GEMM its fused MoE uses (``vllm._custom_ops.cutlass_fp4_moe_mm``): the same
packed e2m1 operands, the same swizzled e4m3 scale factors, fp32 accumulation over k in steps of 64, fp16
output.  Given the same bytes it has to give the same numbers; the test asks for the reference checker's
tolerance (rtol = atol = 1e-3) and reports how many outputs differ at all.  It skips where vLLM or its compiled
op is not usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL_REFERENCE = 1e-3


def _vllm_grouped():
    try:
        from vllm import _custom_ops as ops
    except Exception as exc:                       # noqa: BLE001
        pytest.skip(f"vLLM is not importable here: {str(exc)[:200]}")
    if not hasattr(ops, "cutlass_fp4_moe_mm"):
        pytest.skip("this vLLM has no cutlass_fp4_moe_mm")
    return ops.cutlass_fp4_moe_mm


@pytest.mark.parametrize("rows", [[128, 256, 384, 128], [72, 200, 1000, 40, 513, 8]])
def test_same_numbers_as_vllms_cutlass_grouped_gemm(pkg, oracle, rows):
    grouped = _vllm_grouped()
    experts, n, k = len(rows), 1024, 1536
    data = pkg.inputs.generate_grouped_input(rows, [n] * experts, [k] * experts, experts, 5, dist="reference",
                                             device="cuda", fill_c=100.0)

    def flat_sf(perm):            # the buffer behind a permuted view: [row tile][k tile][32][4][4]
        return perm.view(torch.uint8).permute(5, 2, 4, 0, 1, 3).contiguous().view(-1, k // 16)

    a_cat = torch.cat([abc[0][:, :, 0].view(torch.uint8) for abc in data[0]], dim=0)
    b_all = torch.stack([abc[1][:, :, 0].view(torch.uint8) for abc in data[0]], dim=0)
    sfa_cat = torch.cat([flat_sf(sf[0]) for sf in data[2]], dim=0).view(torch.float8_e4m3fn)
    sfb_all = torch.stack([flat_sf(sf[1]) for sf in data[2]], dim=0).view(torch.float8_e4m3fn)
    first_row, first_sf_row = [0], [0]
    for m in rows:
        first_row.append(first_row[-1] + m)
        first_sf_row.append(first_sf_row[-1] + -(-m // 128) * 128)
    theirs = torch.full((first_row[-1], n), float("nan"), dtype=torch.float16, device="cuda")
    try:
        grouped(theirs, a_cat, b_all, sfa_cat, sfb_all, torch.ones(experts, dtype=torch.float32, device="cuda"),
                torch.tensor([[m, n, k] for m in rows], dtype=torch.int32, device="cuda"),
                torch.tensor(first_row[:-1], dtype=torch.int32, device="cuda"),
                torch.tensor(first_sf_row[:-1], dtype=torch.int32, device="cuda"))
        torch.cuda.synchronize()
    except Exception as exc:                       # noqa: BLE001
        pytest.skip(f"vLLM's grouped GEMM does not run here: {str(exc)[:200]}")
    ours = pkg.group_gemm.custom_kernel(data)
    torch.cuda.synchronize()
    assert pkg._lib.read_status(0) == 0
    different = 0
    for g, (c, m) in enumerate(zip(ours, rows)):
        got, want = c[:, :, 0].cpu(), theirs[first_row[g]:first_row[g] + m].cpu()
        assert oracle.compare(got.unsqueeze(-1), want.unsqueeze(-1), TOL_REFERENCE, TOL_REFERENCE) == [], g
        different += int((got.view(torch.int16) != want.view(torch.int16)).sum())
    assert different <= first_row[-1] * n // 1000, different       # in practice zero: the same bits
