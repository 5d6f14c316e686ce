"""The oracle against vectors produced by the reference's own helper functions
(tests/golden/reference_vectors.npz, see tests/golden/make_golden.py) and
against the reference's analytical known-answer inputs."""
import numpy as np
import pytest
import torch


def test_e2m1_decode_table_and_nibble_order(oracle, golden):
    # reference: nvfp4_to_fp16, group_gemm/group_gemm_cute5_v2.py:4436-4457
    raw = torch.from_numpy(golden["decode_in"])          # [16, 16, 1]: every byte value
    want = torch.from_numpy(golden["decode_out"])        # [16, 16, 2]: (low, high) per byte
    got = oracle.decode_e2m1(raw)                        # [16, 32, 1]
    got = got[:, :, 0].reshape(16, 16, 2)
    assert torch.equal(got, want)
    # -0.0 must stay negative zero
    assert torch.signbit(got[0, 8, 0])


def test_e4m3_decode_matches_format_definition(oracle, c_oracle):
    allb = torch.arange(256, dtype=torch.uint8)
    got = oracle.decode_e4m3(allb)
    for b in range(256):
        want = oracle.e4m3_value(b)
        cval = c_oracle.load().oracle_e4m3_to_f32(b)
        if want != want:
            assert torch.isnan(got[b]) and cval != cval
        else:
            assert got[b].item() == want == cval, b
    assert oracle.e4m3_value(0x38) == 1.0      # the reference's "unit scale factor" byte


def test_to_blocked_matches_reference(oracle, golden):
    # dual_gemm/reference.py:13-24 and the padded copy group_gemm_cute5_v2.py:4461-4483
    got = oracle.to_blocked(torch.from_numpy(golden["to_blocked_in"]))
    assert np.array_equal(got.numpy(), golden["to_blocked_out"])
    got = oracle.to_blocked(torch.from_numpy(golden["to_blocked_pad_in"]))
    assert np.array_equal(got.numpy(), golden["to_blocked_pad_out"])


@pytest.mark.parametrize("name,rows", [("sfa", 128), ("sfb1", 256), ("sfb2", 256)])
def test_permuted_layout_matches_reference_scatter(oracle, golden, name, rows):
    # dual_gemm/reference.py:151-188, generate_input(m=128, n=256, k=512, l=2, seed=1111)
    plain = torch.from_numpy(golden[f"dual_{name}"])               # [rows, 32, 2]
    dense = torch.from_numpy(golden[f"dual_{name}_perm"])          # (L, rest_mn, rest_k, 32, 4, 4)
    shape = tuple(golden[f"dual_{name}_perm_shape"])
    stride = tuple(golden[f"dual_{name}_perm_stride"])
    rest_mn, rest_k = rows // 128, 8
    assert shape == (32, 4, rest_mn, 4, rest_k, 2)
    assert stride == (16, 4, 512 * rest_k, 1, 512, 512 * rest_k * rest_mn)
    perm_view = dense.permute(3, 4, 1, 5, 2, 0)
    assert torch.equal(oracle.unpermute_sf(perm_view, rows, 32), plain)
    assert torch.equal(oracle.permute_sf(plain), perm_view)        # no padding rows here
    flat = dense.flatten()
    for (i, j, b) in [(0, 0, 0), (1, 0, 0), (37, 5, 1), (127, 31, 1), (rows - 1, 17, 0)]:
        assert flat[oracle.sf_offset(i, j, b, rest_mn, rest_k)] == plain[i, j, b]
    # the permuted buffer of one batch is the cuBLAS "blocked" layout of that batch
    for b in range(2):
        assert torch.equal(dense[b].flatten(), oracle.to_blocked(plain[:, :, b]))


def test_grouped_reordered_layout_with_padding(oracle, golden):
    # group_gemm/group_gemm_cute5_v2.py:4489-4535 with M = 72 (padding rows are random)
    plain = torch.from_numpy(golden["grp_sf_in"])                  # [72, 16, 1]
    dense = torch.from_numpy(golden["grp_sf_perm"])
    assert tuple(golden["grp_sf_perm_shape"]) == (32, 4, 1, 4, 4, 1)
    perm_view = dense.permute(3, 4, 1, 5, 2, 0)
    assert torch.equal(oracle.unpermute_sf(perm_view, 72, 16), plain)


def test_reference_operand_distribution(golden):
    # dual_gemm/reference.py:117-121: every nibble has bit 2 cleared
    for name in ("a", "b1", "b2"):
        raw = golden[f"dual_{name}"]
        assert not np.any(raw & 0x44)
    assert tuple(golden["dual_a_shape"]) == (128, 256, 2)
    assert tuple(golden["dual_a_stride"]) == (256, 1, 128 * 256)


def _kat(pkg, **kw):
    return pkg.inputs.generate_grouped_input((128,), (128,), (256,), 1, 5, device="cpu", **kw)


def test_known_answer_constant_inputs(pkg, oracle, c_oracle):
    # constant 1.0 operands with unit scale factors: every output equals K
    data = _kat(pkg, constant_a=True, constant_b=True, unit_sfa=True, unit_sfb=True)
    out = oracle.grouped_gemm(data)[0]
    assert torch.all(out == 256.0)
    (a, b, _), (sfa_p, sfb_p) = data[0][0], data[2][0]
    assert torch.all(c_oracle.gemm(a, b, sfa_p, sfb_p) == 256.0)


def test_known_answer_identity(pkg, oracle):
    # identity A and B, unit scale factors: C = I (128 x 128 corner)
    data = _kat(pkg, identity_a=True, identity_b=True, unit_sfa=True, unit_sfb=True)
    out = oracle.grouped_gemm(data)[0][:, :, 0].float()
    assert torch.equal(out, torch.eye(128))


def test_known_answer_single_element(pkg, oracle):
    # one non-zero element of A (row 3, k 77, value -1.5), constant-1 B, unit SF
    data = _kat(pkg, single_a=(3, 77, -1.5), constant_b=True, unit_sfa=True, unit_sfb=True)
    out = oracle.grouped_gemm(data)[0][:, :, 0].float()
    want = torch.zeros(128, 128)
    want[3, :] = -1.5
    assert torch.equal(out, want)


def test_known_answer_dual_silu(pkg, oracle, c_oracle):
    # A = B1 = B2 = constant 1, unit scale factors: r1 = r2 = K, C = silu(K) * K
    d = list(pkg.inputs.generate_input(128, 128, 256, 1, 0, device="cpu"))
    ones = torch.full((128, 128, 1), 0x22, dtype=torch.uint8)
    unit = torch.full((128, 16, 1), 0x38, dtype=torch.uint8)
    d[0] = d[1] = d[2] = ones
    d[3] = d[4] = d[5] = unit
    d[6] = d[7] = d[8] = oracle.permute_sf(unit)
    want = torch.tensor(256.0 / (1.0 + np.exp(-256.0)) * 256.0).to(torch.float16)   # 65536 -> inf
    assert torch.isinf(want)
    assert torch.all(oracle.dual_gemm(d) == want)
    assert torch.all(c_oracle.dual_gemm(d) == want)


@pytest.mark.parametrize("dist", ["reference", "uniform16"])
def test_c_oracle_equals_python_oracle(pkg, oracle, c_oracle, dist):
    d = pkg.inputs.generate_input(128, 256, 512, 1, 0, dist=dist, device="cpu")
    py = oracle.dual_gemm(d)
    assert oracle.compare(c_oracle.dual_gemm(d), py, 1e-3, 1e-3) == []
    assert torch.equal(oracle.dual_gemm_from_permuted(d).view(torch.int16), py.view(torch.int16))
    if dist == "uniform16":
        # this distribution overflows fp16 for a sizeable fraction of outputs
        frac = torch.isinf(py).float().mean().item()
        assert 0.05 < frac < 0.3


def test_f32_to_f16_rounding(c_oracle):
    f = c_oracle.load().oracle_f32_to_f16
    vals = [0.0, -0.0, 1.0, 65504.0, 65519.99, 65520.0, -65520.0, 1e-8, 5.96e-8, 6.1e-5, 0.1, 1 / 3, 2049.0, 2051.0,
            float("inf"), 2.98e-8, 2.9802325e-8]
    for v in vals:
        want = torch.tensor(v, dtype=torch.float32).to(torch.float16).view(torch.int16).item() & 0xFFFF
        assert f(v) == want, v
    rnd = torch.randn(2000, generator=torch.Generator().manual_seed(3)) * torch.logspace(-9, 5, 2000)
    for v in rnd.tolist():
        want = torch.tensor(v, dtype=torch.float32).to(torch.float16).view(torch.int16).item() & 0xFFFF
        assert f(v) == want, v


def test_compare_rule(oracle):
    e = torch.tensor([1.0, float("inf"), -float("inf"), 100.0], dtype=torch.float16)
    assert oracle.compare(e.clone(), e, 1e-2, 1e-2) == []
    r = e.clone(); r[1] = 65504.0
    assert oracle.compare(r, e, 1e-2, 1e-2) != []                       # inf position mismatch
    fp32 = torch.tensor([1.0, 65525.0, -1e9, 100.0])
    assert oracle.compare(r, e, 1e-2, 1e-2, expected_fp32=fp32) == []   # forgiven: on the overflow boundary
    r = e.clone(); r[3] = 102.0
    assert oracle.compare(r, e, 1e-2, 1e-2) != []
