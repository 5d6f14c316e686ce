"""The MoE oracle's routing against vectors made by executing the reference's own routing
lines (tests/golden/make_moe_golden.py), its planning against first principles, and the host-side
argument checks of the MoE entry points (no GPU needed)."""
import os

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FAKE = 0x7F0000000000


@pytest.fixture(scope="module")
def moe_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "moe_routing_vectors.npz"))


@pytest.fixture(scope="module")
def moe_oracle():
    from oracle import moe_oracle
    return moe_oracle


@pytest.mark.parametrize("case", ["e256", "e256b", "e64"])
def test_oracle_routing_reproduces_the_reference(moe_oracle, moe_golden, case):
    logits = torch.from_numpy(moe_golden[f"{case}_logits"])
    bias = torch.from_numpy(moe_golden[f"{case}_bias"])
    idx, weights = moe_oracle.route(logits, bias, 8, 4, 8, float(moe_golden[f"{case}_scale"]))
    assert np.array_equal(np.sort(idx.numpy(), axis=1), moe_golden[f"{case}_topk_sorted"])
    assert np.array_equal(weights.numpy(), moe_golden[f"{case}_weights"])
    # every token: 8 experts from at most 4 of the 8 groups, weights sum to the scale
    group = idx // (logits.shape[1] // 8)
    assert all(len(set(g.tolist())) <= 4 for g in group)
    assert torch.allclose(weights.sum(1), torch.full((logits.shape[0],), float(moe_golden[f"{case}_scale"])), rtol=1e-5)


def test_oracle_plan(moe_oracle):
    idx = torch.tensor([[0, 3], [3, 1], [0, 1], [3, 0]])
    counts, offsets, tokens_of = moe_oracle.plan(idx, 5)
    assert counts.tolist() == [3, 2, 0, 3, 0] and offsets.tolist() == [0, 3, 5, 5, 8, 8]
    assert tokens_of[0].tolist() == [0, 2, 3] and tokens_of[3].tolist() == [0, 1, 3] and tokens_of[2].numel() == 0


def test_moe_entry_points_reject_bad_arguments(pkg):
    lib = pkg._lib.load()
    E = pkg._lib
    assert lib.b200_moe_route(FAKE, None, 16, 300, 8, 4, 8, 1.0, FAKE, FAKE, None, 0) == E.E_LIMIT
    assert lib.b200_moe_route(FAKE, None, 16, 64, 7, 4, 8, 1.0, FAKE, FAKE, None, 0) == E.E_SHAPE
    assert lib.b200_moe_route(FAKE, None, 16, 64, 8, 1, 16, 1.0, FAKE, FAKE, None, 0) == E.E_SHAPE       # 16 > 8 kept experts
    assert lib.b200_moe_route(None, None, 16, 64, 8, 4, 8, 1.0, FAKE, FAKE, None, 0) == E.E_NULL
    assert lib.b200_moe_plan_scratch_bytes(8192, 64, 8) == 64 * 64 * 4
    assert lib.b200_moe_plan(FAKE, 16, 64, 8, FAKE, FAKE, FAKE, FAKE, FAKE, FAKE, 4, None, 0) == E.E_WORKSPACE
    assert lib.b200_moe_sfa_bytes(8192, 64, 8, 7168) == (512 + 64) * 112 * 512
    assert lib.b200_moe_gather_scratch_bytes(8192, 7168) == 8192 * (3584 + 448)
    assert lib.b200_moe_gather_quantize(FAKE, 0, 16, 100, 128, FAKE, FAKE, FAKE, 64, 8, FAKE, FAKE, FAKE, 1 << 20, None, 0) == E.E_SHAPE
    assert lib.b200_moe_gather_quantize(FAKE, 5, 16, 128, 128, FAKE, FAKE, FAKE, 64, 8, FAKE, FAKE, FAKE, 1 << 20, None, 0) == E.E_VARIANT
    assert lib.b200_moe_gather_quantize(FAKE, 0, 16, 128, 128, FAKE, FAKE, FAKE, 64, 8, FAKE, FAKE, FAKE, 64, None, 0) == E.E_WORKSPACE
    assert lib.b200_moe_quantize_scatter(FAKE, 0, 16, 100, 128, FAKE, FAKE, FAKE, 64, 8, FAKE, FAKE, None, 0) == E.E_SHAPE
    assert lib.b200_moe_quantize_scatter(FAKE, 5, 16, 128, 128, FAKE, FAKE, FAKE, 64, 8, FAKE, FAKE, None, 0) == E.E_VARIANT
    assert lib.b200_moe_quantize_scatter(FAKE, 0, 16, 128, 128, None, FAKE, FAKE, 64, 8, FAKE, FAKE, None, 0) == E.E_NULL
    assert lib.b200_moe_quantize_scatter(FAKE, 0, 16, 128, 100, FAKE, FAKE, FAKE, 64, 8, FAKE, FAKE, None, 0) == E.E_ALIGN
    assert lib.b200_moe_gemm_workspace_bytes(64) == 64 * 512 + 256
    assert lib.b200_moe_combine(FAKE, 2050, FAKE, FAKE, 16, 8, 0, FAKE, 2050, None, 0) == E.E_SHAPE
    assert lib.b200_moe_combine(FAKE, 2048, FAKE, FAKE, 16, 8, 7, FAKE, 2048, None, 0) == E.E_VARIANT


def test_no_cpu_path_for_moe(pkg):
    with pytest.raises(ValueError, match="CUDA"):
        pkg.moe.route(torch.zeros(4, 64), None, 8, 4, 8)
