"""Second pin of the MoE routing, to an implementation that shares no code with the reference.

``b200_moe_route`` restates the reference's no-aux routing (moe/moe_fibench_ref.py:106-134: sigmoid scores, a
per-expert bias for the selection only, groups ranked by the sum of their two best biased scores, ``top_k``
experts out of the best ``topk_group`` groups, weights = unbiased scores renormalised and scaled) and is pinned
to those lines through ``tests/golden/moe_routing_vectors.npz``.  vLLM ships a fused CUDA kernel for the same
DeepSeek-V3 routing (``vllm._custom_ops.grouped_topk``); on the same logits both must choose the same experts
with the same weights.  The test skips where vLLM or its compiled op is not usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,experts,n_group,topk_group,top_k,scale", [(512, 256, 8, 4, 8, 2.5), (300, 64, 8, 4, 8, 1.0)])
def test_same_experts_and_weights_as_vllms_grouped_topk(pkg, tokens, experts, n_group, topk_group, top_k, scale):
    try:
        from vllm import _custom_ops as ops
    except Exception as exc:                       # noqa: BLE001
        pytest.skip(f"vLLM is not importable here: {str(exc)[:200]}")
    if not hasattr(ops, "grouped_topk"):
        pytest.skip("this vLLM has no grouped_topk")
    gen = torch.Generator().manual_seed(tokens + experts)
    logits = torch.randn((tokens, experts), generator=gen).cuda()
    bias = (torch.randn((experts,), generator=gen) * 0.1).cuda()
    try:
        res = ops.grouped_topk(logits, n_group, topk_group, top_k, True, float(scale), bias, 1)
        torch.cuda.synchronize()
    except Exception as exc:                       # noqa: BLE001
        pytest.skip(f"vLLM's grouped_topk does not run here: {str(exc)[:200]}")
    their_idx = next(t for t in res if not t.is_floating_point()).long().cpu()
    their_w = next(t for t in res if t.is_floating_point()).float().cpu()
    idx, w = pkg.moe.route(logits, bias, n_group, topk_group, top_k, scale)
    torch.cuda.synchronize()
    idx, w = idx.long().cpu(), w.cpu()
    # compare per token as expert -> weight maps: the two kernels need not order the slots alike
    ours = torch.zeros((tokens, experts)).scatter_(1, idx, w)
    theirs = torch.zeros((tokens, experts)).scatter_(1, their_idx, their_w)
    same_set = ((ours != 0) == (theirs != 0)).all(dim=1)
    assert same_set.float().mean().item() >= 0.995, same_set.float().mean().item()   # exact score ties aside
    assert torch.allclose(ours[same_set], theirs[same_set], rtol=1e-4, atol=1e-6)
