"""GPU parity of the mixture-of-experts steps (routing, plan, gather + quantise, grouped GEMM
with a device-built table, combine) against the CPU oracle, step by step and end to end at
8192 tokens x 64 experts (N = 2048, K = 7168: the MoE benchmark configuration).

The routing is pinned to the reference (tests/golden/moe_routing_vectors.npz holds what the
reference's own routing lines compute, moe/moe_fibench_ref.py:106-134); the NVFP4 expert
arithmetic has no reference vector (the reference's experts are FP8): parity unpinned there.
Tolerances: integer results exact; weights 1e-6; outputs rtol = atol = 1e-2 on bf16 / fp16."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def moe_oracle():
    from oracle import moe_oracle
    return moe_oracle


def _dense(idx, w, experts):
    dense = torch.zeros((idx.shape[0], experts), dtype=torch.float32)
    dense.scatter_(1, idx.long().cpu(), w.cpu())
    return dense


@pytest.mark.parametrize("case", ["e256", "e256b", "e64"])
def test_routing_matches_the_reference_vectors(pkg, case):
    g = np.load(os.path.join(ROOT, "tests", "golden", "moe_routing_vectors.npz"))
    logits = torch.from_numpy(g[f"{case}_logits"]).cuda()
    bias = torch.from_numpy(g[f"{case}_bias"]).cuda()
    idx, w = pkg.moe.route(logits, bias, 8, 4, 8, float(g[f"{case}_scale"]))
    torch.cuda.synchronize()
    assert np.array_equal(np.sort(idx.cpu().numpy(), axis=1), g[f"{case}_topk_sorted"])
    assert torch.allclose(_dense(idx, w, logits.shape[1]), torch.from_numpy(g[f"{case}_weights"]), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("tokens,experts,n_group,topk_group,top_k", [(8192, 64, 8, 4, 8), (1000, 256, 8, 4, 8),
                                                                     (300, 64, 1, 1, 8), (77, 32, 4, 2, 3)])
def test_routing_and_plan_against_oracle(pkg, moe_oracle, tokens, experts, n_group, topk_group, top_k):
    gen = torch.Generator().manual_seed(tokens)
    logits = torch.randn((tokens, experts), generator=gen)
    bias = torch.randn((experts,), generator=gen) * 0.1
    idx, w = pkg.moe.route(logits.cuda(), bias.cuda(), n_group, topk_group, top_k, 2.5)
    want_idx, want_w = moe_oracle.route(logits, bias, n_group, topk_group, top_k, 2.5, exact_sigmoid=True)
    assert torch.equal(torch.sort(idx.cpu().long(), dim=1).values, torch.sort(want_idx, dim=1).values)
    got_w = _dense(idx, w, experts)
    worst = int((got_w - want_w).abs().max(dim=1).values.argmax())
    assert torch.allclose(got_w, want_w, rtol=1e-5, atol=1e-7), (
        f"token {worst}: experts {idx[worst].tolist()} weights {w[worst].tolist()} "
        f"oracle {want_w[worst][idx[worst].long().cpu()].tolist()} kernel {pkg._lib.last_kernel()}")
    # plan: stable counting sort
    lib = pkg._lib.load()
    i32 = dict(dtype=torch.int32, device="cuda")
    counts, offs, atoms = torch.empty(experts, **i32), torch.empty(experts + 1, **i32), torch.empty(experts + 1, **i32)
    row_of, src = torch.empty(tokens * top_k, **i32), torch.full((tokens * top_k,), -1, **i32)
    scratch = torch.empty(lib.b200_moe_plan_scratch_bytes(tokens, experts, top_k), dtype=torch.uint8, device="cuda")
    pkg._lib.check(lib.b200_moe_plan(idx.data_ptr(), tokens, experts, top_k, counts.data_ptr(), offs.data_ptr(),
                                     atoms.data_ptr(), row_of.data_ptr(), src.data_ptr(), scratch.data_ptr(),
                                     scratch.numel(), torch.cuda.current_stream().cuda_stream, 0))
    torch.cuda.synchronize()
    want_counts, want_offs, tokens_of = moe_oracle.plan(want_idx, experts)
    assert counts.cpu().tolist() == want_counts.tolist() and offs.cpu().tolist() == want_offs.tolist()
    want_atoms = [0]
    for c in want_counts.tolist():
        want_atoms.append(want_atoms[-1] + (c + 127) // 128)
    assert atoms.cpu().tolist() == want_atoms
    src_cpu, row_cpu, idx_cpu = src.cpu(), row_of.cpu().view(tokens, top_k), idx.cpu()
    for e in range(experts):                       # an expert's rows hold its tokens in ascending order
        assert src_cpu[want_offs[e]:want_offs[e + 1]].tolist() == tokens_of[e].tolist()
    t = torch.arange(tokens).view(-1, 1).expand(tokens, top_k)
    assert torch.equal(src_cpu[row_cpu.long()].long(), t)                     # row_of and src_token are inverse maps
    assert torch.all((row_cpu >= offs.cpu()[idx_cpu.long()]) & (row_cpu < offs.cpu()[idx_cpu.long() + 1]))


def _weights(pkg, experts, n, k, seed, device="cuda"):
    data = pkg.inputs.generate_grouped_input([0] * experts, [n] * experts, [k] * experts, experts, seed, dist="uniform16",
                                             device=device)
    b = [abc[1] for abc in data[0]]
    return b, [sf[1] for sf in data[1]], [sf[1] for sf in data[2]]


def _moe_case(pkg, moe_oracle, tokens, experts, n, k, n_group, topk_group, top_k, dtype, seed):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn((tokens, k), generator=gen).to(dtype)
    logits = torch.randn((tokens, experts), generator=gen)
    bias = torch.randn((experts,), generator=gen) * 0.1
    b, sfb, sfb_perm = _weights(pkg, experts, n, k, seed)
    w = pkg.moe.MoEWeights(b, sfb_perm)
    out, buf = pkg.moe.moe_forward(x.cuda(), logits.cuda(), bias.cuda(), w, n_group=n_group, topk_group=topk_group,
                                   top_k=top_k, routed_scaling=2.5, out_dtype=dtype, return_plan=True)
    torch.cuda.synchronize()
    assert pkg._lib.read_status(0) == 0
    want, _idx, _w = moe_oracle.moe_forward(x, logits, bias, [t.cpu() for t in b], sfb, n_group, topk_group, top_k, 2.5,
                                            out_dtype=dtype)
    return x, out, want, buf


@pytest.mark.parametrize("tokens,experts,n,k,dtype", [(200, 16, 256, 512, torch.float16), (96, 32, 128, 256, torch.bfloat16),
                                                      (2048, 8, 1024, 1024, torch.bfloat16)])
def test_moe_layer_small(pkg, oracle, moe_oracle, tokens, experts, n, k, dtype):
    # small cases run the one-CTA grouped kernel; 2048 tokens x top-4 with n = 1024 (32 x 4 pair tiles) is
    # large enough for CTA pairs
    top_k = 4
    x, out, want, buf = _moe_case(pkg, moe_oracle, tokens, experts, n, k, 4, 2, top_k, dtype, seed=tokens)
    assert oracle.compare(out, want, 1e-2, 1e-2) == []
    # the gathered rows are the quantiser applied to the source tokens, byte for byte
    src = buf.src_token.cpu().long()
    packed, _sf = oracle.quantize_nvfp4(x.index_select(0, src))
    assert torch.equal(buf.a_q.cpu(), packed)


def test_moe_layer_8192_tokens_64_experts(pkg, oracle, moe_oracle):
    x, out, want, buf = _moe_case(pkg, moe_oracle, 8192, 64, 2048, 7168, 8, 4, 8, torch.bfloat16, seed=0)
    assert "PairGrouped" in pkg._lib.last_kernel() or "moe_combine" in pkg._lib.last_kernel()
    assert int(buf.counts.sum().item()) == 8192 * 8
    assert oracle.compare(out, want, 1e-2, 1e-2) == []


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("tokens,experts,top_k,k", [(333, 16, 4, 576), (2048, 64, 8, 7168)])
def test_one_pass_scatter_writes_the_two_pass_bytes(pkg, dtype, tokens, experts, top_k, k):
    # b200_moe_quantize_scatter against b200_moe_gather_quantize (whose bytes the layer tests check against the
    # oracle): the same packed rows and the same scale-factor bytes, padding rows of the atoms untouched by both
    lib = pkg._lib.load()
    gen = torch.Generator().manual_seed(tokens + k)
    x = (torch.randn((tokens, k), generator=gen) * 3).to(dtype).cuda()
    idx = torch.stack([torch.randperm(experts, generator=gen)[:top_k] for _ in range(tokens)]).to(torch.int32).cuda()
    i32 = dict(dtype=torch.int32, device="cuda")
    counts, offs, atoms = torch.empty(experts, **i32), torch.empty(experts + 1, **i32), torch.empty(experts + 1, **i32)
    row_of, src = torch.empty(tokens * top_k, **i32), torch.empty(tokens * top_k, **i32)
    scratch = torch.empty(lib.b200_moe_plan_scratch_bytes(tokens, experts, top_k), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    pkg._lib.check(lib.b200_moe_plan(idx.data_ptr(), tokens, experts, top_k, counts.data_ptr(), offs.data_ptr(),
                                     atoms.data_ptr(), row_of.data_ptr(), src.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                     stream, 0))
    code = pkg._lib.DTYPE_F16 if dtype == torch.float16 else pkg._lib.DTYPE_BF16
    sf_bytes = lib.b200_moe_sfa_bytes(tokens, experts, top_k, k)
    out = []
    for one_pass in (False, True):
        a_q = torch.full((tokens * top_k, k // 2), 0xEE, dtype=torch.uint8, device="cuda")
        sfa = torch.full((sf_bytes,), 0xDD, dtype=torch.uint8, device="cuda")
        if one_pass:
            pkg._lib.check(lib.b200_moe_quantize_scatter(x.data_ptr(), code, tokens, k, x.stride(0), row_of.data_ptr(),
                                                         offs.data_ptr(), atoms.data_ptr(), experts, top_k, a_q.data_ptr(),
                                                         sfa.data_ptr(), stream, 0))
        else:
            tmp = torch.empty(lib.b200_moe_gather_scratch_bytes(tokens, k), dtype=torch.uint8, device="cuda")
            pkg._lib.check(lib.b200_moe_gather_quantize(x.data_ptr(), code, tokens, k, x.stride(0), src.data_ptr(),
                                                        offs.data_ptr(), atoms.data_ptr(), experts, top_k, a_q.data_ptr(),
                                                        sfa.data_ptr(), tmp.data_ptr(), tmp.numel(), stream, 0))
        torch.cuda.synchronize()
        out.append((a_q, sfa))
    assert pkg._lib.last_kernel() == "moe_quantize_scatter"
    assert torch.equal(out[0][0], out[1][0])
    assert torch.equal(out[0][1], out[1][1])
    assert not torch.all(out[1][1] == 0xDD)
