"""Host-side logic: input generators in the reference's layouts, sharding, and
the world_size-2 path over gloo."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_dual_generator_layout_matches_reference(pkg, golden):
    d = pkg.inputs.generate_input(128, 256, 512, 2, 1111, device="cpu")
    names = ["a", "b1", "b2", "sfa", "sfb1", "sfb2", "sfa_perm", "sfb1_perm", "sfb2_perm"]
    for name, t in zip(names, d[:9]):
        assert tuple(t.shape) == tuple(golden[f"dual_{name}_shape"]), name
        assert tuple(t.stride()) == tuple(golden[f"dual_{name}_stride"]), name
    assert d[0].dtype == pkg.formats.FP4X2 and d[3].dtype == torch.float8_e4m3fn and d[9].dtype == torch.float16
    assert tuple(d[9].shape) == (128, 256, 2) and tuple(d[9].stride()) == (256, 1, 128 * 256)
    # reference distribution: bit 2 of every nibble is clear; uniform16 uses all codes
    assert not (d[0].view(torch.uint8) & 0x44).any()
    u = pkg.inputs.generate_input(128, 128, 256, 1, 0, dist="uniform16", device="cpu")
    assert len(torch.unique(u[0].view(torch.uint8) & 0xF)) == 16
    sf = u[3].float()
    assert sf.min() >= 0.25 and sf.max() <= 2.0
    # determinism
    again = pkg.inputs.generate_input(128, 256, 512, 2, 1111, device="cpu")
    assert all(torch.equal(x.view(torch.uint8), y.view(torch.uint8)) for x, y in zip(d[:9], again[:9]))


def test_generated_scale_factors_round_trip(pkg, oracle):
    d = pkg.inputs.generate_input(256, 128, 512, 2, 3, device="cpu")
    assert torch.equal(oracle.unpermute_sf(d[6], 256, 32), d[3].view(torch.uint8))
    assert torch.equal(oracle.permute_sf(d[4]).contiguous(), d[7].view(torch.uint8).contiguous())
    flat = d[6].view(torch.uint8).permute(5, 2, 4, 0, 1, 3).contiguous().flatten()
    for (i, j, b) in [(0, 0, 0), (200, 31, 1), (129, 4, 0)]:
        assert flat[pkg.formats.sf_offset(i, j, b, 2, 8)] == d[3].view(torch.uint8)[i, j, b]


def test_grouped_generator(pkg, oracle):
    m, n, k = [40, 0, 384], [512, 128, 256], [256, 512, 768]
    data = pkg.inputs.generate_grouped_input(m, n, k, 3, 1111, device="cpu")
    abc, sfs, perm, sizes = data
    assert sizes == [(40, 512, 256, 1), (0, 128, 512, 1), (384, 256, 768, 1)]
    for (a, b, c), (sfa, sfb), (sfa_p, sfb_p), (mi, ni, ki, _) in zip(abc, sfs, perm, sizes):
        assert tuple(a.shape) == (mi, ki // 2, 1) and tuple(b.shape) == (ni, ki // 2, 1)
        assert tuple(c.shape) == (mi, ni, 1) and c.dtype == torch.float16
        assert tuple(sfa_p.shape) == (32, 4, (mi + 127) // 128, 4, ki // 64, 1)
        assert pkg.formats.is_kernel_sf_layout(sfb_p, ni, ki, 1)
        if mi:
            assert torch.equal(oracle.unpermute_sf(sfa_p, mi, ki // 16), sfa.view(torch.uint8))
    # padding rows of the reordered A scale factors are not all zero (random, like the reference)
    pad = perm[0][0].view(torch.uint8)[8:, 1:, 0]
    assert pad.float().abs().sum() > 0


def test_moe_counts_and_uniform_rows(pkg):
    counts = pkg.inputs.moe_expert_counts(8192, 64, 8, seed=0)
    assert len(counts) == 64 and sum(counts) == 8192 * 8
    assert counts == pkg.inputs.moe_expert_counts(8192, 64, 8, seed=0)
    rows = pkg.inputs.uniform_group_rows(8, seed=0)
    assert len(rows) == 8 and all(r % 64 == 0 and 64 <= r <= 1024 for r in rows)


def test_column_ranges(pkg):
    sh = pkg.shard
    for n, world in [(14336, 8), (14336, 1), (4096, 3), (384, 8), (1792, 4)]:
        spans = [sh.column_range(n, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(lo % 128 == 0 and hi % 128 == 0 for lo, hi in spans)
        widths = [hi - lo for lo, hi in spans]
        assert max(widths) - min(widths) <= 128
    assert sh.column_range(14336, 3, 8) == (5376, 7168)
    with pytest.raises(ValueError):
        sh.column_range(100, 0, 2)


def test_dual_shards_reassemble_on_cpu(pkg, oracle):
    d = pkg.inputs.generate_input(128, 512, 256, 1, 5, device="cpu")
    full = oracle.dual_gemm(d)
    out = torch.zeros_like(full)
    for r in range(4):
        s = pkg.shard.shard_dual_input(d, r, 4)
        lo, hi = pkg.shard.column_range(512, r, 4)
        assert s[9].data_ptr() == d[9][:, lo:hi].data_ptr() and s[9].stride(0) == 512
        assert pkg.formats.is_kernel_sf_layout(s[7], hi - lo, 256, 1)
        out[:, lo:hi] = oracle.dual_gemm_from_permuted(s)       # uses only what a kernel would receive
    assert torch.equal(out.view(torch.int16), full.view(torch.int16))


def test_group_assignment(pkg):
    sizes = [(m, 2048, 7168, 1) for m in (10, 900, 20, 30, 800, 40, 0, 700)]
    blocks = pkg.shard.assign_groups(sizes, 4)
    assert blocks == [[0, 1], [2, 3], [4, 5], [6, 7]]
    bal = pkg.shard.assign_groups(sizes, 4, balance=True)
    assert sorted(i for b in bal for i in b) == list(range(8))
    load = [sum(sizes[i][0] for i in b) for b in bal]
    assert max(load) <= 900
    assert pkg.shard.assign_groups(sizes[:3], 4) == [[0], [1], [2], []]


WORKER = r'''
import importlib, os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
pkg = importlib.import_module("llm-assisted-kernel-dev_b200")
from oracle import nvfp4_oracle as orc
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
# dual GEMM: every rank computes (with the oracle standing in for the kernel) its column shard
d = pkg.inputs.generate_input(128, 768, 256, 1, 9, device="cpu")
s = pkg.shard.shard_dual_input(d, rank, world)
mine = orc.dual_gemm_from_permuted(s).contiguous()
lo, hi = pkg.shard.column_range(768, rank, world)
full = pkg.shard.gather_dual_output(mine, 768)   # optional gather; the data path itself has no collective
assert torch.equal(full.view(torch.int16), orc.dual_gemm(d).view(torch.int16)), "dual shards do not reassemble"
# grouped GEMM: groups are owned by ranks
g = pkg.inputs.generate_grouped_input([40, 0, 136, 64, 8], [128, 256, 128, 384, 128], [256] * 5, 5, 2, device="cpu")
owned = pkg.shard.assign_groups(g[3], world)
local = pkg.shard.shard_grouped_input(g, rank, world)
outs = orc.grouped_gemm(local)
assert len(outs) == len(owned[rank])
want = orc.grouped_gemm(g)
for idx, o in zip(owned[rank], outs):
    assert torch.equal(o.view(torch.int16), want[idx].view(torch.int16))
count = torch.tensor([len(outs)])
dist.all_reduce(count)
assert count.item() == 5
dist.destroy_process_group()
sys.stdout.write(f"rank-{rank}-ok\n")
'''


def test_world_size_two_over_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29731", str(script), ROOT]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert res.stdout.count("rank-0-ok") == 1 and res.stdout.count("rank-1-ok") == 1
