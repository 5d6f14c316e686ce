"""The grouped-GEMM entry point for callers that cannot allocate device memory
(b200_grouped_gemm_nvfp4_static): an inference server that has given the whole
GPU to its own memory pools, or a plugin living inside another runtime's budget,
has no workspace to hand over and may not call cudaMalloc.  The per-group
descriptor table then sits in a fixed array inside the library.

Collected last on purpose (file name), so a run that stops at the first failure
has already executed every other test.  Works alone in a fresh process and after
the rest of the suite: it relies on no state left by other tests."""
import ctypes

import pytest
import torch

FAKE = 0x7F0000000000


def test_more_groups_than_the_table_holds_are_rejected(pkg):
    lib = pkg._lib.load()
    g = pkg._lib.STATIC_MAX_GROUPS + 1
    arr = ctypes.c_void_p * g
    cols = [arr(*[FAKE + 4096 * (5 * i + j) for i in range(g)]) for j in range(5)]
    mnk = (ctypes.c_int * (3 * g))(*([128, 128, 256] * g))
    rc = lib.b200_grouped_gemm_nvfp4_static(g, *cols, mnk, None, 0, None)
    assert rc == pkg._lib.E_LIMIT
    msg = lib.b200_last_error().decode()
    assert str(pkg._lib.STATIC_MAX_GROUPS) in msg and "workspace" in msg
    # the ordinary argument checks apply as well, before any CUDA work
    one = ctypes.c_void_p * 1
    bad = (ctypes.c_int * 3)(64, 100, 256)
    assert lib.b200_grouped_gemm_nvfp4_static(1, *[one(FAKE)] * 5, bad, None, 0, None) == pkg._lib.E_SHAPE
    assert lib.b200_grouped_gemm_nvfp4_static(0, None, None, None, None, None, bad, None, 0, None) == pkg._lib.E_SHAPE


def _through_c_abi(pkg, data):
    """Call the entry point directly through ctypes, as a foreign host would."""
    abc, _, perm, sizes = data
    g = len(sizes)
    arr = ctypes.c_void_p * g
    a = arr(*[t[0].data_ptr() for t in abc])
    b = arr(*[t[1].data_ptr() for t in abc])
    c = arr(*[t[2].data_ptr() for t in abc])
    sfa = arr(*[t[0].data_ptr() for t in perm])
    sfb = arr(*[t[1].data_ptr() for t in perm])
    mnk = (ctypes.c_int * (3 * g))(*[x for s in sizes for x in s[:3]])
    stream = torch.cuda.current_stream().cuda_stream
    rc = pkg._lib.load().b200_grouped_gemm_nvfp4_static(g, a, b, sfa, sfb, c, mnk, stream, torch.cuda.current_device(),
                                                        None)
    pkg._lib.check(rc)


def _oracle_problems(oracle, data, tol):
    want = oracle.grouped_gemm(([tuple(t.cpu() for t in abc) for abc in data[0]], data[1]))
    bad = []
    for g, ((_a, _b, got), w) in enumerate(zip(data[0], want)):
        bad += [(g, msg) for msg in oracle.compare(got, w, tol, tol)]
    return bad


@pytest.mark.gpu
def test_static_table_entry_matches_workspace_entry_twice_in_a_row(pkg, oracle):
    # two different problem lists back to back: the second call must not be
    # affected by the table entries the first one left behind
    cases = [([96, 0, 200, 130], [256, 128, 384, 512], [512, 256, 256, 768]),
             ([72, 384], [512, 256], [256, 1024])]
    tol = 1e-3      # the tolerance of the grouped parity tests (reference distribution)
    for seed, (m, n, k) in enumerate(cases):
        data = pkg.inputs.generate_grouped_input(m, n, k, len(m), 1111 + seed, dist="reference", device="cuda",
                                                 fill_c=100.0)
        # existing entry point (workspace), on the same one-CTA kernels the static entry point runs
        want = [c.clone() for c in pkg.group_gemm.custom_kernel(data, variant=pkg._lib.VARIANT_PERSISTENT)]
        torch.cuda.synchronize()
        for (_a, _b, c) in data[0]:
            c.fill_(-7.0)
        _through_c_abi(pkg, data)
        torch.cuda.synchronize()
        assert pkg._lib.read_status(torch.cuda.current_device()) == 0
        for g, ((_a, _b, got), ref) in enumerate(zip(data[0], want)):
            assert got.shape == ref.shape
            if got.numel() == 0:
                continue
            diff = (got.float() - ref.float()).abs()
            assert torch.all(diff <= tol + tol * ref.float().abs()), (seed, g, diff.max().item())
            assert torch.equal(got, ref), (seed, g)           # same kernel, same order of additions: same bits
        assert _oracle_problems(oracle, data, tol) == []
    # the Python convenience wrapper takes the same route
    data = pkg.inputs.generate_grouped_input([136], [256], [512], 1, 5, dist="reference", device="cuda")
    want = pkg.group_gemm.custom_kernel(data)[0].clone()
    data[0][0][2].zero_()
    got = pkg.group_gemm.custom_kernel_no_alloc(data)[0]
    torch.cuda.synchronize()
    assert torch.equal(got, want)


@pytest.mark.gpu
def test_static_table_entry_allocates_nothing_and_serves_a_full_table(pkg, oracle):
    # 64 groups (the table's capacity), four of them empty, wide enough that the entry point
    # picks its 128 x 256 tiles: 60 groups x 2 x 8 tiles of 128 x 128 = 960 >= 4 per SM
    g = pkg._lib.STATIC_MAX_GROUPS
    m = [0 if i % 16 == 7 else 256 - (i % 5) * 24 for i in range(g)]
    data = pkg.inputs.generate_grouped_input(m, [1024] * g, [256] * g, g, 77, dist="reference", device="cuda",
                                             fill_c=100.0)
    want = [c.clone() for c in pkg.group_gemm.custom_kernel(data, variant=pkg._lib.VARIANT_PERSISTENT, tile_n=256)]
    _through_c_abi(pkg, data)                    # first call on this device may do the one-time set-up
    torch.cuda.synchronize()
    for (_a, _b, c) in data[0]:
        c.fill_(-7.0)
    before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.mem_get_info()[0])
    _through_c_abi(pkg, data)
    torch.cuda.synchronize()
    after = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.mem_get_info()[0])
    assert after == before                       # neither torch's allocator nor the device lost a byte
    assert pkg._lib.read_status(torch.cuda.current_device()) == 0
    for i, ((_a, _b, got), ref) in enumerate(zip(data[0], want)):
        assert torch.equal(got, ref), i
    assert _oracle_problems(oracle, data, 1e-3) == []
