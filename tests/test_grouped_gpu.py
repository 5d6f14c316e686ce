"""GPU parity: the CUDA grouped GEMM (through the C ABI) against the CPU oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL_NORTH_STAR = 1e-2
TOL_REFERENCE = 1e-3
V_AUTO, V_PERSISTENT, V_SERIAL, V_PAIR = 0, 1, 2, 5

# utils/group_gemm/task.yml:47-56 (seed 1111)
REFERENCE_TESTS = [
    ([96, 128], [128, 256], [256, 512]),
    ([256, 72], [512, 384], [256, 256]),
    ([128, 128], [128, 256], [512, 256]),
    ([80, 128, 256], [384, 256, 128], [256, 512, 256]),
    ([64, 72, 96], [128, 384, 512], [512, 512, 256]),
    ([64, 256, 128], [768, 128, 256], [512, 256, 512]),
    ([128, 128, 64], [256, 512, 512], [768, 256, 768]),
    ([128, 128, 128, 128], [128, 128, 128, 128], [512, 256, 512, 256]),
    ([40, 56, 384, 512], [512, 384, 256, 128], [256, 256, 256, 256]),
    ([512, 384, 256, 128], [256, 256, 256, 256], [512, 768, 512, 768]),
]


def _run(pkg, data, variant=V_AUTO, tile_n=0, canary=100.0):
    for (_a, _b, c) in data[0]:
        c.fill_(canary)
    out = pkg.group_gemm.custom_kernel(data, variant=variant, tile_n=tile_n)
    torch.cuda.synchronize()
    assert all(o is c for o, (_a, _b, c) in zip(out, data[0]))
    assert pkg._lib.read_status(torch.cuda.current_device()) == 0
    return out


def _check(oracle, data, out, tol):
    cpu = ([tuple(t.cpu() for t in abc) for abc in data[0]], data[1])
    want = oracle.grouped_gemm(cpu)
    assert len(out) == len(want)
    for g, (o, w) in enumerate(zip(out, want)):
        problems = oracle.compare(o, w, tol, tol)
        assert problems == [], (g, problems)


@pytest.mark.parametrize("case", range(len(REFERENCE_TESTS)))
@pytest.mark.parametrize("variant", [V_SERIAL, V_PERSISTENT])
def test_reference_test_lists(pkg, oracle, case, variant):
    m, n, k = REFERENCE_TESTS[case]
    data = pkg.inputs.generate_grouped_input(m, n, k, len(m), 1111, dist="reference", device="cuda")
    _check(oracle, data, _run(pkg, data, variant), TOL_REFERENCE)


@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("variant", [V_SERIAL, V_PERSISTENT])
def test_tile_widths(pkg, oracle, tile_n, variant):
    # n = 384 with 256-wide tiles exercises the clipped second half-tile
    m, n, k = [200, 64, 384], [512, 384, 256], [512, 256, 768]
    data = pkg.inputs.generate_grouped_input(m, n, k, 3, 5, dist="uniform16", device="cuda")
    _check(oracle, data, _run(pkg, data, variant, tile_n), TOL_NORTH_STAR)


# CTA pairs (256 x 256 tiles): one tile, a group smaller than one CTA's rows, empty groups,
# ragged counts around the 128- and 256-row boundaries, several tiles per pair
PAIR_LISTS = [
    ([256], [256], [256]),
    ([96], [256], [512]),
    ([300, 0, 72], [256, 512, 256], [256, 512, 768]),
    ([40, 56, 384, 512], [512, 256, 256, 256], [256, 256, 256, 256]),
    ([1000, 513, 257, 255], [512, 256, 768, 256], [512, 1024, 256, 512]),
]


@pytest.mark.parametrize("case", range(len(PAIR_LISTS)))
@pytest.mark.parametrize("dist,tol", [("reference", TOL_REFERENCE), ("uniform16", TOL_NORTH_STAR)])
def test_cta_pair_variant(pkg, oracle, case, dist, tol):
    m, n, k = PAIR_LISTS[case]
    data = pkg.inputs.generate_grouped_input(m, n, k, len(m), 7, dist=dist, device="cuda")
    out = [o.clone() for o in _run(pkg, data, V_PAIR)]
    _check(oracle, data, out, tol)
    # same MMAs in the same k order as the one-CTA kernel
    one_cta = _run(pkg, data, V_PERSISTENT)
    for o, w in zip(out, one_cta):
        assert torch.equal(o.view(torch.int16), w.view(torch.int16))


def test_cta_pair_leaves_rows_beyond_m_alone(pkg):
    m, n, k = 72, 256, 256
    data = pkg.inputs.generate_grouped_input([m], [n], [k], 1, 2, dist="reference", device="cuda")
    (a, b, _c) = data[0][0]
    big = torch.full((384, n, 1), 7.0, dtype=torch.float16, device="cuda")
    data[0][0] = (a, b, big[:m])
    pkg.group_gemm.custom_kernel(data, variant=V_PAIR)
    torch.cuda.synchronize()
    assert torch.all(big[m:] == 7.0)
    assert not torch.all(big[:m] == 7.0)


def test_cta_pair_needs_n_multiple_of_256(pkg):
    data = pkg.inputs.generate_grouped_input([64], [384], [256], 1, 0, device="cuda")
    with pytest.raises(ValueError, match="256"):
        pkg.group_gemm.custom_kernel(data, variant=V_PAIR)


def test_large_list_takes_the_pair_kernel_by_default(pkg, oracle):
    # 8 groups x (4 x 4) pair tiles >= one per SM: AUTO and PAIR must agree bit for bit
    m = [1000, 1024, 900, 777, 1024, 513, 1024, 960]
    data = pkg.inputs.generate_grouped_input(m, [1024] * 8, [256] * 8, 8, 5, dist="reference", device="cuda")
    auto = [o.clone() for o in _run(pkg, data)]
    _check(oracle, data, auto, TOL_REFERENCE)
    for o, w in zip(auto, _run(pkg, data, V_PAIR)):
        assert torch.equal(o.view(torch.int16), w.view(torch.int16))


def test_empty_groups_are_skipped(pkg, oracle):
    m, n, k = [0, 136, 0, 64, 0], [256, 256, 128, 384, 256], [256, 512, 256, 256, 512]
    data = pkg.inputs.generate_grouped_input(m, n, k, 5, 9, dist="reference", device="cuda")
    out = _run(pkg, data)
    _check(oracle, data, out, TOL_REFERENCE)
    assert out[0].shape == (0, 256, 1)


def test_all_groups_empty_is_a_no_op(pkg):
    data = pkg.inputs.generate_grouped_input([0, 0], [128, 256], [256, 256], 2, 1, device="cuda")
    before = pkg._lib.launch_count()
    pkg.group_gemm.custom_kernel(data)
    assert pkg._lib.launch_count() == before


def test_rows_beyond_m_are_not_written(pkg):
    # C_g is allocated with guard rows after it: the kernel must not touch them
    m, n, k = 72, 256, 256
    data = pkg.inputs.generate_grouped_input([m], [n], [k], 1, 2, dist="reference", device="cuda")
    (a, b, _c) = data[0][0]
    big = torch.full((128, n, 1), 7.0, dtype=torch.float16, device="cuda")
    data[0][0] = (a, b, big[:m])
    pkg.group_gemm.custom_kernel(data)
    torch.cuda.synchronize()
    assert torch.all(big[m:] == 7.0)
    assert not torch.all(big[:m] == 7.0)


def test_known_answers(pkg):
    kw = dict(unit_sfa=True, unit_sfb=True, device="cuda", fill_c=100.0)
    data = pkg.inputs.generate_grouped_input([128], [128], [256], 1, 0, constant_a=True, constant_b=True, **kw)
    assert torch.all(_run(pkg, data)[0] == 256.0)
    data = pkg.inputs.generate_grouped_input([128], [256], [512], 1, 0, identity_a=True, identity_b=True, **kw)
    out = _run(pkg, data)[0][:, :, 0].float().cpu()
    assert torch.equal(out, torch.eye(128, 256))
    data = pkg.inputs.generate_grouped_input([128], [128], [256], 1, 0, single_a=(3, 77, -1.5), constant_b=True, **kw)
    out = _run(pkg, data)[0][:, :, 0].float().cpu()
    want = torch.zeros(128, 128)
    want[3] = -1.5
    assert torch.equal(out, want)


def test_benchmark_list_g8(pkg, oracle):
    # utils/group_gemm/task.yml:59
    m = [80, 176, 128, 72, 64, 248, 96, 160]
    data = pkg.inputs.generate_grouped_input(m, [4096] * 8, [7168] * 8, 8, 1111, dist="reference", device="cuda")
    _check(oracle, data, _run(pkg, data), TOL_REFERENCE)


def test_moe_routing_shape_with_zero_counts(pkg, oracle):
    # small cousin of the 64-expert MoE configuration: ragged counts incl. zeros
    counts = pkg.inputs.moe_expert_counts(96, 16, 2, seed=4)
    counts[3] = 0
    data = pkg.inputs.generate_grouped_input(counts, [256] * 16, [512] * 16, 16, 3, dist="uniform16", device="cuda")
    _check(oracle, data, _run(pkg, data), TOL_NORTH_STAR)


def test_repeated_calls_reuse_descriptors(pkg, oracle):
    m, n, k = [96, 128], [128, 256], [256, 512]
    data = pkg.inputs.generate_grouped_input(m, n, k, 2, 1111, dist="reference", device="cuda")
    first = [o.clone() for o in _run(pkg, data)]
    second = _run(pkg, data)
    for x, y in zip(first, second):
        assert torch.equal(x, y)
    other = pkg.inputs.generate_grouped_input(m, n, k, 2, 1153, dist="reference", device="cuda")
    _check(oracle, other, _run(pkg, other), TOL_REFERENCE)
    _check(oracle, data, _run(pkg, data), TOL_REFERENCE)


def test_pair_kernel_is_deterministic_over_many_launches(pkg):
    lists = [([300, 0, 72, 1000], [256, 512, 256, 512], [256, 512, 768, 256]),
             ([129, 255, 257], [1024, 256, 512], [512, 1024, 256])]
    inputs = [pkg.inputs.generate_grouped_input(m, n, k, len(m), 3 + i, dist="uniform16", device="cuda")
              for i, (m, n, k) in enumerate(lists)]
    first = [[o.clone() for o in _run(pkg, d, V_PAIR)] for d in inputs]
    for rep in range(40):
        for d in inputs:
            pkg.group_gemm.custom_kernel(d, variant=V_PAIR)
        torch.cuda.synchronize()
        assert pkg._lib.read_status(torch.cuda.current_device()) == 0
        for d, want in zip(inputs, first):
            for (_a, _b, c), w in zip(d[0], want):
                assert torch.equal(c.view(torch.int16), w.view(torch.int16)), rep


def test_every_kernel_gives_the_same_bits_on_random_lists(pkg, oracle):
    # ragged lists (rows from 0 to 700, not multiples of anything) through the library's choice, the one-CTA
    # kernels and the CTA-pair kernel: one set of bits, and it agrees with the oracle
    gen = torch.Generator().manual_seed(77)
    for case in range(6):
        groups = int(torch.randint(1, 7, (1,), generator=gen))
        ms = [int(v) for v in torch.randint(0, 701, (groups,), generator=gen)]
        ns = [256 * int(v) for v in torch.randint(1, 4, (groups,), generator=gen)]
        ks = [256 * int(v) for v in torch.randint(1, 5, (groups,), generator=gen)]
        data = pkg.inputs.generate_grouped_input(ms, ns, ks, groups, 300 + case, dist="reference", device="cuda",
                                                 fill_c=100.0)
        base = [o.clone() for o in _run(pkg, data, V_SERIAL)]
        _check(oracle, data, base, TOL_REFERENCE)
        for variant in (V_AUTO, V_PERSISTENT, V_PAIR):
            out = _run(pkg, data, variant)
            for g, (o, w) in enumerate(zip(out, base)):
                assert torch.equal(o.view(torch.int16), w.view(torch.int16)), (case, variant, g, ms, ns, ks)
