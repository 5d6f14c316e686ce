"""GPU parity: the CUDA dual GEMM (through the C ABI) against the CPU oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

# north-star tolerance on fp16 outputs; the reference's own check uses 1e-3
# (dual_gemm/reference.py:200) and is applied to its own input distribution.
TOL_NORTH_STAR = 1e-2
TOL_REFERENCE = 1e-3

V_AUTO, V_PERSISTENT, V_SERIAL, V_SERIAL_2MMA, V_SPLITK, V_PAIR, V_PAIR_NARROW, V_PAIR_STREAMK = 0, 1, 2, 3, 4, 5, 6, 7


def _run(pkg, data, variant):
    data = tuple(data)
    c = data[9]
    c.fill_(float("nan"))                    # canary: every element must be overwritten
    out = pkg.dual_gemm.custom_kernel(data, variant=variant)
    torch.cuda.synchronize()
    assert out is c
    assert pkg._lib.read_status(c.device.index) == 0
    return out


def _check(oracle, data, out, tol):
    cpu = tuple(t.cpu() for t in data)
    a, b1, b2, sfa, sfb1, sfb2 = cpu[:6]
    fp32 = oracle.dual_gemm_fp32(a, b1, b2, sfa, sfb1, sfb2)
    problems = oracle.compare(out, fp32.to(torch.float16), tol, tol, expected_fp32=fp32)
    assert problems == [], problems


@pytest.mark.parametrize("variant", [V_SERIAL, V_SERIAL_2MMA, V_PERSISTENT])
@pytest.mark.parametrize("dist,tol", [("reference", TOL_REFERENCE), ("uniform16", TOL_NORTH_STAR)])
def test_cfg1_m128_n256_k512(pkg, oracle, variant, dist, tol):
    data = pkg.inputs.generate_input(128, 256, 512, 1, 0, dist=dist, device="cuda")
    _check(oracle, data, _run(pkg, data, variant), tol)


# the reference's test shapes that the CPU oracle finishes in seconds
# (utils/dual_gemm/task.yml:46-56, seed 1111)
@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (1536, 512, 7168), (3072, 1024, 1536), (512, 768, 7168),
                                   (4096, 768, 512), (7168, 384, 2304)])
def test_reference_test_shapes(pkg, oracle, m, n, k):
    data = pkg.inputs.generate_input(m, n, k, 1, 1111, dist="reference", device="cuda")
    _check(oracle, data, _run(pkg, data, V_AUTO), TOL_REFERENCE)


@pytest.mark.parametrize("variant", [V_SERIAL, V_PERSISTENT])
def test_batched_l3(pkg, oracle, variant):
    data = pkg.inputs.generate_input(256, 256, 768, 3, 7, dist="reference", device="cuda")
    _check(oracle, data, _run(pkg, data, variant), TOL_REFERENCE)


def test_many_tiles_per_cta(pkg, oracle):
    # 64 x 24 = 1536 tiles > 148 SMs: every CTA walks several tiles, both TMEM buffers
    data = pkg.inputs.generate_input(8192, 3072, 256, 1, 3, dist="reference", device="cuda")
    one_cta = _run(pkg, data, V_PERSISTENT).clone()
    _check(oracle, data, one_cta, TOL_REFERENCE)
    # with this many tiles the library's own choice is the CTA-pair kernel: same bits
    auto = _run(pkg, data, V_AUTO)
    assert torch.equal(auto.view(torch.int16), one_cta.view(torch.int16))


def test_benchmark_shape_skinny(pkg, oracle):
    data = pkg.inputs.generate_input(256, 4096, 7168, 1, 0, dist="uniform16", device="cuda")
    _check(oracle, data, _run(pkg, data, V_AUTO), TOL_NORTH_STAR)


# shapes with fewer tiles than half the SMs are cut along k (utils/dual_gemm/task.yml:59-62 are all of this kind)
@pytest.mark.parametrize("m,n,k", [(256, 4096, 7168), (512, 4096, 7168), (256, 3072, 4096), (512, 3072, 7168),
                                   (128, 256, 2560), (128, 128, 6400), (256, 512, 1024)])
@pytest.mark.parametrize("variant", [V_SPLITK])
def test_split_k_shapes(pkg, oracle, m, n, k, variant):
    lib = pkg._lib.load()
    data = pkg.inputs.generate_input(m, n, k, 1, 1111, dist="reference", device="cuda")
    expect_split = lib.b200_dual_splitk_workspace_bytes(m, n, k, 1) > 0
    out = _run(pkg, data, variant)
    _check(oracle, data, out, TOL_REFERENCE)
    if expect_split:
        # the split result is bit-identical from run to run (partials are added in unit order) ...
        again = _run(pkg, data, variant).clone()
        assert torch.equal(out.view(torch.int16), again.view(torch.int16))
        # ... and agrees with the unsplit kernel to fp32 re-association error
        whole = _run(pkg, data, V_PERSISTENT)
        assert oracle.compare(again, whole, TOL_REFERENCE, TOL_REFERENCE) == []


def test_split_k_with_overflowing_distribution(pkg, oracle):
    data = pkg.inputs.generate_input(256, 2048, 7168, 1, 5, dist="uniform16", device="cuda")
    _check(oracle, data, _run(pkg, data, V_SPLITK), TOL_NORTH_STAR)


# CTA pairs (2-SM MMA, 256-row tiles): one pair tile, several k-tiles, several tiles per pair, batches
@pytest.mark.parametrize("m,n,k,l", [(256, 128, 256, 1), (256, 256, 2560, 1), (512, 384, 512, 2), (2048, 1024, 1536, 1),
                                     (8192, 3072, 256, 1), (1536, 512, 7168, 1)])
@pytest.mark.parametrize("dist,tol", [("reference", TOL_REFERENCE), ("uniform16", TOL_NORTH_STAR)])
def test_cta_pair_variant(pkg, oracle, m, n, k, l, dist, tol):
    data = pkg.inputs.generate_input(m, n, k, l, 3, dist=dist, device="cuda")
    out = _run(pkg, data, V_PAIR)
    _check(oracle, data, out, tol)
    one_cta = _run(pkg, data, V_PERSISTENT).clone()
    again = _run(pkg, data, V_PAIR)
    # same MMAs in the same k order: the pair kernel reproduces the one-CTA kernel bit for bit
    assert torch.equal(again.view(torch.int16), one_cta.view(torch.int16))


# CTA pairs on 256 x 64 tiles (the library's choice for shapes with few tiles): one tile, both halves of a
# scale-factor atom, several k-tiles and tiles per pair, batches, the reference task's benchmark shapes
@pytest.mark.parametrize("m,n,k,l", [(256, 128, 256, 1), (256, 384, 2560, 1), (512, 256, 512, 2), (2048, 1024, 1536, 1),
                                     (256, 4096, 7168, 1), (256, 3072, 4096, 1)])
@pytest.mark.parametrize("dist,tol", [("reference", TOL_REFERENCE), ("uniform16", TOL_NORTH_STAR)])
def test_narrow_cta_pair_variant(pkg, oracle, m, n, k, l, dist, tol):
    data = pkg.inputs.generate_input(m, n, k, l, 13, dist=dist, device="cuda")
    out = _run(pkg, data, V_PAIR_NARROW)
    _check(oracle, data, out, tol)
    one_cta = _run(pkg, data, V_PERSISTENT).clone()
    again = _run(pkg, data, V_PAIR_NARROW)
    # same products summed in the same k order: the same bits as the one-CTA kernel
    assert torch.equal(again.view(torch.int16), one_cta.view(torch.int16))


def test_library_picks_narrow_tiles_for_few_tiles(pkg):
    for (m, n, k), want in (((256, 4096, 7168), "PairDualNarrow"), ((512, 4096, 7168), "PairDual>"),
                            ((256, 3072, 4096), "PairDualNarrow"), ((512, 3072, 7168), "PairDual>"),
                            ((128, 256, 512), "persistent<Dual>")):
        data = pkg.inputs.generate_input(m, n, k, 1, 0, dist="reference", device="cuda")
        _run(pkg, data, V_AUTO)
        assert want in pkg._lib.last_kernel(), (m, n, k, pkg._lib.last_kernel())


# Stream-k tail: 80 = 74 + 6 pair tiles (everything is cut), 152 = 74 + 78 (one whole round, then the cut part),
# two k-tiles per tile (the smallest that can be cut), ten k-tiles; on a 148-SM GPU
@pytest.mark.parametrize("m,n,k", [(1024, 2560, 1024), (2048, 2432, 512), (512, 5120, 2560), (2048, 2432, 1280)])
@pytest.mark.parametrize("dist,tol", [("reference", TOL_REFERENCE), ("uniform16", TOL_NORTH_STAR)])
def test_stream_k_tail(pkg, oracle, m, n, k, dist, tol):
    data = pkg.inputs.generate_input(m, n, k, 1, 17, dist=dist, device="cuda")
    out = _run(pkg, data, V_PAIR_STREAMK).clone()
    assert "StreamK" in pkg._lib.last_kernel()
    _check(oracle, data, out, tol)
    # the cut is fixed by the shape: a second run gives the same bits
    again = _run(pkg, data, V_PAIR_STREAMK)
    assert torch.equal(again.view(torch.int16), out.view(torch.int16))
    # against whole tiles only the tiles that two pairs share differ, by fp32 re-association
    whole = _run(pkg, data, V_PAIR)
    assert oracle.compare(out, whole, tol, tol) == []


def test_stream_k_needs_its_workspace(pkg):
    lib = pkg._lib.load()
    assert lib.b200_dual_streamk_workspace_bytes(1024, 2560, 1024, 1) == 74 * (256 * 1024) + 2560
    assert lib.b200_dual_streamk_workspace_bytes(8192, 14336 // 8, 4096, 1) > 0      # 448 tiles on 74 pairs
    assert lib.b200_dual_streamk_workspace_bytes(256 * 74, 128, 1024, 1) == 0        # whole rounds: nothing to cut
    d = pkg.inputs.generate_input(1024, 2560, 1024, 1, 0, device="cuda")
    rc = lib.b200_dual_gemm_nvfp4_ex(d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[6].data_ptr(), d[7].data_ptr(),
                                     d[8].data_ptr(), d[9].data_ptr(), 1024, 2560, 1024, 1, 2560, 0, 0, 0, V_PAIR_STREAMK,
                                     None, 0, None, 0, None)
    assert rc == pkg._lib.E_WORKSPACE


def test_cta_pair_needs_even_row_tiles(pkg):
    data = pkg.inputs.generate_input(384, 128, 256, 1, 0, device="cuda")
    with pytest.raises(ValueError, match="256"):
        pkg.dual_gemm.custom_kernel(data, variant=V_PAIR)


def test_known_answer_all_ones_overflows_to_inf(pkg):
    data = list(pkg.inputs.generate_input(128, 128, 256, 1, 0, device="cuda"))
    ones = torch.full((128, 128, 1), 0x22, dtype=torch.uint8, device="cuda")
    unit = torch.full((128, 16, 1), 0x38, dtype=torch.uint8).view(torch.float8_e4m3fn)
    perm = pkg.inputs._to_device_keep_strides(pkg.formats.permute_scale_factors(unit), "cuda")
    data[0] = data[1] = data[2] = ones
    data[6] = data[7] = data[8] = perm
    out = _run(pkg, data, V_PERSISTENT)
    assert torch.all(torch.isposinf(out))       # silu(256) * 256 = 65536 > fp16 max


def test_known_answer_negative_gate_gives_zero(pkg):
    # B1 = -1 everywhere: r1 = -K, silu(-256) underflows to -0, C = -0 * K = -0 (no NaN)
    data = list(pkg.inputs.generate_input(128, 128, 256, 1, 0, device="cuda"))
    ones = torch.full((128, 128, 1), 0x22, dtype=torch.uint8, device="cuda")
    minus = torch.full((128, 128, 1), 0xAA, dtype=torch.uint8, device="cuda")
    unit = torch.full((128, 16, 1), 0x38, dtype=torch.uint8).view(torch.float8_e4m3fn)
    perm = pkg.inputs._to_device_keep_strides(pkg.formats.permute_scale_factors(unit), "cuda")
    data[0], data[1], data[2] = ones, minus, ones
    data[6] = data[7] = data[8] = perm
    out = _run(pkg, data, V_PERSISTENT)
    assert torch.all(out == 0) and not torch.isnan(out).any()


def test_column_shards_reassemble(pkg, oracle):
    # N split over 4 "ranks" on one GPU: each shard writes its own columns of one C
    data = pkg.inputs.generate_input(256, 1024, 512, 1, 11, dist="reference", device="cuda")
    data[9].fill_(float("nan"))
    for r in range(4):
        pkg.dual_gemm.custom_kernel(pkg.shard.shard_dual_input(data, r, 4))
    torch.cuda.synchronize()
    _check(oracle, data, data[9], TOL_REFERENCE)


def test_large_shape_properties(pkg):
    # Full-size SwiGLU shape: no oracle at this size; check size-independent properties.
    m, n, k = 8192, 14336, 4096
    data = pkg.inputs.generate_input(m, n, k, 1, 0, dist="reference", device="cuda")
    out = _run(pkg, data, V_AUTO).clone()
    assert not torch.isnan(out).any()
    # (1) a 256-row x 512-column window recomputed as its own small problem is bit-identical
    a, b1, b2, _, _, _, sfa_p, sfb1_p, sfb2_p, c = data
    r0, c0 = 4096, 7168
    sub_c = torch.empty((256, 512, 1), dtype=torch.float16, device="cuda")
    pkg.dual_gemm.dual_gemm(a[r0:r0 + 256], b1[c0:c0 + 512], b2[c0:c0 + 512],
                            sfa_p[:, :, r0 // 128:r0 // 128 + 2], sfb1_p[:, :, c0 // 128:c0 // 128 + 4],
                            sfb2_p[:, :, c0 // 128:c0 // 128 + 4], sub_c)
    torch.cuda.synchronize()
    assert torch.equal(sub_c[:, :, 0], out[r0:r0 + 256, c0:c0 + 512, 0])
    # (2) determinism: a second run is bit-identical
    out2 = _run(pkg, data, V_AUTO)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))


def test_pair_kernel_is_deterministic_over_many_launches(pkg):
    # alternating shapes back to back: every launch must reproduce its first result bit for bit
    # and leave the device status word clear (a lost hand-over would time out or change bits)
    shapes = [(512, 2048, 1024), (256, 128, 4096), (1024, 4864, 256)]
    inputs = [pkg.inputs.generate_input(m, n, k, 1, 11 + i, dist="uniform16", device="cuda")
              for i, (m, n, k) in enumerate(shapes)]
    first = [_run(pkg, d, V_PAIR).clone() for d in inputs]
    for rep in range(40):
        for d, want in zip(inputs, first):
            out = pkg.dual_gemm.custom_kernel(d, variant=V_PAIR)
        torch.cuda.synchronize()
        assert pkg._lib.read_status(0) == 0
        for d, want in zip(inputs, first):
            assert torch.equal(d[9].view(torch.int16), want.view(torch.int16)), rep


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shards_gathered_by_the_epilogue(pkg, oracle, world):
    # the fused GEMM + all-gather entry point with every "rank" on this one GPU: each rank's launch writes its
    # columns into all `world` full-size C buffers (local ones here, peer-mapped ones on a node)
    m, n, k = 512, 1024, 512
    data = pkg.inputs.generate_input(m, n, k, 1, 23, dist="uniform16", device="cuda")
    full = [torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
    for rank in range(world):
        shard = pkg.shard.shard_dual_input(data, rank, world)
        pkg.shard.dual_gemm_gathered(shard, [c.data_ptr() for c in full], rank, world, n)
    torch.cuda.synchronize()
    assert pkg._lib.read_status(0) == 0
    assert "Gather" in pkg._lib.last_kernel()
    want = _run(pkg, data, V_PAIR)
    for c in full:
        assert torch.equal(c.view(torch.int16), want[:, :, 0].view(torch.int16))
    _check(oracle, data, full[-1].unsqueeze(-1), TOL_NORTH_STAR)


def test_library_choice_equals_the_serial_kernel_on_random_shapes(pkg, oracle):
    # whatever kernel the library picks (one CTA per tile, CTA pairs with wide or narrow tiles), its bits are
    # those of the one-stage serial kernel, and both agree with the oracle
    gen = torch.Generator().manual_seed(2024)
    seen = set()
    for case in range(10):
        m = 128 * int(torch.randint(1, 9, (1,), generator=gen))
        n = 128 * int(torch.randint(1, 13, (1,), generator=gen))
        k = 256 * int(torch.randint(1, 7, (1,), generator=gen))
        l = 1 if case % 4 else 2
        data = pkg.inputs.generate_input(m, n, k, l, 100 + case, dist="reference", device="cuda")
        auto = _run(pkg, data, V_AUTO).clone()
        seen.add(pkg._lib.last_kernel())
        serial = _run(pkg, data, V_SERIAL)
        assert torch.equal(auto.view(torch.int16), serial.view(torch.int16)), (m, n, k, l)
        _check(oracle, data, serial, TOL_REFERENCE)
    assert len(seen) >= 2, seen          # the sweep exercised more than one kernel
