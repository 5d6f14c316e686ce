"""The C-ABI library without a GPU: it loads, exports every symbol the header
declares, and rejects bad arguments on the host before any CUDA work."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "b200_nvfp4.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("b200_dual_gemm_nvfp4", "b200_grouped_gemm_nvfp4", "b200_grouped_workspace_bytes",
                 "b200_last_error", "b200_version", "b200_read_status"):
        assert must in names


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg._lib.load()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/b200_nvfp4.h but not exported"
        assert name in pkg._lib.SIGNATURES, f"{name} has no ctypes signature"
    assert b"sm_100a" in lib.b200_version()


def test_missing_library_fails_loudly(pkg, monkeypatch):
    monkeypatch.setattr(pkg._lib, "_lib", None)
    monkeypatch.setattr(pkg._lib, "LIB_PATH", "/nonexistent/libb200nvfp4.so")
    with pytest.raises(ImportError, match="no CPU fallback"):
        pkg._lib.load()


def test_no_cpu_path(pkg):
    data = pkg.inputs.generate_input(128, 128, 256, 1, 0, device="cpu")
    with pytest.raises(ValueError, match="CUDA"):
        pkg.dual_gemm.custom_kernel(data)
    gdata = pkg.inputs.generate_grouped_input([128], [128], [256], 1, 0, device="cpu")
    with pytest.raises(ValueError, match="CUDA"):
        pkg.group_gemm.custom_kernel(gdata)


FAKE = 0x7F0000000000  # 16-byte aligned fake device address; never dereferenced on the host


def _dual(lib, m=128, n=128, k=256, l=1, ldc=None, ptrs=None):
    p = ptrs or [FAKE + 4096 * i for i in range(7)]
    return lib.b200_dual_gemm_nvfp4(*p, m, n, k, l, ldc if ldc is not None else n, None, 0, None)


@pytest.mark.parametrize("kw,code,needle", [
    (dict(m=100), -2, "m=100"),
    (dict(n=200), -2, "n=200"),
    (dict(k=300), -2, "k=300"),
    (dict(l=0), -2, "positive"),
    (dict(m=-128), -2, "positive"),
    (dict(ldc=64), -3, "ldc"),
    (dict(ldc=132), -3, "ldc"),
    (dict(ptrs=[0] + [FAKE] * 6), -1, "NULL"),
    (dict(ptrs=[FAKE + 8] + [FAKE] * 6), -3, "aligned"),
])
def test_dual_argument_errors(pkg, kw, code, needle):
    lib = pkg._lib.load()
    assert _dual(lib, **kw) == code
    assert needle in lib.b200_last_error().decode()
    with pytest.raises(ValueError):
        pkg._lib.check(code)


def test_dual_unknown_variant(pkg):
    lib = pkg._lib.load()
    p = [FAKE + 4096 * i for i in range(7)]
    for variant in (-1, 9, 99, 100, 164, 400):     # the timing-probe range of instrumented builds included
        rc = lib.b200_dual_gemm_nvfp4_ex(*p, 128, 128, 256, 1, 128, 0, 0, 0, variant, None, 0, None, 0, None)
        assert rc == pkg._lib.E_VARIANT, variant


def test_public_header_has_no_probe_variants():
    text = open(os.path.join(ROOT, "include", "b200_nvfp4.h")).read()
    assert "PROBE" not in text


def test_forgetting_an_unknown_workspace_is_harmless(pkg):
    lib = pkg._lib.load()
    assert lib.b200_grouped_workspace_forget(0, FAKE) == 0
    assert lib.b200_grouped_workspace_forget(3, None) == 0


def _grouped(lib, mnk, ws=FAKE, ws_bytes=1 << 20, null_group=None, misalign=None, tile_n=0, variant=0):
    g = len(mnk)
    arr = ctypes.c_void_p * g
    cols = [arr(*[FAKE + 65536 * (5 * i + j) for i in range(g)]) for j in range(5)]
    if null_group is not None:
        cols[0][null_group] = None
    if misalign is not None:
        cols[4][misalign] = FAKE + 2
    flat = (ctypes.c_int * (3 * g))(*[x for t in mnk for x in t])
    return lib.b200_grouped_gemm_nvfp4_ex(g, *cols, flat, ws, ws_bytes, variant, tile_n, None, 0, None)


def test_grouped_argument_errors(pkg):
    lib = pkg._lib.load()
    E = pkg._lib
    assert _grouped(lib, [(128, 100, 256)]) == E.E_SHAPE
    assert "n=100" in lib.b200_last_error().decode()
    assert _grouped(lib, [(128, 128, 128)]) == E.E_SHAPE
    assert _grouped(lib, [(-1, 128, 256)]) == E.E_SHAPE
    assert _grouped(lib, [(64, 128, 256)], null_group=0) == E.E_NULL
    assert _grouped(lib, [(64, 128, 256)], misalign=0) == E.E_ALIGN
    assert _grouped(lib, [(64, 128, 256)], ws=None) == E.E_WORKSPACE
    assert _grouped(lib, [(64, 128, 256)], ws=FAKE + 64) == E.E_WORKSPACE
    assert _grouped(lib, [(64, 128, 256)] * 3, ws_bytes=100) == E.E_WORKSPACE
    assert _grouped(lib, [(64, 128, 256)], tile_n=192) == E.E_VARIANT
    assert _grouped(lib, [(64, 128, 256)], variant=7) == E.E_VARIANT
    # CTA pairs work on 256-column tiles
    assert _grouped(lib, [(64, 256, 256), (64, 384, 256)], variant=E.VARIANT_PAIR) == E.E_SHAPE
    assert "256" in lib.b200_last_error().decode()
    flat = (ctypes.c_int * 3)(1, 128, 256)
    assert lib.b200_grouped_gemm_nvfp4(0, None, None, None, None, None, flat, FAKE, 0, None, 0, None) == E.E_SHAPE
    # a NULL pointer is fine for an empty group, and all-empty input is a no-op that needs no GPU
    assert _grouped(lib, [(0, 128, 256), (0, 256, 512)], null_group=1) == 0


def test_split_k_workspace_size(pkg):
    lib = pkg._lib.load()
    f = lib.b200_dual_splitk_workspace_bytes
    assert f(8192, 14336, 4096, 1) == 0                       # 7168 tiles: never split
    assert f(512, 4096, 7168, 1) == 0                         # 128 tiles: more than half of the 148 SMs already
    tile = 128 * 256 * 4
    assert f(1536, 512, 7168, 1) == 48 * 32 + 48 * 3 * tile       # 48 tiles, 28 k-tiles -> 3 pieces
    assert f(256, 4096, 7168, 1) == 64 * 32 + 64 * 2 * tile       # 64 tiles, 28 k-tiles -> 2 pieces
    assert f(256, 3072, 4096, 1) == 48 * 32 + 48 * 3 * tile       # 48 tiles, 16 k-tiles -> 3 pieces
    assert f(128, 128, 256, 1) == 0                           # one k-tile cannot be cut
    assert f(100, 128, 256, 1) == 0 and f(128, 128, 0, 1) == 0


def test_workspace_size(pkg):
    lib = pkg._lib.load()
    assert lib.b200_grouped_workspace_bytes(0) == 0
    assert lib.b200_grouped_workspace_bytes(1) == 512
    assert lib.b200_grouped_workspace_bytes(64) == 64 * 512


def test_python_wrappers_validate_layouts(pkg):
    import torch
    # wrong scale-factor layout (plain [M, K/16, L]) is rejected by the host wrapper before the library is called
    d = list(pkg.inputs.generate_input(128, 128, 256, 1, 0, device="cpu"))
    fmt = pkg.formats
    assert fmt.is_kernel_sf_layout(d[6], 128, 256, 1)
    assert not fmt.is_kernel_sf_layout(d[3], 128, 256, 1)
    assert not fmt.is_kernel_sf_layout(d[6].contiguous(), 128, 256, 1)
    assert fmt.sf_perm_bytes(72, 256) == 4 * 512 and fmt.sf_atoms(129, 7168) == (2, 112)
    assert fmt.dual_gemm_flops(128, 256, 512) == 67108864 and fmt.dual_gemm_bytes(128, 256, 512) == 249856
    assert fmt.dual_gemm_flops(256, 4096, 7168) == 30064771072 and fmt.dual_gemm_bytes(256, 4096, 7168) == 36159488
    assert fmt.dual_gemm_flops(8192, 14336, 4096) == 1924145348608
    assert fmt.dual_gemm_bytes(8192, 14336, 4096) == 319815680
    assert fmt.dual_gemm_bytes(8192, 1792, 4096) == 56492032


def test_gather_entry_point_rejects_bad_arguments(pkg):
    lib = pkg._lib.load()
    E = pkg._lib
    ops = [FAKE + 4096 * i for i in range(6)]
    two = (ctypes.c_void_p * 2)(FAKE + 65536, FAKE + 131072)

    def call(c_ranks=two, world=2, rank=0, m=256, n_local=128, n_total=256, col=0, k=256):
        return lib.b200_dual_gemm_nvfp4_gather(*ops, c_ranks, world, rank, m, n_local, n_total, col, k, None, 0, None)
    assert call(c_ranks=None) == E.E_NULL
    assert call(world=9) == E.E_LIMIT
    assert call(rank=2) == E.E_SHAPE
    assert call(m=128) == E.E_SHAPE and "256" in lib.b200_last_error().decode()
    assert call(col=64) == E.E_SHAPE
    assert call(col=256) == E.E_SHAPE                      # columns [256, 384) of a 256-column C
    assert call(k=300) == E.E_SHAPE
    assert call(c_ranks=(ctypes.c_void_p * 2)(FAKE, None)) == E.E_NULL
    assert call(c_ranks=(ctypes.c_void_p * 2)(FAKE, FAKE + 8)) == E.E_ALIGN


def test_feed_probe_rejects_bad_arguments(pkg):
    import ctypes
    lib = pkg._lib.load()
    a, b = ctypes.c_double(0), ctypes.c_double(0)
    assert lib.b200_probe_l2_feed(0, 148, 1, 1, 1200, None, ctypes.byref(b), None) == pkg._lib.E_NULL
    assert lib.b200_probe_l2_feed(0, 0, 1, 1, 1200, ctypes.byref(a), ctypes.byref(b), None) == pkg._lib.E_SHAPE
    assert lib.b200_probe_l2_feed(0, 148, 0, 1, 1200, ctypes.byref(a), ctypes.byref(b), None) == pkg._lib.E_SHAPE
    assert lib.b200_probe_l2_feed(0, 148, 1, 1, 3, ctypes.byref(a), ctypes.byref(b), None) == pkg._lib.E_SHAPE
