"""CPU checks of the activation quantiser: the oracle's restatement of the NVFP4
recipe against hand-computed cases and its own decode side, and the C entry
point's argument checks (no GPU work)."""
import torch

FAKE = 0x7F0000000000


def test_known_answers(oracle):
    x = torch.zeros(2, 32)
    # block amax 6 -> scale 1.0 (e4m3 0x38); values on and between the e2m1 grid points
    x[0, :16] = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.5, -1, -1.5, -2, -3, -4, -6, 0.26])
    # exact ties go to the even code: 0.25->0, 0.75->1, 1.25->1, 1.75->2, 2.5->2, 3.5->4, 5->4
    x[0, 16:] = torch.tensor([6, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5, 0])
    x[1, :16] = 12.0      # amax 12 -> scale 2.0 (0x40), every code 6
    packed, sf = oracle.quantize_nvfp4(x)
    assert sf.tolist() == [[0x38, 0x38], [0x40, 0x00]]
    codes = torch.stack([packed & 0xF, packed >> 4], dim=2).reshape(2, 32)
    assert codes[0, :16].tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 9, 10, 11, 12, 13, 14, 15, 1]
    assert codes[0, 16:].tolist() == [7, 0, 2, 2, 4, 4, 6, 6, 8, 10, 10, 12, 12, 14, 14, 0]
    assert codes[1, :16].tolist() == [7] * 16 and codes[1, 16:].tolist() == [0] * 16


def test_round_trip_error_is_within_half_a_step(oracle):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(64, 256, generator=g) * 5).half()
    packed, sf = oracle.quantize_nvfp4(x)
    values = oracle.decode_e2m1(packed.view(64, 128, 1))[:, :, 0]
    scale = oracle.decode_e4m3(sf.view(64, 16, 1))[:, :, 0].repeat_interleave(16, dim=1)
    err = (values * scale - x.float()).abs()
    # the widest e2m1 step is 2 (between 4 and 6); the scale is amax/6 rounded to e4m3 (relative 2^-4),
    # so |x/s| may exceed 6 by 1/16 at most before saturating
    assert torch.all(err <= scale * (1.0 + 6.0 / 16.0) + 1e-6)
    amax = x.float().abs().reshape(64, 16, 16).amax(dim=2)
    assert torch.all(scale[:, ::16] >= amax / 6.0 * (1 - 2 ** -4))


def test_entry_point_rejects_bad_arguments(pkg):
    lib = pkg._lib.load()
    E = pkg._lib
    ok = (FAKE, E.DTYPE_F16, 128, 256, 256, FAKE + 65536, FAKE + 131072, None, 0)

    def call(**kw):
        names = ("x", "dtype", "rows", "k", "ldx", "q", "sf", "stream", "device")
        args = dict(zip(names, ok))
        args.update(kw)
        return lib.b200_quantize_nvfp4(*[args[n] for n in names])
    assert call(x=None) == E.E_NULL
    assert call(dtype=7) == E.E_VARIANT
    assert call(rows=0) == E.E_SHAPE
    assert call(k=48) == E.E_SHAPE and "64" in lib.b200_last_error().decode()
    assert call(ldx=200) == E.E_ALIGN
    assert call(ldx=260) == E.E_ALIGN
    assert call(q=FAKE + 8) == E.E_ALIGN
    assert lib.b200_quantize_sf_bytes(128, 256) == 2048
    assert lib.b200_quantize_sf_bytes(129, 256) == 4096
    assert lib.b200_quantize_sf_bytes(128, 100) == 0


def test_quantised_output_entry_point_rejects_bad_arguments(pkg):
    lib = pkg._lib.load()
    E = pkg._lib
    ptrs = [FAKE + 65536 * i for i in range(8)]
    assert lib.b200_dual_gemm_nvfp4_quant(*ptrs, 128, 128, 256, None, 0, None) == E.E_SHAPE
    assert "256" in lib.b200_last_error().decode()
    assert lib.b200_dual_gemm_nvfp4_quant(*ptrs[:6], None, ptrs[7], 256, 128, 256, None, 0, None) == E.E_NULL
    assert lib.b200_dual_gemm_nvfp4_quant(*ptrs[:7], FAKE + 4, 256, 128, 256, None, 0, None) == E.E_ALIGN
    assert lib.b200_dual_gemm_nvfp4_quant(*ptrs, 256, 100, 256, None, 0, None) == E.E_SHAPE
