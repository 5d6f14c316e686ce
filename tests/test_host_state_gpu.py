"""GPU tests of the library's host-side state: the tensor-map cache of the dual GEMM, the
descriptor-table cache of the grouped GEMM (workspace reuse, other streams, stream capture)
and the failure path of a bounded on-device wait.  Nothing here faults, traps or hangs the
GPU: the one induced failure is a wait that runs out after about a millisecond."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL_REFERENCE = 1e-3


def _dual_problems(oracle, data, out, tol=TOL_REFERENCE):
    cpu = tuple(t.cpu() for t in data[:6])
    fp32 = oracle.dual_gemm_fp32(*cpu)
    return oracle.compare(out, fp32.to(torch.float16), tol, tol, expected_fp32=fp32)


def test_plain_call_after_quantised_call_at_the_same_address(pkg, oracle):
    # The quantised-output entry point passes its packed output where the plain one passes C.  A plain
    # call whose C starts at that address, with the same operands and shape, must get an fp16 store
    # map of its own (8 x 38 = 304 tiles: the library picks the CTA-pair kernel, which stores by TMA).
    m, n, k = 1024, 4864, 256
    data = list(pkg.inputs.generate_input(m, n, k, 1, 1, dist="reference", device="cuda"))
    buf = torch.zeros(m * n * 2, dtype=torch.uint8, device="cuda")
    lib = pkg._lib.load()
    sf = torch.empty(lib.b200_quantize_sf_bytes(m, n), dtype=torch.uint8, device="cuda")
    rc = lib.b200_dual_gemm_nvfp4_quant(data[0].data_ptr(), data[1].data_ptr(), data[2].data_ptr(), data[6].data_ptr(),
                                        data[7].data_ptr(), data[8].data_ptr(), buf.data_ptr(), sf.data_ptr(), m, n, k,
                                        torch.cuda.current_stream().cuda_stream, 0, None)
    pkg._lib.check(rc)
    torch.cuda.synchronize()
    c = buf.view(torch.float16).view(1, m, n).permute(1, 2, 0)
    assert c.data_ptr() == buf.data_ptr()
    c.fill_(float("nan"))
    data[9] = c
    out = pkg.dual_gemm.custom_kernel(tuple(data))
    torch.cuda.synchronize()
    assert pkg._lib.read_status(0) == 0
    assert _dual_problems(oracle, data, out) == []


def _tiny_list(pkg, seed):
    return pkg.inputs.generate_grouped_input([72], [128], [256], 1, seed, dist="reference", device="cuda", fill_c=100.0)


def _grouped_ok(oracle, data):
    want = oracle.grouped_gemm(([tuple(t.cpu() for t in abc) for abc in data[0]], data[1]))
    return all(oracle.compare(c, w, TOL_REFERENCE, TOL_REFERENCE) == [] for (_a, _b, c), w in zip(data[0], want))


def test_evicted_workspace_is_never_trusted_again(pkg, oracle):
    gg = pkg.group_gemm
    first = _tiny_list(pkg, 0)
    gg.custom_kernel(first)
    torch.cuda.synchronize()
    assert _grouped_ok(oracle, first)
    keep = [first]
    for seed in range(1, gg._MAX_PLANS + 2):            # pushes the first plan out of the cache
        other = _tiny_list(pkg, seed)
        keep.append(other)
        gg.custom_kernel(other)
    torch.cuda.synchronize()
    # whatever memory evicted plans left behind now holds garbage
    for pool in gg._free_workspaces.values():
        for ws in pool:
            ws.fill_(0xFF)
    for plan in gg._plans.values():
        assert plan.workspace is not None
    first[0][0][2].fill_(100.0)
    gg.custom_kernel(first)                               # a new plan: its table must be uploaded again
    torch.cuda.synchronize()
    assert pkg._lib.read_status(0) == 0
    assert _grouped_ok(oracle, first)
    # and a workspace that the caller overwrote is re-uploaded once the library is told
    plan = next(reversed(gg._plans.values()))
    plan.workspace.fill_(0xFF)
    pkg._lib.check(pkg._lib.load().b200_grouped_workspace_forget(0, gg._workspace_ptr(plan)))
    first[0][0][2].fill_(100.0)
    gg.custom_kernel(first)
    torch.cuda.synchronize()
    assert pkg._lib.read_status(0) == 0
    assert _grouped_ok(oracle, first)


def test_cached_table_is_ordered_behind_its_upload_on_another_stream(pkg, oracle):
    data = pkg.inputs.generate_grouped_input([200, 64], [256, 128], [512, 256], 2, 21, dist="reference", device="cuda",
                                             fill_c=100.0)
    side = torch.cuda.Stream()
    pkg.group_gemm.custom_kernel(data)                   # uploads on the current stream ...
    with torch.cuda.stream(side):
        pkg.group_gemm.custom_kernel(data)               # ... and launches again, at once, on another one
    torch.cuda.synchronize()
    assert pkg._lib.read_status(0) == 0
    assert _grouped_ok(oracle, data)


def test_upload_is_refused_while_the_stream_is_captured(pkg, oracle):
    gg = pkg.group_gemm
    data = pkg.inputs.generate_grouped_input([136, 40], [256, 128], [256, 512], 2, 33, dist="reference", device="cuda",
                                             fill_c=100.0)
    fresh = pkg.inputs.generate_grouped_input([96], [128], [256], 1, 34, dist="reference", device="cuda", fill_c=100.0)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        gg.custom_kernel(data)                           # table uploaded from the stream that will be captured
        gg.custom_kernel_no_alloc(fresh)                 # per-device set-up of the static entry point done
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    refused = []
    with torch.cuda.stream(stream):
        graph.capture_begin()
        try:
            for call in (lambda: gg.custom_kernel(fresh), lambda: gg.custom_kernel_no_alloc(fresh)):
                try:
                    call()                               # both would have to copy a table from dying host memory
                    refused.append(None)
                except ValueError as exc:
                    refused.append(getattr(exc, "code", None))
            gg.custom_kernel(data)                       # table already in its workspace: only a launch
        finally:
            graph.capture_end()
    assert refused == [pkg._lib.E_CAPTURE, pkg._lib.E_CAPTURE]
    for (_a, _b, c) in data[0]:
        c.fill_(100.0)
    graph.replay()
    torch.cuda.synchronize()
    assert pkg._lib.read_status(0) == 0
    assert _grouped_ok(oracle, data)


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(pkg, oracle):
    # failure detection without a fault: the self-test variant drops one k-tile's loads and limits every
    # on-device wait to about a millisecond; the roles give up, the launch ends, the status word says so
    data = pkg.inputs.generate_input(128, 128, 1024, 1, 5, dist="reference", device="cuda")
    c = data[9]
    c.fill_(7.0)
    assert pkg._lib.read_status(0) == 0
    pkg.dual_gemm.custom_kernel(data, variant=pkg._lib.VARIANT_SELFTEST_LOST_LOAD)
    with pytest.raises(pkg._lib.B200Error, match="wait ran out"):
        pkg._lib.raise_on_status(0)
    assert torch.all(c == 7.0)                           # nothing was stored
    assert pkg._lib.read_status(0) == 0                  # reading clears the word
    # the same context keeps working
    out = pkg.dual_gemm.custom_kernel(data)
    torch.cuda.synchronize()
    pkg._lib.raise_on_status(0)
    assert _dual_problems(oracle, data, out) == []


def test_probe_variants_are_not_part_of_the_library(pkg):
    lib = pkg._lib.load()
    d = pkg.inputs.generate_input(128, 128, 256, 1, 0, device="cuda")
    for variant in (9, 100, 164, 400):
        rc = lib.b200_dual_gemm_nvfp4_ex(d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[6].data_ptr(),
                                         d[7].data_ptr(), d[8].data_ptr(), d[9].data_ptr(), 128, 128, 256, 1, 128, 0, 0, 0,
                                         variant, None, 0, None, 0, None)
        assert rc == pkg._lib.E_VARIANT


def test_launch_cycle_counter(pkg):
    d = pkg.inputs.generate_input(256, 512, 1024, 1, 0, device="cuda")
    pkg.dual_gemm.custom_kernel(d)
    cycles = pkg._lib.last_launch_cycles(0)
    assert 1_000 < cycles < 50_000_000


def test_l2_feed_probe_reports_a_plausible_rate(pkg):
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    alone = pkg._lib.probe_l2_feed(0, 1, 1, True, copies_per_cta=1200)
    every = pkg._lib.probe_l2_feed(0, sms, 2, True, copies_per_cta=1200)
    bulk = pkg._lib.probe_l2_feed(0, sms, 1, False, copies_per_cta=1200)
    assert pkg._lib.read_status(0) == 0
    for r in (alone, every, bulk):
        assert 20.0 < r["bytes_per_clk_per_sm"] < 400.0, r       # one SM: tens of bytes per clock, not thousands
        assert 500.0 < r["sm_mhz"] < 2500.0, r
    assert every["tb_per_s"] > 20 * alone["tb_per_s"]            # the aggregate grows with the SMs used
    with pytest.raises(ValueError):
        pkg._lib.probe_l2_feed(0, 0, 1, True)
