"""The bounded-wait mechanism of the tensor-core kernels, exercised without hanging anything.

Every device-side wait of the library (mbarrier waits of the producer, MMA, scale and promotion
warps) gives up after a time limit, records which wait it was in a device status word and lets
the kernel return.  ``gg_selftest_wait_timeout`` runs that same wait on a barrier nothing ever
completes, with a limit of a few milliseconds: the kernel must come back, report "did not
complete", and ``gg_device_status`` must return the self-test's site code once and then zero.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_that_nothing_completes_times_out_and_reports():
    from grain_gemm_b200 import _loader

    lib = _loader.library()
    assert _loader.device_status() == 0
    result = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    status = lib.gg_selftest_wait_timeout(2_000_000, _loader.pointer(result),
                                          _loader.stream_pointer(result.device))
    stop.record()
    assert status == 0
    torch.cuda.synchronize()
    assert int(result.item()) == 0                     # the wait reported failure, not success
    assert start.elapsed_time(stop) < 1000.0           # and gave up promptly (limit 2 ms)
    assert _loader.device_status() == (15 << 8) | 1    # site code of the self-test, code 1
    assert _loader.device_status() == 0                # reading clears the word
    # The context is still usable: a normal kernel runs and reports no status.
    from grain_gemm_b200 import int8_gemm
    a = torch.ones((128, 256), dtype=torch.int8, device="cuda")
    b = torch.ones((64, 256), dtype=torch.int8, device="cuda").t()
    out = int8_gemm(a, b, torch.ones((128, 1), device="cuda"), torch.ones((1, 64), device="cuda"),
                    output_dtype=torch.float32)
    assert torch.equal(out, torch.full((128, 64), 256.0, device="cuda"))
    assert _loader.device_status() == 0


def test_selftest_rejects_unbounded_limits():
    from grain_gemm_b200 import _loader

    lib = _loader.library()
    result = torch.zeros((1,), dtype=torch.int32, device="cuda")
    for limit in (0, -5, 100_000_001):
        assert lib.gg_selftest_wait_timeout(limit, _loader.pointer(result), None) == 1
    assert lib.gg_selftest_wait_timeout(1000, ctypes.c_void_p(0), None) == 1


def test_report_to_host_stores_words_in_pinned_memory():
    """The routing statistics reach the host through a kernel store into page-locked memory
    (no copy engine involved); memory the device cannot address is refused with the driver's
    error before any launch."""
    from grain_gemm_b200 import _loader

    lib = _loader.library()
    values = torch.arange(100, 137, dtype=torch.int32, device="cuda")
    host = torch.zeros((37,), dtype=torch.int32).pin_memory()
    status = lib.gg_report_to_host(_loader.pointer(values), 37, host.data_ptr(),
                                   _loader.stream_pointer(values.device))
    assert status == 0
    torch.cuda.synchronize()
    assert host.tolist() == list(range(100, 137))
    pageable = torch.zeros((64,), dtype=torch.int32)
    refused = lib.gg_report_to_host(_loader.pointer(values), 3, pageable.data_ptr(),
                                    _loader.stream_pointer(values.device))
    torch.cuda.synchronize()
    # Either the driver has no device address for pageable memory (the usual answer: nothing is
    # launched, nothing is written) or the system maps all host memory and the words arrive.
    assert pageable[:3].tolist() == ([0, 0, 0] if refused else [100, 101, 102])
    assert _loader.device_status() == 0
