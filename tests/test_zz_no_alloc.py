"""The allocation-free statistics entry point against the list-based one.

Collected last on purpose (file name), so that a run that stops at the first failure has
already exercised everything else.  The entry point serves callers that cannot allocate device
memory (a trainer running after the inference engine has taken the free memory for its KV
cache; hot paths that must stay out of the allocator): its reduction scratch is a fixed array
inside the library, shared by every call, so two calls in a row are checked to make sure
nothing left behind by the first one leaks into the second."""
import numpy as np
import pytest

from helpers import read_stat

pytestmark = pytest.mark.gpu

NORM_BAR = 1e-5      # relative, the bar the other statistics tests use


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available(), "this test needs a CUDA device"
    torch.cuda.set_device(0)
    return torch


def list_based(pkg, torch, g, dtype, unscale, max_norm):
    tl = pkg.TensorList([pkg.TensorDesc(None, g.data_ptr(), None, None, None, g.numel(), 0.0, dtype,
                                        pkg.TENSOR_NORM_ONLY, 0)])
    stat = torch.zeros(16, device="cuda")
    tl.gradstat(stat.data_ptr(), unscale, max_norm)
    torch.cuda.synchronize()
    tl.close()
    return read_stat(pkg, stat)


def no_alloc(pkg, torch, g, dtype, unscale, max_norm):
    stat = torch.full((16,), 7.0, device="cuda")          # stale contents must be overwritten
    pkg.gradstat_flat_noalloc(g.data_ptr(), dtype, g.numel(), stat.data_ptr(), unscale, max_norm)
    torch.cuda.synchronize()
    return read_stat(pkg, stat)


def agree(a, b):
    assert a.found_inf == b.found_inf
    if a.found_inf:
        return
    assert a.clip_active == b.clip_active
    assert abs(a.norm - b.norm) <= NORM_BAR * b.norm
    assert abs(a.sum_sq - b.sum_sq) <= 2 * NORM_BAR * b.sum_sq
    assert abs(a.coef - b.coef) <= NORM_BAR * abs(b.coef)


def test_two_calls_in_a_row_match_the_list_based_pass(pkg, torch):
    gen = torch.Generator(device="cuda").manual_seed(3)
    big = (torch.randn(20_000_003, device="cuda", generator=gen) * 1e-4).half()      # ragged size
    small = (torch.randn(70_001, device="cuda", generator=gen) * 3e-2).half()
    # first call: large buffer, loss-scale style unscale, clip inactive
    agree(no_alloc(pkg, torch, big, pkg.F16, 0.5, 10.0), list_based(pkg, torch, big, pkg.F16, 0.5, 10.0))
    # second call right after: smaller buffer (fewer scratch slots than the first call used),
    # clip active
    second = no_alloc(pkg, torch, small, pkg.F16, 1.0, 1.0)
    agree(second, list_based(pkg, torch, small, pkg.F16, 1.0, 1.0))
    assert second.clip_active == 1
    exact = float(torch.sqrt((small.double() ** 2).sum()))
    assert abs(second.norm - exact) <= NORM_BAR * exact


def test_overflow_then_clean_and_fp32_and_misaligned(pkg, torch):
    gen = torch.Generator(device="cuda").manual_seed(4)
    g = (torch.randn(1_000_000, device="cuda", generator=gen) * 1e-2).half()
    bad = g.clone()
    bad[123_456] = float("inf")
    assert no_alloc(pkg, torch, bad, pkg.F16, 1.0 / 65536, 1.0).found_inf == 1
    clean = no_alloc(pkg, torch, g, pkg.F16, 1.0, 1.0)       # the flag must not stick
    agree(clean, list_based(pkg, torch, g, pkg.F16, 1.0, 1.0))
    g32 = torch.randn(300_007, device="cuda", generator=gen) * 1e-3
    agree(no_alloc(pkg, torch, g32, pkg.F32, 1.0, 0.1), list_based(pkg, torch, g32, pkg.F32, 1.0, 0.1))
    off = g[3:200_000]                                       # pointer off the 16-byte grid
    agree(no_alloc(pkg, torch, off, pkg.F16, 1.0, 0.0), list_based(pkg, torch, off, pkg.F16, 1.0, 0.0))
    empty = no_alloc(pkg, torch, g[:0], pkg.F16, 1.0, 1.0)
    assert empty.norm == 0.0 and empty.found_inf == 0 and empty.coef == 1.0


def test_two_pools_of_one_step_combine_into_one_record(pkg, torch):
    """RL.cu's clip norm covers its FP16 gradient pool and its FP32 one (trainer.h:331-337): the
    first call leaves only its sum (STAT_PARTIAL), the second adds its own and finishes the
    record (STAT_ACCUMULATE); the result is the list-based pass over both tensors."""
    gen = torch.Generator(device="cuda").manual_seed(5)
    g16 = (torch.randn(3_000_001, device="cuda", generator=gen) * 1e-3).half()
    g32 = torch.randn(65_536 + 777, device="cuda", generator=gen) * 1e-2
    stat = torch.full((16,), 7.0, device="cuda")
    for _ in range(2):                                     # twice: the record is reused every step
        pkg.gradstat_flat_noalloc(g16.data_ptr(), pkg.F16, g16.numel(), stat.data_ptr(), 1.0, 1.0, pkg.STAT_PARTIAL)
        pkg.gradstat_flat_noalloc(g32.data_ptr(), pkg.F32, g32.numel(), stat.data_ptr(), 1.0, 1.0, pkg.STAT_ACCUMULATE)
        torch.cuda.synchronize()
        got = read_stat(pkg, stat)
        tl = pkg.TensorList([
            pkg.TensorDesc(None, g16.data_ptr(), None, None, None, g16.numel(), 0.0, pkg.F16, pkg.TENSOR_NORM_ONLY, 0),
            pkg.TensorDesc(None, g32.data_ptr(), None, None, None, g32.numel(), 0.0, pkg.F32, pkg.TENSOR_NORM_ONLY, 0)])
        want = torch.zeros(16, device="cuda")
        tl.gradstat(want.data_ptr(), 1.0, 1.0)
        torch.cuda.synchronize()
        tl.close()
        agree(got, read_stat(pkg, want))
        assert got.clip_active == 1
    # an inf in the first pool survives the second call
    bad = g16.clone()
    bad[17] = float("-inf")
    pkg.gradstat_flat_noalloc(bad.data_ptr(), pkg.F16, bad.numel(), stat.data_ptr(), 1.0, 1.0, pkg.STAT_PARTIAL)
    pkg.gradstat_flat_noalloc(g32.data_ptr(), pkg.F32, g32.numel(), stat.data_ptr(), 1.0, 1.0, pkg.STAT_ACCUMULATE)
    torch.cuda.synchronize()
    assert read_stat(pkg, stat).found_inf == 1


def test_second_device_in_the_same_process_has_its_own_scratch(pkg, torch):
    """The scratch address is resolved once per device (with that device current): calls on two
    devices of one process each use their own copy of the array and give their own results."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    results = []
    try:
        for dev in (0, 1, 0):
            torch.cuda.set_device(dev)
            gen = torch.Generator(device=f"cuda:{dev}").manual_seed(10 + dev)
            g = (torch.randn(1_000_003, device=f"cuda:{dev}", generator=gen) * 1e-2).half()
            stat = torch.full((16,), 7.0, device=f"cuda:{dev}")
            pkg.gradstat_flat_noalloc(g.data_ptr(), pkg.F16, g.numel(), stat.data_ptr(), 1.0, 1.0)
            torch.cuda.synchronize(dev)
            got = read_stat(pkg, stat)
            exact = float(torch.sqrt((g.double() ** 2).sum()))
            assert abs(got.norm - exact) <= NORM_BAR * exact and got.found_inf == 0
            results.append(got.norm)
    finally:
        torch.cuda.set_device(0)
    assert results[0] == results[2] and results[0] != results[1]


def test_sizes_beyond_the_fixed_scratch_are_refused(pkg, torch):
    g = torch.zeros(16, device="cuda").half()
    stat = torch.zeros(16, device="cuda")
    with pytest.raises(pkg.RlcuError) as err:
        pkg.gradstat_flat_noalloc(g.data_ptr(), pkg.F16, pkg.NOALLOC_MAX_ELEMS + 1, stat.data_ptr())
    assert err.value.code == pkg.ERR_INVALID and "exceed the fixed scratch" in str(err.value)
