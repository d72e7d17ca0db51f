"""GPU parity tests of the single-tensor entry points (the launch_adamw_* replacements),
called through the C ABI.  Bars: FP16 parameters within 1 ulp, FP32 moments and masters
within 1e-6 relative.  The kernels are written to reproduce the reference bit for bit, and
the tests also assert that stronger property."""
import numpy as np
import pytest

from helpers import DevBuf, fresh_grad, max_rel, seeded_case, ulp16

pytestmark = pytest.mark.gpu

ULP_BAR = 1          # FP16 parameters
REL_BAR = 1e-6       # FP32 moments and master weights


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch


def check_state(got, want, exact=True):
    for name in want:
        a, b = got[name], want[name]
        if a.dtype == np.uint16:
            assert ulp16(a, b).max(initial=0) <= ULP_BAR, f"{name}: more than {ULP_BAR} ulp"
        else:
            assert max_rel(a, b) <= REL_BAR, f"{name}: relative error above {REL_BAR}"
        if exact:
            assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), f"{name}: not bit-identical"


def test_config1_ten_steps_fp16_master(pkg, O, torch):
    """Single tensor, N=1,048,576, seed 0, ten steps with fresh seeded gradients:
    new kernel vs CPU oracle vs the reference's own CUDA kernel."""
    n, lr, b1, b2, eps, wd = 1 << 20, 1e-5, 0.9, 0.999, 1e-8, 0.01
    p0, _, m0, v0 = seeded_case(O, n, seed=0)
    host = dict(master=O.h2f(p0), p=p0.copy(), m=m0.copy(), v=v0.copy())
    dev = {k: DevBuf(a, torch) for k, a in host.items()}
    ref = {k: DevBuf(a, torch) for k, a in host.items()} if O.ref_available() else None
    for t in range(1, 11):
        g = fresh_grad(O, n, seed=0, step=t)
        gd = DevBuf(g, torch)
        bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)
        pkg.adamw_fp16_master(dev["master"].ptr, dev["p"].ptr, gd.ptr, dev["m"].ptr, dev["v"].ptr,
                              n, lr, b1, b2, eps, wd, bc1, bc2)
        O.adamw_fp16_master(host["master"], host["p"], g, host["m"], host["v"],
                            lr, b1, b2, eps, wd, bc1, bc2, O.NVCC, 0)
        if ref:
            rc = O.ref_lib().ref_launch_adamw_fp16(ref["master"].ptr, ref["p"].ptr, gd.ptr, ref["m"].ptr,
                                                   ref["v"].ptr, n, lr, b1, b2, eps, wd, bc1, bc2, None)
            assert rc == 0
        torch.cuda.synchronize()
        assert gd.guards_intact()
    got = {k: d.get() for k, d in dev.items()}
    check_state(got, host)
    if ref:
        check_state(got, {k: d.get() for k, d in ref.items()})
    assert all(d.guards_intact() for d in dev.values())


@pytest.mark.parametrize("tail", [0, 4099])
def test_large_tensor_with_master_takes_the_bulk_copy_kernel(pkg, O, torch, tail):
    """rlcu_adamw_fp16_master on a tensor large enough for the bulk-copy kernel (at least four
    work items per SM), with and without a ragged last item: three steps against the CPU oracle
    and the reference's own kernel, bit for bit, guard bytes intact, no bounded wait gave up."""
    n, lr, b1, b2, eps, wd = 8192 * 700 + tail, 1e-4, 0.9, 0.999, 1e-8, 0.01
    p0, _, m0, v0 = seeded_case(O, n, seed=3, warm=True)
    host = dict(master=O.h2f(p0), p=p0.copy(), m=m0.copy(), v=v0.copy())
    dev = {k: DevBuf(a, torch) for k, a in host.items()}
    ref = {k: DevBuf(a, torch) for k, a in host.items()} if O.ref_available() else None
    for t in range(1, 4):
        g = fresh_grad(O, n, seed=3, step=t, g_std=1e-2)
        gd = DevBuf(g, torch)
        bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)
        pkg.adamw_fp16_master(dev["master"].ptr, dev["p"].ptr, gd.ptr, dev["m"].ptr, dev["v"].ptr,
                              n, lr, b1, b2, eps, wd, bc1, bc2)
        O.adamw_fp16_master(host["master"], host["p"], g, host["m"], host["v"],
                            lr, b1, b2, eps, wd, bc1, bc2, O.NVCC, 0)
        if ref:
            assert O.ref_lib().ref_launch_adamw_fp16(ref["master"].ptr, ref["p"].ptr, gd.ptr, ref["m"].ptr,
                                                     ref["v"].ptr, n, lr, b1, b2, eps, wd, bc1, bc2, None) == 0
        torch.cuda.synchronize()
        assert gd.guards_intact() and np.array_equal(gd.get(), g)
    assert pkg.lib().rlcu_tensor_list_check(None) == pkg.OK
    got = {k: d.get() for k, d in dev.items()}
    check_state(got, host)
    if ref:
        check_state(got, {k: d.get() for k, d in ref.items()})
    assert all(d.guards_intact() for d in dev.values())


def test_config1_masterless(pkg, O, torch):
    n, lr, b1, b2, eps, wd = 1 << 20, 1e-5, 0.9, 0.999, 1e-8, 0.01
    p0, _, m0, v0 = seeded_case(O, n, seed=0)
    host = dict(p=p0.copy(), m=m0.copy(), v=v0.copy())
    dev = {k: DevBuf(a, torch) for k, a in host.items()}
    for t in range(1, 11):
        g = fresh_grad(O, n, seed=0, step=t)
        gd = DevBuf(g, torch)
        bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)
        pkg.adamw_fp16(dev["p"].ptr, gd.ptr, dev["m"].ptr, dev["v"].ptr, n, lr, b1, b2, eps, wd, bc1, bc2)
        O.adamw_fp16(host["p"], g, host["m"], host["v"], lr, b1, b2, eps, wd, bc1, bc2, O.NVCC, 0)
    torch.cuda.synchronize()
    check_state({k: d.get() for k, d in dev.items()}, host)
    assert all(d.guards_intact() for d in dev.values())


def test_fp32_tensor_vs_oracle_and_reference(pkg, O, torch):
    n, lr, b1, b2, eps = 65536, 1e-5, 0.9, 0.999, 1e-8
    rng = np.random.default_rng(7)
    host = dict(w=(1 + rng.standard_normal(n) * 0.01).astype(np.float32),
                m=np.zeros(n, np.float32), v=np.zeros(n, np.float32))
    dev = {k: DevBuf(a, torch) for k, a in host.items()}
    ref = {k: DevBuf(a, torch) for k, a in host.items()} if O.ref_available() else None
    for t in range(1, 6):
        g = (np.random.default_rng([7, t]).standard_normal(n) * 1e-3).astype(np.float32)
        gd = DevBuf(g, torch)
        bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)
        pkg.adamw_fp32(dev["w"].ptr, gd.ptr, dev["m"].ptr, dev["v"].ptr, n, lr, b1, b2, eps, 0.0, bc1, bc2)
        O.adamw_fp32(host["w"], g, host["m"], host["v"], lr, b1, b2, eps, 0.0, bc1, bc2, O.NVCC, 0)
        if ref:
            assert O.ref_lib().ref_launch_adamw_fp32(ref["w"].ptr, gd.ptr, ref["m"].ptr, ref["v"].ptr, n,
                                                     lr, b1, b2, eps, 0.0, bc1, bc2, None) == 0
        torch.cuda.synchronize()
    got = {k: d.get() for k, d in dev.items()}
    check_state(got, host)
    if ref:
        check_state(got, {k: d.get() for k, d in ref.items()})


RAGGED = [1, 2, 7, 8, 9, 63, 64, 65, 255, 2047, 2048, 2049, 8191, 8192, 8193, 16385, 100_003]


@pytest.mark.parametrize("offset", [0, 1, 3, 8])
def test_ragged_sizes_and_misaligned_pointers(pkg, O, torch, offset):
    """Every size around the vector width and the work-item size, with pointers shifted off
    their 16-byte alignment: vector path, tails and the scalar path against the oracle,
    guard bytes around every buffer intact."""
    lr, b1, b2, eps, wd, t = 1e-3, 0.9, 0.999, 1e-8, 0.01, 3
    bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)
    for n in RAGGED:
        p, g, m, v = seeded_case(O, n, seed=n, warm=True)
        # FP16 with master
        host = dict(master=O.h2f(p), p=p.copy(), m=m.copy(), v=v.copy())
        dev = {k: DevBuf(a, torch, offset) for k, a in host.items()}
        gd = DevBuf(g, torch, offset)
        pkg.adamw_fp16_master(dev["master"].ptr, dev["p"].ptr, gd.ptr, dev["m"].ptr, dev["v"].ptr,
                              n, lr, b1, b2, eps, wd, bc1, bc2)
        O.adamw_fp16_master(host["master"], host["p"], g, host["m"], host["v"], lr, b1, b2, eps, wd, bc1, bc2)
        torch.cuda.synchronize()
        check_state({k: d.get() for k, d in dev.items()}, host)
        assert all(d.guards_intact() for d in dev.values()) and gd.guards_intact(), n
        # FP16 without master
        host = dict(p=p.copy(), m=m.copy(), v=v.copy())
        dev = {k: DevBuf(a, torch, offset) for k, a in host.items()}
        pkg.adamw_fp16(dev["p"].ptr, gd.ptr, dev["m"].ptr, dev["v"].ptr, n, lr, b1, b2, eps, wd, bc1, bc2)
        O.adamw_fp16(host["p"], g, host["m"], host["v"], lr, b1, b2, eps, wd, bc1, bc2)
        torch.cuda.synchronize()
        check_state({k: d.get() for k, d in dev.items()}, host)
        assert all(d.guards_intact() for d in dev.values()), n
        # FP32
        g32 = O.h2f(g)
        host = dict(w=O.h2f(p), m=m.copy(), v=v.copy())
        dev = {k: DevBuf(a, torch, offset) for k, a in host.items()}
        gd32 = DevBuf(g32, torch, offset)
        pkg.adamw_fp32(dev["w"].ptr, gd32.ptr, dev["m"].ptr, dev["v"].ptr, n, lr, b1, b2, eps, wd, bc1, bc2)
        O.adamw_fp32(host["w"], g32, host["m"], host["v"], lr, b1, b2, eps, wd, bc1, bc2)
        torch.cuda.synchronize()
        check_state({k: d.get() for k, d in dev.items()}, host)
        assert all(d.guards_intact() for d in dev.values()) and gd32.guards_intact(), n


def test_mixed_alignment_falls_back_correctly(pkg, O, torch):
    """Pointers with different misalignments (no common vector phase)."""
    n, lr, b1, b2, eps, wd, t = 10_007, 1e-3, 0.9, 0.999, 1e-8, 0.0, 2
    bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)
    p, g, m, v = seeded_case(O, n, seed=99, warm=True)
    host = dict(p=p.copy(), m=m.copy(), v=v.copy())
    dev = dict(p=DevBuf(p, torch, 1), m=DevBuf(m, torch, 2), v=DevBuf(v, torch, 0))
    gd = DevBuf(g, torch, 5)
    pkg.adamw_fp16(dev["p"].ptr, gd.ptr, dev["m"].ptr, dev["v"].ptr, n, lr, b1, b2, eps, wd, bc1, bc2)
    O.adamw_fp16(host["p"], g, host["m"], host["v"], lr, b1, b2, eps, wd, bc1, bc2)
    torch.cuda.synchronize()
    check_state({k: d.get() for k, d in dev.items()}, host)
    assert all(d.guards_intact() for d in dev.values())


def test_half_to_float_master_init(pkg, O, torch):
    """fp16_to_fp32 of include/training/optimizer.h:46-57."""
    for n, off in ((1, 0), (7, 1), (8192, 0), (100_003, 0), (100_003, 3)):
        p, _, _, _ = seeded_case(O, n, seed=n)
        src = DevBuf(p, torch, off)
        dst = DevBuf(np.zeros(n, np.float32), torch, off)
        pkg.half_to_float(dst.ptr, src.ptr, n)
        torch.cuda.synchronize()
        assert np.array_equal(dst.get(), O.h2f(p))
        assert dst.guards_intact()


def test_cxx_launchers_forward(pkg, O, torch):
    """The C++-linkage launch_adamw_fp16 (RL.cu's signature, `int n`) gives the same result."""
    import ctypes as C
    n, lr, b1, b2, eps, wd, t = 50_000, 1e-4, 0.9, 0.999, 1e-8, 0.01, 2
    bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)
    p, g, m, v = seeded_case(O, n, seed=3, warm=True)
    host = dict(master=O.h2f(p), p=p.copy(), m=m.copy(), v=v.copy())
    dev = {k: DevBuf(a, torch) for k, a in host.items()}
    gd = DevBuf(g, torch)
    fn = getattr(pkg.lib(), pkg.CXX_EXPORTS[0])
    fn.argtypes = [C.c_void_p] * 5 + [C.c_int] + [C.c_float] * 7 + [C.c_void_p]
    fn.restype = None
    fn(dev["master"].ptr, dev["p"].ptr, gd.ptr, dev["m"].ptr, dev["v"].ptr, n, lr, b1, b2, eps, wd, bc1, bc2, None)
    O.adamw_fp16_master(host["master"], host["p"], g, host["m"], host["v"], lr, b1, b2, eps, wd, bc1, bc2)
    torch.cuda.synchronize()
    check_state({k: d.get() for k, d in dev.items()}, host)


def test_runs_on_a_side_stream(pkg, O, torch):
    n, lr, b1, b2, eps, wd, t = 300_000, 1e-4, 0.9, 0.999, 1e-8, 0.01, 5
    bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)
    p, g, m, v = seeded_case(O, n, seed=4, warm=True)
    host = dict(p=p.copy(), m=m.copy(), v=v.copy())
    dev = {k: DevBuf(a, torch) for k, a in host.items()}
    gd = DevBuf(g, torch)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    pkg.adamw_fp16(dev["p"].ptr, gd.ptr, dev["m"].ptr, dev["v"].ptr, n, lr, b1, b2, eps, wd, bc1, bc2,
                   stream=s.cuda_stream)
    s.synchronize()
    O.adamw_fp16(host["p"], g, host["m"], host["v"], lr, b1, b2, eps, wd, bc1, bc2)
    check_state({k: d.get() for k, d in dev.items()}, host)


def test_invalid_arguments_are_rejected(pkg, torch):
    a = torch.zeros(64, device="cuda")
    L = pkg.lib()
    rc = L.rlcu_adamw_fp16_master(None, a.data_ptr(), a.data_ptr(), a.data_ptr(), a.data_ptr(), 8,
                                  1e-3, .9, .999, 1e-8, 0, .1, .001, None)
    assert rc == pkg.ERR_INVALID
    rc = L.rlcu_adamw_fp32(a.data_ptr() + 2, a.data_ptr(), a.data_ptr(), a.data_ptr(), 8,
                           1e-3, .9, .999, 1e-8, 0, .1, .001, None)
    assert rc == pkg.ERR_INVALID and b"aligned" in L.rlcu_last_error()
