"""GPU parity tests of the fused step: statistics pass (unscale, non-finite, norm, clip
factor) + multi-tensor update, through the C ABI.  Bars: FP16 parameters within 1 ulp,
FP32 moments within 1e-6 relative, gradient norm within 1e-5 relative; bit identity is
asserted as well wherever the reference's own result is deterministic."""
import ctypes as C

import numpy as np
import pytest

from helpers import DevBuf, max_rel, qwen3_0p6b, read_stat, seeded_case, ulp16

pytestmark = pytest.mark.gpu

NORM_BAR = 1e-5


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch


def make_case(O, torch, pkg, specs, seed, g_std=1e-2, offset=0):
    """specs: list of (n, kind, wd, flags) with kind in {'h', 'hm', 'f', 'hg', 'hmg'}: FP16,
    FP16 with FP32 master, FP32, and the two FP16 kinds with an FP32 gradient.  Returns the
    host entries (oracle side), device buffers and the product's descriptors."""
    host, dev, descs = [], [], []
    for k, (n, kind, wd, flags) in enumerate(specs):
        p, g, m, v = seeded_case(O, n, seed=[seed, k], g_std=g_std, warm=True)
        e = dict(wd=wd, flags=flags)
        if kind == "f":
            e.update(p=O.h2f(p), g=O.h2f(g), m=m, v=v)
        else:
            e.update(p=p, g=g, m=m, v=v)
            if kind in ("hm", "hmg"):
                e["master"] = O.h2f(p)
            if kind in ("hg", "hmg"):
                # an FP32 gradient with bits below FP16 resolution, as FP32 accumulation leaves them
                fine = np.random.default_rng([seed, k, 9]).standard_normal(n).astype(np.float32)
                e["g"] = (O.h2f(g) * (np.float32(1) + np.float32(2.0 ** -14) * fine)).astype(np.float32)
                e["grad_dtype"] = O.GRAD_F32
        d = {name: DevBuf(e[name], torch, offset) for name in ("p", "g", "m", "v", "master") if name in e}
        host.append(e)
        dev.append(d)
        descs.append(pkg.TensorDesc(d["p"].ptr, d["g"].ptr, d["m"].ptr, d["v"].ptr,
                                    d["master"].ptr if "master" in d else None, n, wd,
                                    pkg.F32 if kind == "f" else pkg.F16, flags,
                                    pkg.GRAD_F32 if kind in ("hg", "hmg") else pkg.GRAD_AS_PARAM))
    return host, dev, descs


def assert_same(host, dev, exact=True):
    for e, d in zip(host, dev):
        for name in ("p", "m", "v", "master"):
            if name not in d:
                continue
            got, want = d[name].get(), e[name]
            if got.dtype == np.uint16:
                assert ulp16(got, want).max(initial=0) <= 1, f"{name}: more than 1 ulp"
            else:
                assert max_rel(got, want) <= 1e-6, f"{name}: relative error above 1e-6"
            if exact:
                assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), f"{name} not bit-identical"
        assert all(b.guards_intact() for b in d.values())


MIXED = [(70_001, "h", 0.01, 0), (1024, "hm", 0.0, 0), (8192 * 3, "hm", 0.01, 0), (129, "f", 0.0, 0),
         (1, "h", 0.0, 0), (8192, "h", 0.01, 0), (8193, "f", 0.01, 0), (0, "h", 0.0, 0), (40_000, "hm", 0.02, 0)]


@pytest.mark.parametrize("max_norm,flags_round", [(1.0, True), (1.0, False), (0.0, False), (1e6, True)])
def test_fused_step_vs_oracle(pkg, O, torch, max_norm, flags_round):
    host, dev, descs = make_case(O, torch, pkg, MIXED, seed=11)
    stat = torch.zeros(16, device="cuda")
    tl = pkg.TensorList(descs)
    assert tl.numel == sum(s[0] for s in MIXED)
    lr, b1, b2, eps, t = 1e-4, 0.9, 0.999, 1e-8, 6
    hp = pkg.hparams(lr, b1, b2, eps, t)
    flags = pkg.STEP_ROUND_CLIP_FP16 if flags_round else 0
    tl.gradstat(stat.data_ptr(), 1.0, max_norm)
    tl.step(hp, stat.data_ptr(), flags)
    torch.cuda.synchronize()
    got = read_stat(pkg, stat)

    ot = O.make_tensors(host)
    want = O.gradstat(ot, 1.0, max_norm)
    assert got.found_inf == 0
    assert abs(got.norm - want.norm) <= NORM_BAR * want.norm
    assert abs(got.sum_sq - want.sum_sq) <= NORM_BAR * want.sum_sq
    assert got.clip_active == want.clip_active == (1 if 0 < max_norm < 100 else 0)
    # the update is checked bit for bit given the statistics record the device produced
    dev_stat = O.gradstat_finalize(got.sum_sq, 0, 1.0, max_norm)
    assert dev_stat.coef == got.coef and dev_stat.norm == got.norm
    O.multi_step(ot, O.HParams(lr, b1, b2, eps, hp.bias_correction1, hp.bias_correction2), dev_stat,
                 O.STEP_ROUND_CLIP_FP16 if flags_round else 0)
    assert_same(host, dev)
    tl.close()


def test_update_without_statistics_is_plain_adamw(pkg, O, torch):
    host, dev, descs = make_case(O, torch, pkg, MIXED, seed=12, offset=0)
    tl = pkg.TensorList(descs)
    hp = pkg.hparams(3e-4, 0.9, 0.999, 1e-8, 2)
    tl.step(hp)
    torch.cuda.synchronize()
    O.multi_step(O.make_tensors(host), O.HParams(3e-4, 0.9, 0.999, 1e-8, hp.bias_correction1, hp.bias_correction2), None)
    assert_same(host, dev)


@pytest.mark.parametrize("offset", [1, 3])
def test_fused_step_misaligned_tensors(pkg, O, torch, offset):
    host, dev, descs = make_case(O, torch, pkg, MIXED, seed=13, offset=offset)
    stat = torch.zeros(16, device="cuda")
    tl = pkg.TensorList(descs)
    hp = pkg.hparams(1e-4, 0.9, 0.999, 1e-8, 3)
    tl.gradstat(stat.data_ptr(), 1.0, 0.5)
    tl.step(hp, stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16)
    torch.cuda.synchronize()
    got = read_stat(pkg, stat)
    ot = O.make_tensors(host)
    want = O.gradstat(ot, 1.0, 0.5)
    assert abs(got.norm - want.norm) <= NORM_BAR * want.norm
    O.multi_step(ot, O.HParams(1e-4, 0.9, 0.999, 1e-8, hp.bias_correction1, hp.bias_correction2),
                 O.gradstat_finalize(got.sum_sq, 0, 1.0, 0.5), O.STEP_ROUND_CLIP_FP16)
    assert_same(host, dev)


def test_statistics_are_deterministic(pkg, O, torch):
    """Same inputs, same bits, run after run (the reference's atomic sum is not)."""
    n = 3_000_017
    g = (torch.randn(n, device="cuda") * 1e-2).half()
    tl = pkg.TensorList([pkg.TensorDesc(None, g.data_ptr(), None, None, None, n, 0.0, pkg.F16, pkg.TENSOR_NORM_ONLY, 0)])
    stat = torch.zeros(16, device="cuda")
    seen = set()
    for _ in range(5):
        tl.gradstat(stat.data_ptr(), 1.0, 1.0)
        torch.cuda.synchronize()
        seen.add(stat.cpu().numpy().tobytes())
    assert len(seen) == 1
    s = read_stat(pkg, stat)
    exact = float((g.double() ** 2).sum())
    assert abs(s.sum_sq - exact) <= NORM_BAR * exact


def test_reference_sequence_bit_exact_when_its_sum_is_exact(pkg, O, torch):
    """clip_grad_norm_ then the three launch_adamw_* calls of RL.cu, run with the reference's
    own kernels, against one statistics pass + one update launch.  The gradients are powers
    of two so the reference's unordered FP32 atomic sum is exact and its result is well defined."""
    if not O.ref_available():
        pytest.skip("reference kernels were not built")
    R = O.ref_lib()
    rng = np.random.default_rng(21)
    n16a, n16b, n32 = 60_000, 30_000, 4_000
    def pow2(n):
        return (rng.choice([-1.0, 1.0], n) * np.exp2(-rng.integers(5, 9, n))).astype(np.float32)
    g16 = O.f2h(pow2(n16a + n16b))
    g32 = pow2(n32)
    p16, _, m16, v16 = seeded_case(O, n16a + n16b, seed=22, warm=True)
    w32 = (1 + rng.standard_normal(n32) * 0.01).astype(np.float32)
    m32, v32 = np.zeros(n32, np.float32), np.zeros(n32, np.float32)
    lr, b1, b2, eps, wd, t, max_norm = 1e-4, 0.9, 0.999, 1e-8, 0.01, 3, 1.0
    bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)

    def buffers():
        return dict(g16=DevBuf(g16, torch), g32=DevBuf(g32, torch), p=DevBuf(p16, torch),
                    master=DevBuf(O.h2f(p16), torch), m=DevBuf(m16, torch), v=DevBuf(v16, torch),
                    w32=DevBuf(w32, torch), m32=DevBuf(m32, torch), v32=DevBuf(v32, torch))
    ref, mine = buffers(), buffers()

    acc = torch.zeros(1, device="cuda")
    norm = C.c_float()
    assert R.ref_clip_grad_norm(ref["g16"].ptr, n16a + n16b, ref["g32"].ptr, n32, max_norm, acc.data_ptr(), C.byref(norm)) == 0
    # optimizer.h:126-146: projections with weight decay, embedding without, norms without
    assert R.ref_launch_adamw_fp16(ref["master"].ptr, ref["p"].ptr, ref["g16"].ptr, ref["m"].ptr, ref["v"].ptr,
                                   n16a, lr, b1, b2, eps, wd, bc1, bc2, None) == 0
    assert R.ref_launch_adamw_fp16(ref["master"].ptr + 4 * n16a, ref["p"].ptr + 2 * n16a, ref["g16"].ptr + 2 * n16a,
                                   ref["m"].ptr + 4 * n16a, ref["v"].ptr + 4 * n16a,
                                   n16b, lr, b1, b2, eps, 0.0, bc1, bc2, None) == 0
    assert R.ref_launch_adamw_fp32(ref["w32"].ptr, ref["g32"].ptr, ref["m32"].ptr, ref["v32"].ptr,
                                   n32, lr, b1, b2, eps, 0.0, bc1, bc2, None) == 0

    d = mine
    descs = [pkg.TensorDesc(d["p"].ptr, d["g16"].ptr, d["m"].ptr, d["v"].ptr, d["master"].ptr, n16a, wd, pkg.F16, 0, 0),
             pkg.TensorDesc(d["p"].ptr + 2 * n16a, d["g16"].ptr + 2 * n16a, d["m"].ptr + 4 * n16a, d["v"].ptr + 4 * n16a,
                            d["master"].ptr + 4 * n16a, n16b, 0.0, pkg.F16, 0, 0),
             pkg.TensorDesc(d["w32"].ptr, d["g32"].ptr, d["m32"].ptr, d["v32"].ptr, None, n32, 0.0, pkg.F32, 0, 0)]
    tl = pkg.TensorList(descs)
    stat = torch.zeros(16, device="cuda")
    tl.gradstat(stat.data_ptr(), 1.0, max_norm)
    tl.step(pkg.HParams(lr, b1, b2, eps, bc1, bc2), stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16)
    torch.cuda.synchronize()
    s = read_stat(pkg, stat)
    assert s.norm == norm.value and s.clip_active == 1          # pre-clip norm, bit for bit
    for name in ("p", "master", "m", "v", "w32", "m32", "v32"):
        assert np.array_equal(mine[name].get().view(np.uint8), ref[name].get().view(np.uint8)), name
    # the fused path leaves the gradients as they were; the reference scaled them in place
    assert np.array_equal(mine["g16"].get(), g16)


def test_norm_vs_reference_kernels_on_random_gradients(pkg, O, torch):
    if not O.ref_available():
        pytest.skip("reference kernels were not built")
    n16, n32 = 5_000_000, 65_536
    g16 = (torch.randn(n16, device="cuda") * 1e-4).half()
    g32 = torch.randn(n32, device="cuda") * 1e-4
    acc, out = torch.zeros(1, device="cuda"), C.c_float()
    assert O.ref_lib().ref_grad_sum_sq(g16.data_ptr(), n16, g32.data_ptr(), n32, acc.data_ptr(), C.byref(out)) == 0
    tl = pkg.TensorList([pkg.TensorDesc(None, g16.data_ptr(), None, None, None, n16, 0.0, pkg.F16, pkg.TENSOR_NORM_ONLY, 0),
                         pkg.TensorDesc(None, g32.data_ptr(), None, None, None, n32, 0.0, pkg.F32, pkg.TENSOR_NORM_ONLY, 0)])
    stat = torch.zeros(16, device="cuda")
    tl.gradstat(stat.data_ptr(), 1.0, 0.0)
    torch.cuda.synchronize()
    s = read_stat(pkg, stat)
    ref_norm = float(np.sqrt(np.float32(out.value)))
    exact = float(torch.sqrt((g16.double() ** 2).sum() + (g32.double() ** 2).sum()))
    assert abs(s.norm - ref_norm) <= NORM_BAR * ref_norm
    assert abs(s.norm - exact) <= NORM_BAR * exact
    assert s.coef == 1.0 and s.clip_active == 0


@pytest.mark.parametrize("bad", [0x7C00, 0xFC00, 0x7E00])
def test_non_finite_gradient_skips_the_step(pkg, O, torch, bad):
    specs = [(20_000, "h", 0.01, 0), (9_000, "hm", 0.0, 0), (500, "f", 0.0, 0)]
    host, dev, descs = make_case(O, torch, pkg, specs, seed=31, g_std=1.0)
    g = host[1]["g"].copy()
    g[4321] = bad
    dev[1]["g"].set(g)
    before = [{k: b.get() for k, b in d.items()} for d in dev]
    tl = pkg.TensorList(descs)
    stat = torch.zeros(16, device="cuda")
    tl.gradstat(stat.data_ptr(), 1.0 / 65536, 1.0)
    tl.step(pkg.hparams(1e-3, 0.9, 0.999, 1e-8, 1), stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16)
    torch.cuda.synchronize()
    assert read_stat(pkg, stat).found_inf == 1
    for d, b in zip(dev, before):
        for k in d:
            assert np.array_equal(d[k].get().view(np.uint8), b[k].view(np.uint8)), f"{k} changed on a skipped step"
    # FP32 gradient overflow is caught too
    g32 = host[2]["g"].copy()
    g32[7] = np.inf
    dev[2]["g"].set(g32)
    dev[1]["g"].set(host[1]["g"])
    tl.gradstat(stat.data_ptr(), 1.0, 1.0)
    torch.cuda.synchronize()
    assert read_stat(pkg, stat).found_inf == 1


def test_unscale_of_scaled_gradients_matches_unscaled_run(pkg, O, torch):
    """Gradients multiplied by a loss scale of 65536 and unscaled in the kernels give the same
    bits as the unscaled gradients (powers of two scale FP16 exactly)."""
    specs = [(50_003, "h", 0.01, 0), (8192, "hm", 0.0, 0)]
    host_a, dev_a, descs_a = make_case(O, torch, pkg, specs, seed=41, g_std=1e-4)
    host_b, dev_b, descs_b = make_case(O, torch, pkg, specs, seed=41, g_std=1e-4)
    for e, d in zip(host_b, dev_b):
        # scale in FP32 and round once to FP16: what a scaled backward pass would have produced
        scaled = O.f2h(O.h2f(e["g"]) * np.float32(65536))
        # keep only elements that scale exactly (FP16 subnormals become normal: still exact)
        assert np.array_equal(O.h2f(scaled), O.h2f(e["g"]) * np.float32(65536))
        d["g"].set(scaled)
    stat_a, stat_b = torch.zeros(16, device="cuda"), torch.zeros(16, device="cuda")
    hp = pkg.hparams(1e-4, 0.9, 0.999, 1e-8, 2)
    ta, tb = pkg.TensorList(descs_a), pkg.TensorList(descs_b)
    ta.gradstat(stat_a.data_ptr(), 1.0, 0.01)
    ta.step(hp, stat_a.data_ptr(), 0)
    tb.gradstat(stat_b.data_ptr(), 1.0 / 65536, 0.01)
    tb.step(hp, stat_b.data_ptr(), 0)
    torch.cuda.synchronize()
    sa, sb = read_stat(pkg, stat_a), read_stat(pkg, stat_b)
    assert sa.norm == sb.norm and sa.clip_active == sb.clip_active == 1
    for da, db in zip(dev_a, dev_b):
        for k in ("p", "m", "v"):
            a, b = da[k].get(), db[k].get()
            if a.dtype == np.uint16:
                assert ulp16(a, b).max() <= 1
            else:
                assert max_rel(a, b) <= 1e-6


def test_flags_norm_only_grad_zero_and_zero_grads(pkg, O, torch):
    specs = [(30_000, "h", 0.01, 0), (10_000, "hm", 0.0, pkg.TENSOR_GRAD_ZERO),
             (5_000, "f", 0.0, pkg.TENSOR_NORM_ONLY), (3_001, "f", 0.0, 0)]
    host, dev, descs = make_case(O, torch, pkg, specs, seed=51)
    tl = pkg.TensorList(descs)
    assert tl.numel == 30_000 + 10_000 + 3_001 and tl.stat_numel == 30_000 + 5_000 + 3_001
    stat = torch.zeros(16, device="cuda")
    hp = pkg.hparams(1e-4, 0.9, 0.999, 1e-8, 4)
    norm_only_before = {k: b.get() for k, b in dev[2].items()}
    frozen_grad_before = dev[1]["g"].get()
    tl.gradstat(stat.data_ptr(), 1.0, 1.0)
    tl.step(hp, stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16 | pkg.STEP_ZERO_GRADS)
    torch.cuda.synchronize()
    got = read_stat(pkg, stat)
    ot = O.make_tensors(host)
    want = O.gradstat(ot, 1.0, 1.0)
    assert abs(got.norm - want.norm) <= NORM_BAR * want.norm
    O.multi_step(ot, O.HParams(1e-4, 0.9, 0.999, 1e-8, hp.bias_correction1, hp.bias_correction2),
                 O.gradstat_finalize(got.sum_sq, 0, 1.0, 1.0), O.STEP_ROUND_CLIP_FP16)
    assert_same([host[0], host[1], host[3]], [dev[0], dev[1], dev[3]])
    for k, b in dev[2].items():                       # NORM_ONLY: read, never written
        assert np.array_equal(b.get().view(np.uint8), norm_only_before[k].view(np.uint8))
    assert not dev[0]["g"].get().any() and not dev[3]["g"].get().any()   # ZERO_GRADS
    assert np.array_equal(dev[1]["g"].get(), frozen_grad_before)          # GRAD_ZERO: never touched


def test_partial_then_finalize_equals_direct(pkg, O, torch):
    specs = [(100_000, "h", 0.0, 0), (777, "f", 0.0, 0)]
    _, dev, descs = make_case(O, torch, pkg, specs, seed=61)
    tl = pkg.TensorList(descs)
    a, b = torch.zeros(16, device="cuda"), torch.zeros(16, device="cuda")
    tl.gradstat(a.data_ptr(), 0.5, 0.3)
    tl.gradstat(b.data_ptr(), 0.5, 0.3, flags=pkg.STAT_PARTIAL)
    pkg.gradstat_finalize(b.data_ptr(), 0.5, 0.3)
    torch.cuda.synchronize()
    sa, sb = read_stat(pkg, a), read_stat(pkg, b)
    assert (sa.sum_sq, sa.norm, sa.coef, sa.found_inf, sa.clip_active) == \
           (sb.sum_sq, sb.norm, sb.coef, sb.found_inf, sb.clip_active)


def test_device_scaler_state_machine(pkg, O, torch):
    """Loss scale and step counter kept on the device: halve on overflow, double after the
    growth interval, skipped steps do not advance t; bias corrections equal the host's powf."""
    n = 4096
    specs = [(n, "h", 0.01, 0)]
    host, dev, descs = make_case(O, torch, pkg, specs, seed=71, g_std=1.0)
    tl = pkg.TensorList(descs)
    stat = torch.zeros(16, device="cuda")
    b1, b2, interval = 0.9, 0.999, 3
    sc_host = np.zeros(1, dtype=[("scale", "f4"), ("gt", "i4"), ("step", "i4"), ("skipped", "i4"),
                                 ("interval", "i4"), ("b1", "f4"), ("b2", "f4"), ("mul", "f4")])
    sc_host["scale"], sc_host["interval"], sc_host["b1"], sc_host["b2"] = 1024.0, interval, b1, b2
    scaler = torch.from_numpy(sc_host.view(np.uint8).copy()).cuda()
    osc = O.Scaler(1024.0, 0, 0, 0)
    clean = dev[0]["g"].get()
    dirty = clean.copy()
    dirty[5] = 0x7C00
    hp = pkg.HParams(1e-3, b1, b2, 1e-8, 1.0, 1.0)     # bias corrections come from the device
    for i in range(14):
        overflow = i in (2, 3, 9)
        dev[0]["g"].set(dirty if overflow else clean)
        scale_before = osc.scale
        tl.gradstat(stat.data_ptr(), 123.0, 0.0, scaler_ptr=scaler.data_ptr())
        tl.step(hp, stat.data_ptr(), pkg.STEP_DEVICE_BIAS_CORRECTION)
        torch.cuda.synchronize()
        s = read_stat(pkg, stat)
        O.scaler_update(osc, 1 if overflow else 0, interval)
        assert s.found_inf == (1 if overflow else 0)
        assert s.loss_scale == scale_before
        if not overflow:
            assert s.coef == 1.0 / scale_before
            assert s.step == osc.step
            assert s.bias_correction1 == pkg.bias_correction(b1, osc.step)
            assert s.bias_correction2 == pkg.bias_correction(b2, osc.step)
            e = host[0]
            g_host = O.make_tensors([e])
            O.multi_step(g_host, O.HParams(1e-3, b1, b2, 1e-8, s.bias_correction1, s.bias_correction2),
                         O.gradstat_finalize(s.sum_sq, 0, 1.0 / scale_before, 0.0), 0)
        got = np.frombuffer(scaler.cpu().numpy().tobytes(), dtype=sc_host.dtype)[0]
        assert (got["scale"], got["gt"], got["step"], got["skipped"]) == \
               (osc.scale, osc.growth_tracker, osc.step, osc.skipped)
    assert_same(host, dev)


def test_device_bias_correction_matches_host_for_many_steps(pkg, torch):
    """1 - beta^t computed on the device (FP64 pow rounded once to FP32) for every t up to
    100,000 and five betas.  It equals the correctly rounded FP32 power everywhere, and the
    host's powf (optimizer.h:121-122) everywhere except the few steps at which the C library's
    powf is itself one ulp off the correctly rounded value (glibc 2.39: beta 0.999, t = 2958 and
    3606); there the two differ by one ulp of the bias correction, 6e-8 relative, far inside
    the parity bars.  Also: the scale doubles after 1000 clean steps."""
    import ctypes as C
    g = torch.full((64,), 0.5, device="cuda").half()
    tl = pkg.TensorList([pkg.TensorDesc(None, g.data_ptr(), None, None, None, 64, 0.0, pkg.F16, pkg.TENSOR_NORM_ONLY, 0)])
    dt = np.dtype([("scale", "f4"), ("gt", "i4"), ("step", "i4"), ("skipped", "i4"),
                   ("interval", "i4"), ("b1", "f4"), ("b2", "f4"), ("mul", "f4")])
    rec = np.dtype([("sum_sq", "f8"), ("norm", "f4"), ("coef", "f4"), ("found_inf", "u4"), ("clip", "u4"),
                    ("bc1", "f4"), ("bc2", "f4"), ("step", "i4"), ("loss_scale", "f4"), ("pad", "u4", 6)])
    T = 100_000
    gradstat, handle = pkg.lib().rlcu_gradstat, tl.handle
    off_by_one = 0
    for b1, b2 in ((0.8, 0.999), (0.9, 0.99), (0.95, 0.9)):
        sc = np.zeros(1, dt)
        sc["scale"], sc["interval"], sc["b1"], sc["b2"] = 65536.0, 1 << 30, b1, b2
        scaler = torch.from_numpy(sc.view(np.uint8).copy()).cuda()
        stats = torch.zeros(T, 16, device="cuda")
        base, sp = stats.data_ptr(), scaler.data_ptr()
        for t in range(T):
            assert gradstat(handle, 1.0, 0.0, sp, base + 64 * t, 0, None) == 0
        torch.cuda.synchronize()
        got = np.frombuffer(stats.cpu().numpy().tobytes(), dtype=rec)
        steps = np.arange(1, T + 1)
        assert np.array_equal(got["step"], steps)
        for beta, field in ((b1, "bc1"), (b2, "bc2")):
            b32 = np.float32(beta)
            rounded_once = np.float32(1.0) - np.power(np.float64(b32), steps.astype(np.float64)).astype(np.float32)
            assert np.array_equal(got[field], rounded_once.astype(np.float32)), (beta, "device vs correctly rounded power")
            host = np.array([pkg.bias_correction(float(b32), int(t)) for t in steps[:20_000]], np.float32)
            diff = np.nonzero(got[field][:20_000] != host)[0]
            for i in diff:
                assert abs(float(got[field][i]) - float(host[i])) <= float(np.spacing(host[i])), (beta, int(i) + 1)
            off_by_one += len(diff)
            # past t = 20,000 every beta here has beta^t < 2^-25 and both give exactly 1.0
            assert (got[field][20_000:] == 1.0).all() and pkg.bias_correction(float(b32), 20_001) == 1.0
    assert off_by_one <= 4
    # growth: the scale doubles after `interval` clean steps
    sc = np.zeros(1, dt)
    sc["scale"], sc["interval"], sc["b1"], sc["b2"] = 65536.0, 1000, 0.9, 0.999
    scaler = torch.from_numpy(sc.view(np.uint8).copy()).cuda()
    stats = torch.zeros(1200, 16, device="cuda")
    for t in range(1200):
        tl.gradstat(stats[t].data_ptr(), 1.0, 0.0, scaler_ptr=scaler.data_ptr())
    torch.cuda.synchronize()
    got = np.frombuffer(stats.cpu().numpy().tobytes(), dtype=rec)
    assert (got["loss_scale"][:1000] == 65536.0).all() and (got["loss_scale"][1000:] == 131072.0).all()


def test_list_argument_checks(pkg, torch):
    a = torch.zeros(64, device="cuda")
    with pytest.raises(pkg.RlcuError):
        pkg.TensorList([pkg.TensorDesc(a.data_ptr(), None, a.data_ptr(), a.data_ptr(), None, 8, 0.0, pkg.F16, 0, 0)])
    with pytest.raises(pkg.RlcuError):
        pkg.TensorList([pkg.TensorDesc(a.data_ptr(), a.data_ptr(), a.data_ptr(), a.data_ptr(), a.data_ptr(), 8, 0.0, pkg.F32, 0, 0)])
    with pytest.raises(pkg.RlcuError):
        pkg.TensorList([pkg.TensorDesc(a.data_ptr(), a.data_ptr(), a.data_ptr(), a.data_ptr(), None, 8, 0.0, 7, 0, 0)])
    empty = pkg.TensorList([])
    stat = torch.zeros(16, device="cuda")
    empty.gradstat(stat.data_ptr(), 1.0, 1.0)
    empty.step(pkg.hparams(1e-3, 0.9, 0.999, 1e-8, 1), stat.data_ptr())
    torch.cuda.synchronize()
    s = read_stat(pkg, stat)
    assert s.norm == 0.0 and s.found_inf == 0 and s.coef == 1.0


def test_config2_full_size_vs_reference_kernels(pkg, O, torch):
    """Qwen3-0.6B-shaped parameter set (596,049,920 parameters, 310 tensors) in RL.cu's
    layout: FP16 projections + embedding with FP32 masters, FP32 norm weights.  One
    statistics pass + one update launch against the reference's scale kernels and its three
    launch_adamw_* calls, compared on the device bit for bit."""
    if not O.ref_available():
        pytest.skip("reference kernels were not built")
    R = O.ref_lib()
    shapes = qwen3_0p6b()
    proj = [(nm, n, wd) for nm, n, wd in shapes if wd]
    norms = [(nm, n, wd) for nm, n, wd in shapes if "norm" in nm]
    embed = [(nm, n, wd) for nm, n, wd in shapes if nm == "embed"]
    n_proj, n_embed, n32 = sum(x[1] for x in proj), embed[0][1], sum(x[1] for x in norms)
    n16 = n_proj + n_embed
    assert n16 + n32 == 596_049_920
    gen = torch.Generator(device="cuda").manual_seed(0)
    lr, b1, b2, eps, wd, t, max_norm = 1e-6, 0.9, 0.999, 1e-8, 0.01, 6, 1.0
    bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)

    master = torch.randn(n16, device="cuda", generator=gen) * 0.02
    g16 = (torch.randn(n16, device="cuda", generator=gen) * 1e-4).half()
    m16 = torch.randn(n16, device="cuda", generator=gen) * 3e-5
    v16 = torch.rand(n16, device="cuda", generator=gen) * 1e-8
    w32 = torch.ones(n32, device="cuda")
    g32 = torch.randn(n32, device="cuda", generator=gen) * 1e-4
    m32 = torch.randn(n32, device="cuda", generator=gen) * 3e-5
    v32 = torch.rand(n32, device="cuda", generator=gen) * 1e-8
    p16 = master.half()
    mine = dict(master=master.clone(), p=p16.clone(), m=m16.clone(), v=v16.clone(),
                w32=w32.clone(), m32=m32.clone(), v32=v32.clone())
    ref = dict(master=master, p=p16, m=m16, v=v16, w32=w32, m32=m32, v32=v32)

    # ours: one descriptor per tensor, in pool order
    descs, off16, off32 = [], 0, 0
    for nm, n, decays in proj + embed:
        descs.append(pkg.TensorDesc(mine["p"].data_ptr() + 2 * off16, g16.data_ptr() + 2 * off16,
                                    mine["m"].data_ptr() + 4 * off16, mine["v"].data_ptr() + 4 * off16,
                                    mine["master"].data_ptr() + 4 * off16, n, wd if decays else 0.0, pkg.F16, 0, 0))
        off16 += n
    for nm, n, _ in norms:
        descs.append(pkg.TensorDesc(mine["w32"].data_ptr() + 4 * off32, g32.data_ptr() + 4 * off32,
                                    mine["m32"].data_ptr() + 4 * off32, mine["v32"].data_ptr() + 4 * off32,
                                    None, n, 0.0, pkg.F32, 0, 0))
        off32 += n
    assert len(descs) == 310
    tl = pkg.TensorList(descs)
    stat = torch.zeros(16, device="cuda")
    tl.gradstat(stat.data_ptr(), 1.0, max_norm)
    tl.step(pkg.HParams(lr, b1, b2, eps, bc1, bc2), stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16)
    torch.cuda.synchronize()
    s = read_stat(pkg, stat)
    exact = float(torch.sqrt((g16.double() ** 2).sum() + (g32.double() ** 2).sum()))
    assert abs(s.norm - exact) <= NORM_BAR * exact
    assert s.clip_active == 1 and 2.3 < s.norm < 2.6          # ~1e-4 * sqrt(P)

    # reference: its sum-of-squares kernels for the norm, then its scale kernels with the clip
    # factor of this run (its own atomic sum differs from run to run in the last bits), then
    # optimizer.h:126-146
    acc, out = torch.zeros(1, device="cuda"), C.c_float()
    assert R.ref_grad_sum_sq(g16.data_ptr(), n16, g32.data_ptr(), n32, acc.data_ptr(), C.byref(out)) == 0
    ref_norm = float(np.sqrt(np.float32(out.value)))
    # At this size the reference's own sum (16,384 FP32 atomic adds into one word) is off the
    # exact FP64 value by more than the 1e-5 bar and changes from run to run, so the bar is
    # applied against the exact value (above); the reference must agree to the accuracy it has.
    ref_err = abs(ref_norm - exact) / exact
    assert abs(s.norm - ref_norm) <= max(NORM_BAR, 2 * ref_err) * ref_norm
    assert abs(s.norm - exact) <= ref_err * exact + 1e-7 * exact   # never worse than the reference
    rg16, rg32 = g16.clone(), g32.clone()
    assert R.ref_scale_grads(rg16.data_ptr(), n16, rg32.data_ptr(), n32, s.coef) == 0
    assert R.ref_launch_adamw_fp16(ref["master"].data_ptr(), ref["p"].data_ptr(), rg16.data_ptr(),
                                   ref["m"].data_ptr(), ref["v"].data_ptr(), n_proj, lr, b1, b2, eps, wd, bc1, bc2, None) == 0
    assert R.ref_launch_adamw_fp16(ref["master"].data_ptr() + 4 * n_proj, ref["p"].data_ptr() + 2 * n_proj,
                                   rg16.data_ptr() + 2 * n_proj, ref["m"].data_ptr() + 4 * n_proj,
                                   ref["v"].data_ptr() + 4 * n_proj, n_embed, lr, b1, b2, eps, 0.0, bc1, bc2, None) == 0
    assert R.ref_launch_adamw_fp32(ref["w32"].data_ptr(), rg32.data_ptr(), ref["m32"].data_ptr(), ref["v32"].data_ptr(),
                                   n32, lr, b1, b2, eps, 0.0, bc1, bc2, None) == 0
    torch.cuda.synchronize()
    for name in mine:
        a, b = mine[name], ref[name]
        view = torch.int16 if a.dtype == torch.float16 else torch.int32
        assert torch.equal(a.view(view), b.view(view)), f"{name}: differs from the reference kernels"


@pytest.mark.parametrize("extra", [0, "zero_grads"])
def test_bulk_copy_update_equals_the_direct_update(pkg, O, torch, extra):
    """The cp.async.bulk (TMA) variant of the update kernel against the per-thread load/store
    one, bit for bit, on a list that mixes full work items with ragged, unaligned, FP32 and
    statistics-only entries."""
    specs = [(8192 * 5, "h", 0.01, 0), (100, "h", 0.0, 0), (8192 * 3 + 17, "hm", 0.01, 0), (8192, "hm", 0.0, 0),
             (8192 * 9, "h", 0.01, 0), (5, "f", 0.0, 0), (8192 * 2, "f", 0.01, 0), (8192 * 4, "hm", 0.0, pkg.TENSOR_GRAD_ZERO),
             (3000, "f", 0.0, pkg.TENSOR_NORM_ONLY)]
    flags = pkg.STEP_ROUND_CLIP_FP16 | (pkg.STEP_ZERO_GRADS if extra else 0)
    results = []
    stat = None
    for bulk in (0, pkg.STEP_BULK_COPY):
        host, dev, descs = make_case(O, torch, pkg, specs, seed=81)
        tl = pkg.TensorList(descs)
        if stat is None:                 # one record for both runs (the sum's order depends on addresses)
            stat = torch.zeros(16, device="cuda")
            tl.gradstat(stat.data_ptr(), 1.0, 1.0)
        for t in (2, 3, 4):
            tl.step(pkg.hparams(1e-4, 0.9, 0.999, 1e-8, t), stat.data_ptr(), flags | bulk)
        tl.check()
        results.append([{k: b.get() for k, b in d.items()} for d in dev])
        assert all(b.guards_intact() for d in dev for b in d.values())
    for a, b in zip(*results):
        for k in a:
            assert np.array_equal(a[k].view(np.uint8), b[k].view(np.uint8)), k


def test_master_lists_default_to_the_bulk_copy_kernel_with_the_same_bits(pkg, O, torch):
    """A list that is mostly FP16 weights with FP32 masters and has at least four work items per
    SM runs through the bulk-copy kernel unless RLCU_STEP_DIRECT is given; both give the bits
    of the oracle."""
    specs = [(8192 * 400 + 11, "hm", 0.01, 0), (8192 * 300, "hm", 0.0, 0), (5000, "f", 0.0, 0), (8192 * 20 + 3, "h", 0.01, 0)]
    results = []
    stat = None
    for forced in (0, pkg.STEP_DIRECT):
        host, dev, descs = make_case(O, torch, pkg, specs, seed=171)
        tl = pkg.TensorList(descs)
        hp = pkg.hparams(1e-4, 0.9, 0.999, 1e-8, 3)
        if stat is None:                 # one record for both runs (the sum's order depends on addresses)
            stat = torch.zeros(16, device="cuda")
            tl.gradstat(stat.data_ptr(), 1.0, 1.0)
        tl.step(hp, stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16 | forced)
        tl.check()
        got = read_stat(pkg, stat)
        ot = O.make_tensors(host)
        O.multi_step(ot, O.HParams(1e-4, 0.9, 0.999, 1e-8, hp.bias_correction1, hp.bias_correction2),
                     O.gradstat_finalize(got.sum_sq, 0, 1.0, 1.0), O.STEP_ROUND_CLIP_FP16)
        assert_same(host, dev)
        results.append([{k: b.get() for k, b in d.items()} for d in dev])
    for a, b in zip(*results):
        for k in a:
            assert np.array_equal(a[k].view(np.uint8), b[k].view(np.uint8)), k
    with pytest.raises(pkg.RlcuError):
        tl.step(hp, stat.data_ptr(), pkg.STEP_DIRECT | pkg.STEP_BULK_COPY)


@pytest.mark.parametrize("side_stream", [False, True])
def test_bounded_wait_gives_up_and_reports(pkg, torch, side_stream):
    """A device-side wait that nothing satisfies runs out of tries, the kernel returns, the host
    reads RLCU_ERR_TIMEOUT, and the GPU keeps working.  With a stream that does not synchronise
    with the legacy stream (torch's pool streams are non-blocking) the check still sees it."""
    a = torch.zeros(64, device="cuda")
    tl = pkg.TensorList([pkg.TensorDesc(a.data_ptr(), a.data_ptr(), a.data_ptr(), a.data_ptr(), None, 8, 0.0, pkg.F32, 0, 0)])
    stream = torch.cuda.Stream() if side_stream else None
    rc = pkg.lib().rlcu_selftest_bounded_wait(tl.handle, stream.cuda_stream if stream else None)
    assert rc == pkg.ERR_TIMEOUT and b"gave up" in pkg.lib().rlcu_last_error()
    tl.check()                                           # the condition was cleared
    tl.step(pkg.hparams(1e-3, 0.9, 0.999, 1e-8, 1))      # and the device still runs kernels
    torch.cuda.synchronize()


def test_step_replays_from_a_cuda_graph(pkg, O, torch):
    """The whole step (statistics + update, step counter and bias corrections kept on the
    device) has no host round trip, so it can be captured once and replayed: five replays give
    the bits of five eager steps."""
    specs = [(8192 * 6 + 40, "h", 0.01, 0), (5000, "hm", 0.0, 0), (700, "f", 0.0, 0)]
    dt = np.dtype([("scale", "f4"), ("gt", "i4"), ("step", "i4"), ("skipped", "i4"),
                   ("interval", "i4"), ("b1", "f4"), ("b2", "f4"), ("mul", "f4")])

    def scaler():
        sc = np.zeros(1, dt)
        sc["scale"], sc["interval"], sc["b1"], sc["b2"] = 1.0, 1 << 30, 0.9, 0.999
        return torch.from_numpy(sc.view(np.uint8).copy()).cuda()

    hp = pkg.HParams(1e-4, 0.9, 0.999, 1e-8, 1.0, 1.0)
    flags = pkg.STEP_DEVICE_BIAS_CORRECTION | pkg.STEP_ROUND_CLIP_FP16
    _, dev_a, descs_a = make_case(O, torch, pkg, specs, seed=91)
    _, dev_b, descs_b = make_case(O, torch, pkg, specs, seed=91)
    ta, tb = pkg.TensorList(descs_a), pkg.TensorList(descs_b)
    sa, sb, stat_a, stat_b = scaler(), scaler(), torch.zeros(16, device="cuda"), torch.zeros(16, device="cuda")
    for _ in range(5):                                   # eager
        ta.gradstat(stat_a.data_ptr(), 1.0, 0.5, scaler_ptr=sa.data_ptr())
        ta.step(hp, stat_a.data_ptr(), flags)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        tb.gradstat(stat_b.data_ptr(), 1.0, 0.5, scaler_ptr=sb.data_ptr(), stream=side.cuda_stream)   # set-up outside capture
        tb.step(hp, stat_b.data_ptr(), flags, stream=side.cuda_stream)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            s = torch.cuda.current_stream().cuda_stream
            tb.gradstat(stat_b.data_ptr(), 1.0, 0.5, scaler_ptr=sb.data_ptr(), stream=s)
            tb.step(hp, stat_b.data_ptr(), flags, stream=s)
    for _ in range(4):
        graph.replay()
    torch.cuda.synchronize()
    assert read_stat(pkg, stat_a).step == read_stat(pkg, stat_b).step == 5
    for da, db in zip(dev_a, dev_b):
        for k in da:
            assert np.array_equal(da[k].get().view(np.uint8), db[k].get().view(np.uint8)), k


@pytest.mark.parametrize("bulk", [False, True])
def test_skipped_step_still_clears_gradients_when_asked(pkg, O, torch, bulk):
    specs = [(8192 * 2 + 5, "h", 0.01, 0), (900, "f", 0.0, 0), (8192, "hm", 0.0, pkg.TENSOR_GRAD_ZERO)]
    host, dev, descs = make_case(O, torch, pkg, specs, seed=101)
    g = host[0]["g"].copy()
    g[77] = 0x7C00
    dev[0]["g"].set(g)
    frozen_grad = dev[2]["g"].get()
    before = [{k: b.get() for k, b in d.items() if k != "g"} for d in dev]
    tl = pkg.TensorList(descs)
    stat = torch.zeros(16, device="cuda")
    tl.gradstat(stat.data_ptr(), 1.0, 1.0)
    tl.step(pkg.hparams(1e-3, 0.9, 0.999, 1e-8, 1), stat.data_ptr(),
            pkg.STEP_ZERO_GRADS | (pkg.STEP_BULK_COPY if bulk else 0))
    tl.check()
    assert read_stat(pkg, stat).found_inf == 1
    for d, b in zip(dev, before):
        for k in b:
            assert np.array_equal(d[k].get().view(np.uint8), b[k].view(np.uint8)), k
    assert not dev[0]["g"].get().any() and not dev[1]["g"].get().any()
    assert np.array_equal(dev[2]["g"].get(), frozen_grad)      # a GRAD_ZERO tensor's buffer is never touched


# ---------------------------------------------------------------------------------------------
# FP32 gradients for 16-bit parameters (RLCU_GRAD_F32)
# ---------------------------------------------------------------------------------------------

GF32_MIXED = [(70_001, "hg", 0.01, 0), (1024, "hmg", 0.0, 0), (8192 * 3, "hmg", 0.01, 0), (129, "f", 0.0, 0),
              (1, "hg", 0.0, 0), (8192, "hg", 0.01, 0), (8192 * 2 + 5, "h", 0.01, 0), (0, "hg", 0.0, 0),
              (40_000, "hm", 0.02, 0), (8192 * 4, "hmg", 0.0, 0)]


@pytest.mark.parametrize("offset", [0, 1])
@pytest.mark.parametrize("max_norm", [1.0, 0.0])
def test_fp32_gradients_for_fp16_parameters(pkg, O, torch, max_norm, offset):
    """A list that mixes FP16 and FP32 gradients for FP16 parameters (with and without a master
    copy): statistics within the norm bar, update bit for bit against the oracle.  The clip is
    applied to FP32 gradients in FP32 (trainer.h:142-145): STEP_ROUND_CLIP_FP16 re-rounds only
    the gradients that are stored in FP16."""
    host, dev, descs = make_case(O, torch, pkg, GF32_MIXED, seed=111, offset=offset)
    stat = torch.zeros(16, device="cuda")
    tl = pkg.TensorList(descs)
    lr, b1, b2, eps, t = 1e-4, 0.9, 0.999, 1e-8, 5
    hp = pkg.hparams(lr, b1, b2, eps, t)
    tl.gradstat(stat.data_ptr(), 1.0, max_norm)
    tl.step(hp, stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16)
    torch.cuda.synchronize()
    got = read_stat(pkg, stat)
    ot = O.make_tensors(host)
    want = O.gradstat(ot, 1.0, max_norm)
    assert got.found_inf == 0 and got.clip_active == want.clip_active == (1 if max_norm else 0)
    assert abs(got.norm - want.norm) <= NORM_BAR * want.norm
    O.multi_step(ot, O.HParams(lr, b1, b2, eps, hp.bias_correction1, hp.bias_correction2),
                 O.gradstat_finalize(got.sum_sq, 0, 1.0, max_norm), O.STEP_ROUND_CLIP_FP16)
    assert_same(host, dev)
    for e, d in zip(host, dev):                      # gradients are read, never written
        assert np.array_equal(d["g"].get().view(np.uint8), e["g"].view(np.uint8))


def test_fp32_gradient_keeps_what_fp16_would_round_away(pkg, O, torch):
    """The point of the variant: a gradient below FP16's smallest subnormal still moves the
    moments when it arrives in FP32, and is lost when it is rounded to FP16 first."""
    n = 8192 * 2 + 3
    p, _, _, _ = seeded_case(O, n, seed=121)
    tiny = np.full(n, 1e-9, np.float32)              # FP16 rounds this to zero
    out = {}
    for kind in ("hg", "h"):
        g = tiny if kind == "hg" else O.f2h(tiny)
        bufs = dict(p=DevBuf(p, torch), g=DevBuf(g, torch), m=DevBuf(np.zeros(n, np.float32), torch),
                    v=DevBuf(np.zeros(n, np.float32), torch))
        tl = pkg.TensorList([pkg.TensorDesc(bufs["p"].ptr, bufs["g"].ptr, bufs["m"].ptr, bufs["v"].ptr, None, n, 0.0,
                                            pkg.F16, 0, pkg.GRAD_F32 if kind == "hg" else 0)])
        tl.step(pkg.hparams(1e-3, 0.9, 0.999, 1e-8, 1))
        torch.cuda.synchronize()
        out[kind] = bufs["m"].get()
    assert not out["h"].any()
    assert np.array_equal(out["hg"], np.full(n, np.float32(1.0 - np.float32(0.9)) * np.float32(1e-9), np.float32))


def test_fp32_gradients_zeroed_after_the_update_and_on_a_skipped_step(pkg, O, torch):
    specs = [(8192 * 2 + 5, "hg", 0.01, 0), (3000, "hmg", 0.0, 0), (8192, "hg", 0.0, pkg.TENSOR_GRAD_ZERO)]
    host, dev, descs = make_case(O, torch, pkg, specs, seed=131)
    tl = pkg.TensorList(descs)
    stat = torch.zeros(16, device="cuda")
    hp = pkg.hparams(1e-4, 0.9, 0.999, 1e-8, 2)
    frozen = dev[2]["g"].get()
    tl.gradstat(stat.data_ptr(), 1.0, 1.0)
    tl.step(hp, stat.data_ptr(), pkg.STEP_ZERO_GRADS)
    torch.cuda.synchronize()
    got = read_stat(pkg, stat)
    ot = O.make_tensors(host)
    O.multi_step(ot, O.HParams(1e-4, 0.9, 0.999, 1e-8, hp.bias_correction1, hp.bias_correction2),
                 O.gradstat_finalize(got.sum_sq, 0, 1.0, 1.0), 0)
    assert_same(host, dev)
    assert not dev[0]["g"].get().any() and not dev[1]["g"].get().any()
    assert np.array_equal(dev[2]["g"].get(), frozen)
    # overflowed step: nothing but the gradients changes
    bad = host[0]["g"].copy()
    bad[11] = np.nan
    dev[0]["g"].set(bad)
    dev[1]["g"].set(host[1]["g"])
    before = [{k: b.get() for k, b in d.items() if k != "g"} for d in dev]
    tl.gradstat(stat.data_ptr(), 1.0, 1.0)
    tl.step(hp, stat.data_ptr(), pkg.STEP_ZERO_GRADS)
    torch.cuda.synchronize()
    assert read_stat(pkg, stat).found_inf == 1
    for d, b in zip(dev, before):
        for k in b:
            assert np.array_equal(d[k].get().view(np.uint8), b[k].view(np.uint8)), k
    assert not dev[0]["g"].get().any() and not dev[1]["g"].get().any()


@pytest.mark.parametrize("zero_grads", [False, True])
def test_bulk_copy_update_takes_fp32_gradients(pkg, O, torch, zero_grads):
    """FP32 gradients for FP16 parameters through the bulk-copy kernel: the bits of the direct kernel."""
    specs = [(8192 * 5 + 9, "hg", 0.01, 0), (8192 * 3, "hmg", 0.0, 0), (8192 * 2, "hm", 0.01, 0), (777, "hg", 0.0, 0),
             (8192 * 4, "hmg", 0.0, pkg.TENSOR_GRAD_ZERO)]
    flags = pkg.STEP_ROUND_CLIP_FP16 | (pkg.STEP_ZERO_GRADS if zero_grads else 0)
    results = []
    stat = None
    for how in (pkg.STEP_DIRECT, pkg.STEP_BULK_COPY):
        host, dev, descs = make_case(O, torch, pkg, specs, seed=141)
        tl = pkg.TensorList(descs)
        if stat is None:
            # one record for both runs: work items are cut by address, so the squares of two
            # copies of the same data at other addresses are added in another order
            stat = torch.zeros(16, device="cuda")
            tl.gradstat(stat.data_ptr(), 1.0, 1.0)
        for t in (2, 3):
            tl.step(pkg.hparams(1e-4, 0.9, 0.999, 1e-8, t), stat.data_ptr(), flags | how)
        tl.check()
        results.append([{k: b.get() for k, b in d.items()} for d in dev])
        assert all(b.guards_intact() for d in dev for b in d.values())
    for a, b in zip(*results):
        for k in a:
            assert np.array_equal(a[k].view(np.uint8), b[k].view(np.uint8)), k
    if zero_grads:
        assert not results[1][0]["g"].any() and not results[1][1]["g"].any() and results[1][4]["g"].any()


# ---------------------------------------------------------------------------------------------
# what counts as an overflowed step
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("kind", ["f", "hg"])
def test_finite_fp32_gradient_with_an_overflowing_square_is_not_an_overflow(pkg, O, torch, kind):
    """The non-finite test looks at the stored gradient, like the oracle, not at its square: an
    FP32 gradient of 1e20 is finite (its square is not), so the step is not skipped; the norm is
    +inf and the clip scales every gradient to zero, which is what RL.cu's own sequence does
    with such a value.  A true +inf skips the step."""
    specs = [(8192 + 7, kind, 0.01, 0), (5000, "h", 0.0, 0)]
    host, dev, descs = make_case(O, torch, pkg, specs, seed=151)
    g = host[0]["g"].copy()
    g[3] = np.float32(1e20)
    host[0]["g"] = g
    dev[0]["g"].set(g)
    tl = pkg.TensorList(descs)
    stat = torch.zeros(16, device="cuda")
    hp = pkg.hparams(1e-4, 0.9, 0.999, 1e-8, 3)
    tl.gradstat(stat.data_ptr(), 1.0, 1.0)
    tl.step(hp, stat.data_ptr(), 0)
    torch.cuda.synchronize()
    got = read_stat(pkg, stat)
    ot = O.make_tensors(host)
    want = O.gradstat(ot, 1.0, 1.0)
    assert want.found_inf == 0 and np.isinf(want.norm) and want.coef == 0.0 and want.clip_active == 1
    assert got.found_inf == 0 and np.isinf(got.norm) and got.coef == 0.0 and got.clip_active == 1
    O.multi_step(ot, O.HParams(1e-4, 0.9, 0.999, 1e-8, hp.bias_correction1, hp.bias_correction2), want, 0)
    assert_same(host, dev)
    # without a clip the value is used as it is (RL.cu does the same when max_grad_norm <= 0)
    tl.gradstat(stat.data_ptr(), 1.0, 0.0)
    torch.cuda.synchronize()
    got = read_stat(pkg, stat)
    assert got.found_inf == 0 and got.coef == 1.0 and got.clip_active == 0
    # a real infinity is an overflow
    g[3] = np.inf
    dev[0]["g"].set(g)
    tl.gradstat(stat.data_ptr(), 1.0, 1.0)
    torch.cuda.synchronize()
    assert read_stat(pkg, stat).found_inf == 1
    g[3] = np.float32(-1e20)
    g[100] = np.nan
    dev[0]["g"].set(g)
    tl.gradstat(stat.data_ptr(), 1.0, 1.0)
    torch.cuda.synchronize()
    assert read_stat(pkg, stat).found_inf == 1
