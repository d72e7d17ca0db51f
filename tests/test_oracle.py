"""Self-checks of the CPU oracle that need no fixture: conversions, the closed form of the
first step that the reference's own test uses, the clip rule, the fused multi-tensor step
against its per-tensor parts, and the loss-scale state machine."""
import numpy as np
import pytest


def test_half_to_float_exhaustive(O):
    h = np.arange(65536, dtype=np.uint16)
    mine, ref = O.h2f(h), h.view(np.float16).astype(np.float32)
    nan = np.isnan(ref)
    assert np.array_equal(mine[~nan].view(np.uint32), ref[~nan].view(np.uint32))
    assert np.isnan(mine[nan]).all()


def test_float_to_half_rounding(O):
    rng = np.random.default_rng(1)
    parts = [rng.standard_normal(200_000).astype(np.float32) * np.float32(s)
             for s in (1e-8, 1e-6, 6e-5, 1e-3, 1.0, 300.0, 7e4)]
    h = np.arange(65536, dtype=np.uint16)
    finite = np.sort(h[(h & 0x7C00) != 0x7C00].view(np.float16).astype(np.float64))
    ties = ((finite[:-1] + finite[1:]) / 2).astype(np.float32)       # exact midpoints
    edge = np.array([65504, 65519.996, 65520, 65536, -65520, np.inf, -np.inf,
                     2.0 ** -25, np.nextafter(np.float32(2.0 ** -25), np.float32(1)), 2.0 ** -24, 0.0, -0.0],
                    np.float32)
    x = np.concatenate(parts + [ties, edge])
    with np.errstate(over="ignore"):
        ref = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(O.f2h(x), ref)
    assert O.f2h(np.array([np.nan], np.float32))[0] & 0x7C00 == 0x7C00


def test_hardware_half_conversions_equal_the_bit_level_definition(O):
    """The timed loops of the oracle convert with the CPU's F16C instructions when they are
    there; the bit-level functions stay the definition.  Every binary16 value one way, the
    rounding cases of the test above plus NaN the other way, and one whole update both ways."""
    if not O.hw_half_available():
        pytest.skip("no F16C on this CPU: the loops already use the bit-level functions")
    L = O.lib()
    for h in range(65536):
        a, b = L.orc_h2f(h), L.orc_h2f_hw(h)
        assert (np.isnan(a) and np.isnan(b)) or np.float32(a).view(np.uint32) == np.float32(b).view(np.uint32), h
    rng = np.random.default_rng(2)
    h = np.arange(65536, dtype=np.uint16)
    finite = np.sort(h[(h & 0x7C00) != 0x7C00].view(np.float16).astype(np.float64))
    ties = ((finite[:-1] + finite[1:]) / 2).astype(np.float32)
    xs = np.concatenate([rng.standard_normal(20_000).astype(np.float32) * np.float32(s) for s in (1e-8, 6e-5, 1.0, 7e4)]
                        + [ties[::7], np.array([65504, 65519.996, 65520, np.inf, -np.inf, np.nan, 2.0 ** -25, 0.0, -0.0], np.float32)])
    for x in xs:
        assert L.orc_f2h(float(x)) == L.orc_f2h_hw(float(x)), x
    n = 50_001
    p = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(0.02))
    g = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(1e-2))
    out = []
    try:
        for on in (True, False):
            O.use_hw_half(on)
            e = dict(p=p.copy(), g=g, m=np.zeros(n, np.float32), v=np.zeros(n, np.float32), wd=0.01)
            ts = O.make_tensors([e])
            st = O.gradstat(ts, 1.0, 0.5)
            O.multi_step(ts, O.HParams(1e-3, 0.9, 0.999, 1e-8, 0.1, 0.001), st, O.STEP_ROUND_CLIP_FP16)
            out.append((st.sum_sq, e["p"].copy(), e["m"].copy(), e["v"].copy()))
    finally:
        O.use_hw_half(True)
    assert out[0][0] == out[1][0]
    for a, b in zip(out[0][1:], out[1][1:]):
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_bias_correction_matches_float32_powf(O):
    """include/training/optimizer.h:121-122: 1.0f - powf(beta, (float)t), all in FP32."""
    for beta in (0.9, 0.999, 0.95, 0.8):
        for t in (1, 2, 3, 10, 100, 1000, 5000):
            b = np.float32(beta)
            power = np.float32(np.float64(b) ** t)            # correctly rounded powf
            want = np.float32(1.0) - power
            assert O.bias_correction(beta, t) == float(want), (beta, t)


def test_first_step_closed_form_fp32(O):
    """tests/test_adamw.cu:195-206 of RL.cu: m=v=0, no weight decay, FP32 parameter."""
    rng = np.random.default_rng(2)
    n, lr, b1, b2, eps = 1024, np.float32(1e-3), np.float32(0.9), np.float32(0.999), np.float32(1e-8)
    w0 = (1 + rng.standard_normal(n) * 0.05).astype(np.float32)
    g = (rng.standard_normal(n) * 1e-2).astype(np.float32)
    one = np.float32(1)
    mi = (one - b1) * g
    vi = (one - b2) * g * g
    want = w0 - lr * (mi / (one - b1)) / (np.sqrt(vi / (one - b2)) + eps)
    w, m, v = w0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    O.adamw_fp32(w, g, m, v, float(lr), float(b1), float(b2), float(eps), 0.0,
                 O.bias_correction(float(b1), 1), O.bias_correction(float(b2), 1), O.UNFUSED)
    assert np.abs(w - want).max() < 1e-6            # the reference test's bar (:224)
    assert np.array_equal(m, mi) and np.array_equal(v, vi)


def test_first_step_closed_form_fp16(O):
    """tests/test_adamw.cu:277-293 of RL.cu: FP16 parameter with FP32 master, wd=0.01."""
    rng = np.random.default_rng(3)
    n = 4096
    lr, b1, b2, eps, wd = (np.float32(x) for x in (1e-3, 0.9, 0.999, 1e-8, 0.01))
    p0 = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(0.02))
    g16 = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(1e-3))
    w0, g = O.h2f(p0), O.h2f(g16)
    one = np.float32(1)
    mi, vi = (one - b1) * g, (one - b2) * g * g
    want = w0 * (one - lr * wd) - lr * (mi / (one - b1)) / (np.sqrt(vi / (one - b2)) + eps)
    master, p = w0.copy(), p0.copy()
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    O.adamw_fp16_master(master, p, g16, m, v, float(lr), float(b1), float(b2), float(eps), float(wd),
                        O.bias_correction(float(b1), 1), O.bias_correction(float(b2), 1), O.UNFUSED)
    assert np.abs(master - want).max() < 1e-6       # the reference test's bar (:324)
    assert np.array_equal(p, O.f2h(master))
    # master-less variant starts from the same weight: identical on the first step
    p2, m2, v2 = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    O.adamw_fp16(p2, g16, m2, v2, float(lr), float(b1), float(b2), float(eps), float(wd),
                 O.bias_correction(float(b1), 1), O.bias_correction(float(b2), 1), O.UNFUSED)
    assert np.array_equal(p2, p)


def test_empty_is_noop(O):
    e16, e32 = np.zeros(0, np.uint16), np.zeros(0, np.float32)
    O.adamw_fp16_master(e32, e16, e16, e32, e32, 1e-3, 0.9, 0.999, 1e-8, 0.0, 0.1, 0.001)
    O.adamw_fp32(e32, e32, e32, e32, 1e-3, 0.9, 0.999, 1e-8, 0.0, 0.1, 0.001)
    assert O.clip_grad_norm(None, None, 1.0) == 0.0


def test_clip_rule(O):
    """include/training/trainer.h:339-349: scale only above the threshold, +1e-6 in the divisor."""
    g = np.full(10_000, 0.01, np.float32)                # norm = 1.0 exactly-ish
    norm = O.clip_grad_norm(None, g.copy(), 2.0)
    assert abs(norm - 1.0) < 1e-5
    g2 = g.copy()
    O.clip_grad_norm(None, g2, 2.0)
    assert np.array_equal(g2, g)                         # below the threshold: untouched
    g3 = g.copy()
    norm3 = O.clip_grad_norm(None, g3, 0.5)
    scale = np.float32(0.5) / (np.float32(norm3) + np.float32(1e-6))
    assert np.array_equal(g3, g * scale)
    st = O.gradstat_finalize(float(np.float32(norm3)) ** 2, 0, 1.0, 0.5)
    assert st.clip_active == 1 and st.coef == pytest.approx(float(scale), rel=1e-6)


def test_multi_step_equals_reference_sequence(O):
    """statistics + fused update == clip_grad_norm_ followed by per-tensor AdamW, the order
    RL.cu's training_step runs them in (trainer.h:279-286)."""
    rng = np.random.default_rng(4)
    sizes = [5000, 129, 8192, 1]
    lr, b1, b2, eps, t = 1e-4, 0.9, 0.999, 1e-8, 4
    bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)
    A, B = [], []
    for k, n in enumerate(sizes):
        p = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(0.02))
        g = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(0.02))
        m = (rng.standard_normal(n) * 1e-3).astype(np.float32)
        v = (rng.random(n) * 1e-5).astype(np.float32)
        e = dict(p=p, g=g, m=m, v=v, master=O.h2f(p), wd=0.01 * (k % 2))
        A.append({k2: (a.copy() if isinstance(a, np.ndarray) else a) for k2, a in e.items()})
        B.append({k2: (a.copy() if isinstance(a, np.ndarray) else a) for k2, a in e.items()})
    f32 = dict(p=(1 + rng.standard_normal(300) * 0.01).astype(np.float32),
               g=(rng.standard_normal(300) * 0.02).astype(np.float32),
               m=np.zeros(300, np.float32), v=np.zeros(300, np.float32), wd=0.0)
    A.append({k2: (a.copy() if isinstance(a, np.ndarray) else a) for k2, a in f32.items()})
    B.append({k2: (a.copy() if isinstance(a, np.ndarray) else a) for k2, a in f32.items()})

    ta = O.make_tensors(A)
    st = O.gradstat(ta, 1.0, 1.0)
    assert st.clip_active == 1 and st.found_inf == 0
    O.multi_step(ta, O.HParams(lr, b1, b2, eps, bc1, bc2), st, O.STEP_ROUND_CLIP_FP16)

    half_pool = np.concatenate([e["g"] for e in B[:-1]])
    norm = O.clip_grad_norm(half_pool, B[-1]["g"], 1.0)
    assert norm == pytest.approx(st.norm, rel=1e-6)
    off = 0
    for e in B[:-1]:
        n = e["p"].size
        g = half_pool[off:off + n].copy()
        off += n
        O.adamw_fp16_master(e["master"], e["p"], g, e["m"], e["v"], lr, b1, b2, eps, e["wd"], bc1, bc2)
    e = B[-1]
    O.adamw_fp32(e["p"], e["g"], e["m"], e["v"], lr, b1, b2, eps, 0.0, bc1, bc2)
    for a, b in zip(A, B):
        for name in ("p", "m", "v", "master"):
            if name in a and a[name] is not None:
                assert np.array_equal(a[name], b[name]), name


def test_overflow_skips_and_flags(O):
    rng = np.random.default_rng(5)
    n = 1000
    e = dict(p=O.f2h(rng.standard_normal(n).astype(np.float32)), g=O.f2h(rng.standard_normal(n).astype(np.float32)),
             m=np.ones(n, np.float32), v=np.ones(n, np.float32), wd=0.01)
    for bad in (0x7C00, 0xFC00, 0x7E00):
        e["g"][17] = bad
        before = {k: e[k].copy() for k in ("p", "m", "v")}
        ts = O.make_tensors([e])
        st = O.gradstat(ts, 1.0 / 65536, 1.0)
        assert st.found_inf == 1
        assert O.multi_step(ts, O.HParams(1e-3, 0.9, 0.999, 1e-8, 0.1, 0.001), st) == 1
        for k in before:
            assert np.array_equal(before[k], e[k])


def test_scaler_state_machine(O):
    s = O.Scaler(65536.0, 0, 0, 0)
    O.scaler_update(s, 1, 1000)
    assert (s.scale, s.growth_tracker, s.step, s.skipped) == (32768.0, 0, 0, 1)
    for _ in range(999):
        O.scaler_update(s, 0, 1000)
    assert (s.scale, s.growth_tracker, s.step) == (32768.0, 999, 999)
    O.scaler_update(s, 0, 1000)
    assert (s.scale, s.growth_tracker, s.step) == (65536.0, 0, 1000)
    # an overflow every fourth step never lets the tracker reach the interval
    s = O.Scaler(65536.0, 0, 0, 0)
    for i in range(40):
        O.scaler_update(s, 1 if i % 4 == 3 else 0, 1000)
    assert s.scale == 65536.0 / 2 ** 10 and s.step == 30 and s.skipped == 10


def test_fp32_gradient_branch_equals_the_fp16_branch_on_exact_values(O):
    """A 16-bit parameter with an FP32 gradient (ORC_GRAD_F32): with gradients that are exactly
    representable in FP16 and no clip re-rounding, the statistics and the update equal those of
    the FP16-gradient branch bit for bit; with the clip active the FP32 branch skips the FP16
    re-rounding (trainer.h:142-145 against :136-139)."""
    rng = np.random.default_rng(5)
    n = 20_011
    p = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(0.02))
    g16 = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(1e-2))
    g32 = O.h2f(g16)
    hp = O.HParams(1e-3, 0.9, 0.999, 1e-8, O.bias_correction(0.9, 2), O.bias_correction(0.999, 2))

    def run(grad, grad_dtype, max_norm, flags, master):
        e = dict(p=p.copy(), g=grad, m=np.full(n, 1e-4, np.float32), v=np.full(n, 1e-6, np.float32), wd=0.01,
                 dtype=O.F16, grad_dtype=grad_dtype)
        if master:
            e["master"] = O.h2f(p)
        ts = O.make_tensors([e])
        st = O.gradstat(ts, 1.0, max_norm)
        O.multi_step(ts, hp, st, flags)
        return st, e

    for master in (False, True):
        sa, a = run(g16, O.GRAD_AS_PARAM, 0.0, 0, master)
        sb, b = run(g32, O.GRAD_F32, 0.0, 0, master)
        assert (sa.sum_sq, sa.norm, sa.coef) == (sb.sum_sq, sb.norm, sb.coef)
        for k in ("p", "m", "v") + (("master",) if master else ()):
            assert np.array_equal(a[k].view(np.uint8), b[k].view(np.uint8)), k
        # clip active: identical without the re-rounding flag, different with it (FP16 branch only)
        sa, a = run(g16, O.GRAD_AS_PARAM, 0.5, 0, master)
        sb, b = run(g32, O.GRAD_F32, 0.5, O.STEP_ROUND_CLIP_FP16, master)
        assert sa.clip_active == sb.clip_active == 1
        assert np.array_equal(a["m"].view(np.uint8), b["m"].view(np.uint8))
        sc, c = run(g16, O.GRAD_AS_PARAM, 0.5, O.STEP_ROUND_CLIP_FP16, master)
        assert not np.array_equal(c["m"].view(np.uint8), b["m"].view(np.uint8))


def test_overflow_is_judged_on_the_stored_gradient(O):
    """found_inf looks at the gradient element, not at its square: 1e20 in an FP32 gradient is
    finite; its square is not, so the sum and the norm are +inf and a clip scales to zero."""
    g = np.full(100, 1e-3, np.float32)
    g[7] = 1e20
    e = dict(p=np.zeros(100, np.float32), g=g, m=np.zeros(100, np.float32), v=np.zeros(100, np.float32))
    st = O.gradstat(O.make_tensors([e]), 1.0, 1.0)
    assert st.found_inf == 0 and np.isinf(st.sum_sq) and np.isinf(st.norm) and st.clip_active == 1 and st.coef == 0.0
    st = O.gradstat(O.make_tensors([e]), 1.0, 0.0)
    assert st.found_inf == 0 and st.clip_active == 0 and st.coef == 1.0
    g[8] = np.inf
    st = O.gradstat(O.make_tensors([e]), 1.0, 1.0)
    assert st.found_inf == 1
    h = np.full(64, 0x3C00, np.uint16)
    h[3] = 0x7E00                                     # NaN in FP16
    e16 = dict(p=h.copy(), g=h, m=np.zeros(64, np.float32), v=np.zeros(64, np.float32))
    st = O.gradstat(O.make_tensors([e16]), 1.0, 1.0)
    assert st.found_inf == 1 and st.sum_sq == 63.0    # the non-finite element is left out of the sum
