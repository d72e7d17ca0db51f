"""Size-independent properties of the optimizer step, checked on the CPU oracle with
hypothesis: the update is elementwise (splitting or reordering tensors changes nothing), the
norm is a global quantity (splitting changes nothing either), and FP16 rounding is monotone."""
import numpy as np
from hypothesis import given, settings, strategies as st


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 4000), st.integers(0, 2 ** 31 - 1), st.floats(1e-6, 1e-2), st.integers(1, 50))
def test_splitting_a_tensor_changes_nothing(O, n, seed, lr, t):
    rng = np.random.default_rng(seed)
    p = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(0.02))
    g = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(0.05))
    m = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    v = (rng.random(n) * 1e-5).astype(np.float32)
    cut = int(rng.integers(0, n + 1))
    hp = O.HParams(lr, 0.9, 0.999, 1e-8, O.bias_correction(0.9, t), O.bias_correction(0.999, t))

    whole = dict(p=p.copy(), g=g.copy(), m=m.copy(), v=v.copy(), wd=0.01)
    tw = O.make_tensors([whole])
    sw = O.gradstat(tw, 1.0, 1.0)
    O.multi_step(tw, hp, sw, O.STEP_ROUND_CLIP_FP16)

    a = dict(p=p[:cut].copy(), g=g[:cut].copy(), m=m[:cut].copy(), v=v[:cut].copy(), wd=0.01)
    b = dict(p=p[cut:].copy(), g=g[cut:].copy(), m=m[cut:].copy(), v=v[cut:].copy(), wd=0.01)
    ts = O.make_tensors([b, a])                      # reordered as well
    ss = O.gradstat(ts, 1.0, 1.0)
    assert abs(ss.sum_sq - sw.sum_sq) <= 1e-12 * max(sw.sum_sq, 1e-300)
    O.multi_step(ts, hp, sw, O.STEP_ROUND_CLIP_FP16)   # same record: the update itself must be identical
    for k in ("p", "m", "v"):
        assert np.array_equal(np.concatenate([a[k], b[k]]), whole[k]), k


@settings(max_examples=30, deadline=None)
@given(st.integers(1, 3000), st.integers(0, 2 ** 31 - 1), st.sampled_from([2.0, 256.0, 65536.0]))
def test_power_of_two_loss_scale_is_transparent(O, n, seed, scale):
    """Scaling FP16 gradients by a power of two and unscaling in the step gives the bits of the
    unscaled run, as long as the scaled values stay finite."""
    rng = np.random.default_rng(seed)
    p = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(0.02))
    g = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(1e-4))
    gs = O.f2h(O.h2f(g) * np.float32(scale))
    hp = O.HParams(1e-4, 0.9, 0.999, 1e-8, O.bias_correction(0.9, 3), O.bias_correction(0.999, 3))
    out = []
    for grad, unscale in ((g, 1.0), (gs, 1.0 / scale)):
        e = dict(p=p.copy(), g=grad.copy(), m=np.zeros(n, np.float32), v=np.zeros(n, np.float32), wd=0.01)
        ts = O.make_tensors([e])
        s = O.gradstat(ts, unscale, 0.0)
        O.multi_step(ts, hp, s, 0)
        out.append((e, s))
    assert out[0][1].norm == out[1][1].norm
    for k in ("p", "m", "v"):
        assert np.array_equal(out[0][0][k], out[1][0][k]), k


@settings(max_examples=200, deadline=None)
@given(st.floats(-70000, 70000, width=32), st.floats(-70000, 70000, width=32))
def test_half_rounding_is_monotone(O, a, b):
    lo, hi = (a, b) if a <= b else (b, a)
    h = O.h2f(O.f2h(np.array([lo, hi], np.float32)))
    assert h[0] <= h[1]
