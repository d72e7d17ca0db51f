"""Pins the CPU oracle against outputs of the reference's own CUDA kernels.

tests/golden/adamw_ref_b200.npz was produced by tests/golden/make_golden.py, which runs
RL.cu's src/kernels/adamw.cu and the static clip kernels of include/training/trainer.h
(compiled unmodified) on a B200.  The oracle must reproduce them bit for bit under its
ORC_NVCC rounding model; under ORC_UNFUSED (the reference's host-side check loop) it must
stay inside the reference test's own bars (tests/test_adamw.cu:224, 324).
"""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "adamw_ref_b200.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN)


def bits(a):
    return a.view(np.uint32) if a.dtype == np.float32 else a.view(np.uint16)


@pytest.mark.parametrize("tag", ["h_a", "h_b", "h_c"])
def test_fp16_master_bit_exact(O, gold, tag):
    lr, b1, b2, eps, wd = (float(x) for x in gold[f"{tag}_hyper"])
    p0, grads = gold[f"{tag}_p0"], gold[f"{tag}_grads"]
    snap_steps = list(gold[f"{tag}_snap_steps"])
    master, p = O.h2f(p0), p0.copy()
    m, v = np.zeros(p0.size, np.float32), np.zeros(p0.size, np.float32)
    for t in range(1, grads.shape[0] + 1):
        O.adamw_fp16_master(master, p, grads[t - 1], m, v, lr, b1, b2, eps, wd,
                            O.bias_correction(b1, t), O.bias_correction(b2, t), O.NVCC)
        if t in snap_steps:
            k = snap_steps.index(t)
            for name, mine in (("master", master), ("p", p), ("m", m), ("v", v)):
                ref = gold[f"{tag}_{name}"][k]
                assert np.array_equal(bits(mine), bits(ref)), f"{tag} step {t}: {name} differs"


def test_fp16_master_unfused_within_reference_test_bars(O, gold):
    """The reference's CPU check rounds every operation separately and passes at
    max |err| < 1e-6 on the master and zero FP16 mismatches after one step."""
    tag = "h_b"
    lr, b1, b2, eps, wd = (float(x) for x in gold[f"{tag}_hyper"])
    p0, grads = gold[f"{tag}_p0"], gold[f"{tag}_grads"]
    master, p = O.h2f(p0), p0.copy()
    m, v = np.zeros(p0.size, np.float32), np.zeros(p0.size, np.float32)
    O.adamw_fp16_master(master, p, grads[0], m, v, lr, b1, b2, eps, wd,
                        O.bias_correction(b1, 1), O.bias_correction(b2, 1), O.UNFUSED)
    assert np.abs(master - gold[f"{tag}_master"][0]).max() < 1e-6
    assert np.array_equal(p, gold[f"{tag}_p"][0])


def test_fp32_bit_exact(O, gold):
    lr, b1, b2, eps, wd = (float(x) for x in gold["f_hyper"])
    w, grads = gold["f_w0"].copy(), gold["f_grads"]
    snap_steps = list(gold["f_snap_steps"])
    m, v = np.zeros(w.size, np.float32), np.zeros(w.size, np.float32)
    for t in range(1, grads.shape[0] + 1):
        O.adamw_fp32(w, grads[t - 1], m, v, lr, b1, b2, eps, wd,
                     O.bias_correction(b1, t), O.bias_correction(b2, t), O.NVCC)
        if t in snap_steps:
            k = snap_steps.index(t)
            for name, mine in (("w", w), ("m", m), ("v", v)):
                assert np.array_equal(bits(mine), bits(gold[f"f_{name}"][k])), f"step {t}: {name}"


@pytest.mark.parametrize("tag,clipped", [("c_hi", True), ("c_lo", False)])
def test_clip_grad_norm(O, gold, tag, clipped):
    g16, g32 = gold[f"{tag}_g16"].copy(), gold[f"{tag}_g32"].copy()
    max_norm = float(gold[f"{tag}_max_norm"][0])
    ref_norm = np.float32(gold[f"{tag}_norm"][0])
    # the reference adds FP32 partial sums with atomics in no fixed order: the norm is
    # compared at the 1e-5 relative bar, the scaling bit for bit given the norm it used
    norm = O.clip_grad_norm(g16.copy(), g32.copy(), max_norm)
    assert abs(norm - ref_norm) <= 1e-5 * ref_norm
    assert (ref_norm > max_norm) == clipped
    if clipped:
        scale = np.float32(max_norm) / (ref_norm + np.float32(1e-6))
        O.lib().orc_scale_half(g16.ctypes.data, g16.size, float(scale), 1)
        O.lib().orc_scale_float(g32.ctypes.data, g32.size, float(scale), 1)
    assert np.array_equal(g16, gold[f"{tag}_g16_out"])
    assert np.array_equal(bits(g32), bits(gold[f"{tag}_g32_out"]))
