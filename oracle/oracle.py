"""ctypes front end of the CPU oracle (``liboracle.so``) and, when it was built,
of the reference's own CUDA kernels (``_ref/libref_adamw.so``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, by the smoke check and by
the benchmark's CPU-baseline leg.  The product package never imports it.

Arrays are numpy: FP16 data travels as ``uint16`` bit patterns (``arr.view(np.uint16)``)
so that nothing depends on numpy's own half conversions.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")
REF_LIB_PATH = os.path.join(_HERE, "_ref", "libref_adamw.so")

UNFUSED = 0


def rounding(m_mode, v_mode, w_fused, d_fused):
    """ORC_ROUNDING bit field (see adamw_oracle.h)."""
    return m_mode | (v_mode << 2) | (w_fused << 4) | (d_fused << 5)


NVCC = rounding(2, 2, 0, 0)
F16, F32, BF16 = 0, 1, 2
FLAG_NORM_ONLY, FLAG_GRAD_ZERO = 1, 2
GRAD_AS_PARAM, GRAD_F32 = 0, 1
STEP_ROUND_CLIP_FP16 = 1


class Tensor(C.Structure):
    """Binary layout of ``orc_tensor`` (and of the product's ``rlcu_tensor_desc``)."""
    _fields_ = [("param", C.c_void_p), ("grad", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
                ("master", C.c_void_p), ("n", C.c_uint64), ("weight_decay", C.c_float),
                ("dtype", C.c_uint32), ("flags", C.c_uint32), ("grad_dtype", C.c_uint32)]


class HParams(C.Structure):
    _fields_ = [("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
                ("bias_correction1", C.c_float), ("bias_correction2", C.c_float)]


class Stat(C.Structure):
    _fields_ = [("sum_sq", C.c_double), ("norm", C.c_float), ("coef", C.c_float),
                ("found_inf", C.c_uint32), ("clip_active", C.c_uint32)]


class Scaler(C.Structure):
    _fields_ = [("scale", C.c_float), ("growth_tracker", C.c_int32), ("step", C.c_int32),
                ("skipped", C.c_int32)]


def build(force: bool = False) -> None:
    """Compile the checkers with the Makefile beside this file."""
    if force or not os.path.exists(LIB_PATH):
        subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.DEVNULL)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB_PATH)
        f, i64, i32, vp = C.c_float, C.c_int64, C.c_int, C.c_void_p
        hyper = [f] * 7
        L.orc_f2h.argtypes, L.orc_f2h.restype = [f], C.c_uint16
        L.orc_h2f.argtypes, L.orc_h2f.restype = [C.c_uint16], f
        L.orc_f2h_hw.argtypes, L.orc_f2h_hw.restype = [f], C.c_uint16
        L.orc_h2f_hw.argtypes, L.orc_h2f_hw.restype = [C.c_uint16], f
        L.orc_hw_half_available.restype = i32
        L.orc_use_hw_half.argtypes = [i32]
        L.orc_f2h_array.argtypes = [vp, vp, i64]
        L.orc_h2f_array.argtypes = [vp, vp, i64]
        L.orc_f2bf_array.argtypes = [vp, vp, i64]
        L.orc_bf2f_array.argtypes = [vp, vp, i64]
        L.orc_bias_correction.argtypes, L.orc_bias_correction.restype = [f, i32], f
        L.orc_adamw_fp16_master.argtypes = [vp, vp, vp, vp, vp, i64] + hyper + [i32, i32]
        L.orc_adamw_fp16.argtypes = [vp, vp, vp, vp, i64] + hyper + [i32, i32]
        L.orc_adamw_fp32.argtypes = [vp, vp, vp, vp, i64] + hyper + [i32, i32]
        L.orc_sum_sq_half.argtypes, L.orc_sum_sq_half.restype = [vp, i64, f, i32], C.c_double
        L.orc_sum_sq_float.argtypes, L.orc_sum_sq_float.restype = [vp, i64, f, i32], C.c_double
        L.orc_count_nonfinite_half.argtypes, L.orc_count_nonfinite_half.restype = [vp, i64], i64
        L.orc_count_nonfinite_float.argtypes, L.orc_count_nonfinite_float.restype = [vp, i64], i64
        L.orc_scale_half.argtypes = [vp, i64, f, i32]
        L.orc_scale_float.argtypes = [vp, i64, f, i32]
        L.orc_clip_grad_norm.argtypes = [vp, i64, vp, i64, f, i32]
        L.orc_clip_grad_norm.restype = f
        L.orc_gradstat.argtypes = [vp, C.c_uint64, f, f, C.c_double, C.c_uint32, i32, vp]
        L.orc_gradstat_finalize.argtypes = [C.c_double, C.c_uint32, f, f, vp]
        L.orc_multi_step.argtypes = [vp, C.c_uint64, vp, vp, C.c_uint32, i32, i32]
        L.orc_multi_step.restype = i32
        L.orc_scaler_update.argtypes = [vp, C.c_uint32, i32]
        _lib = L
    return _lib


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def f2h(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f2h_array(_p(x), _p(out), x.size)
    return out


def h2f(h: np.ndarray) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, dtype=np.float32)
    lib().orc_h2f_array(_p(h), _p(out), h.size)
    return out


def f2bf(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f2bf_array(_p(x), _p(out), x.size)
    return out


def bf2f(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    out = np.empty(b.shape, dtype=np.float32)
    lib().orc_bf2f_array(_p(b), _p(out), b.size)
    return out


def hw_half_available() -> bool:
    """Whether the timed loops convert halves with the CPU's F16C instructions."""
    return bool(lib().orc_hw_half_available())


def use_hw_half(on: bool) -> None:
    lib().orc_use_hw_half(1 if on else 0)


def bias_correction(beta: float, step: int) -> float:
    return float(lib().orc_bias_correction(beta, step))


def adamw_fp16_master(master, model_w, grad, m, v, lr, beta1, beta2, eps, wd, bc1, bc2,
                      rounding=NVCC, threads=1):
    lib().orc_adamw_fp16_master(_p(master), _p(model_w), _p(grad), _p(m), _p(v), master.size,
                                lr, beta1, beta2, eps, wd, bc1, bc2, rounding, threads)


def adamw_fp16(param, grad, m, v, lr, beta1, beta2, eps, wd, bc1, bc2, rounding=NVCC, threads=1):
    lib().orc_adamw_fp16(_p(param), _p(grad), _p(m), _p(v), param.size,
                         lr, beta1, beta2, eps, wd, bc1, bc2, rounding, threads)


def adamw_fp32(w, grad, m, v, lr, beta1, beta2, eps, wd, bc1, bc2, rounding=NVCC, threads=1):
    lib().orc_adamw_fp32(_p(w), _p(grad), _p(m), _p(v), w.size,
                         lr, beta1, beta2, eps, wd, bc1, bc2, rounding, threads)


def sum_sq(g: np.ndarray, unscale: float = 1.0, threads: int = 1) -> float:
    if g.dtype == np.uint16:
        return float(lib().orc_sum_sq_half(_p(g), g.size, unscale, threads))
    assert g.dtype == np.float32
    return float(lib().orc_sum_sq_float(_p(g), g.size, unscale, threads))


def clip_grad_norm(half_pool, float_pool, max_norm: float, threads: int = 1) -> float:
    n16 = 0 if half_pool is None else half_pool.size
    n32 = 0 if float_pool is None else float_pool.size
    return float(lib().orc_clip_grad_norm(_p(half_pool), n16, _p(float_pool), n32, max_norm, threads))


def make_tensors(entries) -> C.Array:
    """entries: iterable of dicts with numpy arrays p, g, m, v, optional master, wd, flags."""
    entries = list(entries)
    arr = (Tensor * len(entries))()
    for k, e in enumerate(entries):
        p = e["p"]
        t = arr[k]
        t.param, t.grad, t.m, t.v = _p(p), _p(e.get("g")), _p(e.get("m")), _p(e.get("v"))
        t.master = _p(e.get("master"))
        t.n = p.size if p is not None else e["g"].size
        t.weight_decay = e.get("wd", 0.0)
        t.dtype = e.get("dtype", F16 if (p if p is not None else e["g"]).dtype == np.uint16 else F32)
        t.flags = e.get("flags", 0)
        t.grad_dtype = e.get("grad_dtype", GRAD_AS_PARAM)
    return arr


def gradstat(tensors, unscale=1.0, max_norm=0.0, extra_sum_sq=0.0, extra_found_inf=0, threads=1) -> Stat:
    out = Stat()
    lib().orc_gradstat(C.addressof(tensors), len(tensors), unscale, max_norm, extra_sum_sq,
                       extra_found_inf, threads, C.addressof(out))
    return out


def gradstat_finalize(sum_sq_total, found_inf, unscale, max_norm) -> Stat:
    out = Stat()
    lib().orc_gradstat_finalize(sum_sq_total, found_inf, unscale, max_norm, C.addressof(out))
    return out


def multi_step(tensors, hp: HParams, stat: Stat | None, step_flags=0, rounding=NVCC, threads=1) -> int:
    return lib().orc_multi_step(C.addressof(tensors), len(tensors), C.addressof(hp),
                                C.addressof(stat) if stat is not None else None,
                                step_flags, rounding, threads)


def scaler_update(s: Scaler, found_inf: int, growth_interval: int) -> None:
    lib().orc_scaler_update(C.addressof(s), found_inf, growth_interval)


# ---------------------------------------------------------------------------
# the reference's own CUDA kernels (GPU only; pointers are device addresses)
# ---------------------------------------------------------------------------
_ref = None


def ref_available() -> bool:
    return os.path.exists(REF_LIB_PATH)


def ref_lib() -> C.CDLL:
    """``libref_adamw.so``: src/kernels/adamw.cu of RL.cu compiled unmodified, plus the
    static clip kernels of include/training/trainer.h behind a C doorway."""
    global _ref
    if _ref is None:
        R = C.CDLL(REF_LIB_PATH)
        f, i32, vp = C.c_float, C.c_int, C.c_void_p
        R.ref_launch_adamw_fp16.argtypes = [vp, vp, vp, vp, vp, i32] + [f] * 7 + [vp]
        R.ref_launch_adamw_fp32.argtypes = [vp, vp, vp, vp, i32] + [f] * 7 + [vp]
        R.ref_grad_sum_sq.argtypes = [vp, i32, vp, i32, vp, C.POINTER(f)]
        R.ref_clip_grad_norm.argtypes = [vp, i32, vp, i32, f, vp, C.POINTER(f)]
        R.ref_scale_grads.argtypes = [vp, i32, vp, i32, f]
        _ref = R
    return _ref
