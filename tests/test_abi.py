"""The C-ABI shared library loads without a GPU and exports every symbol that
include/rlcu_adamw.h declares, plus the two C++ launchers with RL.cu's signatures;
struct layouts match the header; compute entry points fail loudly without a device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(rlcu_[a-z0-9_]+)\s*\(", text))
    return names


def test_exports_every_declared_symbol(pkg):
    L = pkg.lib()
    declared = declared_symbols()
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} is declared in include/ but not exported"
    assert declared == set(pkg.EXPORTS), "the binding's export list and the header disagree"


def test_missing_library_fails_loudly(pkg, monkeypatch):
    """No fallback implementation: without the shared library the binding refuses to work."""
    monkeypatch.setattr(pkg, "_lib", None)
    monkeypatch.setattr(pkg, "LIB_PATH", "/nonexistent/librlcu_b200.so")
    with pytest.raises(ImportError):
        pkg.lib()


def test_exports_reference_launchers(pkg):
    """launch_adamw_fp16 / launch_adamw_fp32 with the mangled names of RL.cu's
    include/kernels/adamw.cuh:24-57, so its objects link unchanged."""
    L = pkg.lib()
    for name in pkg.CXX_EXPORTS:
        assert hasattr(L, name), name


def test_struct_layouts(pkg):
    assert C.sizeof(pkg.TensorDesc) == 64
    assert C.sizeof(pkg.Stat) == 64
    assert C.sizeof(pkg.ScalerState) == 32
    assert C.sizeof(pkg.HParams) == 24
    assert pkg.TensorDesc.n.offset == 40 and pkg.TensorDesc.flags.offset == 56
    assert pkg.Stat.coef.offset == 12 and pkg.Stat.found_inf.offset == 16
    assert pkg.lib().rlcu_abi_version() == 2


def test_bias_correction_host_helper(pkg, O):
    for beta in (0.9, 0.999):
        for t in (1, 6, 10, 1000):
            assert pkg.bias_correction(beta, t) == O.bias_correction(beta, t)


def test_non_positive_n_is_noop(pkg):
    """adamw.cu:49 and :99 of RL.cu: n <= 0 returns before touching anything."""
    assert pkg.lib().rlcu_adamw_fp16_master(None, None, None, None, None, 0, 1e-3, .9, .999, 1e-8, 0, .1, .001, None) == 0
    assert pkg.lib().rlcu_adamw_fp32(None, None, None, None, -5, 1e-3, .9, .999, 1e-8, 0, .1, .001, None) == 0
    assert pkg.lib().rlcu_adamw_fp16(None, None, None, None, 0, 1e-3, .9, .999, 1e-8, 0, .1, .001, None) == 0


def test_no_cpu_fallback(pkg):
    """Without a CUDA device a compute call must fail with an error, never compute on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import numpy as np
    a = np.zeros(64, np.float32)
    rc = pkg.lib().rlcu_adamw_fp32(a.ctypes.data, a.ctypes.data, a.ctypes.data, a.ctypes.data, 64,
                                   1e-3, .9, .999, 1e-8, 0, .1, .001, None)
    assert rc == pkg.ERR_CUDA
    assert pkg.lib().rlcu_last_error()
    with pytest.raises(pkg.RlcuError):
        pkg.TensorList([pkg.TensorDesc(a.ctypes.data, a.ctypes.data, a.ctypes.data, a.ctypes.data, None, 64, 0.0, pkg.F32, 0, 0)])


def test_product_does_not_touch_the_oracle():
    """The package and its sources never import, link or load anything under oracle/."""
    pkg_dir = os.path.join(ROOT, "rl.cu_b200")
    for base, _, files in os.walk(pkg_dir):
        if os.path.basename(base) == "lib":
            continue
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h", ".cpp", "Makefile")):
                text = open(os.path.join(base, fn), errors="ignore").read()
                assert "oracle" not in text.lower(), f"{fn} mentions the oracle"
