"""Generates tests/golden/adamw_ref_b200.npz: inputs and outputs of the REFERENCE's own
CUDA kernels (RL.cu src/kernels/adamw.cu and the static clip kernels of
include/training/trainer.h, compiled unmodified into oracle/_ref/libref_adamw.so) run on a
B200.  The CPU oracle is pinned against these vectors by tests/test_oracle_golden.py.

Run on a machine with a B200 after `make -C oracle` has built the reference library
(that step needs a checkout of RL.cu; this script itself does not):

    python tests/golden/make_golden.py [output.npz]

Inputs are seeded synthetic data with the shapes and distributions of the benchmark
configurations (FP16 params ~N(0,0.02), FP16 grads ~N(0,1e-3) / N(0,1e-4), FP32 moments
starting at zero); no dataset or checkpoint is involved.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402


def dev(a):
    return torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda()


def host(t):
    a = t.cpu().numpy()
    return a.view(np.uint16) if a.dtype == np.int16 else a


def main(out_path):
    R = O.ref_lib()
    out = {}

    # ---- launch_adamw_fp16: ten steps, the single-tensor configuration's hyper-parameters
    for tag, n, lr, b1, b2, eps, wd, steps, gstd in (
            ("h_a", 4133, 1e-5, 0.9, 0.999, 1e-8, 0.01, 10, 1e-3),
            ("h_b", 2051, 1e-3, 0.9, 0.999, 1e-8, 0.01, 4, 1e-4),
            ("h_c", 1024, 1.7e-2, 0.8, 0.99, 1e-6, 0.37, 3, 1e-2)):
        rng = np.random.default_rng([20, n])
        p0 = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(0.02))
        grads = np.stack([O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(gstd))
                          for _ in range(steps)])
        master, p = dev(O.h2f(p0)), dev(p0.copy())
        m, v = dev(np.zeros(n, np.float32)), dev(np.zeros(n, np.float32))
        snaps = []
        for t in range(1, steps + 1):
            g = dev(grads[t - 1])
            bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)
            rc = R.ref_launch_adamw_fp16(master.data_ptr(), p.data_ptr(), g.data_ptr(), m.data_ptr(),
                                         v.data_ptr(), n, lr, b1, b2, eps, wd, bc1, bc2, None)
            assert rc == 0
            torch.cuda.synchronize()
            snaps.append((host(master).copy(), host(p).copy(), host(m).copy(), host(v).copy()))
        out[f"{tag}_hyper"] = np.array([lr, b1, b2, eps, wd], np.float64)
        out[f"{tag}_p0"] = p0
        out[f"{tag}_grads"] = grads
        keep = sorted({1, 2, steps})          # snapshots after these steps
        out[f"{tag}_snap_steps"] = np.array(keep, np.int32)
        for name, idx in (("master", 0), ("p", 1), ("m", 2), ("v", 3)):
            out[f"{tag}_{name}"] = np.stack([snaps[t - 1][idx] for t in keep])

    # ---- launch_adamw_fp32: norm-weight shaped, no weight decay (optimizer.h:143-146)
    n, lr, b1, b2, eps, wd, steps = 2304 + 5, 1e-5, 0.9, 0.999, 1e-8, 0.0, 5
    rng = np.random.default_rng([21, n])
    w0 = (1.0 + rng.standard_normal(n) * 0.01).astype(np.float32)
    grads = (rng.standard_normal((steps, n)) * 1e-3).astype(np.float32)
    w, m, v = dev(w0.copy()), dev(np.zeros(n, np.float32)), dev(np.zeros(n, np.float32))
    snaps = []
    for t in range(1, steps + 1):
        g = dev(grads[t - 1])
        bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)
        rc = R.ref_launch_adamw_fp32(w.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), n,
                                     lr, b1, b2, eps, wd, bc1, bc2, None)
        assert rc == 0
        torch.cuda.synchronize()
        snaps.append((host(w).copy(), host(m).copy(), host(v).copy()))
    out["f_hyper"] = np.array([lr, b1, b2, eps, wd], np.float64)
    out["f_w0"], out["f_grads"] = w0, grads
    keep = sorted({1, 2, steps})
    out["f_snap_steps"] = np.array(keep, np.int32)
    for name, idx in (("w", 0), ("m", 1), ("v", 2)):
        out[f"f_{name}"] = np.stack([snaps[t - 1][idx] for t in keep])

    # ---- clip_grad_norm_: one case above the threshold (scaled), one below (untouched)
    for tag, gstd, max_norm in (("c_hi", 1e-2, 1.0), ("c_lo", 1e-4, 1.0)):
        n16, n32 = 20001, 2309
        rng = np.random.default_rng([22, n16])
        g16 = O.f2h(rng.standard_normal(n16).astype(np.float32) * np.float32(gstd))
        g32 = (rng.standard_normal(n32) * gstd).astype(np.float32)
        d16, d32 = dev(g16.copy()), dev(g32.copy())
        acc = torch.zeros(1, device="cuda")
        norm = C.c_float()
        rc = R.ref_clip_grad_norm(d16.data_ptr(), n16, d32.data_ptr(), n32, max_norm, acc.data_ptr(),
                                  C.byref(norm))
        assert rc == 0
        torch.cuda.synchronize()
        out[f"{tag}_g16"], out[f"{tag}_g32"] = g16, g32
        out[f"{tag}_norm"] = np.array([norm.value], np.float32)
        out[f"{tag}_max_norm"] = np.array([max_norm], np.float32)
        out[f"{tag}_g16_out"], out[f"{tag}_g32_out"] = host(d16).copy(), host(d32).copy()

    out["meta"] = np.array([f"reference kernels on {torch.cuda.get_device_name(0)}, "
                            f"CUDA runtime {torch.version.cuda}"])
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    default = os.path.join(ROOT, "tests", "golden", "adamw_ref_b200.npz")
    target = sys.argv[1] if len(sys.argv) > 1 else default
    os.makedirs(os.path.dirname(target), exist_ok=True)
    main(target)
