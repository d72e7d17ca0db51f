"""bfloat16 parameters and gradients (RLCU_BF16).  RL.cu trains in FP16 only, so there is no
reference result to pin this against (parity unpinned): the oracle's conversions are checked
against PyTorch's, and the kernels against the oracle, bit for bit."""
import numpy as np
import pytest

from helpers import DevBuf, read_stat


def test_oracle_bfloat16_conversions_match_pytorch(O):
    import torch
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(200_000).astype(np.float32) * np.float32(s) for s in (1e-30, 1e-6, 1.0, 1e20)]
                       + [np.array([np.inf, -np.inf, 0.0, -0.0, 3.3895314e38, 1.0039062, 1.0117188], np.float32)])
    want = torch.from_numpy(x).bfloat16().view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.f2bf(x), want)
    h = np.arange(65536, dtype=np.uint16)
    back = torch.from_numpy(h.view(np.int16)).view(torch.bfloat16).float().numpy()
    mine = O.bf2f(h)
    ok = ~np.isnan(back)
    assert np.array_equal(mine[ok].view(np.uint32), back[ok].view(np.uint32)) and np.isnan(mine[~ok]).all()
    assert O.f2bf(np.array([np.nan], np.float32))[0] & 0x7F80 == 0x7F80


def bf_case(O, n, seed, master):
    rng = np.random.default_rng(seed)
    p = O.f2bf(rng.standard_normal(n).astype(np.float32) * np.float32(0.02))
    e = dict(p=p, g=O.f2bf(rng.standard_normal(n).astype(np.float32) * np.float32(1e-2)),
             m=(rng.standard_normal(n) * 1e-3).astype(np.float32), v=(rng.random(n) * 1e-5).astype(np.float32),
             wd=0.01, dtype=O.BF16)
    if master:
        e["master"] = O.bf2f(p)
    return e


@pytest.mark.gpu
@pytest.mark.parametrize("offset", [0, 3])
def test_fused_step_bfloat16_vs_oracle(pkg, O, offset):
    import torch
    torch.cuda.set_device(0)
    sizes = [(70_001, False), (8192 * 3, True), (8192, False), (129, True), (1, False)]
    host = [bf_case(O, n, 300 + k, master) for k, (n, master) in enumerate(sizes)]
    f32 = dict(p=(1 + np.random.default_rng(9).standard_normal(500) * 0.01).astype(np.float32),
               g=(np.random.default_rng(10).standard_normal(500) * 1e-2).astype(np.float32),
               m=np.zeros(500, np.float32), v=np.zeros(500, np.float32), wd=0.0)
    host.append(f32)
    dev, descs = [], []
    for e in host:
        d = {k: DevBuf(e[k], torch, offset) for k in ("p", "g", "m", "v", "master") if k in e}
        dev.append(d)
        descs.append(pkg.TensorDesc(d["p"].ptr, d["g"].ptr, d["m"].ptr, d["v"].ptr,
                                    d["master"].ptr if "master" in d else None, e["p"].size, e["wd"],
                                    e.get("dtype", pkg.F32) if e["p"].dtype == np.uint16 else pkg.F32, 0, 0))
    tl = pkg.TensorList(descs)
    stat = torch.zeros(16, device="cuda")
    lr, b1, b2, eps = 1e-4, 0.9, 0.999, 1e-8
    ot = O.make_tensors(host)
    for t in (3, 4):
        hp = pkg.hparams(lr, b1, b2, eps, t)
        tl.gradstat(stat.data_ptr(), 1.0, 1.0)
        tl.step(hp, stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16)
        torch.cuda.synchronize()
        got = read_stat(pkg, stat)
        want = O.gradstat(ot, 1.0, 1.0)
        assert got.clip_active == 1 and abs(got.norm - want.norm) <= 1e-5 * want.norm
        O.multi_step(ot, O.HParams(lr, b1, b2, eps, hp.bias_correction1, hp.bias_correction2),
                     O.gradstat_finalize(got.sum_sq, 0, 1.0, 1.0), O.STEP_ROUND_CLIP_FP16)
    for e, d in zip(host, dev):
        for k in d:
            assert np.array_equal(d[k].get().view(np.uint8), e[k].view(np.uint8)), k
        assert all(b.guards_intact() for b in d.values())


@pytest.mark.gpu
def test_single_tensor_bfloat16_entry_points(pkg, O):
    import torch
    torch.cuda.set_device(0)
    n, lr, b1, b2, eps, wd, t = 100_003, 1e-4, 0.9, 0.999, 1e-8, 0.01, 2
    bc1, bc2 = O.bias_correction(b1, t), O.bias_correction(b2, t)
    for master in (False, True):
        e = bf_case(O, n, 400, master)
        d = {k: DevBuf(e[k], torch) for k in ("p", "g", "m", "v", "master") if k in e}
        if master:
            pkg.adamw_bf16_master(d["master"].ptr, d["p"].ptr, d["g"].ptr, d["m"].ptr, d["v"].ptr, n, lr, b1, b2, eps, wd, bc1, bc2)
        else:
            pkg.adamw_bf16(d["p"].ptr, d["g"].ptr, d["m"].ptr, d["v"].ptr, n, lr, b1, b2, eps, wd, bc1, bc2)
        torch.cuda.synchronize()
        O.multi_step(O.make_tensors([e]), O.HParams(lr, b1, b2, eps, bc1, bc2), None)
        for k in d:
            assert np.array_equal(d[k].get().view(np.uint8), e[k].view(np.uint8)), k
