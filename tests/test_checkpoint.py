"""Optimizer-state checkpoint: file-format checks that need no GPU, and on the GPU the
property that matters -- a run that saves, reloads into fresh buffers and continues is
bit-identical to the run that never stopped (RL.cu has only a stub here,
include/training/trainer.h:317-319)."""
import struct

import numpy as np
import pytest

from helpers import seeded_case


def test_missing_and_foreign_files_are_rejected(pkg, tmp_path):
    with pytest.raises(pkg.RlcuError):
        pkg.checkpoint_peek(tmp_path / "nope.ckpt")
    bad = tmp_path / "bad.ckpt"
    bad.write_bytes(b"NOTACKPT" + bytes(200))
    with pytest.raises(pkg.RlcuError) as e:
        pkg.checkpoint_peek(bad)
    assert "bad magic" in str(e.value)
    short = tmp_path / "short.ckpt"
    short.write_bytes(b"RLCU")
    with pytest.raises(pkg.RlcuError):
        pkg.checkpoint_peek(short)
    future = tmp_path / "future.ckpt"
    future.write_bytes(b"RLCUOPT1" + struct.pack("<II", 9, 128) + bytes(112))
    with pytest.raises(pkg.RlcuError) as e:
        pkg.checkpoint_peek(future)
    assert e.value.code == pkg.ERR_UNSUPPORTED


def test_empty_state_round_trip_on_the_host(pkg, tmp_path):
    """state_elems == 0 touches no device memory: header and checksum only."""
    path = tmp_path / "empty.ckpt"
    info = pkg.CheckpointInfo(0, 17, 32768.0, 5, 2, 3, 8, 0, 0)
    pkg.checkpoint_save(path, info, None, None)
    got = pkg.checkpoint_peek(path)
    assert (got.state_elems, got.step, got.loss_scale, got.growth_tracker, got.skipped, got.rank, got.world) == \
           (0, 17, 32768.0, 5, 2, 3, 8)
    assert path.stat().st_size == 128 + 8
    again = pkg.checkpoint_load(path, None, None, None, 0)
    assert again.step == 17


def test_failed_save_keeps_the_previous_checkpoint(pkg, tmp_path):
    """The file is written beside the target and renamed over it when complete: a save that
    cannot finish (here: the temporary name is taken by a directory) leaves the old file alone."""
    path = tmp_path / "opt.ckpt"
    pkg.checkpoint_save(path, pkg.CheckpointInfo(0, 3, 1024.0, 0, 0, 0, 1, 0, 0), None, None)
    old = path.read_bytes()
    (tmp_path / "opt.ckpt.tmp").mkdir()
    with pytest.raises(pkg.RlcuError):
        pkg.checkpoint_save(path, pkg.CheckpointInfo(0, 4, 2048.0, 0, 0, 0, 1, 0, 0), None, None)
    assert path.read_bytes() == old and pkg.checkpoint_peek(path).step == 3
    (tmp_path / "opt.ckpt.tmp").rmdir()
    pkg.checkpoint_save(path, pkg.CheckpointInfo(0, 4, 2048.0, 0, 0, 0, 1, 0, 0), None, None)
    assert pkg.checkpoint_peek(path).step == 4 and not (tmp_path / "opt.ckpt.tmp").exists()


@pytest.mark.gpu
@pytest.mark.parametrize("with_master", [False, True])
def test_resume_is_bit_identical(pkg, O, tmp_path, with_master):
    import torch
    torch.cuda.set_device(0)
    n, lr, b1, b2, eps, wd = 300_011, 1e-4, 0.9, 0.999, 1e-8, 0.01
    p0, _, _, _ = seeded_case(O, n, seed=5)

    def dev(a):
        return torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda()

    def grads(t):
        return dev(O.f2h(np.random.default_rng([6, t]).standard_normal(n).astype(np.float32) * np.float32(1e-2)))

    def make_state():
        return dict(p=dev(p0.copy()), m=torch.zeros(n, device="cuda"), v=torch.zeros(n, device="cuda"),
                    master=dev(O.h2f(p0)) if with_master else None)

    def step(st, t):
        g = grads(t)
        tl = pkg.TensorList([pkg.TensorDesc(st["p"].data_ptr(), g.data_ptr(), st["m"].data_ptr(), st["v"].data_ptr(),
                                            st["master"].data_ptr() if with_master else None, n, wd, pkg.F16, 0, 0)])
        stat = torch.zeros(16, device="cuda")
        tl.gradstat(stat.data_ptr(), 1.0, 1.0)
        tl.step(pkg.hparams(lr, b1, b2, eps, t), stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16)
        torch.cuda.synchronize()
        tl.close()

    a = make_state()
    for t in (1, 2, 3):
        step(a, t)
    path = tmp_path / "opt.ckpt"
    info = pkg.CheckpointInfo(n, 3, 65536.0, 7, 1, 0, 1, 1 if with_master else 0, 0)
    pkg.checkpoint_save(path, info, a["m"].data_ptr(), a["v"].data_ptr(),
                        a["master"].data_ptr() if with_master else None)
    p_at_save = a["p"].clone()
    for t in (4, 5):
        step(a, t)

    b = make_state()
    b["p"].copy_(p_at_save)                      # the FP16 weights are the model's checkpoint, not ours
    got = pkg.checkpoint_load(path, b["m"].data_ptr(), b["v"].data_ptr(),
                              b["master"].data_ptr() if with_master else None, n)
    assert (got.state_elems, got.step, got.loss_scale, got.growth_tracker, got.skipped) == (n, 3, 65536.0, 7, 1)
    for t in (got.step + 1, got.step + 2):
        step(b, t)
    for k in ("p", "m", "v", "master"):
        if a[k] is not None:
            view = torch.int16 if a[k].dtype == torch.int16 else torch.int32
            assert torch.equal(a[k].view(view), b[k].view(view)), f"{k} differs after resume"

    # wrong buffer shape and corruption are refused
    with pytest.raises(pkg.RlcuError):
        pkg.checkpoint_load(path, b["m"].data_ptr(), b["v"].data_ptr(),
                            b["master"].data_ptr() if with_master else None, n - 1)
    with pytest.raises(pkg.RlcuError):
        pkg.checkpoint_load(path, b["m"].data_ptr(), b["v"].data_ptr(),
                            None if with_master else b["m"].data_ptr(), n)
    # a corrupt or truncated file is refused before anything reaches the live state
    good = path.read_bytes()
    raw = bytearray(good)
    raw[128 + 1000] ^= 0x40
    path.write_bytes(bytes(raw))
    before = {k: b[k].clone() for k in ("m", "v", "master") if b[k] is not None}
    with pytest.raises(pkg.RlcuError) as e:
        pkg.checkpoint_load(path, b["m"].data_ptr(), b["v"].data_ptr(),
                            b["master"].data_ptr() if with_master else None, n)
    assert "checksum" in str(e.value)
    path.write_bytes(good[:len(good) // 2])
    with pytest.raises(pkg.RlcuError) as e:
        pkg.checkpoint_load(path, b["m"].data_ptr(), b["v"].data_ptr(),
                            b["master"].data_ptr() if with_master else None, n)
    assert "truncated" in str(e.value)
    for k, t in before.items():
        assert torch.equal(t.view(torch.int32), b[k].view(torch.int32)), f"{k} was touched by a refused load"
