"""ZeRO-1 sharded step on real GPUs through the C ABI (NCCL reduce-scatter / all-gather).

world = 1 runs on any box.  world >= 2 spawns one process per GPU and is skipped when the
box has fewer GPUs.  Contract: (i) the sharded update equals, bit for bit, a single-GPU step
fed the reduce-scattered (summed) gradients with 1/world as the unscale factor; (ii) the
reduce-scatter itself equals the FP32 sum of the replicas rounded to FP16 within 1 FP16 ulp
per hop (exact for two ranks)."""
import os
import socket

import numpy as np
import pytest

from helpers import read_stat, ulp16

pytestmark = pytest.mark.gpu

SEGS = [(300_000, 0.01, 0), (200_037, 0.0, 0), (8_192, 0.02, 0)]
LR, B1, B2, EPS, T, MAX_NORM = 1e-4, 0.9, 0.999, 1e-8, 4, 1.0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(O, world, bf=False):
    total = sum(s[0] for s in SEGS)
    rng = np.random.default_rng(200)
    if bf:
        p = O.f2bf(rng.standard_normal(total).astype(np.float32) * np.float32(0.02))
        m = (rng.standard_normal(total) * 1e-3).astype(np.float32)
        v = (rng.random(total) * 1e-5).astype(np.float32)
        grads = [O.f2bf(np.random.default_rng([201, r]).standard_normal(total).astype(np.float32) * np.float32(5e-3))
                 for r in range(world)]
        return total, p, m, v, grads
    p = O.f2h(rng.standard_normal(total).astype(np.float32) * np.float32(0.02))
    m = (rng.standard_normal(total) * 1e-3).astype(np.float32)
    v = (rng.random(total) * 1e-5).astype(np.float32)
    grads = [O.f2h(np.random.default_rng([201, r]).standard_normal(total).astype(np.float32) * np.float32(5e-3))
             for r in range(world)]
    return total, p, m, v, grads


def _run_rank(rank, world, uid, pkg, O, torch, use_master, mode=0, bf=False, extra_flags=0):
    """Runs one sharded step on this process's GPU; returns host copies of everything."""
    total, p, m, v, grads = _inputs(O, world, bf)
    plan = pkg.zero1_plan(SEGS, rank, world)
    S, padded = int(plan.shard_elems), int(plan.padded_elems)
    lo = rank * S

    def pool16(a):
        out = np.zeros(padded, np.uint16)
        out[:total] = a
        return torch.from_numpy(out.view(np.int16)).cuda()

    def shard32(a):
        out = np.zeros(padded, np.float32)
        out[:total] = a
        return torch.from_numpy(out[lo:lo + S].copy()).cuda()

    p_pool, g_pool = pool16(p), pool16(grads[rank])
    m_sh, v_sh = shard32(m), shard32(v)
    master_sh = shard32((O.bf2f if bf else O.h2f)(p)) if use_master else None
    stat = torch.zeros(16, device="cuda")
    z = pkg.Zero1(uid, rank, world, p_pool.data_ptr(), g_pool.data_ptr(), SEGS, m_sh.data_ptr(), v_sh.data_ptr(),
                  master_sh.data_ptr() if use_master else None, mode=mode | (pkg.ZERO1_POOLS_BF16 if bf else 0))
    hp = pkg.hparams(LR, B1, B2, EPS, T)
    z.step(hp, stat.data_ptr(), 1.0, MAX_NORM, None, pkg.STEP_ROUND_CLIP_FP16 | extra_flags)
    torch.cuda.synchronize()
    z.check()
    out = dict(p=p_pool.cpu().numpy().view(np.uint16), g=g_pool.cpu().numpy().view(np.uint16),
               m=m_sh.cpu().numpy(), v=v_sh.cpu().numpy(), stat=stat.cpu().numpy(), lo=lo, S=S)
    if use_master:
        out["master"] = master_sh.cpu().numpy()
    z.close()
    return out


def _check(pkg, O, world, outs, use_master, mode=0, bf=False):
    total, p, m, v, grads = _inputs(O, world, bf)
    to_f, to_16 = (O.bf2f, O.f2bf) if bf else (O.h2f, O.f2h)
    S = outs[0]["S"]
    # (ii) the reduce-scattered shard against the FP32 sum (rank order) rounded once to 16 bits
    acc = to_f(grads[0]).copy()
    for g in grads[1:]:
        acc = acc + to_f(g)
    exact = to_16(acc)
    g_sum = np.zeros(total, np.uint16)
    for r, o in enumerate(outs):
        lo, hi = o["lo"], min(o["lo"] + S, total)
        g_sum[lo:hi] = o["g"][lo:hi]
    if world <= 2 or mode == 1:
        # two ranks: one correctly rounded addition; peer-to-peer mode: FP32 sum, one rounding
        assert np.array_equal(g_sum, exact)
    else:
        # NCCL adds in FP16 hop by hop in an order of its choosing: each of the world-1
        # additions can lose half an FP16 ulp of the partial sum it produces
        ulp = 2.0 ** (-8 if bf else -11)
        bound = (world - 1) * ulp * np.sum([np.abs(to_f(g)) for g in grads], axis=0) + 2.0 ** -24
        assert (np.abs(to_f(g_sum).astype(np.float64) - acc) <= bound).all()
    # (i) single-rank oracle step on the summed gradients, unscale = 1/world
    master = to_f(p)
    entries, off = [], 0
    for n, wd, fl in SEGS:
        e = dict(p=p[off:off + n], g=g_sum[off:off + n], m=m[off:off + n], v=v[off:off + n], wd=wd, flags=fl,
                 dtype=O.BF16 if bf else O.F16)
        if use_master:
            e["master"] = master[off:off + n]
        entries.append(e)
        off += n
    ts = O.make_tensors(entries)
    want = O.gradstat(ts, 1.0 / world, MAX_NORM)
    got = pkg.Stat.from_buffer_copy(outs[0]["stat"].tobytes())
    assert got.found_inf == 0 and got.clip_active == want.clip_active == 1
    assert abs(got.norm - want.norm) <= 1e-5 * want.norm
    hp = O.HParams(LR, B1, B2, EPS, O.bias_correction(B1, T), O.bias_correction(B2, T))
    O.multi_step(ts, hp, O.gradstat_finalize(got.sum_sq, 0, 1.0 / world, MAX_NORM), O.STEP_ROUND_CLIP_FP16)
    for r, o in enumerate(outs):
        st = pkg.Stat.from_buffer_copy(o["stat"].tobytes())
        assert (st.sum_sq, st.norm, st.coef) == (got.sum_sq, got.norm, got.coef), "ranks disagree on the norm"
        assert np.array_equal(o["p"][:total], p), f"rank {r}: parameters after all-gather differ"
        lo, hi = o["lo"], min(o["lo"] + S, total)
        assert np.array_equal(o["m"][:hi - lo], m[lo:hi]) and np.array_equal(o["v"][:hi - lo], v[lo:hi])
        if use_master:
            assert np.array_equal(o["master"][:hi - lo], master[lo:hi])
        assert not o["p"][total:].any()              # padding stays zero


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("use_master", [False, True])
def test_world_one_equals_unsharded_step(pkg, O, use_master, mode):
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    out = _run_rank(0, 1, pkg.zero1_unique_id(), pkg, O, torch, use_master, mode)
    _check(pkg, O, 1, [out], use_master, mode)


@pytest.mark.parametrize("mode", [0, 1], ids=["nccl", "p2p"])
def test_world_one_bfloat16_pools(pkg, O, mode):
    import torch
    torch.cuda.set_device(0)
    out = _run_rank(0, 1, pkg.zero1_unique_id(), pkg, O, torch, True, mode, bf=True)
    _check(pkg, O, 1, [out], True, mode, bf=True)


def _worker(rank, world, port, out_dir, use_master, mode, bf=False):
    import sys
    import torch
    import torch.distributed as dist
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    import __graft_entry__ as entry
    from oracle import oracle as O
    pkg = entry.load_package()
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    box = [pkg.zero1_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    out = _run_rank(rank, world, box[0], pkg, O, torch, use_master, mode, bf)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", [0, 1], ids=["nccl", "p2p"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_step_on_several_gpus(pkg, O, tmp_path, world, mode):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), world == 2, mode), nprocs=world, join=True)
    outs = []
    for r in range(world):
        z = np.load(tmp_path / f"rank{r}.npz")
        outs.append({k: (z[k] if z[k].ndim else z[k].item()) for k in z.files})
    _check(pkg, O, world, outs, world == 2, mode)


@pytest.mark.parametrize("mode", [0, 1], ids=["nccl", "p2p"])
def test_bfloat16_pools_on_two_gpus(pkg, O, tmp_path, mode):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), False, mode, True), nprocs=2, join=True)
    outs = []
    for r in range(2):
        z = np.load(tmp_path / f"rank{r}.npz")
        outs.append({k: (z[k] if z[k].ndim else z[k].item()) for k in z.files})
    _check(pkg, O, 2, outs, False, mode, bf=True)


def _leaver(rank, world, port, out_dir):
    """Rank 1 leaves after the first step, between steps, with nothing in flight.  The ranks agree
    on the host (gloo) before every launch who is still there; when someone has left, nobody
    launches, and the survivors abort the communicator instead of waiting on it."""
    import sys
    import torch
    import torch.distributed as dist
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    import __graft_entry__ as entry
    from oracle import oracle as O
    pkg = entry.load_package()
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    box = [pkg.zero1_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    total, p, m, v, grads = _inputs(O, world)
    plan = pkg.zero1_plan(SEGS, rank, world)
    S, padded = int(plan.shard_elems), int(plan.padded_elems)
    pool = lambda a: torch.from_numpy(np.concatenate([a, np.zeros(padded - total, np.uint16)]).view(np.int16)).cuda()
    p_pool, g_pool = pool(p), pool(grads[rank])
    m_sh, v_sh = torch.zeros(S, device="cuda"), torch.zeros(S, device="cuda")
    stat = torch.zeros(16, device="cuda")
    z = pkg.Zero1(box[0], rank, world, p_pool.data_ptr(), g_pool.data_ptr(), SEGS, m_sh.data_ptr(), v_sh.data_ptr(), None)
    steps_done = 0
    for t in (1, 2, 3):
        staying = not (rank == 1 and t == 2)
        votes = [None] * world
        dist.all_gather_object(votes, staying)            # the host-side heartbeat
        if not all(votes):
            break
        z.step(pkg.hparams(LR, B1, B2, EPS, t), stat.data_ptr(), 1.0, MAX_NORM, None, 0)
        torch.cuda.synchronize()
        z.poll_error()
        steps_done += 1
    after = p_pool.cpu().numpy().copy()
    z.close(abort=True)                                    # no collective is pending on any rank
    np.savez(os.path.join(out_dir, f"leave{rank}.npz"), steps=steps_done, p=after.view(np.uint16))
    dist.destroy_process_group()


def test_rank_leaving_between_steps_is_handled_on_the_host(pkg, O, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    mp.spawn(_leaver, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    a, b = np.load(tmp_path / "leave0.npz"), np.load(tmp_path / "leave1.npz")
    assert int(a["steps"]) == int(b["steps"]) == 1         # nobody launched the second step
    assert np.array_equal(a["p"], b["p"])                  # and both hold the same parameters


@pytest.mark.parametrize("mode", [0, 1], ids=["nccl", "p2p"])
def test_sharded_step_with_device_scaler_skips_on_overflow(pkg, O, mode):
    """Loss scaling through the sharded step (world 1 here): the scaler's grad_mul carries
    1/world, a non-finite gradient makes every rank skip and halve the scale, a clean step
    matches the oracle."""
    import torch
    torch.cuda.set_device(0)
    total, p, m, v, grads = _inputs(O, 1)
    plan = pkg.zero1_plan(SEGS, 0, 1)
    S, padded = int(plan.shard_elems), int(plan.padded_elems)
    scale = 1024.0

    def pool(a):
        out = np.zeros(padded, np.uint16)
        out[:total] = a
        return torch.from_numpy(out.view(np.int16)).cuda()

    g_scaled = O.f2h(O.h2f(grads[0]) * np.float32(scale))
    p_pool, g_pool = pool(p), pool(g_scaled)
    m_sh = torch.from_numpy(np.concatenate([m, np.zeros(padded - total, np.float32)])).cuda()
    v_sh = torch.from_numpy(np.concatenate([v, np.zeros(padded - total, np.float32)])).cuda()
    dt = np.dtype([("scale", "f4"), ("gt", "i4"), ("step", "i4"), ("skipped", "i4"),
                   ("interval", "i4"), ("b1", "f4"), ("b2", "f4"), ("mul", "f4")])
    sc = np.zeros(1, dt)
    sc["scale"], sc["interval"], sc["b1"], sc["b2"], sc["mul"], sc["step"] = scale, 1000, B1, B2, 1.0, T - 1
    scaler = torch.from_numpy(sc.view(np.uint8).copy()).cuda()
    stat = torch.zeros(16, device="cuda")
    z = pkg.Zero1(pkg.zero1_unique_id(), 0, 1, p_pool.data_ptr(), g_pool.data_ptr(), SEGS,
                  m_sh.data_ptr(), v_sh.data_ptr(), None, mode=mode)
    hp = pkg.HParams(LR, B1, B2, EPS, 1.0, 1.0)
    # overflowing step first
    bad = g_scaled.copy()
    bad[12345] = 0x7C00
    g_pool.copy_(pool(bad))
    before = (p_pool.clone(), m_sh.clone(), v_sh.clone())
    z.step(hp, stat.data_ptr(), 1.0, MAX_NORM, scaler.data_ptr(), pkg.STEP_DEVICE_BIAS_CORRECTION)
    torch.cuda.synchronize()
    s = read_stat(pkg, stat)
    got = np.frombuffer(scaler.cpu().numpy().tobytes(), dtype=dt)[0]
    assert s.found_inf == 1 and got["scale"] == scale / 2 and got["step"] == T - 1 and got["skipped"] == 1
    assert torch.equal(before[0], p_pool) and torch.equal(before[1], m_sh) and torch.equal(before[2], v_sh)
    # clean step with gradients carrying the halved scale
    g_half = O.f2h(O.h2f(grads[0]) * np.float32(scale / 2))
    g_pool.copy_(pool(g_half))
    z.step(hp, stat.data_ptr(), 1.0, MAX_NORM, scaler.data_ptr(), pkg.STEP_DEVICE_BIAS_CORRECTION)
    torch.cuda.synchronize()
    s = read_stat(pkg, stat)
    assert s.found_inf == 0 and s.step == T and s.loss_scale == scale / 2
    entries, off = [], 0
    for n, wd, fl in SEGS:
        entries.append(dict(p=p[off:off + n], g=g_half[off:off + n], m=m[off:off + n], v=v[off:off + n], wd=wd, flags=fl))
        off += n
    ts = O.make_tensors(entries)
    want = O.gradstat(ts, 2.0 / scale, MAX_NORM)
    assert abs(s.norm - want.norm) <= 1e-5 * want.norm
    O.multi_step(ts, O.HParams(LR, B1, B2, EPS, s.bias_correction1, s.bias_correction2),
                 O.gradstat_finalize(s.sum_sq, 0, 2.0 / scale, MAX_NORM), 0)
    assert np.array_equal(p_pool.cpu().numpy().view(np.uint16)[:total], p)
    assert np.array_equal(m_sh.cpu().numpy()[:total], m) and np.array_equal(v_sh.cpu().numpy()[:total], v)
    z.close()


def _overflow_worker(rank, world, port, out_dir, mode):
    import sys
    import torch
    import torch.distributed as dist
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    import __graft_entry__ as entry
    from oracle import oracle as O
    pkg = entry.load_package()
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    box = [pkg.zero1_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    total, p, m, v, grads = _inputs(O, world)
    plan = pkg.zero1_plan(SEGS, rank, world)
    S, padded = int(plan.shard_elems), int(plan.padded_elems)
    lo = rank * S
    scale = 256.0

    def pool(a):
        out = np.zeros(padded, np.uint16)
        out[:total] = a
        return torch.from_numpy(out.view(np.int16)).cuda()

    def shard(a):
        out = np.zeros(padded, np.float32)
        out[:total] = a
        return torch.from_numpy(out[lo:lo + S].copy()).cuda()

    mine = O.f2h(O.h2f(grads[rank]) * np.float32(scale))
    bad = mine.copy()
    if rank == 1:
        bad[7] = 0xFC00                     # -inf in ONE rank's replica, in the OTHER rank's shard
    p_pool, g_pool = pool(p), pool(bad)
    m_sh, v_sh = shard(m), shard(v)
    dt = np.dtype([("scale", "f4"), ("gt", "i4"), ("step", "i4"), ("skipped", "i4"),
                   ("interval", "i4"), ("b1", "f4"), ("b2", "f4"), ("mul", "f4")])
    sc = np.zeros(1, dt)
    sc["scale"], sc["interval"], sc["b1"], sc["b2"], sc["mul"], sc["step"] = scale, 1000, B1, B2, 1.0 / world, T - 1
    scaler = torch.from_numpy(sc.view(np.uint8).copy()).cuda()
    stat = torch.zeros(16, device="cuda")
    z = pkg.Zero1(box[0], rank, world, p_pool.data_ptr(), g_pool.data_ptr(), SEGS, m_sh.data_ptr(), v_sh.data_ptr(),
                  None, mode=mode)
    hp = pkg.HParams(LR, B1, B2, EPS, 1.0, 1.0)
    z.step(hp, stat.data_ptr(), 1.0, MAX_NORM, scaler.data_ptr(), pkg.STEP_DEVICE_BIAS_CORRECTION)
    torch.cuda.synchronize()
    s1 = stat.cpu().numpy().copy()
    sc1 = scaler.cpu().numpy().copy()
    untouched = bool(np.array_equal(p_pool.cpu().numpy().view(np.uint16)[:total], p))
    g_pool.copy_(pool(O.f2h(O.h2f(grads[rank]) * np.float32(scale / 2))))
    z.step(hp, stat.data_ptr(), 1.0, MAX_NORM, scaler.data_ptr(), pkg.STEP_DEVICE_BIAS_CORRECTION)
    torch.cuda.synchronize()
    np.savez(os.path.join(out_dir, f"ovf{rank}.npz"), s1=s1, sc1=sc1, untouched=untouched, s2=stat.cpu().numpy(),
             sc2=scaler.cpu().numpy(), p=p_pool.cpu().numpy().view(np.uint16), g=g_pool.cpu().numpy().view(np.uint16),
             m=m_sh.cpu().numpy(), v=v_sh.cpu().numpy(), lo=lo, S=S)
    z.close()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", [0, 1], ids=["nccl", "p2p"])
def test_overflow_in_one_replica_skips_every_rank(pkg, O, tmp_path, mode):
    """A non-finite gradient in one rank's replica reaches every rank through the reduced sum of
    squares: all ranks skip, all halve the scale; the next clean step equals the oracle."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world = 2
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_overflow_worker, args=(world, _free_port(), str(tmp_path), mode), nprocs=world, join=True)
    dt = np.dtype([("scale", "f4"), ("gt", "i4"), ("step", "i4"), ("skipped", "i4"),
                   ("interval", "i4"), ("b1", "f4"), ("b2", "f4"), ("mul", "f4")])
    outs = [np.load(tmp_path / f"ovf{r}.npz") for r in range(world)]
    total, p, m, v, grads = _inputs(O, world)
    scale = 256.0
    for o in outs:
        s1 = pkg.Stat.from_buffer_copy(o["s1"].tobytes())
        sc1 = np.frombuffer(o["sc1"].tobytes(), dtype=dt)[0]
        assert s1.found_inf == 1 and bool(o["untouched"])
        assert sc1["scale"] == scale / 2 and sc1["skipped"] == 1 and sc1["step"] == T - 1
        s2 = pkg.Stat.from_buffer_copy(o["s2"].tobytes())
        assert s2.found_inf == 0 and s2.step == T and s2.loss_scale == scale / 2
    S = int(outs[0]["S"])
    g_sum = np.zeros(total, np.uint16)
    for o in outs:
        lo, hi = int(o["lo"]), min(int(o["lo"]) + S, total)
        g_sum[lo:hi] = o["g"][lo:hi]
    s2 = pkg.Stat.from_buffer_copy(outs[0]["s2"].tobytes())
    entries, off = [], 0
    for n, wd, fl in SEGS:
        entries.append(dict(p=p[off:off + n], g=g_sum[off:off + n], m=m[off:off + n], v=v[off:off + n], wd=wd, flags=fl))
        off += n
    ts = O.make_tensors(entries)
    unscale = (1.0 / world) / (scale / 2)
    O.multi_step(ts, O.HParams(LR, B1, B2, EPS, s2.bias_correction1, s2.bias_correction2),
                 O.gradstat_finalize(s2.sum_sq, 0, unscale, MAX_NORM), 0)
    for o in outs:
        assert np.array_equal(o["p"][:total], p)
        lo, hi = int(o["lo"]), min(int(o["lo"]) + S, total)
        assert np.array_equal(o["m"][:hi - lo], m[lo:hi]) and np.array_equal(o["v"][:hi - lo], v[lo:hi])


def _bad_create_worker(rank, world, port, out_dir):
    import sys
    import torch
    import torch.distributed as dist
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    import __graft_entry__ as entry
    pkg = entry.load_package()
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    box = [pkg.zero1_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    plan = pkg.zero1_plan(SEGS, rank, world)
    S, padded = int(plan.shard_elems), int(plan.padded_elems)
    p_pool = torch.zeros(padded, dtype=torch.float16, device="cuda")
    g_pool = torch.zeros(padded, dtype=torch.float16, device="cuda")
    m_sh, v_sh = torch.zeros(S + 8, device="cuda"), torch.zeros(S, device="cuda")
    skew = 4 if rank == 1 else 0                      # rank 1 hands in a misaligned state array
    message = ""
    try:
        pkg.Zero1(box[0], rank, world, p_pool.data_ptr(), g_pool.data_ptr(), SEGS, m_sh.data_ptr() + skew,
                  v_sh.data_ptr(), None, mode=pkg.ZERO1_P2P)
    except pkg.RlcuError as exc:
        message = str(exc)
    with open(os.path.join(out_dir, f"create{rank}.txt"), "w") as f:
        f.write(message)
    dist.barrier()
    dist.destroy_process_group()


def test_create_fails_on_every_rank_when_one_rank_cannot_set_up(pkg, tmp_path):
    """One rank's local set-up fails after the communicator is joined: every rank gets an error
    back (the failing one its own message, the others "another rank failed") and nobody waits
    in a collective the failing rank never enters."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_bad_create_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    m0, m1 = ((tmp_path / f"create{r}.txt").read_text() for r in range(2))
    assert "another rank failed" in m0
    assert "32-byte aligned" in m1


def _flags_worker(rank, world, port, out_dir, mode, extra_flags, plain_flags=0):
    """The same step twice, with `plain_flags` and with `extra_flags`, each on fresh buffers."""
    import sys
    import torch
    import torch.distributed as dist
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    import __graft_entry__ as entry
    from oracle import oracle as O
    pkg = entry.load_package()
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    for tag, fl in (("plain", plain_flags), ("flagged", extra_flags)):
        box = [pkg.zero1_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        out = _run_rank(rank, world, box[0], pkg, O, torch, False, mode, False, fl)
        np.savez(os.path.join(out_dir, f"{tag}{rank}.npz"), **out)
        dist.barrier()
    dist.destroy_process_group()


def _compare_flag_runs(pkg, tmp_path, world, grads_cleared, same_sum_order=True):
    """same_sum_order False: the flagged run adds the squares in another order (another kernel
    with another partition of the shard), so its sum may differ in the last bits: the norm is
    held to 1e-6 relative, and p, m, v to bit identity only if the clip factor came out equal."""
    for r in range(world):
        a, b = np.load(tmp_path / f"plain{r}.npz"), np.load(tmp_path / f"flagged{r}.npz")
        sa, sb = pkg.Stat.from_buffer_copy(a["stat"].tobytes()), pkg.Stat.from_buffer_copy(b["stat"].tobytes())
        if same_sum_order:
            assert np.array_equal(a["stat"].view(np.uint8), b["stat"].view(np.uint8)), f"rank {r}: record differs"
        else:
            assert abs(sa.norm - sb.norm) <= 1e-6 * sa.norm and (sa.found_inf, sa.clip_active) == (sb.found_inf, sb.clip_active)
        for k in ("p", "m", "v"):
            if sa.coef == sb.coef:
                assert np.array_equal(a[k].view(np.uint8), b[k].view(np.uint8)), f"rank {r}: {k} differs"
            elif a[k].dtype == np.uint16:
                assert ulp16(a[k], b[k]).max() <= 1, f"rank {r}: {k} differs by more than 1 ulp"
            else:
                assert np.all(np.abs(a[k] - b[k]) <= 1e-6 * np.abs(a[k]) + 1e-30), f"rank {r}: {k} differs"
        if grads_cleared:
            assert not b["g"].any(), f"rank {r}: gradient pool not cleared"
            assert a["g"].any()
        else:
            assert np.array_equal(a["g"], b["g"])


@pytest.mark.parametrize("mode", [0, 1], ids=["nccl", "p2p"])
@pytest.mark.parametrize("world", [1, 2])
def test_sharded_step_clears_the_whole_gradient_pool_when_asked(pkg, O, tmp_path, world, mode):
    """RLCU_STEP_ZERO_GRADS in the sharded step (RL.cu's qwen3_gradients_zero, qwen3.cu:1109-1112,
    folded in): same parameters, moments and record as without it, and every element of every
    rank's gradient pool, inside and outside its shard, is zero afterwards."""
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_flags_worker, args=(world, _free_port(), str(tmp_path), mode, pkg.STEP_ZERO_GRADS), nprocs=world, join=True)
    _compare_flag_runs(pkg, tmp_path, world, grads_cleared=True)


@pytest.mark.parametrize("world", [1, 2])
def test_sharded_step_through_the_bulk_copy_engine(pkg, O, tmp_path, world):
    """The two pairs of exchange kernels of peer-to-peer mode against each other: RLCU_STEP_DIRECT
    (per-thread loads and stores) and RLCU_STEP_BULK_COPY (the peers' gradients fetched, and the
    update's traffic with the copies into the peers' pools issued, by cp.async.bulk; the default
    for FP16 pools on several ranks).  Reduced gradients are bit-identical; the sum of squares
    is taken in another order."""
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_flags_worker, args=(world, _free_port(), str(tmp_path), 1, pkg.STEP_BULK_COPY, pkg.STEP_DIRECT),
             nprocs=world, join=True)
    _compare_flag_runs(pkg, tmp_path, world, grads_cleared=False, same_sum_order=False)
    mp.spawn(_flags_worker, args=(world, _free_port(), str(tmp_path), 1, pkg.STEP_BULK_COPY | pkg.STEP_ZERO_GRADS, pkg.STEP_DIRECT),
             nprocs=world, join=True)
    _compare_flag_runs(pkg, tmp_path, world, grads_cleared=True, same_sum_order=False)


# ---------------------------------------------------------------------------------------------
# FP32 gradient pools (RLCU_ZERO1_GRADS_F32)
# ---------------------------------------------------------------------------------------------

def _f32_grads(O, world):
    total, p, m, v, grads = _inputs(O, world)
    out = []
    for r, g in enumerate(grads):
        fine = np.random.default_rng([202, r]).standard_normal(total).astype(np.float32)
        out.append((O.h2f(g) * (np.float32(1) + np.float32(2.0 ** -13) * fine)).astype(np.float32))
    return total, p, m, v, out


def _f32_worker(rank, world, port, out_dir, mode, use_master):
    import sys
    import torch
    import torch.distributed as dist
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    import __graft_entry__ as entry
    from oracle import oracle as O
    pkg = entry.load_package()
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    box = [pkg.zero1_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    total, p, m, v, grads = _f32_grads(O, world)
    plan = pkg.zero1_plan(SEGS, rank, world)
    S, padded = int(plan.shard_elems), int(plan.padded_elems)
    lo = rank * S

    def padded_of(a, dtype):
        out = np.zeros(padded, dtype)
        out[:total] = a
        return out

    p_pool = torch.from_numpy(padded_of(p, np.uint16).view(np.int16)).cuda()
    g_pool = torch.from_numpy(padded_of(grads[rank], np.float32)).cuda()
    m_sh = torch.from_numpy(padded_of(m, np.float32)[lo:lo + S].copy()).cuda()
    v_sh = torch.from_numpy(padded_of(v, np.float32)[lo:lo + S].copy()).cuda()
    master_sh = torch.from_numpy(padded_of(O.h2f(p), np.float32)[lo:lo + S].copy()).cuda() if use_master else None
    stat = torch.zeros(16, device="cuda")
    z = pkg.Zero1(box[0], rank, world, p_pool.data_ptr(), g_pool.data_ptr(), SEGS, m_sh.data_ptr(), v_sh.data_ptr(),
                  master_sh.data_ptr() if use_master else None, mode=mode | pkg.ZERO1_GRADS_F32)
    z.step(pkg.hparams(LR, B1, B2, EPS, T), stat.data_ptr(), 1.0, MAX_NORM, None, pkg.STEP_ROUND_CLIP_FP16)
    torch.cuda.synchronize()
    z.poll_error()
    out = dict(p=p_pool.cpu().numpy().view(np.uint16), g=g_pool.cpu().numpy(), m=m_sh.cpu().numpy(), v=v_sh.cpu().numpy(),
               stat=stat.cpu().numpy(), lo=lo, S=S)
    if use_master:
        out["master"] = master_sh.cpu().numpy()
    z.close()
    np.savez(os.path.join(out_dir, f"f32rank{rank}.npz"), **out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", [0, 1], ids=["nccl", "p2p"])
@pytest.mark.parametrize("world,use_master", [(1, False), (2, True), (4, False)])
def test_sharded_step_with_fp32_gradient_pools(pkg, O, tmp_path, world, use_master, mode):
    """FP16 parameters whose gradients arrive in FP32 (RL.cu accumulates dW in FP16,
    src/kernels/linear.cu:85-98; this is the variant for a caller that accumulates in FP32):
    the reduce-scatter adds in FP32 and rounds nothing, and the sharded update equals the
    oracle's step with FP32 gradients on the summed gradients, bit for bit."""
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_f32_worker, args=(world, _free_port(), str(tmp_path), mode, use_master), nprocs=world, join=True)
    outs = []
    for r in range(world):
        zf = np.load(tmp_path / f"f32rank{r}.npz")
        outs.append({k: (zf[k] if zf[k].ndim else zf[k].item()) for k in zf.files})
    total, p, m, v, grads = _f32_grads(O, world)
    S = outs[0]["S"]
    acc = grads[0].copy()
    for g in grads[1:]:
        acc = (acc + g).astype(np.float32)            # FP32 adds in rank order
    g_sum = np.zeros(total, np.float32)
    for o in outs:
        lo, hi = o["lo"], min(o["lo"] + S, total)
        g_sum[lo:hi] = o["g"][lo:hi]
    if mode == 1 or world <= 2:
        assert np.array_equal(g_sum.view(np.uint32), acc.view(np.uint32)), "reduced gradients are not the rank-order FP32 sum"
    else:
        assert np.all(np.abs(g_sum - acc) <= 4e-7 * np.sum([np.abs(g) for g in grads], axis=0) + 1e-30)
    master = O.h2f(p)
    entries, off = [], 0
    for n, wd, fl in SEGS:
        e = dict(p=p[off:off + n], g=g_sum[off:off + n], m=m[off:off + n], v=v[off:off + n], wd=wd, flags=fl,
                 dtype=O.F16, grad_dtype=O.GRAD_F32)
        if use_master:
            e["master"] = master[off:off + n]
        entries.append(e)
        off += n
    ts = O.make_tensors(entries)
    want = O.gradstat(ts, 1.0 / world, MAX_NORM)
    got = pkg.Stat.from_buffer_copy(outs[0]["stat"].tobytes())
    assert got.found_inf == 0 and got.clip_active == want.clip_active == 1
    assert abs(got.norm - want.norm) <= 1e-5 * want.norm
    O.multi_step(ts, O.HParams(LR, B1, B2, EPS, O.bias_correction(B1, T), O.bias_correction(B2, T)),
                 O.gradstat_finalize(got.sum_sq, 0, 1.0 / world, MAX_NORM), O.STEP_ROUND_CLIP_FP16)
    for r, o in enumerate(outs):
        assert np.array_equal(o["p"][:total], p), f"rank {r}: parameters after all-gather differ"
        lo, hi = o["lo"], min(o["lo"] + S, total)
        assert np.array_equal(o["m"][:hi - lo], m[lo:hi]) and np.array_equal(o["v"][:hi - lo], v[lo:hi])
        if use_master:
            assert np.array_equal(o["master"][:hi - lo], master[lo:hi])
