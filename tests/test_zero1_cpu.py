"""ZeRO-1 host logic without a GPU: the shard geometry computed by the library
(rlcu_zero1_make_plan / rlcu_zero1_plan_pieces are pure host arithmetic) and the step
protocol run by two gloo ranks on the CPU, with the oracle standing in for the kernels.
The contract (configuration 3 of the benchmark specification): the sharded result equals the single-rank step on the
averaged gradients."""
import os
import socket

import numpy as np
import pytest

CASES = [
    [(440_401_920, 0.01, 0), (155_582_464, 0.0, 0), (65_536, 0.0, 0)],
    [(1, 0.0, 0)],
    [(1023, 0.1, 0), (1, 0.0, 0), (0, 0.5, 0), (4097, 0.0, 2)],
    [(3000, 0.01, 0), (5000, 0.0, 0), (100_000, 0.02, 0), (77, 0.0, 0)],
]


@pytest.mark.parametrize("segments", CASES)
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_shards_partition_the_element_space(pkg, segments, world):
    total = sum(s[0] for s in segments)
    covered = 0
    plans = [pkg.zero1_plan(segments, r, world) for r in range(world)]
    shard = plans[0].shard_elems
    assert shard % 1024 == 0 and shard * world >= total and (shard - 1024) * world < max(total, 1)
    seg_of = []
    begin = 0
    for n, wd, fl in segments:
        seg_of.append((begin, begin + n, wd, fl))
        begin += n
    for r, plan in enumerate(plans):
        assert (plan.total, plan.shard_elems, plan.padded_elems) == (total, shard, shard * world)
        assert plan.lo == min(r * shard, total) and plan.hi == min((r + 1) * shard, total)
        pieces = pkg.zero1_pieces(segments, r, world)
        assert len(pieces) == plan.pieces
        pos = plan.lo
        for off, state_off, n, wd, fl in pieces:
            assert n > 0 and off >= pos            # in order, no overlap
            assert state_off == off - r * shard    # state arrays start at the shard's first element
            owner = [s for s in seg_of if s[0] <= off and off + n <= s[1]]
            assert len(owner) == 1, "a piece never spans two segments"
            assert np.float32(owner[0][2]) == np.float32(wd) and owner[0][3] == fl
            pos = off + n
            covered += n
        assert pos <= plan.hi
    assert covered == total                        # every element owned exactly once


def test_bad_geometry_is_rejected(pkg):
    with pytest.raises(pkg.RlcuError):
        pkg.zero1_plan([(10, 0.0, 0)], 2, 2)
    with pytest.raises(pkg.RlcuError):
        pkg.zero1_plan([(10, 0.0, 0)], 0, 0)
    with pytest.raises(pkg.RlcuError):
        pkg.zero1_plan([(10, 0.0, 1)], 0, 1)       # NORM_ONLY is not a pool segment flag


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


SEGS = [(70_000, 0.01, 0), (30_011, 0.0, 0), (5_000, 0.02, 0)]


def _rank_inputs(O, world):
    """Same parameters on every rank, one seeded gradient replica per rank."""
    total = sum(s[0] for s in SEGS)
    rng = np.random.default_rng(100)
    p = O.f2h(rng.standard_normal(total).astype(np.float32) * np.float32(0.02))
    m = (rng.standard_normal(total) * 1e-3).astype(np.float32)
    v = (rng.random(total) * 1e-5).astype(np.float32)
    grads = [O.f2h(np.random.default_rng([101, r]).standard_normal(total).astype(np.float32) * np.float32(2e-2))
             for r in range(world)]
    return total, p, m, v, grads


def padded_elems(pkg, world):
    return int(pkg.zero1_plan(SEGS, 0, world).padded_elems)


def _worker(rank, world, port, out_dir):
    import sys
    import torch
    import torch.distributed as dist
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    import __graft_entry__ as entry
    from oracle import oracle as O
    pkg = entry.load_package()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    total, p, m, v, grads = _rank_inputs(O, world)
    plan = pkg.zero1_plan(SEGS, rank, world)
    S = int(plan.shard_elems)
    pad = int(plan.padded_elems) - total
    p_pool = np.concatenate([p, np.zeros(pad, np.uint16)])
    g_pool = np.concatenate([grads[rank], np.zeros(pad, np.uint16)])

    # reduce-scatter (sum): FP32 sum in rank order rounded once to FP16 (with two ranks this is
    # also what a single FP16 addition gives)
    parts32 = [torch.empty(padded_elems(pkg, world), dtype=torch.float32) for _ in range(world)]
    dist.all_gather(parts32, torch.from_numpy(O.h2f(g_pool)))
    acc = parts32[0].numpy().copy()
    for q in parts32[1:]:
        acc = acc + q.numpy()
    g_sum = O.f2h(acc)
    lo = rank * S
    g_pool[lo:lo + S] = g_sum[lo:lo + S]

    # statistics on the shard, all-reduce of one double, finalize with 1/world folded in
    m_shard = np.concatenate([m, np.zeros(pad, np.float32)])[lo:lo + S].copy()
    v_shard = np.concatenate([v, np.zeros(pad, np.float32)])[lo:lo + S].copy()
    entries = []
    for off, soff, n, wd, fl in pkg.zero1_pieces(SEGS, rank, world):
        entries.append(dict(p=p_pool[off:off + n], g=g_pool[off:off + n], m=m_shard[soff:soff + n],
                            v=v_shard[soff:soff + n], wd=wd, flags=fl))
    ts = O.make_tensors(entries)
    unscale, max_norm = 1.0 / world, 1.0
    part = O.gradstat(ts, unscale, 0.0)
    s = torch.tensor([part.sum_sq], dtype=torch.float64)
    dist.all_reduce(s)
    stat = O.gradstat_finalize(float(s[0]), 0, unscale, max_norm)
    hp = O.HParams(1e-3, 0.9, 0.999, 1e-8, O.bias_correction(0.9, 3), O.bias_correction(0.999, 3))
    O.multi_step(ts, hp, stat, O.STEP_ROUND_CLIP_FP16)

    # all-gather of the updated parameter shards
    mine = torch.from_numpy(p_pool[lo:lo + S].view(np.uint8).copy())      # raw bytes: gloo has no 16-bit types
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    full = np.concatenate([x.numpy().view(np.uint16) for x in parts])[:total]
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), p=full, m=m_shard, v=v_shard,
             norm=np.float32(stat.norm), clip=stat.clip_active, lo=lo, S=S)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_ranks_equal_single_rank_on_averaged_gradients(pkg, O, tmp_path, world):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)

    total, p, m, v, grads = _rank_inputs(O, world)
    acc = O.h2f(grads[0]).copy()
    for g in grads[1:]:
        acc = acc + O.h2f(g)
    g_sum = O.f2h(acc)
    entries, off = [], 0
    for n, wd, fl in SEGS:
        entries.append(dict(p=p[off:off + n], g=g_sum[off:off + n], m=m[off:off + n], v=v[off:off + n], wd=wd, flags=fl))
        off += n
    ts = O.make_tensors(entries)
    stat = O.gradstat(ts, 1.0 / world, 1.0)
    assert stat.clip_active == 1
    hp = O.HParams(1e-3, 0.9, 0.999, 1e-8, O.bias_correction(0.9, 3), O.bias_correction(0.999, 3))
    O.multi_step(ts, hp, stat, O.STEP_ROUND_CLIP_FP16)

    outs = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    for r, o in enumerate(outs):
        assert abs(float(o["norm"]) - stat.norm) <= 1e-6 * stat.norm and int(o["clip"]) == 1
        assert np.array_equal(o["p"], p), f"rank {r}: gathered parameters differ from the single-rank step"
        lo, S = int(o["lo"]), int(o["S"])
        hi = min(lo + S, total)
        assert np.array_equal(o["m"][:hi - lo], m[lo:hi]) and np.array_equal(o["v"][:hi - lo], v[lo:hi])
    for o in outs[1:]:
        assert np.array_equal(outs[0]["p"], o["p"])
