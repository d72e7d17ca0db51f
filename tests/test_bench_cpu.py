"""bench.py's reference arm (the CPU restatement timed on the host cores) runs without a GPU
and prints one JSON line with the agreed keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    env = dict(os.environ, RLCU_BENCH_SAMPLE=str(1 << 20))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2",
                        "--warmup", "3"], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "params/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "params/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["steps"] == 2 and line["warmup"] == 3 and line["higher_is_better"] is True
    # the same `config` object the GPU arm of the same command prints
    sys.path.insert(0, ROOT)
    import argparse
    import bench
    want = bench.config_for(argparse.Namespace(workload="qwen3-0.6b", gpus=1))
    assert line["config"] == want and want["params"] == 596_049_920 and want["tensors"] == 310
    assert line["scaling"] == "strong"


def test_reference_arm_other_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", RLCU_BENCH_SAMPLE=str(1 << 20))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_pool_hash_sees_single_bit_and_order_changes():
    """The hash the sharded arm all-reduces (MIN and MAX) to check that every rank holds the same
    parameter pool: equal pools give equal hashes, one flipped bit or two swapped words do not."""
    import torch
    sys.path.insert(0, ROOT)
    import bench
    g = torch.Generator().manual_seed(0)
    a = torch.randint(-30000, 30000, (1 << 18,), generator=g, dtype=torch.int16)
    h = bench.pool_hash(torch, a)
    assert torch.equal(h, bench.pool_hash(torch, a.clone()))
    b = a.clone()
    b[12345] ^= 1
    assert not torch.equal(h, bench.pool_hash(torch, b))
    c = a.clone().view(torch.int64)
    c[[7, 9000]] = c[[9000, 7]]
    assert not torch.equal(h, bench.pool_hash(torch, c.view(torch.int16)))
