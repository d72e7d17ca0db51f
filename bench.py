"""Benchmark of the optimizer step (statistics pass + multi-tensor AdamW update).

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

N = 1   : Qwen3-0.6B-shaped parameter set (596,049,920 FP16 parameters in 310 tensors,
          FP32 moments warmed by 5 prior steps, global-norm clip at 1.0, lr 1e-6) updated
          on one GPU.  One step = one statistics launch + one update launch.
N > 1   : the same parameter set with the FP32 moments partitioned ZeRO-1 style over the N
          ranks (launched by torch.distributed.run, one rank per GPU): reduce-scatter of the
          FP16 gradients, sharded statistics + update, all-gather of the FP16 parameters,
          by fused peer-to-peer kernels (default) or NCCL.  Total work is fixed ("strong"
          scaling).  After the timed region one more step is run from known gradients and
          checked (`parity` in the JSON line); a mismatch ends the run with a non-zero status.

Rank 0 prints one JSON line.  `value` is parameters updated per second with everything
resident in HBM; `e2e` is the same step driven from host memory (the step's FP16 gradients
copied from pinned host memory, the statistics record read back, both inside the timed
region); `roofline` is the update kernel's algorithmic bytes (22 per parameter) over its
CUDA-event time against the measured HBM copy bandwidth; `cpu_baseline` is the CPU
restatement of the reference algorithm timed on this machine's cores.

`--impl reference` times that CPU restatement (all host threads) instead of the GPU path.
Data are synthetic (seeded normal values with the shapes above); no checkpoint is read.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

BYTES_PER_PARAM = 22          # read p,g (2+2) m,v (4+4); write p (2) m,v (4+4)
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 * 1024 * 1024
L2_NOTE = "every step streams its whole working set (12 bytes per parameter or more), far larger than the 126 MB L2; no flush needed"


def ncu_dram_bytes_per_param(kernel="adamw_table_kernel"):
    """DRAM bytes per parameter that ncu measured for `kernel` (profiles/dram_traffic.json, kept
    next to the capture's summary), or None when no capture of it is on file."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            return float(json.load(f)[kernel]["bytes_per_param"])
    except Exception:
        return None


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def shapes_for(workload):
    from helpers import qwen3_0p6b, qwen3_8b
    if workload == "qwen3-0.6b":
        return qwen3_0p6b()
    if workload == "qwen3-8b":
        return qwen3_8b()
    if workload == "qwen3-0.6b-4l":     # 4 of the 28 layers + embedding: the profiler-sized case
        from helpers import qwen3_shapes
        return qwen3_shapes(1024, 3072, 4, 151936, 16, 8, 128, tied=True)
    if workload in ("ragged-20k", "ragged-600"):   # sizes log-uniform in [64, 4,194,304], seed 0
        import numpy as np
        rng = np.random.default_rng(0)
        count = 20_000 if workload == "ragged-20k" else 600        # 600: the profiler-sized cut
        sizes = np.floor(np.exp(rng.uniform(np.log(64), np.log(4_194_304), count))).astype(np.int64)
        return [(f"t{k}", int(n), True) for k, n in enumerate(sizes)]
    raise SystemExit(f"unknown workload {workload}")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def report(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "note": "NVML unavailable"}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def build_pools(torch, shapes, dev, seed, align=8):
    """Flat pools in RL.cu's order with one descriptor per tensor, every tensor starting on a
    16-byte boundary (a no-op for the Qwen3 shapes, padding for ragged ones).  FP16 params
    ~N(0,0.02) with norm weights 1.0, FP16 grads ~N(0,1e-4), FP32 moments zero."""
    params = sum(n for _, n, _ in shapes)
    pad = lambda n: (n + align - 1) // align * align
    total = sum(pad(n) for _, n, _ in shapes)
    gen = torch.Generator(device=dev).manual_seed(seed)
    p = torch.empty(total, dtype=torch.float16, device=dev)
    g = torch.empty(total, dtype=torch.float16, device=dev)
    step = 1 << 26
    for lo in range(0, total, step):
        hi = min(total, lo + step)
        p[lo:hi] = (torch.randn(hi - lo, device=dev, generator=gen) * 0.02).half()
        g[lo:hi] = (torch.randn(hi - lo, device=dev, generator=gen) * 1e-4).half()
    off = 0
    for name, n, _ in shapes:
        if "norm" in name:
            p[off:off + n] = 1.0
        off += pad(n)
    m = torch.zeros(total, dtype=torch.float32, device=dev)
    v = torch.zeros(total, dtype=torch.float32, device=dev)
    return dict(p=p, g=g, m=m, v=v, total=params, arena=total)


def fresh_grads(torch, g, gen):
    step = 1 << 26
    for lo in range(0, g.numel(), step):
        hi = min(g.numel(), lo + step)
        g[lo:hi] = (torch.randn(hi - lo, device=g.device, generator=gen) * 1e-4).half()


def make_descs(pkg, pools, shapes, wd, align=8):
    descs, off = [], 0
    for _, n, decays in shapes:
        descs.append(pkg.TensorDesc(pools["p"].data_ptr() + 2 * off, pools["g"].data_ptr() + 2 * off,
                                    pools["m"].data_ptr() + 4 * off, pools["v"].data_ptr() + 4 * off,
                                    None, n, wd if decays else 0.0, pkg.F16, 0, 0))
        off += (n + align - 1) // align * align
    return descs


# ----------------------------------------------------------------------------------------
# CPU restatement of the reference (the reported baseline and the `--impl reference` arm)
# ----------------------------------------------------------------------------------------

def cpu_port_step_rate(sample_params, steps, warmup, threads=0):
    """Times gradient statistics + clip + AdamW of the CPU oracle on `sample_params` parameters
    of the workload (one FP16 tensor with the workload's value distributions)."""
    import numpy as np
    from oracle import oracle as O
    rng = np.random.default_rng(0)
    n = sample_params
    p, g = np.empty(n, np.uint16), np.empty(n, np.uint16)
    g_std = np.float32(1e-4 * (596_049_920 / n) ** 0.5)      # keeps the norm, and so the clip, as in the full set
    for lo in range(0, n, 1 << 25):
        hi = min(n, lo + (1 << 25))
        p[lo:hi] = O.f2h(rng.standard_normal(hi - lo, dtype=np.float32) * np.float32(0.02))
        g[lo:hi] = O.f2h(rng.standard_normal(hi - lo, dtype=np.float32) * g_std)
    e = dict(p=p, g=g, m=np.zeros(n, np.float32), v=np.zeros(n, np.float32), wd=0.01)
    ts = O.make_tensors([e])
    # an explicit thread count: launchers such as torch.distributed.run export OMP_NUM_THREADS=1
    if threads == 0:
        threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    cores = threads
    times = []
    for i in range(warmup + steps):
        t = 6 + i
        hp = O.HParams(1e-6, 0.9, 0.999, 1e-8, O.bias_correction(0.9, t), O.bias_correction(0.999, t))
        t0 = time.perf_counter()
        st = O.gradstat(ts, 1.0, 1.0, threads=threads)
        O.multi_step(ts, hp, st, O.STEP_ROUND_CLIP_FP16, O.NVCC, threads)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    return n / (sum(times) / len(times)), sum(times) / len(times), cores


def workload_params(workload):
    return sum(n for _, n, _ in shapes_for(workload))


def config_for(args):
    """The `config` object, identical in the GPU arm and in the reference arm of one command."""
    shapes = shapes_for(args.workload)
    return {"workload": workload_name(args), "params": sum(n for _, n, _ in shapes), "tensors": len(shapes),
            "l2": L2_NOTE}


def run_reference_arm(args):
    """The reference's algorithm on this machine's host cores: the CPU restatement (statistics +
    clip + update) with OpenMP over all host threads.  One step covers the whole parameter set
    of the workload unless RLCU_BENCH_SAMPLE bounds it (the 8 B-parameter sets are sampled)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    P = workload_params(args.workload)
    sample = int(os.environ.get("RLCU_BENCH_SAMPLE", min(P, 1 << 30)))     # parameters per timed step
    rate, sec, cores = cpu_port_step_rate(sample, args.steps, args.warmup, threads=0)
    whole = sample == P
    line = {
        "impl": "reference", "metric": "adamw_params_per_sec", "value": rate, "unit": "params/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3 * (P / sample),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "storage": "f16 params and grads, f32 moments", "data": "synthetic",
        "config": config_for(args),
        "cpu_baseline": {"value": rate, "unit": "params/s", "cores": cores, "kind": "port",
                         "sample": (f"the whole workload, {sample} parameters per step" if whole else
                                    f"{sample} of the workload's {P} parameters per step, rate extrapolated") +
                                   " (statistics + clip + update), OpenMP over all host threads, "
                                   f"half conversions by {'F16C instructions' if O.hw_half_available() else 'bit arithmetic'}"},
        "e2e": {"value": rate, "unit": "params/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_name(args):
    base = {"ragged-600": "600 FP16 tensors with log-uniform sizes in [64, 4,194,304] (profiling cut of ragged-20k), clip 1.0",
            "ragged-20k": "20,000 FP16 tensors with log-uniform sizes in [64, 4,194,304] (7,544,329,889 params), clip 1.0",
            "qwen3-0.6b-4l": "Qwen3-0.6B shapes cut to 4 layers + embedding (profiling case), clip 1.0",
            "qwen3-0.6b": "Qwen3-0.6B-shaped multi-tensor AdamW step, 596,049,920 params in 310 tensors, clip 1.0",
            "qwen3-8b": "Qwen3-8B-shaped multi-tensor AdamW step, 8,190,735,360 params in 399 tensors, clip 1.0"}[args.workload]
    if args.gpus > 1:
        base += f", ZeRO-1 over {args.gpus} GPUs (reduce-scatter grads, sharded update, all-gather params)"
    return base


# ----------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------

def mean_launch_ms(torch, fn, reps=20, warm=3):
    """Mean CUDA-event time of `fn` (which enqueues on torch's current stream) over `reps` calls."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    for a, b in ev:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return statistics.mean(a.elapsed_time(b) for a, b in ev)


def time_variants(torch, pkg, pools, shapes, wd, hp, stat, stream, peak, only=""):
    """The other forms of the update a caller can ask for, each with its own algorithmic bytes
    and fraction of the measured HBM bandwidth: what RL.cu itself would run (FP32 master copy:
    28 bytes per parameter, through the multi-tensor list and through its own three launches
    per step), the bulk-copy kernel, and FP32 gradients for FP16 parameters."""
    P, arena = pools["total"], pools["arena"]
    out = {}
    want = lambda name: not only or name in only.split(",")

    def entry(ms, bytes_per_param, params, what, launches, ncu_key=None):
        gbs = bytes_per_param * params / (ms * 1e-3) / 1e9
        e = {"ms": ms, "bytes_per_param": bytes_per_param, "params": params, "launches_per_step": launches,
             "achieved_gbs": gbs, "frac_of_measured": gbs / peak, "what": what}
        per_param = ncu_dram_bytes_per_param(ncu_key) if ncu_key else None
        if per_param is not None:
            e["traffic"] = per_param * params          # DRAM bytes per step, from the ncu capture of this kernel
        return e

    def descs(master=None, g32=None, align=8):
        d, off = [], 0
        for _, n, decays in shapes:
            d.append(pkg.TensorDesc(pools["p"].data_ptr() + 2 * off,
                                    (g32.data_ptr() + 4 * off) if g32 is not None else (pools["g"].data_ptr() + 2 * off),
                                    pools["m"].data_ptr() + 4 * off, pools["v"].data_ptr() + 4 * off,
                                    (master.data_ptr() + 4 * off) if master is not None else None,
                                    n, wd if decays else 0.0, pkg.F16, 0,
                                    pkg.GRAD_F32 if g32 is not None else pkg.GRAD_AS_PARAM))
            off += (n + align - 1) // align * align
        return d

    master = pools["p"].float()
    # (i) the multi-tensor kernel with an FP32 master copy
    if want("multi_tensor_fp32_master") or want("bulk_copy_fp32_master"):
        tl = pkg.TensorList(descs(master=master))
        ms = mean_launch_ms(torch, lambda: tl.step(hp, stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16, stream=stream))
        out["multi_tensor_fp32_master"] = entry(ms, 28, P, "the kernel rlcu_adamw_multi_step picks for this list (adamw_table_bulk_kernel), "
                                                "FP16 weights written from an FP32 master (read master,g,m,v; write master,p,m,v)",
                                                1, "adamw_table_bulk_kernel_fp32_master")
        ms = mean_launch_ms(torch, lambda: tl.step(hp, stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16 | pkg.STEP_DIRECT, stream=stream))
        out["direct_fp32_master"] = entry(ms, 28, P, "adamw_table_kernel (per-thread loads and stores) forced on the same list", 1)
        ms = mean_launch_ms(torch, lambda: tl.step(hp, stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16 | pkg.STEP_BULK_COPY, stream=stream))
        tl.check()
        out["bulk_copy_fp32_master"] = entry(ms, 28, P, "adamw_table_bulk_kernel with an FP32 master", 1)
        tl.close()
    # (ii) RL.cu's own call sequence through the drop-in launchers: projections, embedding, norms
    if want("reference_layout_three_launches") and any(name == "embed" for name, _, _ in shapes):
        # RL.cu's pools: projections (weight decay), then the embedding, and the norm weights in FP32
        # (Qwen3-0.6B: 440,401,920 + 155,582,464 FP16 elements and 65,536 FP32 ones)
        n_proj = sum(n for name, n, decays in shapes if decays)
        n_embed = sum(n for name, n, _ in shapes if name == "embed")
        n32 = sum(n for name, n, _ in shapes if "norm" in name)
        w32, g32n, m32, v32 = (torch.zeros(n32, device=master.device) for _ in range(4))
        a = (hp.lr, hp.beta1, hp.beta2, hp.eps)
        bc = (hp.bias_correction1, hp.bias_correction2)

        def three_launches():
            pkg.adamw_fp16_master(master.data_ptr(), pools["p"].data_ptr(), pools["g"].data_ptr(), pools["m"].data_ptr(),
                                  pools["v"].data_ptr(), n_proj, *a, wd, *bc, stream)
            pkg.adamw_fp16_master(master.data_ptr() + 4 * n_proj, pools["p"].data_ptr() + 2 * n_proj,
                                  pools["g"].data_ptr() + 2 * n_proj, pools["m"].data_ptr() + 4 * n_proj,
                                  pools["v"].data_ptr() + 4 * n_proj, n_embed, *a, 0.0, *bc, stream)
            pkg.adamw_fp32(w32.data_ptr(), g32n.data_ptr(), m32.data_ptr(), v32.data_ptr(), n32, *a, 0.0, *bc, stream)

        ms = mean_launch_ms(torch, three_launches)
        out["reference_layout_three_launches"] = entry(
            ms, 28, n_proj + n_embed + n32,
            f"adamw_flat_bulk_kernel behind launch_adamw_fp16 x2 ({n_proj} + {n_embed} elements) and "
            f"launch_adamw_fp32 ({n32}), as AdamWOptimizer::step issues them", 3, "adamw_flat_bulk_kernel")
    # (iii) the bulk-copy (cp.async.bulk) form of the multi-tensor kernel
    if want("bulk_copy"):
        tl = pkg.TensorList(descs())
        ms = mean_launch_ms(torch, lambda: tl.step(hp, stat.data_ptr(), pkg.STEP_ROUND_CLIP_FP16 | pkg.STEP_BULK_COPY, stream=stream))
        tl.check()
        out["bulk_copy"] = entry(ms, 22, P, "adamw_table_bulk_kernel: the same update with its traffic issued by cp.async.bulk", 1)
        tl.close()
    if not want("fp32_gradients"):
        return out
    # (iv) FP32 gradients for the FP16 parameters
    g32 = pools["g"].float()
    tl = pkg.TensorList(descs(g32=g32))
    ms = mean_launch_ms(torch, lambda: tl.step(hp, stat.data_ptr(), 0, stream=stream))
    out["fp32_gradients"] = entry(ms, 24, P, "adamw_table_kernel with FP32 gradients (read p 2, g 4, m 4, v 4; write p 2, m 4, v 4)", 1)
    ms = mean_launch_ms(torch, lambda: tl.gradstat(stat.data_ptr(), 1.0, 1.0, stream=stream))
    out["fp32_gradients_statistics"] = entry(ms, 4, P, "gradstat_kernel over FP32 gradients", 1)
    tl.close()
    tl = pkg.TensorList(descs(master=master, g32=g32))
    ms = mean_launch_ms(torch, lambda: tl.step(hp, stat.data_ptr(), 0, stream=stream))
    out["fp32_gradients_fp32_master"] = entry(ms, 30, P, "adamw_table_kernel with FP32 gradients and an FP32 master", 1)
    tl.close()
    return out


def run_single(args):
    import numpy as np
    import torch
    import __graft_entry__ as entry
    pkg = entry.load_package()
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    shapes = shapes_for(args.workload)
    pools = build_pools(torch, shapes, dev, seed=0, align=args.align)
    P = pools["total"]
    lr, b1, b2, eps, wd, max_norm = 1e-6, 0.9, 0.999, 1e-8, 0.01, 1.0
    tl = pkg.TensorList(make_descs(pkg, pools, shapes, wd, align=args.align))
    stat = torch.zeros(16, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    flags = pkg.STEP_ROUND_CLIP_FP16 | (pkg.STEP_BULK_COPY if args.bulk else 0)

    def step(t):
        tl.gradstat(stat.data_ptr(), 1.0, max_norm, stream=stream)
        tl.step(pkg.hparams(lr, b1, b2, eps, t), stat.data_ptr(), flags, stream=stream)

    # moments warmed by five prior steps on fresh gradients (untimed)
    gen = torch.Generator(device=dev).manual_seed(1)
    for t in range(1, 6):
        fresh_grads(torch, pools["g"], gen)
        step(t)
    fresh_grads(torch, pools["g"], gen)
    torch.cuda.synchronize()

    t = 6
    for _ in range(args.warmup):
        step(t)
        t += 1
    torch.cuda.synchronize()

    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    with ClockSampler(0) as clocks:
        torch.cuda.synchronize()
        for k in range(K):
            ev[k][0].record()
            tl.gradstat(stat.data_ptr(), 1.0, max_norm, stream=stream)
            ev[k][1].record()
            tl.step(pkg.hparams(lr, b1, b2, eps, t), stat.data_ptr(), flags, stream=stream)
            ev[k][2].record()
            t += 1
        torch.cuda.synchronize()
    total_ms = ev[0][0].elapsed_time(ev[K - 1][2])
    stat_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    upd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    ms_per_step = total_ms / K
    value = P / (ms_per_step * 1e-3)
    final = pkg.Stat.from_buffer_copy(stat.cpu().numpy().tobytes())

    if args.quick:
        quick = {"metric": "adamw_params_per_sec", "value": value, "unit": "params/s", "n_gpus": 1,
                 "steps": K, "warmup": args.warmup, "ms_per_step": ms_per_step,
                 "kernels_ms": {"gradstat_kernel": stat_ms, "adamw_table_kernel": upd_ms},
                 "config": config_for(args), "quick": True}
        if args.variants:
            quick["variants"] = time_variants(torch, pkg, pools, shapes, wd, pkg.hparams(lr, b1, b2, eps, t), stat, stream,
                                              measured_peak()[0], only=args.variants)
        print(json.dumps(quick), flush=True)
        return

    # ---- end to end from host memory: H2D of the step's gradients, step, D2H of the record
    host_g = torch.empty(pools["g"].numel(), dtype=torch.float16).pin_memory()
    host_g.copy_(pools["g"])
    host_stat = torch.empty(16, dtype=torch.float32).pin_memory()
    e2e_steps = max(3, min(K, 20))

    def e2e_step(tt):
        pools["g"].copy_(host_g, non_blocking=True)
        tl.gradstat(stat.data_ptr(), 1.0, max_norm, stream=stream)
        tl.step(pkg.hparams(lr, b1, b2, eps, tt), stat.data_ptr(), flags, stream=stream)
        host_stat.copy_(stat, non_blocking=True)

    for _ in range(2):
        e2e_step(t)
        t += 1
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step(t)
        t += 1
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    assert pkg.Stat.from_buffer_copy(host_stat.numpy().tobytes()).found_inf == 0

    # ---- the reference's own CUDA kernels on the same GPU (when they were built): context only
    ref_cuda = None
    try:
        from oracle import oracle as O
        if O.ref_available() and P < 2 ** 31:
            ref_cuda = time_reference_cuda(torch, O, pools, shapes, lr, b1, b2, eps, wd, max_norm)
    except Exception as exc:   # the checker is optional here
        ref_cuda = {"unavailable": str(exc)[:120]}

    peak, peak_kind = measured_peak()
    achieved = BYTES_PER_PARAM * P / (upd_ms * 1e-3) / 1e9
    # DRAM bytes per launch: bytes per parameter measured with ncu (dram__bytes_read.sum +
    # dram__bytes_write.sum) on a 218,507,264-parameter cut of this workload, read from the
    # file kept beside that capture's summary and scaled by the element count of this launch.
    per_param = ncu_dram_bytes_per_param("adamw_table_kernel" if not args.bulk else "adamw_table_bulk_kernel")
    traffic = per_param * P if per_param is not None else None

    variants = None
    if not args.bulk and args.workload in ("qwen3-0.6b", "qwen3-0.6b-4l"):
        variants = time_variants(torch, pkg, pools, shapes, wd, pkg.hparams(lr, b1, b2, eps, t), stat, stream, peak)
        variants["statistics"] = {"ms": stat_ms, "bytes_per_param": 2, "params": P, "launches_per_step": 1,
                                  "achieved_gbs": 2 * P / (stat_ms * 1e-3) / 1e9,
                                  "frac_of_measured": 2 * P / (stat_ms * 1e-3) / 1e9 / peak,
                                  "what": "gradstat_kernel of the timed step (FP16 gradients read once)"}

    # ---- CPU restatement on this machine's cores (bounded sample)
    cpu_sample, cpu_steps = min(P, 1 << 27), 5
    cpu_rate, cpu_sec, cores = cpu_port_step_rate(cpu_sample, cpu_steps, 1, threads=0)
    cpu_rate_1t, _, _ = cpu_port_step_rate(1 << 24, 3, 1, threads=1)

    line = {
        "metric": "adamw_params_per_sec", "value": value, "unit": "params/s", "n_gpus": 1,
        "steps": K, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "storage": "f16 params and grads, f32 moments",
        "data": "synthetic",
        "config": config_for(args),
        "run_info": {"launches_per_step": 2, "grad_norm": final.norm, "clip_active": int(final.clip_active)},
        "kernels_ms": {"gradstat_kernel": stat_ms, "adamw_table_kernel": upd_ms},
        "hbm_gbs_whole_step": (BYTES_PER_PARAM + 2) * P / (ms_per_step * 1e-3) / 1e9,
        "roofline": {"bound": "hbm", "kernel": "adamw_table_kernel", "achieved": achieved, "peak": peak,
                     "peak_kind": f"{peak_kind} copy bandwidth", "unit": "GB/s", "frac": achieved / peak,
                     "frac_of_nominal_8000": achieved / 8000.0, "traffic": traffic,
                     "algorithmic_bytes_per_launch": BYTES_PER_PARAM * P},
        "e2e": {"value": P / (e2e_ms * 1e-3), "unit": "params/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": 2 * P, "d2h_bytes_per_step": 64,
                "what": "pinned-host FP16 gradients copied in, statistics + update, statistics record copied out"},
        "gpu_launches": 2 * K,
        "clocks": clocks.report(),
        "cpu_baseline": {"value": cpu_rate, "unit": "params/s", "cores": cores, "kind": "port",
                         "single_thread_value": cpu_rate_1t,
                         "sample": f"{cpu_sample} parameters per step, {cpu_steps} steps, statistics + clip + update, "
                                   f"OpenMP over all host threads; single thread on {1 << 24} parameters"},
    }
    if variants is not None:
        line["variants"] = variants
    if ref_cuda is not None:
        line["reference_cuda_same_gpu"] = ref_cuda
    print(json.dumps(line), flush=True)


def time_reference_cuda(torch, O, pools, shapes, lr, b1, b2, eps, wd, max_norm):
    """RL.cu's own sequence (sum of squares, read-back, scale, launch_adamw_fp16 with FP32
    master) on the same FP16 pools, timed with CUDA events.  28 bytes per parameter in the
    update plus the read-back stall; shown beside the new path for context."""
    R = O.ref_lib()
    P = pools["total"]
    master = pools["p"].float()
    p, m, v = pools["p"].clone(), pools["m"].clone(), pools["v"].clone()
    g0 = pools["g"]
    g = g0.clone()
    acc = torch.zeros(1, device=g.device)
    norm = C.c_float()
    bc1, bc2 = O.bias_correction(b1, 7), O.bias_correction(b2, 7)

    def step():
        g.copy_(g0)       # the reference scales gradients in place; restore (untimed below)
    times = []
    for i in range(8):
        step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        R.ref_clip_grad_norm(g.data_ptr(), P, None, 0, max_norm, acc.data_ptr(), C.byref(norm))
        R.ref_launch_adamw_fp16(master.data_ptr(), p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
                                P, lr, b1, b2, eps, wd, bc1, bc2, None)
        e1.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(e0.elapsed_time(e1))
    ms = statistics.mean(times)
    return {"ms_per_step": ms, "value": P / (ms * 1e-3), "unit": "params/s",
            "what": "RL.cu kernels rebuilt for sm_100a: sum_sq + D2H + scale + launch_adamw_fp16 (FP32 master)"}


def pool_hash(torch, pool):
    """Two 64-bit sums over the pool's bytes taken as int64 words (plain, and weighted by the
    word's position): equal on two GPUs only if the pools are equal, for any practical purpose."""
    words = pool.view(torch.int64)
    h1 = torch.zeros((), dtype=torch.int64, device=pool.device)
    h2 = torch.zeros((), dtype=torch.int64, device=pool.device)
    step = 1 << 24
    for lo in range(0, words.numel(), step):
        w = words[lo:lo + step]
        h1 += w.sum()
        h2 += (w * (torch.arange(lo, lo + w.numel(), device=pool.device, dtype=torch.int64) * 2 + 1)).sum()
    return torch.stack([h1, h2])


def checked_step(torch, dist, pkg, z, mode, rank, world, segments, P, S, p_pool, g_pool, g_fresh, m_sh, v_sh,
                 stat, hp, flags, max_norm, stream):
    """One sharded step from known gradients, outside every timed interval, compared with what
    the step is defined to equal.  Returns the `parity` object of the JSON line; `ok` false
    means the run must fail.
      ranks_agree            every rank holds the same parameter pool afterwards (64-bit hashes,
                             all-reduced MIN and MAX) and the same statistics record
      reduce_scatter         each rank's reduced gradient shard against the FP32 sum of all
                             ranks' replicas in rank order, rounded once to FP16 (peer-to-peer
                             mode: bit for bit; NCCL adds hop by hop in FP16: bounded error)
      shard_vs_single_gpu    the shard's p, m, v after the step against the single-GPU statistics
                             + update kernels run on copies of the shard, fed the reduced
                             gradients with unscale = 1/world and the step's own record
      norm_rel_err           the step's global norm against an FP64 sum over the reduced gradients"""
    dev = p_pool.device
    lo = rank * S
    hi = min(lo + S, P)
    p_before = p_pool[lo:lo + S].clone()
    m_before, v_before = m_sh.clone(), v_sh.clone()
    g_pool.copy_(g_fresh)
    torch.cuda.synchronize()
    dist.barrier()
    z.step(hp, stat.data_ptr(), 1.0, max_norm, None, flags, 0, stream)
    torch.cuda.synchronize()
    dist.barrier()
    rec = pkg.Stat.from_buffer_copy(stat.cpu().numpy().tobytes())
    out = {}

    # -- every rank holds the same parameters and the same record
    h = pool_hash(torch, p_pool)
    hmin, hmax = h.clone(), h.clone()
    dist.all_reduce(hmin, op=dist.ReduceOp.MIN)
    dist.all_reduce(hmax, op=dist.ReduceOp.MAX)
    sbits = stat.view(torch.int32).to(torch.int64)
    smin, smax = sbits.clone(), sbits.clone()
    dist.all_reduce(smin, op=dist.ReduceOp.MIN)
    dist.all_reduce(smax, op=dist.ReduceOp.MAX)
    out["ranks_agree"] = bool(torch.equal(hmin, hmax) and torch.equal(smin, smax))

    # -- the reduced gradient shard against the FP32 rank-order sum rounded once
    mine = None
    for owner in range(world):
        piece = g_fresh[owner * S:(owner + 1) * S].contiguous()
        got = [torch.empty_like(piece) for _ in range(world)] if rank == owner else None
        dist.gather(piece, got, dst=owner)
        if rank == owner:
            mine = got
    acc = mine[0].float()
    for r in range(1, world):
        acc += mine[r].float()
    want = acc.half()
    reduced = g_pool[lo:lo + S]
    if mode == pkg.ZERO1_P2P or world <= 2:
        rs_ok = bool(torch.equal(reduced.view(torch.int16), want.view(torch.int16)))
        out["reduce_scatter"] = "bit-exact vs the FP32 rank-order sum rounded once" if rs_ok else "MISMATCH"
    else:
        mag = torch.zeros_like(acc)
        for r in range(world):
            mag += mine[r].float().abs()
        bound = (world - 1) * 2.0 ** -11 * mag + 2.0 ** -24
        rs_ok = bool(((reduced.float() - acc).abs() <= bound).all())
        out["reduce_scatter"] = "within (world-1) half-ulps per hop of the FP32 sum (FP16 hop-by-hop adds)" if rs_ok else "MISMATCH"
    del mine, acc, want

    # -- the shard's update against the single-GPU kernels on copies of the shard
    p_chk, m_chk, v_chk = p_before.clone(), m_before.clone(), v_before.clone()
    descs = []
    for pool_off, state_off, n, wd, fl in pkg.zero1_pieces(segments, rank, world):
        descs.append(pkg.TensorDesc(p_chk.data_ptr() + 2 * (pool_off - lo), reduced.data_ptr() + 2 * (pool_off - lo),
                                    m_chk.data_ptr() + 4 * state_off, v_chk.data_ptr() + 4 * state_off, None,
                                    n, wd, pkg.F16, fl, 0))
    tl = pkg.TensorList(descs)
    part = torch.zeros(16, dtype=torch.float32, device=dev)
    tl.gradstat(part.data_ptr(), 1.0 / world, max_norm, flags=pkg.STAT_PARTIAL, stream=stream)
    tl.step(hp, stat.data_ptr(), flags, stream=stream)          # same record, so the same clip factor
    torch.cuda.synchronize()
    same = (torch.equal(p_chk.view(torch.int16), p_pool[lo:lo + S].view(torch.int16)) and
            torch.equal(m_chk.view(torch.int32), m_sh.view(torch.int32)) and
            torch.equal(v_chk.view(torch.int32), v_sh.view(torch.int32)))
    moved = not torch.equal(p_chk.view(torch.int16), p_before.view(torch.int16)) if hi > lo else True
    local_sum = torch.tensor([pkg.Stat.from_buffer_copy(part.cpu().numpy().tobytes()).sum_sq], dtype=torch.float64, device=dev)
    exact = (reduced[:max(hi - lo, 0)].double() / world).square().sum().reshape(1)
    both = torch.cat([local_sum, exact])
    dist.all_reduce(both)
    flag = torch.tensor([1 if (same and moved and rs_ok) else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    sum_kernels, sum_exact = float(both[0]), float(both[1])
    out["shard_vs_single_gpu"] = "bit-exact (p, m, v of every rank's shard)" if int(flag[0]) == 1 else "MISMATCH"
    out["sum_sq_rel_err_vs_single_gpu_kernels"] = abs(rec.sum_sq - sum_kernels) / sum_kernels
    out["norm_rel_err"] = abs(rec.norm - sum_exact ** 0.5) / sum_exact ** 0.5
    out["grad_norm"] = rec.norm
    out["clip_active"] = int(rec.clip_active)
    out["ok"] = bool(out["ranks_agree"] and int(flag[0]) == 1 and out["norm_rel_err"] <= 1e-5 and
                     out["sum_sq_rel_err_vs_single_gpu_kernels"] <= 1e-5 and rec.found_inf == 0)
    tl.close()
    return out


def run_sharded(args):
    """N > 1: ZeRO-1 step, one rank per GPU (launched by torch.distributed.run)."""
    import numpy as np
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg = entry.load_package()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)

    shapes = shapes_for(args.workload)
    # pool order of the sharded path: runs of equal weight decay (projections | norms ... ) --
    # one segment per tensor keeps RL.cu's per-tensor policy
    segments = [(n, 0.01 if decays else 0.0, 0) for _, n, decays in shapes]
    P = sum(n for n, _, _ in segments)
    plan = pkg.zero1_plan(segments, rank, world)
    S, padded = int(plan.shard_elems), int(plan.padded_elems)

    def rand_into(t, std, gen):
        step = 1 << 26
        for lo in range(0, P, step):
            hi = min(P, lo + step)
            t[lo:hi] = (torch.randn(hi - lo, device=dev, generator=gen) * std).half()

    p_pool = torch.zeros(padded, dtype=torch.float16, device=dev)
    g_pool = torch.zeros(padded, dtype=torch.float16, device=dev)
    g_fresh = torch.zeros(padded, dtype=torch.float16, device=dev)     # this rank's replica
    rand_into(p_pool, 0.02, torch.Generator(device=dev).manual_seed(0))        # same on every rank
    off = 0
    for name, n, _ in shapes:
        if "norm" in name:
            p_pool[off:off + n] = 1.0
        off += n
    ggen = torch.Generator(device=dev).manual_seed(1000 + rank)                # one replica per rank
    m_sh = torch.zeros(S, dtype=torch.float32, device=dev)
    v_sh = torch.zeros(S, dtype=torch.float32, device=dev)
    stat = torch.zeros(16, dtype=torch.float32, device=dev)

    def create(mode):
        box = [pkg.zero1_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return pkg.Zero1(box[0], rank, world, p_pool.data_ptr(), g_pool.data_ptr(), segments,
                         m_sh.data_ptr(), v_sh.data_ptr(), None, mode=mode)

    mode = pkg.ZERO1_P2P if args.zero1_mode == "p2p" else pkg.ZERO1_NCCL
    mode_note = None
    try:
        z = create(mode)
    except pkg.RlcuError as exc:
        # Peer mapping needs pools that came from cudaMalloc (CUDA IPC); it fails on every rank
        # alike, e.g. under an allocator that uses virtual-memory segments.  The NCCL exchange
        # still runs the same kernels and is reported as what it is.
        if mode != pkg.ZERO1_P2P:
            raise
        mode_note = f"peer-to-peer exchange unavailable ({exc}); ran the NCCL exchange"
        mode = pkg.ZERO1_NCCL
        z = create(mode)
    stream = torch.cuda.current_stream().cuda_stream
    lr, b1, b2, eps, max_norm = 1e-6, 0.9, 0.999, 1e-8, 1.0
    flags = pkg.STEP_ROUND_CLIP_FP16 | (pkg.STEP_BULK_COPY if args.bulk else 0) | (pkg.STEP_DIRECT if args.direct else 0)

    def step(t, phases=0):
        z.step(pkg.hparams(lr, b1, b2, eps, t), stat.data_ptr(), 1.0, max_norm, None, flags, phases, stream)

    # The reduce-scatter is in place, so every step needs its gradients back: the device copy
    # below stands in for the backward pass that regenerates them and is outside the timed
    # intervals.
    def restore():
        g_pool.copy_(g_fresh)

    t = 1
    for _ in range(5):                       # moments warmed by five steps on fresh gradients
        rand_into(g_fresh, 1e-4, ggen)
        restore()
        step(t)
        t += 1
    rand_into(g_fresh, 1e-4, ggen)
    for _ in range(args.warmup):
        restore()
        step(t)
        t += 1
    torch.cuda.synchronize()

    def timed(phases, steps):
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        nonlocal t
        dist.barrier()
        torch.cuda.synchronize()
        for a, b in ev:
            restore()
            a.record()
            step(t, phases)
            b.record()
            t += 1
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([sum(a.elapsed_time(b) for a, b in ev) / steps], dtype=torch.float64, device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms[0])

    K = args.steps
    with ClockSampler(local) as clocks:
        ms_per_step = timed(0, K)
    z.check()
    final = pkg.Stat.from_buffer_copy(stat.cpu().numpy().tobytes())
    ks = max(3, min(K, 10))
    if mode == pkg.ZERO1_P2P:
        phase_ms = {"reduce_scatter_statistics_fused": timed(1, ks), "allreduce_finalize": timed(2, ks),
                    "update_allgather_fused": timed(4, ks)}
    else:
        phase_ms = {"reduce_scatter": timed(1, ks), "statistics_allreduce": timed(2, ks),
                    "update": timed(4, ks), "all_gather": timed(8, ks)}

    if args.quick:                     # device-resident timing only (sweeps, profiler runs)
        if rank == 0:
            wire = 2.0 * P * (world - 1) / world
            print(json.dumps({"metric": "adamw_params_per_sec", "value": P / (ms_per_step * 1e-3), "unit": "params/s",
                              "n_gpus": world, "steps": K, "warmup": args.warmup, "ms_per_step": ms_per_step,
                              "phases_ms": phase_ms, "config": config_for(args), "quick": True,
                              "link_gbs_per_direction": {k: wire / (v * 1e-3) / 1e9 for k, v in phase_ms.items()
                                                         if "reduce_scatter" in k or "gather" in k},
                              "env": {k: v for k, v in os.environ.items() if k.startswith("RLCU_")}}), flush=True)
        z.close()
        dist.barrier()
        dist.destroy_process_group()
        return

    # end to end: this rank's gradient replica comes from pinned host memory every step
    host_g = torch.empty(padded, dtype=torch.float16).pin_memory()
    host_g.copy_(g_fresh)
    host_stat = torch.empty(16, dtype=torch.float32).pin_memory()
    e2e_steps = max(3, min(K, 10))
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        g_pool.copy_(host_g, non_blocking=True)
        step(t)
        host_stat.copy_(stat, non_blocking=True)
        t += 1
    e1.record()
    torch.cuda.synchronize()
    e2e = torch.tensor([e0.elapsed_time(e1) / e2e_steps], dtype=torch.float64, device=dev)
    dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e[0])
    del host_g

    # ---- one checked step (not timed): the sharded result against its definition
    parity = checked_step(torch, dist, pkg, z, mode, rank, world, segments, P, S, p_pool, g_pool, g_fresh, m_sh, v_sh,
                          stat, pkg.hparams(lr, b1, b2, eps, t), flags, max_norm, stream)
    t += 1

    # ---- the sharded update alone against the same update on one GPU (no exchange in either)
    def shard_list():
        descs = []
        lo = rank * S
        for pool_off, state_off, n, wd, fl in pkg.zero1_pieces(segments, rank, world):
            descs.append(pkg.TensorDesc(p_pool.data_ptr() + 2 * pool_off, g_pool.data_ptr() + 2 * pool_off,
                                        m_sh.data_ptr() + 4 * state_off, v_sh.data_ptr() + 4 * state_off, None,
                                        n, wd, pkg.F16, fl, 0))
        return pkg.TensorList(descs)

    # (This runs last: it steps the shard and the full set on their own, after which the ranks'
    # pools no longer agree.)
    update_only = None
    if P * 8 < 70e9:                                    # full-size m and v on every GPU: 8 bytes per parameter
        hp_now = pkg.hparams(lr, b1, b2, eps, t)
        tl_sh = shard_list()
        shard_ms = mean_launch_ms(torch, lambda: tl_sh.step(hp_now, stat.data_ptr(), flags, stream=stream), reps=10)
        tl_sh.close()
        torch.cuda.empty_cache()
        m_full = torch.zeros(P, dtype=torch.float32, device=dev)
        v_full = torch.zeros(P, dtype=torch.float32, device=dev)
        descs, off = [], 0
        for n, wd_, fl in segments:
            descs.append(pkg.TensorDesc(p_pool.data_ptr() + 2 * off, g_pool.data_ptr() + 2 * off, m_full.data_ptr() + 4 * off,
                                        v_full.data_ptr() + 4 * off, None, n, wd_, pkg.F16, fl, 0))
            off += n
        tl_full = pkg.TensorList(descs)
        full_ms = mean_launch_ms(torch, lambda: tl_full.step(hp_now, stat.data_ptr(), flags, stream=stream), reps=10)
        tl_full.close()
        del m_full, v_full
        both = torch.tensor([shard_ms, full_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(both, op=dist.ReduceOp.MAX)
        update_only = {"one_gpu_ms": float(both[1]), "shard_ms": float(both[0]), "speedup": float(both[1] / both[0]),
                       "what": "adamw_table_kernel over all parameters on one GPU against the same kernel over one "
                               "rank's shard (max over ranks), no exchange in either"}

    if rank == 0:
        peak, peak_kind = measured_peak()
        link = 770.0                                   # measured peer copy, GB/s per direction per GPU
        wire = 2.0 * P * (world - 1) / world           # bytes each GPU sends (and receives) per collective
        upd_bytes = BYTES_PER_PARAM * S
        per_param = ncu_dram_bytes_per_param("adamw_table_kernel")
        traffic = per_param * S if per_param is not None else None     # local HBM bytes of the shard's update

        def floor_for(rate):
            if mode == pkg.ZERO1_P2P:
                # both exchanges ride inside a kernel; each is bounded by the slower of its HBM
                # traffic and the bytes it moves over NVLink
                return (max(wire / (rate * 1e9), 4.0 * S / (peak * 1e9)) +
                        max(wire / (rate * 1e9), upd_bytes / (peak * 1e9))) * 1e3
            return (2 * wire / (rate * 1e9) + (upd_bytes + 2 * S) / (peak * 1e9)) * 1e3

        floor_ms = floor_for(link)
        if mode == pkg.ZERO1_P2P:
            link_rates = {"reduce_scatter_statistics_fused": wire / (phase_ms["reduce_scatter_statistics_fused"] * 1e-3) / 1e9,
                          "update_allgather_fused": wire / (phase_ms["update_allgather_fused"] * 1e-3) / 1e9}
            upd_ms = phase_ms["update_allgather_fused"]
            roof = {"bound": "nvlink" if wire / link > upd_bytes / peak else "hbm",
                    "kernel": ("adamw_table_peer_kernel" if args.direct else "adamw_table_bulk_peer_kernel") + " (shard update + all-gather)",
                    "achieved": link_rates["update_allgather_fused"], "peak": link,
                    "peak_kind": "measured peer copy, GB/s per direction per GPU", "unit": "GB/s",
                    "frac": link_rates["update_allgather_fused"] / link,
                    "hbm_gbs": upd_bytes / (upd_ms * 1e-3) / 1e9, "traffic": traffic}
        else:
            link_rates = {"reduce_scatter": wire / (phase_ms["reduce_scatter"] * 1e-3) / 1e9,
                          "all_gather": wire / (phase_ms["all_gather"] * 1e-3) / 1e9}
            roof = {"bound": "hbm", "kernel": "adamw_table_kernel (shard)",
                    "achieved": upd_bytes / (phase_ms["update"] * 1e-3) / 1e9, "peak": peak,
                    "peak_kind": f"{peak_kind} copy bandwidth", "unit": "GB/s",
                    "frac": upd_bytes / (phase_ms["update"] * 1e-3) / 1e9 / peak,
                    "traffic": traffic}
        line = {
            "metric": "adamw_params_per_sec", "value": P / (ms_per_step * 1e-3), "unit": "params/s",
            "n_gpus": world, "steps": K, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "storage": "f16 params and grads, f32 moments", "data": "synthetic",
            "config": config_for(args),
            "run_info": {"shard_params": S,
                         "exchange": ("peer-to-peer kernels over NVLink: fused reduce-scatter+statistics, fused update+all-gather "
                                      f"({'per-thread loads and stores' if args.direct else 'cp.async.bulk through shared memory'}), "
                                      "8-byte NCCL all-reduces for ordering and the norm") if mode == pkg.ZERO1_P2P else
                                     "ncclReduceScatter(sum, f16) + ncclAllReduce(1 double) + ncclAllGather(f16)",
                         "grad_restore": "device copy of the rank's gradient replica before each step, outside the timed intervals",
                         "grad_norm": final.norm, "clip_active": int(final.clip_active),
                         **({"note": mode_note} if mode_note else {})},
            "parity": parity,
            **({"update_only": update_only} if update_only else {}),
            "phases_ms": phase_ms,
            "link_gbs_per_direction": link_rates,
            "roofline": roof,
            "nvlink_roofline": {"floor_ms": floor_ms, "frac": floor_ms / ms_per_step,
                                "what": "two exchanges of (N-1)/N x 2 bytes/param per GPU per direction at 770 GB/s (one-direction peer copy) and the shard's HBM traffic at the measured peak; overlapped inside the fused kernels in p2p mode, back to back in nccl mode"},
            "e2e": {"value": P / (e2e_ms * 1e-3), "unit": "params/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": 2 * padded * world, "d2h_bytes_per_step": 64 * world,
                    "what": "each rank copies its FP16 gradient replica from pinned host memory, runs the sharded step, reads the "
                            "record back; the N ranks' copies share the host's PCIe paths (about 22 GB/s per GPU with 8 ranks "
                            "against 50 GB/s alone), which is what bounds this number, not the kernels"},
            "gpu_launches": (3 if mode == pkg.ZERO1_P2P else 3) * K * world,
            "clocks": clocks.report(),
        }
        print(json.dumps(line), flush=True)
    z.close()
    dist.barrier()
    dist.destroy_process_group()
    if not parity["ok"]:
        raise SystemExit(f"rank {rank}: the checked step does not match its definition: {parity}")


def probe_links(args):
    """Copy-engine bandwidth between GPU 0 and GPU 1 of this box, one direction alone and both
    directions at once (one process, two devices, cudaMemcpyPeerAsync through torch): what the
    NVLink figures of the sharded step are compared with."""
    import torch
    assert torch.cuda.device_count() >= 2, "needs two visible GPUs"
    n = 596_049_920
    a0, b0 = (torch.empty(n, dtype=torch.float16, device="cuda:0") for _ in range(2))
    a1, b1 = (torch.empty(n, dtype=torch.float16, device="cuda:1") for _ in range(2))
    s0, s1 = torch.cuda.Stream(device=0), torch.cuda.Stream(device=1)

    def one_way():
        with torch.cuda.device(0), torch.cuda.stream(s0):
            b1.copy_(a0, non_blocking=True)

    def two_way():
        one_way()
        with torch.cuda.device(1), torch.cuda.stream(s1):
            b0.copy_(a1, non_blocking=True)

    out = {}
    for name, fn in (("one_direction", one_way), ("both_directions", two_way)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(0), torch.cuda.synchronize(1)
        t0 = time.perf_counter()
        for _ in range(10):
            fn()
        torch.cuda.synchronize(0), torch.cuda.synchronize(1)
        out[name] = 2 * n / ((time.perf_counter() - t0) / 10) / 1e9
    print(json.dumps({"probe": "peer copy, GB/s per direction", **out}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="qwen3-0.6b", choices=["qwen3-0.6b", "qwen3-8b", "qwen3-0.6b-4l", "ragged-20k", "ragged-600"])
    ap.add_argument("--zero1-mode", default="p2p", choices=["p2p", "nccl"],
                    help="N>1: fused peer-to-peer kernels (default) or NCCL reduce-scatter/all-gather")
    ap.add_argument("--align", type=int, default=8,
                    help="N=1: elements every tensor start is aligned to inside the pools (8 = 16 bytes)")
    ap.add_argument("--bulk", action="store_true",
                    help="N=1: run the update through the cp.async.bulk variant of the kernel")
    ap.add_argument("--direct", action="store_true",
                    help="N>1: force the per-thread load/store exchange kernels (the default for FP16 pools is the bulk-copy pair)")
    ap.add_argument("--variants", default="", help="with --quick: also time these variants of the update (comma-separated "
                    "names of the `variants` object: multi_tensor_fp32_master, reference_layout_three_launches, bulk_copy, fp32_gradients)")
    ap.add_argument("--quick", action="store_true",
                    help="device-resident timing only (no end-to-end, CPU or reference-kernel legs): for profiler runs")
    ap.add_argument("--probe-links", action="store_true",
                    help="measure copy-engine peer bandwidth between GPU 0 and 1 (one and both directions) and exit")
    args = ap.parse_args()
    if args.probe_links:
        probe_links(args)
        return
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        run_single(args)
    else:
        run_sharded(args)


if __name__ == "__main__":
    main()
