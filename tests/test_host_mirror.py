"""The C++ AdamWOptimizer mirror (include/training/optimizer.h).

CPU: it compiles against a stand-in for RL.cu's model header, and -- when a checkout of RL.cu
is found (RLCU_REFERENCE, or a directory named "reference" beside this repository) -- RL.cu's own tests/test_adamw.cu compiles
unchanged against it.  GPU: the mirror's test program runs and reports no failure."""
import os
import shutil
import subprocess

import pytest

from helpers import reference_checkout

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "tests", "cpp")
REF = reference_checkout() or ""
NVCC = ["nvcc", "-std=c++17", "-O2", "--expt-relaxed-constexpr", "-gencode", "arch=compute_100a,code=sm_100a"]


def _third_party_shim(dest):
    """RL.cu expects nlohmann/json and xxhash under third_party/ and does not vendor them; installed
    copies of the same libraries are put on the include path through symlinks (nothing is copied)."""
    import glob
    import sysconfig
    site = sysconfig.get_paths()["purelib"]
    json_hpp = glob.glob(os.path.join(site, "include", "cudnn_frontend", "thirdparty", "nlohmann", "json.hpp"))
    xxhash_h = glob.glob(os.path.join(site, "pyarrow", "include", "arrow", "vendored", "xxhash", "xxhash.h"))
    if not json_hpp or not xxhash_h:
        pytest.skip("nlohmann/json or xxhash, which RL.cu expects under third_party/, is not installed")
    shim = dest / "third_party"
    shim.mkdir(parents=True)
    os.symlink(json_hpp[0], shim / "json.hpp")
    os.symlink(xxhash_h[0], shim / "xxhash.h")
    return str(dest)


def _patched_training_headers(dest):
    """A copy of RL.cu's include/training/ in which trainer.h and GRPO_trainer.h carry
    include/training/trainer_fused_step.patch and optimizer.h is this repository's."""
    tdir = dest / "include" / "training"
    tdir.mkdir(parents=True)
    ref_training = os.path.join(REF, "include", "training")
    for name in os.listdir(ref_training):
        if name in ("trainer.h", "GRPO_trainer.h"):
            shutil.copy(os.path.join(ref_training, name), tdir / name)
            os.chmod(tdir / name, 0o644)
        elif name == "optimizer.h":
            os.symlink(os.path.join(ROOT, "include", "training", "optimizer.h"), tdir / name)
        else:
            os.symlink(os.path.join(ref_training, name), tdir / name)
    with open(os.path.join(ROOT, "include", "training", "trainer_fused_step.patch")) as patch:
        subprocess.run(["patch", "-p1", "-d", str(dest)], stdin=patch, check=True)
    return str(dest / "include")


@pytest.fixture(scope="module")
def reference_objects(tmp_path_factory):
    """Every RL.cu source of its `kernels` and `model` libraries except src/kernels/adamw.cu
    (CMakeLists.txt:58-79), compiled once for the link tests below."""
    import glob
    if not REF or shutil.which("nvcc") is None:
        pytest.skip("no checkout of RL.cu here")
    work = tmp_path_factory.mktemp("refobj")
    shim = _third_party_shim(work / "shim")
    sources = [s for pat in ("src/kernels/*.cu", "src/kernels/*.cpp", "src/model/*.cu")
               for s in sorted(glob.glob(os.path.join(REF, pat))) if not s.endswith("kernels/adamw.cu")]
    objs = []
    procs = []
    for src in sources:
        obj = str(work / (os.path.basename(src) + ".o"))
        objs.append(obj)
        procs.append(subprocess.Popen(["nvcc", "-std=c++17", "-O0", "--expt-relaxed-constexpr", "-w", "-gencode",
                                       "arch=compute_100a,code=sm_100a", "-I", os.path.join(REF, "include"), "-I", shim,
                                       "-c", src, "-o", obj]))
    for pr in procs:
        assert pr.wait() == 0
    return objs, shim


@pytest.fixture(scope="module")
def mirror_binary(pkg, tmp_path_factory):
    if shutil.which("nvcc") is None:
        pytest.skip("nvcc not available")
    out = str(tmp_path_factory.mktemp("mirror") / "test_optimizer_mirror")
    lib_dir = os.path.join(ROOT, "rl.cu_b200", "lib")
    cmd = NVCC + ["-I", os.path.join(ROOT, "include"), "-I", os.path.join(CPP, "stub"),
                  os.path.join(CPP, "test_optimizer_mirror.cu"), "-o", out,
                  "-L", lib_dir, "-lrlcu_b200", "-Xlinker", f"-rpath={lib_dir}"]
    subprocess.run(cmd, check=True)
    return out


def test_mirror_builds_against_the_stand_in_model_header(mirror_binary):
    assert os.path.exists(mirror_binary)


def test_reference_test_source_compiles_against_the_mirror(tmp_path):
    """RL.cu's tests/test_adamw.cu, unchanged, with this repository's include/ first."""
    src = os.path.join(REF, "tests", "test_adamw.cu")
    if not os.path.exists(src) or shutil.which("nvcc") is None:
        pytest.skip("no checkout of RL.cu here")
    cmd = NVCC + ["-I", os.path.join(ROOT, "include"), "-I", os.path.join(REF, "include"),
                  "-c", src, "-o", str(tmp_path / "test_adamw.o")]
    subprocess.run(cmd, check=True)
    syms = subprocess.run(["nm", "-C", str(tmp_path / "test_adamw.o")], check=True, capture_output=True, text=True).stdout
    assert "rlcu_adamw_multi_step" in syms          # the mirror, not RL.cu's header, was picked up


@pytest.mark.gpu
def test_mirror_program_passes_on_the_gpu(mirror_binary):
    r = subprocess.run([mirror_binary], capture_output=True, text=True)
    print(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "[FAIL]" not in r.stdout and r.stdout.count("[PASS]") >= 17


def test_reference_test_binary_links_against_the_library(pkg, tmp_path, reference_objects):
    """Link-level drop-in: RL.cu's tests/test_adamw.cu with RL.cu's own headers and every RL.cu
    source except src/kernels/adamw.cu links into an executable whose launch_adamw_fp16 /
    launch_adamw_fp32 come from librlcu_b200.so.  (Running it needs real Qwen3-0.6B weights, which
    are not here; it exits at once without them, tests/test_adamw.cu:507-510.)"""
    objs, shim = reference_objects
    src = os.path.join(REF, "tests", "test_adamw.cu")
    lib_dir = os.path.join(ROOT, "rl.cu_b200", "lib")
    exe = str(tmp_path / "test_adamw")
    cmd = ["nvcc", "-std=c++17", "-O0", "--expt-relaxed-constexpr", "-w", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", os.path.join(REF, "include"), "-I", shim, src] + objs + \
          ["-o", exe, "-lcublas", "-L", lib_dir, "-lrlcu_b200", "-Xlinker", f"-rpath={lib_dir}"]
    subprocess.run(cmd, check=True)
    undefined = subprocess.run(["nm", "-D", "--undefined-only", exe], check=True, capture_output=True, text=True).stdout
    for sym in pkg.CXX_EXPORTS:
        assert sym in undefined, f"{sym} is not taken from the shared library"
    needed = subprocess.run(["ldd", exe], check=True, capture_output=True, text=True).stdout
    assert "librlcu_b200.so" in needed


@pytest.mark.parametrize("program", ["train_sft", "train_grpo"])
def test_reference_trainers_link_with_the_fused_step(pkg, tmp_path, reference_objects, program):
    """The whole trainer binary: RL.cu's tests/train_sft.cu / tests/train_grpo.cu, compiled against
    the patched trainer headers and this repository's optimizer.h, link with RL.cu's own model and
    kernel objects (without src/kernels/adamw.cu) and librlcu_b200.so; the executable takes the
    statistics pass and the multi-tensor update from the shared library and no longer needs
    RL.cu's launch_adamw_* at all."""
    if shutil.which("patch") is None:
        pytest.skip("patch is not installed")
    objs, shim = reference_objects
    src = os.path.join(REF, "tests", f"{program}.cu")
    patched = _patched_training_headers(tmp_path / "patched")
    lib_dir = os.path.join(ROOT, "rl.cu_b200", "lib")
    exe = str(tmp_path / program)
    cmd = ["nvcc", "-std=c++17", "-O0", "--expt-relaxed-constexpr", "-w", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", os.path.join(ROOT, "include"), "-I", patched, "-I", os.path.join(REF, "include"), "-I", shim, src] + objs + \
          ["-o", exe, "-lcublas", "-L", lib_dir, "-lrlcu_b200", "-Xlinker", f"-rpath={lib_dir}"]
    subprocess.run(cmd, check=True)
    undefined = subprocess.run(["nm", "-D", "--undefined-only", exe], check=True, capture_output=True, text=True).stdout
    for sym in ("rlcu_gradstat", "rlcu_adamw_multi_step", "rlcu_tensor_list_create", "rlcu_half_to_float"):
        assert sym in undefined, f"{sym} is not taken from the shared library"
    for sym in pkg.CXX_EXPORTS:
        assert sym not in undefined, "the patched trainer still calls RL.cu's launchers"
    assert "librlcu_b200.so" in subprocess.run(["ldd", exe], check=True, capture_output=True, text=True).stdout


@pytest.mark.parametrize("program", ["train_sft", "train_grpo"])
def test_reference_trainers_compile_with_the_fused_step_patch(tmp_path, program):
    """The trainer side of the drop-in: include/training/trainer_fused_step.patch, applied to
    copies of RL.cu's trainer.h and GRPO_trainer.h, replaces clip_grad_norm_ + optimizer_.step
    (trainer.h:279-286, GRPO_trainer.h:507-514) and the freeze_embed memset (trainer.h:271-277)
    by AdamWOptimizer::clip_and_step of this repository's optimizer.h.  RL.cu's own
    tests/train_sft.cu and tests/train_grpo.cu then compile, call the fused library entry
    points, and no longer contain RL.cu's sum-of-squares and scale kernels."""
    src = os.path.join(REF, "tests", f"{program}.cu")
    if not os.path.exists(src) or shutil.which("nvcc") is None or shutil.which("patch") is None:
        pytest.skip("no checkout of RL.cu here")
    shim = _third_party_shim(tmp_path / "shim")
    patched = _patched_training_headers(tmp_path / "patched")
    obj = str(tmp_path / f"{program}.o")
    cmd = ["nvcc", "-std=c++17", "-O0", "--expt-relaxed-constexpr", "-w", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", os.path.join(ROOT, "include"), "-I", patched,
           "-I", os.path.join(REF, "include"), "-I", shim, "-c", src, "-o", obj]
    subprocess.run(cmd, check=True)
    syms = subprocess.run(["nm", "-C", obj], check=True, capture_output=True, text=True).stdout
    for wanted in ("U rlcu_gradstat", "U rlcu_adamw_multi_step", "clip_and_step"):
        assert wanted in syms, wanted
    for gone in ("sum_sq_half_kernel", "sum_sq_float_kernel", "scale_half_kernel", "clip_grad_norm_", "launch_adamw_fp16"):
        assert gone not in syms, gone


@pytest.fixture(scope="module")
def zero1_threads_binary(pkg, tmp_path_factory):
    if shutil.which("nvcc") is None:
        pytest.skip("nvcc not available")
    out = str(tmp_path_factory.mktemp("zero1") / "test_zero1_threads")
    lib_dir = os.path.join(ROOT, "rl.cu_b200", "lib")
    cmd = NVCC + ["-I", os.path.join(ROOT, "include"), os.path.join(CPP, "test_zero1_threads.cu"), "-o", out,
                  "-L", lib_dir, "-lrlcu_b200", "-Xlinker", f"-rpath={lib_dir}", "-Xcompiler", "-pthread"]
    subprocess.run(cmd, check=True)
    return out


def test_cxx_sharded_driver_builds(zero1_threads_binary):
    """The C ABI of the sharded step is usable from plain C++ (no Python, no PyTorch)."""
    assert os.path.exists(zero1_threads_binary)


@pytest.mark.gpu
def test_cxx_sharded_driver_runs_on_several_gpus(zero1_threads_binary):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([zero1_threads_binary], capture_output=True, text=True, env=env, timeout=600)
    print(r.stdout, r.stderr[-2000:])
    assert r.returncode == 0, r.stdout + r.stderr[-2000:]
    assert "[FAIL]" not in r.stdout and r.stdout.count("[PASS]") == 4
