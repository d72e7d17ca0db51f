"""ctypes binding of ``librlcu_b200.so`` (the C ABI declared in ``include/rlcu_adamw.h``).

The directory name contains a dot, so it cannot be imported by name; load it with
``importlib`` under the module name ``rlcu_b200`` (``load_package()`` in
``__graft_entry__.py`` does that).

Everything that computes runs in the CUDA library.  There is no CPU fallback
here: if the shared library is missing, importing fails; if no GPU is present,
every compute call returns ``RLCU_ERR_CUDA`` and the wrappers raise ``RlcuError``.
PyTorch is used by callers only to own device memory and streams; this module
itself needs nothing but ``ctypes``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "lib", "librlcu_b200.so")

OK, ERR_INVALID, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_UNSUPPORTED = range(6)
F16, F32, BF16 = 0, 1, 2
GRAD_AS_PARAM, GRAD_F32 = 0, 1
TENSOR_NORM_ONLY, TENSOR_GRAD_ZERO = 1, 2
STEP_ROUND_CLIP_FP16, STEP_DEVICE_BIAS_CORRECTION, STEP_ZERO_GRADS, STEP_BULK_COPY, STEP_DIRECT = 1, 2, 4, 8, 16
STAT_PARTIAL, STAT_ACCUMULATE = 1, 2

# every symbol include/rlcu_adamw.h declares
EXPORTS = [
    "rlcu_abi_version", "rlcu_last_error", "rlcu_adamw_fp16_master", "rlcu_adamw_fp16",
    "rlcu_adamw_bf16_master", "rlcu_adamw_bf16", "rlcu_adamw_fp32", "rlcu_half_to_float", "rlcu_tensor_list_create",
    "rlcu_tensor_list_destroy", "rlcu_tensor_list_check", "rlcu_selftest_bounded_wait", "rlcu_tensor_list_numel", "rlcu_tensor_list_stat_numel",
    "rlcu_tensor_list_work_items", "rlcu_gradstat", "rlcu_gradstat_finalize",
    "rlcu_adamw_multi_step", "rlcu_bias_correction", "rlcu_gradstat_flat_noalloc",
    "rlcu_zero1_make_plan", "rlcu_zero1_plan_pieces", "rlcu_zero1_unique_id", "rlcu_zero1_create",
    "rlcu_zero1_step", "rlcu_zero1_poll_error", "rlcu_zero1_check", "rlcu_zero1_destroy",
    "rlcu_checkpoint_save", "rlcu_checkpoint_peek", "rlcu_checkpoint_load",
]
UNIQUE_ID_BYTES = 128
PHASE_REDUCE_SCATTER, PHASE_STATISTICS, PHASE_UPDATE, PHASE_ALL_GATHER = 1, 2, 4, 8
ZERO1_NCCL, ZERO1_P2P = 0, 1
ZERO1_POOLS_BF16 = 0x100
ZERO1_GRADS_F32 = 0x200
NOALLOC_MAX_ELEMS = 1 << 31
# C++-linkage launchers with RL.cu's signatures (include/kernels/adamw.cuh)
CXX_EXPORTS = [
    "_Z17launch_adamw_fp16PfP6__halfPKS0_S_S_ifffffffP11CUstream_st",
    "_Z17launch_adamw_fp32PfPKfS_S_ifffffffP11CUstream_st",
]


class RlcuError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"rlcu error {code}: {message}")
        self.code = code


class TensorDesc(C.Structure):
    """``rlcu_tensor_desc`` (64 bytes)."""
    _fields_ = [("param", C.c_void_p), ("grad", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
                ("master", C.c_void_p), ("n", C.c_uint64), ("weight_decay", C.c_float),
                ("dtype", C.c_uint32), ("flags", C.c_uint32), ("grad_dtype", C.c_uint32)]


class HParams(C.Structure):
    """``rlcu_hparams``."""
    _fields_ = [("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
                ("bias_correction1", C.c_float), ("bias_correction2", C.c_float)]


class Stat(C.Structure):
    """``rlcu_stat`` (64 bytes, lives in device memory; this is its host image)."""
    _fields_ = [("sum_sq", C.c_double), ("norm", C.c_float), ("coef", C.c_float),
                ("found_inf", C.c_uint32), ("clip_active", C.c_uint32),
                ("bias_correction1", C.c_float), ("bias_correction2", C.c_float),
                ("step", C.c_int32), ("loss_scale", C.c_float), ("reserved", C.c_uint32 * 6)]


class ScalerState(C.Structure):
    """``rlcu_scaler_state`` (32 bytes, device memory)."""
    _fields_ = [("scale", C.c_float), ("growth_tracker", C.c_int32), ("step", C.c_int32),
                ("skipped", C.c_int32), ("growth_interval", C.c_int32),
                ("beta1", C.c_float), ("beta2", C.c_float), ("grad_mul", C.c_float)]


class Zero1Segment(C.Structure):
    """``rlcu_zero1_segment``."""
    _fields_ = [("n", C.c_uint64), ("weight_decay", C.c_float), ("flags", C.c_uint32)]


class Zero1Plan(C.Structure):
    """``rlcu_zero1_plan``."""
    _fields_ = [("total", C.c_uint64), ("shard_elems", C.c_uint64), ("padded_elems", C.c_uint64),
                ("lo", C.c_uint64), ("hi", C.c_uint64), ("pieces", C.c_uint64)]


class CheckpointInfo(C.Structure):
    """``rlcu_checkpoint_info``."""
    _fields_ = [("state_elems", C.c_uint64), ("step", C.c_int32), ("loss_scale", C.c_float),
                ("growth_tracker", C.c_int32), ("skipped", C.c_int32), ("rank", C.c_int32),
                ("world", C.c_int32), ("has_master", C.c_uint32), ("reserved", C.c_uint32)]


assert C.sizeof(TensorDesc) == 64 and C.sizeof(Stat) == 64 and C.sizeof(ScalerState) == 32
assert C.sizeof(CheckpointInfo) == 40
assert C.sizeof(Zero1Segment) == 16 and C.sizeof(Zero1Plan) == 48


def build(force: bool = False, extra_flags: str = "") -> None:
    """Compile the CUDA library for sm_100a with the Makefile in ``csrc/``."""
    cmd = ["make", "-C", CSRC]
    if force:
        cmd.append("-B")
    if extra_flags:
        cmd.append(f"EXTRA_NVCCFLAGS={extra_flags}")
    subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL)


_lib = None


def lib() -> C.CDLL:
    """The loaded library, with argument types set.  Raises if it was not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `make -C {CSRC}` "
                          "(there is no fallback implementation)")
    L = C.CDLL(LIB_PATH)
    f, i64, u64, u32, vp = C.c_float, C.c_int64, C.c_uint64, C.c_uint32, C.c_void_p
    hyper = [f] * 7
    L.rlcu_abi_version.restype = C.c_int
    L.rlcu_last_error.restype = C.c_char_p
    L.rlcu_adamw_fp16_master.argtypes = [vp, vp, vp, vp, vp, i64] + hyper + [vp]
    L.rlcu_adamw_fp16.argtypes = [vp, vp, vp, vp, i64] + hyper + [vp]
    L.rlcu_adamw_fp32.argtypes = [vp, vp, vp, vp, i64] + hyper + [vp]
    L.rlcu_adamw_bf16_master.argtypes = [vp, vp, vp, vp, vp, i64] + hyper + [vp]
    L.rlcu_adamw_bf16.argtypes = [vp, vp, vp, vp, i64] + hyper + [vp]
    L.rlcu_half_to_float.argtypes = [vp, vp, i64, vp]
    L.rlcu_tensor_list_create.argtypes = [vp, u64, C.POINTER(vp)]
    L.rlcu_tensor_list_destroy.argtypes = [vp]
    L.rlcu_tensor_list_check.argtypes = [vp]
    L.rlcu_selftest_bounded_wait.argtypes = [vp, vp]
    for name in ("rlcu_tensor_list_numel", "rlcu_tensor_list_stat_numel", "rlcu_tensor_list_work_items"):
        getattr(L, name).argtypes = [vp]
        getattr(L, name).restype = u64
    L.rlcu_gradstat.argtypes = [vp, f, f, vp, vp, u32, vp]
    L.rlcu_gradstat_finalize.argtypes = [vp, f, f, vp, vp]
    L.rlcu_adamw_multi_step.argtypes = [vp, vp, vp, u32, vp]
    L.rlcu_gradstat_flat_noalloc.argtypes = [vp, u32, u64, f, f, vp, u32, vp]
    L.rlcu_zero1_make_plan.argtypes = [vp, u64, C.c_int, C.c_int, vp]
    L.rlcu_zero1_plan_pieces.argtypes = [vp, u64, C.c_int, C.c_int, vp, vp, vp, vp, vp]
    L.rlcu_zero1_unique_id.argtypes = [vp]
    L.rlcu_zero1_create.argtypes = [vp, C.c_int, C.c_int, vp, vp, vp, u64, vp, vp, vp, u32, C.POINTER(vp)]
    L.rlcu_zero1_step.argtypes = [vp, vp, f, f, vp, vp, u32, u32, vp]
    L.rlcu_zero1_poll_error.argtypes = [vp]
    L.rlcu_zero1_check.argtypes = [vp]
    L.rlcu_zero1_destroy.argtypes = [vp, C.c_int]
    L.rlcu_checkpoint_save.argtypes = [C.c_char_p, vp, vp, vp, vp, vp]
    L.rlcu_checkpoint_peek.argtypes = [C.c_char_p, vp]
    L.rlcu_checkpoint_load.argtypes = [C.c_char_p, vp, vp, vp, vp, u64, vp]
    L.rlcu_bias_correction.argtypes = [f, C.c_int]
    L.rlcu_bias_correction.restype = f
    _lib = L
    return L


def check(rc: int) -> None:
    if rc != OK:
        raise RlcuError(rc, lib().rlcu_last_error().decode())


def bias_correction(beta: float, step: int) -> float:
    return float(lib().rlcu_bias_correction(beta, step))


def hparams(lr, beta1, beta2, eps, step) -> HParams:
    """Hyper-parameters for Adam step ``step`` (1-based), bias corrections as RL.cu's
    AdamWOptimizer::step computes them (include/training/optimizer.h:121-122)."""
    return HParams(lr, beta1, beta2, eps, bias_correction(beta1, step), bias_correction(beta2, step))


def adamw_fp16_master(master, model_w, grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, stream=None):
    check(lib().rlcu_adamw_fp16_master(master, model_w, grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, stream))


def adamw_fp16(param, grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, stream=None):
    check(lib().rlcu_adamw_fp16(param, grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, stream))


def adamw_bf16_master(master, model_w, grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, stream=None):
    check(lib().rlcu_adamw_bf16_master(master, model_w, grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, stream))


def adamw_bf16(param, grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, stream=None):
    check(lib().rlcu_adamw_bf16(param, grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, stream))


def adamw_fp32(w, grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, stream=None):
    check(lib().rlcu_adamw_fp32(w, grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, stream))


def half_to_float(dst, src, n, stream=None):
    check(lib().rlcu_half_to_float(dst, src, n, stream))


class TensorList:
    """Owner of an ``rlcu_tensor_list`` handle.  ``descs`` is a sequence of ``TensorDesc``
    holding device addresses."""

    def __init__(self, descs):
        descs = list(descs)
        arr = (TensorDesc * max(len(descs), 1))(*descs)
        handle = C.c_void_p()
        check(lib().rlcu_tensor_list_create(C.addressof(arr), len(descs), C.byref(handle)))
        self.handle = handle
        self.count = len(descs)

    @property
    def numel(self) -> int:
        return lib().rlcu_tensor_list_numel(self.handle)

    @property
    def stat_numel(self) -> int:
        return lib().rlcu_tensor_list_stat_numel(self.handle)

    @property
    def work_items(self) -> int:
        return lib().rlcu_tensor_list_work_items(self.handle)

    def gradstat(self, stat_ptr, unscale=1.0, max_norm=0.0, scaler_ptr=None, flags=0, stream=None):
        check(lib().rlcu_gradstat(self.handle, unscale, max_norm, scaler_ptr, stat_ptr, flags, stream))

    def step(self, hp: HParams, stat_ptr=None, step_flags=0, stream=None):
        check(lib().rlcu_adamw_multi_step(self.handle, C.addressof(hp), stat_ptr, step_flags, stream))

    def check(self):
        """Synchronise and raise if a bounded device-side wait gave up (bulk-copy update only)."""
        check(lib().rlcu_tensor_list_check(self.handle))

    def close(self):
        if self.handle:
            check(lib().rlcu_tensor_list_destroy(self.handle))
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def gradstat_finalize(stat_ptr, unscale=1.0, max_norm=0.0, scaler_ptr=None, stream=None):
    check(lib().rlcu_gradstat_finalize(stat_ptr, unscale, max_norm, scaler_ptr, stream))


def gradstat_flat_noalloc(grad_ptr, dtype, n, stat_ptr, unscale=1.0, max_norm=0.0, flags=0, stream=None):
    """Statistics of one flat gradient buffer without any device allocation (see the header:
    fixed scratch inside the library, at most ``NOALLOC_MAX_ELEMS`` elements, calls must not
    overlap on the GPU).  Two buffers of one step: ``STAT_PARTIAL`` on the first call,
    ``STAT_ACCUMULATE`` on the second."""
    check(lib().rlcu_gradstat_flat_noalloc(grad_ptr, dtype, n, unscale, max_norm, stat_ptr, flags, stream))


# ---------------------------------------------------------------------------
# ZeRO-1
# ---------------------------------------------------------------------------

def _segments(segments):
    segments = list(segments)
    arr = (Zero1Segment * max(len(segments), 1))()
    for k, (n, wd, flags) in enumerate(segments):
        arr[k] = Zero1Segment(n, wd, flags)
    return arr, len(segments)


def zero1_plan(segments, rank, world) -> Zero1Plan:
    """Shard geometry of ``rank`` (host arithmetic; works without a GPU)."""
    arr, n = _segments(segments)
    plan = Zero1Plan()
    check(lib().rlcu_zero1_make_plan(C.addressof(arr), n, rank, world, C.addressof(plan)))
    return plan


def zero1_pieces(segments, rank, world):
    """[(pool_offset, state_offset, n, weight_decay, flags)] that ``rank`` updates."""
    arr, n = _segments(segments)
    plan = zero1_plan(segments, rank, world)
    k = max(int(plan.pieces), 1)
    po, so, nn = (C.c_uint64 * k)(), (C.c_uint64 * k)(), (C.c_uint64 * k)()
    wd, fl = (C.c_float * k)(), (C.c_uint32 * k)()
    check(lib().rlcu_zero1_plan_pieces(C.addressof(arr), n, rank, world, C.addressof(po), C.addressof(so),
                                       C.addressof(nn), C.addressof(wd), C.addressof(fl)))
    return [(po[i], so[i], nn[i], wd[i], fl[i]) for i in range(int(plan.pieces))]


def zero1_unique_id() -> bytes:
    buf = C.create_string_buffer(UNIQUE_ID_BYTES)
    check(lib().rlcu_zero1_unique_id(buf))
    return buf.raw


class Zero1:
    """Owner of an ``rlcu_zero1`` context (one per rank; creation is collective)."""

    def __init__(self, unique_id: bytes, rank, world, param_pool_ptr, grad_pool_ptr, segments,
                 m_shard_ptr, v_shard_ptr, master_shard_ptr=None, mode=ZERO1_NCCL):
        arr, n = _segments(segments)
        self.plan = zero1_plan(segments, rank, world)
        self.rank, self.world = rank, world
        handle = C.c_void_p()
        idbuf = C.create_string_buffer(unique_id, UNIQUE_ID_BYTES)
        check(lib().rlcu_zero1_create(idbuf, rank, world, param_pool_ptr, grad_pool_ptr, C.addressof(arr), n,
                                      m_shard_ptr, v_shard_ptr, master_shard_ptr, mode, C.byref(handle)))
        self.handle = handle
        self.mode = mode

    def step(self, hp: HParams, stat_ptr, unscale=1.0, max_norm=0.0, scaler_ptr=None, step_flags=0,
             phases=0, stream=None):
        check(lib().rlcu_zero1_step(self.handle, C.addressof(hp), unscale, max_norm, scaler_ptr, stat_ptr,
                                    step_flags, phases, stream))

    def poll_error(self):
        check(lib().rlcu_zero1_poll_error(self.handle))

    def check(self):
        """Wait for the device and raise if a bounded wait of an exchange kernel gave up or NCCL failed."""
        check(lib().rlcu_zero1_check(self.handle))

    def close(self, abort=False):
        if self.handle:
            h, self.handle = self.handle, C.c_void_p()
            check(lib().rlcu_zero1_destroy(h, 1 if abort else 0))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------------------
# optimizer-state checkpoint
# ---------------------------------------------------------------------------

def checkpoint_save(path, info: CheckpointInfo, m_ptr, v_ptr, master_ptr=None, stream=None):
    check(lib().rlcu_checkpoint_save(os.fsencode(path), C.addressof(info), m_ptr, v_ptr, master_ptr, stream))


def checkpoint_peek(path) -> CheckpointInfo:
    info = CheckpointInfo()
    check(lib().rlcu_checkpoint_peek(os.fsencode(path), C.addressof(info)))
    return info


def checkpoint_load(path, m_ptr, v_ptr, master_ptr, capacity_elems, stream=None) -> CheckpointInfo:
    info = CheckpointInfo()
    check(lib().rlcu_checkpoint_load(os.fsencode(path), C.addressof(info), m_ptr, v_ptr, master_ptr,
                                     capacity_elems, stream))
    return info
