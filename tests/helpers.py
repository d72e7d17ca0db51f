"""Shared plumbing of the GPU parity tests: seeded inputs, device buffers with
guard words, descriptor construction, and comparison in the units the parity
bars are stated in (FP16 ulps, relative FP32 error)."""
from __future__ import annotations

import os

import numpy as np


def reference_checkout():
    """Path of a checkout of KJLdefeated/RL.cu, or None: the directory RLCU_REFERENCE names,
    else a directory called ``reference`` beside this repository."""
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for cand in (os.environ.get("RLCU_REFERENCE"), os.path.join(os.path.dirname(here), "reference")):
        if cand and os.path.exists(os.path.join(cand, "src", "kernels", "adamw.cu")):
            return cand
    return None


GUARD = 64          # guard elements before and after every device buffer
GUARD_BYTE = 0x5A


def seeded_case(O, n, seed, p_std=0.02, g_std=1e-3, warm=False):
    """FP16 params ~N(0,p_std), FP16 grads ~N(0,g_std), FP32 moments zero or warm."""
    rng = np.random.default_rng(seed)
    p = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(p_std))
    g = O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(g_std))
    if warm:
        m = (rng.standard_normal(n) * g_std * 0.3).astype(np.float32)
        v = (rng.random(n) * g_std * g_std).astype(np.float32)
    else:
        m = np.zeros(n, np.float32)
        v = np.zeros(n, np.float32)
    return p, g, m, v


def fresh_grad(O, n, seed, step, g_std=1e-3):
    rng = np.random.default_rng([seed, step, 1])
    return O.f2h(rng.standard_normal(n).astype(np.float32) * np.float32(g_std))


class DevBuf:
    """A device copy of a numpy array with guard bytes on both sides and an
    optional element offset (to produce deliberately misaligned pointers)."""

    def __init__(self, arr, torch, offset_elems=0):
        self.torch = torch
        self.dtype = arr.dtype
        self.n = arr.size
        self.itemsize = arr.dtype.itemsize
        pad = (GUARD + offset_elems) * self.itemsize
        raw = np.full(pad + self.n * self.itemsize + GUARD * self.itemsize, GUARD_BYTE, np.uint8)
        raw[pad:pad + self.n * self.itemsize] = arr.view(np.uint8).reshape(-1)
        self.pad = pad
        self.raw = torch.from_numpy(raw).cuda()

    @property
    def ptr(self):
        return self.raw.data_ptr() + self.pad

    def get(self):
        host = self.raw.cpu().numpy()
        return host[self.pad:self.pad + self.n * self.itemsize].view(self.dtype).copy()

    def set(self, arr):
        assert arr.size == self.n and arr.dtype == self.dtype
        t = self.torch.from_numpy(arr.view(np.uint8).reshape(-1).copy()).cuda()
        self.raw[self.pad:self.pad + self.n * self.itemsize] = t

    def guards_intact(self):
        host = self.raw.cpu().numpy()
        return bool((host[:self.pad] == GUARD_BYTE).all()
                    and (host[self.pad + self.n * self.itemsize:] == GUARD_BYTE).all())


def ulp16(a, b):
    """Distance between two binary16 bit-pattern arrays in units in the last place
    (monotone integer mapping of sign-magnitude patterns)."""
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, 0x8000 - x, x)
    return np.abs(key(a) - key(b))


def rel_err(a, b):
    a = a.astype(np.float64)
    b = b.astype(np.float64)
    denom = np.maximum(np.abs(b), 1e-38)
    return np.abs(a - b) / denom


def max_rel(a, b):
    if a.size == 0:
        return 0.0
    return float(rel_err(a, b).max())


def read_stat(pkg, stat_tensor):
    return pkg.Stat.from_buffer_copy(stat_tensor.cpu().numpy().tobytes())


def qwen3_shapes(hidden, inter, layers, vocab, q_heads, kv_heads, head_dim, tied):
    """(name, numel, weight_decay_applies) in RL.cu's pool order: per layer
    [q,k,v,o,gate,up,down] then embed (include/model/weights.h:43-61), with the
    norm weights listed after the projections they belong to."""
    out = []
    q_dim, kv_dim = q_heads * head_dim, kv_heads * head_dim
    for l in range(layers):
        out += [(f"l{l}.q", q_dim * hidden, True), (f"l{l}.k", kv_dim * hidden, True),
                (f"l{l}.v", kv_dim * hidden, True), (f"l{l}.o", hidden * q_dim, True),
                (f"l{l}.gate", inter * hidden, True), (f"l{l}.up", inter * hidden, True),
                (f"l{l}.down", hidden * inter, True),
                (f"l{l}.in_norm", hidden, False), (f"l{l}.q_norm", head_dim, False),
                (f"l{l}.k_norm", head_dim, False), (f"l{l}.post_norm", hidden, False)]
    out.append(("embed", vocab * hidden, False))
    if not tied:
        out.append(("lm_head", vocab * hidden, False))
    out.append(("final_norm", hidden, False))
    return out


def qwen3_0p6b():
    return qwen3_shapes(1024, 3072, 28, 151936, 16, 8, 128, tied=True)


def qwen3_8b():
    return qwen3_shapes(4096, 12288, 36, 151936, 32, 8, 128, tied=False)
