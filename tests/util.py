"""Shared helpers of the test-suite: the reference tests' RNG, seeded inputs, error metrics and a
numpy -> CUDA -> C-ABI -> numpy runner."""
from __future__ import annotations

import numpy as np

MAX_ABS_TOL = 2e-3   # the path's stated tolerance: max-abs error against the CPU operator
REL_L2_TOL = 1e-3    # the path's stated tolerance: relative L2 error


class XorShift:
    """The Rng of tests/test-core-cross-attn.cpp:26-31 and tests/test-kv-quant-roundtrip.cpp."""

    def __init__(self, seed):
        self.s = seed & 0xFFFFFFFFFFFFFFFF

    def nx(self):
        s = self.s
        s ^= (s << 13) & 0xFFFFFFFFFFFFFFFF
        s ^= s >> 7
        s ^= (s << 17) & 0xFFFFFFFFFFFFFFFF
        self.s = s
        return (s >> 11) & 0xFFFFFFFF

    def sym(self):
        return np.float32((self.nx() % 20001) / 10000.0 - 1.0)

    def fill(self, n):
        return np.array([self.sym() for _ in range(n)], np.float32)


def errors(got, ref):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    max_abs = float(np.abs(got - ref).max()) if got.size else 0.0
    den = float(np.sqrt((ref ** 2).sum()))
    rel = float(np.sqrt(((got - ref) ** 2).sum()) / den) if den > 0 else max_abs
    return max_abs, rel


def assert_close(got, ref, what="", max_abs=MAX_ABS_TOL, rel_l2=REL_L2_TOL):
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    ma, rl = errors(got, ref)
    assert ma <= max_abs and rl <= rel_l2, f"{what}: max-abs {ma:.3e} (tol {max_abs}) rel-L2 {rl:.3e} (tol {rel_l2})"
    return ma, rl


def randn_f16(rng, shape, scale=1.0):
    return (rng.standard_normal(shape).astype(np.float32) * np.float32(scale)).astype(np.float16)


def cuda_view(view, base):
    """The same strided window of `base` (numpy, C-contiguous) that `view` is, on the GPU."""
    import torch
    assert base.flags.c_contiguous and view.dtype == base.dtype
    off = (view.__array_interface__["data"][0] - base.__array_interface__["data"][0]) // view.itemsize
    tb = torch.from_numpy(base.reshape(-1)).cuda()
    return torch.as_strided(tb, view.shape, [st // view.itemsize for st in view.strides], off)


def gpu_op(b200, q, k, v, mask=None, **kw):
    """Run the CUDA operator through the C-ABI. numpy inputs are copied contiguously; torch CUDA
    tensors (e.g. from cuda_view) are passed with their strides."""
    import torch

    def dev(a):
        if a is None:
            return None
        if isinstance(a, torch.Tensor):
            return a if a.is_cuda else a.cuda()
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    kw = dict(kw)
    for name in ("q_v", "r", "pos_bias_u", "pos_bias_v"):
        if kw.get(name) is not None:
            kw[name] = dev(kw[name])
    for name in ("kv_len", "q_len", "kv_index"):
        if kw.get(name) is not None and not isinstance(kw[name], torch.Tensor):
            kw[name] = torch.as_tensor(np.ascontiguousarray(kw[name], np.int32)).cuda()
    out = b200.flash_attn_ext(dev(q), dev(k), dev(v), dev(mask), **kw)
    torch.cuda.synchronize()
    return out.cpu().numpy()
