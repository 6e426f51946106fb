"""The allocation-free decode entry point, b200_fattn_launch_static.

It exists for hosts that cannot allocate device memory where they run the operator (a decode loop inside
a real-time audio callback, an embedder with a fixed memory budget, a caller that hands over a stream but
has no allocator): the split-KV partials live in a fixed 8 MiB array inside the loaded library instead of
a caller-provided workspace.  The test calls it through the C-ABI several times in a row — each later call finds
the earlier calls' bytes in the shared array — and compares each result with b200_fattn_launch on the same
operands, within the parity tolerance of the suite.  This file sorts last so a run that stops at the
first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from crispasr_b200 import abi
from tests.util import MAX_ABS_TOL, REL_L2_TOL, errors

pytestmark = pytest.mark.gpu


def _descs(q, k, v, dst, kv_type=None):
    return abi.from_torch(q), abi.from_torch(k, kv_type), abi.from_torch(v, kv_type), abi.from_torch(dst)


def _launch_ws(L, q, k, v, kv_type, scale, kv_len=None):
    """The existing entry point, with a caller-allocated workspace."""
    dst = torch.empty((q.shape[0], q.shape[2], q.shape[1], q.shape[3]), dtype=torch.float32, device="cuda")
    tq, tk, tv, td = _descs(q, k, v, dst, kv_type)
    p = abi.Params(scale, 0.0, 0.0, 0)
    e = abi.Ext()
    if kv_len is not None:
        e.kv_len = kv_len.data_ptr()
    n = C.c_size_t(0)
    assert L.b200_fattn_workspace_bytes(C.byref(tq), C.byref(tk), C.byref(tv), None, C.byref(td), C.byref(p), C.byref(e), C.byref(n)) == 0
    ws = torch.empty(max(n.value, 256), dtype=torch.uint8, device="cuda")
    rc = L.b200_fattn_launch(C.byref(tq), C.byref(tk), C.byref(tv), None, C.byref(td), C.byref(p), C.byref(e),
                             ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.b200_strerror(rc)
    torch.cuda.synchronize()
    return dst, n.value


def _launch_static(L, q, k, v, kv_type, scale, kv_len=None):
    dst = torch.empty((q.shape[0], q.shape[2], q.shape[1], q.shape[3]), dtype=torch.float32, device="cuda")
    tq, tk, tv, td = _descs(q, k, v, dst, kv_type)
    p = abi.Params(scale, 0.0, 0.0, 0)
    e = abi.Ext()
    if kv_len is not None:
        e.kv_len = kv_len.data_ptr()
    rc = L.b200_fattn_launch_static(C.byref(tq), C.byref(tk), C.byref(tv), None, C.byref(td), C.byref(p), C.byref(e),
                                    torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, dst


def _plan(L, q, k, v, kv_type, scale):
    dst = torch.empty((q.shape[0], q.shape[2], q.shape[1], q.shape[3]), dtype=torch.float32, device="cuda")
    tq, tk, tv, td = _descs(q, k, v, dst, kv_type)
    p = abi.Params(scale, 0.0, 0.0, 0)
    kern, ns = C.c_int(0), C.c_int(0)
    assert L.b200_fattn_plan(C.byref(tq), C.byref(tk), C.byref(tv), None, C.byref(td), C.byref(p), None, C.byref(kern), C.byref(ns)) == 0
    return kern.value, ns.value


def test_static_scratch_matches_workspace_launch_twice(b200, orc):
    """Three calls in a row on the shared array, every one a form whose splits really travel through it: more than
    eight splits per (stream, kv-head), so the partials go to the scratch and a merge kernel reads them back (up to
    eight splits of a resident grid would merge inside thread-block clusters and never touch it).  Call 1 leaves the
    largest footprint, so calls 2 and 3 find stale bytes both inside and beyond the range they use; call 3 repeats
    call 1's geometry with other data."""
    L = b200.lib()
    assert L.b200_fattn_static_scratch_bytes() == 8 << 20
    assert L.b200_set_decode_splits(12) == 0
    try:
        _static_scratch_three_calls(L, orc)
    finally:
        assert L.b200_set_decode_splits(0) == 0


def _static_scratch_three_calls(L, orc):
    rng = np.random.default_rng(77)
    S, H, Hkv, hd, Lk = 8, 32, 8, 128, 663
    lens = torch.tensor([663, 408, 500, 64, 1, 650, 129, 333], dtype=torch.int32, device="cuda")

    def llm_case():
        k = torch.from_numpy(rng.standard_normal((S, Hkv, Lk, hd)).astype(np.float16)).cuda()
        v = torch.from_numpy(rng.standard_normal((S, Hkv, Lk, hd)).astype(np.float16)).cuda()
        q = torch.from_numpy(rng.standard_normal((S, H, 1, hd)).astype(np.float16)).cuda()
        return q, k, v

    q1, k1, v1 = llm_case()
    kern, ns1 = _plan(L, q1, k1, v1, None, hd ** -0.5)
    assert kern == abi.KERNEL_DECODE_SPLIT and ns1 > 1, "call 1 must split the KV range"
    want1, ws1 = _launch_ws(L, q1, k1, v1, None, hd ** -0.5, lens)
    assert ws1 > 0, "call 1 must merge through scratch memory"
    rc, got1 = _launch_static(L, q1, k1, v1, None, hd ** -0.5, lens)
    assert rc == 0, L.b200_strerror(rc)
    # call 2, directly after: Whisper cross-attention, 5 beams share one F16 cache; other geometry, smaller footprint
    k2 = torch.from_numpy((rng.standard_normal((1, 20, 1500, 64)) * 0.5).astype(np.float16)).cuda()
    v2 = torch.from_numpy((rng.standard_normal((1, 20, 1500, 64)) * 0.5).astype(np.float16)).cuda()
    q2 = torch.from_numpy((rng.standard_normal((1, 20, 5, 64)) * 0.5).astype(np.float32)).cuda()
    assert _plan(L, q2, k2, v2, None, 64 ** -0.25)[1] > 1
    rc, got2 = _launch_static(L, q2, k2, v2, None, 64 ** -0.25)
    assert rc == 0, L.b200_strerror(rc)
    want2, ws2 = _launch_ws(L, q2, k2, v2, None, 64 ** -0.25)
    assert 0 < ws2 < ws1
    # call 3: call 1's geometry again, new data, on top of what calls 1 and 2 left behind
    q3, k3, v3 = llm_case()
    rc, got3 = _launch_static(L, q3, k3, v3, None, hd ** -0.5, lens)
    assert rc == 0, L.b200_strerror(rc)
    want3, _ = _launch_ws(L, q3, k3, v3, None, hd ** -0.5, lens)
    for name, got, want in (("call 1", got1, want1), ("call 2", got2, want2), ("call 3", got3, want3)):
        ma, rl = errors(got.cpu().numpy(), want.cpu().numpy())
        assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL, f"{name}: max-abs {ma:.3e} rel-L2 {rl:.3e}"
    # and the results agree with the oracle
    for q, k, v, got in ((q1, k1, v1, got1), (q3, k3, v3, got3)):
        ref = orc.flash_attn_ext(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), scale=hd ** -0.5, kv_len=lens.cpu().numpy())
        ma, rl = errors(got.cpu().numpy(), ref)
        assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL


def test_static_scratch_rejects_what_it_cannot_hold(b200):
    L = b200.lib()
    # 591 (stream, kv-head) units with 2 splits each: 1182 partials x 16 rows x 128 floats = 9.7 MB > 8 MiB.  The
    # automatic choice keeps single-wave grids, whose partials always fit, so the split count is forced here.
    q = torch.zeros((3, 197, 1, 128), dtype=torch.float16, device="cuda")
    k = torch.zeros((3, 197, 128, 128), dtype=torch.float16, device="cuda")
    assert L.b200_set_decode_splits(2) == 0
    try:
        need = b200.workspace_bytes(q, k, k, scale=1.0)
        assert need > (8 << 20)
        rc, _ = _launch_static(L, q, k, k, None, 1.0)
        assert rc == abi.E_LIMIT and b"limit" in L.b200_strerror(rc)
    finally:
        assert L.b200_set_decode_splits(0) == 0
    assert L.b200_set_decode_splits(65) == abi.E_LIMIT
    # a prefill-shaped call is not the decode kernel: refused, not silently rerouted
    qp = torch.zeros((1, 4, 300, 64), dtype=torch.float16, device="cuda")
    kp = torch.zeros((1, 4, 300, 64), dtype=torch.float16, device="cuda")
    rc, _ = _launch_static(L, qp, kp, kp, None, 0.125)
    assert rc == abi.E_UNSUPPORTED
