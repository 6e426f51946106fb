"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol, validates operands
with error codes (never aborts), plans kernels, and the segment scheduler's host logic."""
import ctypes as C
import os
import re
import threading

import numpy as np
import pytest
import torch

from crispasr_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200_fattn.h")).read()
    return sorted(set(re.findall(r"B200_API\s+[\w\s\*]+?\b(b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(b200):
    names = declared_symbols()
    assert len(names) >= 18
    lib = C.CDLL(b200.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/b200_fattn.h but not exported"
    assert set(names) == set(abi.SYMBOLS), "ctypes mirror and header disagree"
    assert b"sm_100a" in b200.lib().b200_version()


def test_library_was_built_from_the_sources_in_the_tree(b200):
    """The stamp written beside the library at link time equals the hash of the sources now in the tree."""
    from crispasr_b200 import build
    assert build.built_hash() == build.source_hash()


def test_missing_library_fails_loudly(b200, monkeypatch):
    import crispasr_b200
    monkeypatch.setattr(crispasr_b200, "_LIB", None)
    monkeypatch.setattr(crispasr_b200, "LIB_PATH", "/nonexistent/libb200_fattn.so")
    with pytest.raises(ImportError):
        crispasr_b200.lib()


def _desc(shape, dtype=torch.float16):
    return torch.zeros(shape, dtype=dtype)


def _supports(b200, q, k, v, mask=None, dst=None, **kw):
    from crispasr_b200.op import _make, _dst_like
    c = _make(q, k, v, mask, dst if dst is not None else _dst_like(q), dict(scale=1.0, **kw), abi.from_torch)
    why = C.c_int(0)
    ok = b200.lib().b200_fattn_supports(*c.args(), C.byref(why))
    return bool(ok), why.value


def test_validator_codes(b200):
    q = _desc((1, 8, 10, 64), torch.float32)
    k = _desc((1, 8, 20, 64))
    assert _supports(b200, q, k, k) == (True, 0)
    assert _supports(b200, q, k, _desc((1, 8, 20, 64), torch.float32))[1] == abi.E_TYPE      # K/V types differ
    assert _supports(b200, q, _desc((1, 8, 20, 32)), _desc((1, 8, 20, 32)))[1] == abi.E_SHAPE  # head dims
    assert _supports(b200, q, _desc((1, 3, 20, 64)), _desc((1, 3, 20, 64)))[1] == abi.E_SHAPE  # 8 % 3
    assert _supports(b200, q, k, k, _desc((1, 1, 10, 20), torch.float32))[1] == abi.E_TYPE    # mask must be F16
    assert _supports(b200, q, k, k, _desc((1, 1, 10, 19)))[1] == abi.E_SHAPE                  # mask ne0 != Lk
    assert _supports(b200, q, k, k, _desc((1, 5, 10, 20)))[1] == abi.E_SHAPE                  # mask heads
    assert _supports(b200, q, k, k, _desc((1, 8, 10, 20)))[0]                                 # per-head mask ok
    big = _desc((1, 8, 10, 160), torch.float32)
    assert _supports(b200, big, _desc((1, 8, 20, 160)), _desc((1, 8, 20, 160)))[1] == abi.E_UNSUPPORTED
    # dst must be contiguous [hd,H,Tq,B]
    bad_dst = torch.zeros((1, 10, 8, 128), dtype=torch.float32)[..., :64]
    assert _supports(b200, q, k, k, dst=bad_dst)[1] == abi.E_STRIDE
    # dst rows are written with 128-bit stores by the tensor-core prefill: a base that is only 4-byte aligned is refused
    buf = torch.zeros(1 * 10 * 8 * 64 + 4, dtype=torch.float32)
    assert _supports(b200, q, k, k, dst=buf[1:1 + 10 * 8 * 64].view(1, 10, 8, 64))[1] == abi.E_ALIGN
    assert _supports(b200, q, k, k, dst=buf[4:4 + 10 * 8 * 64].view(1, 10, 8, 64)) == (True, 0)
    # Q8_0 rows: nb0 must be one block and hd a multiple of 32
    kq = torch.zeros((1, 2, 20, 136), dtype=torch.uint8)
    q128 = _desc((1, 8, 1, 128), torch.float32)
    assert _supports(b200, q128, kq, kq, kv_type=abi.Q8_0)[0]
    # relpos needs both operands and Lk == Tq
    qq = _desc((1, 8, 20, 64), torch.float32)
    r = _desc((1, 8, 39, 64))
    assert _supports(b200, qq, k, k, q_v=qq, r=r)[0]
    assert _supports(b200, q, k, k, q_v=q, r=r)[1] == abi.E_SHAPE
    # position biases folded into the Q load: both, F32 [hd, H], with r and without q_v
    bu = _desc((8, 64), torch.float32)
    kk = _desc((1, 8, 20, 64))
    assert _supports(b200, qq, kk, kk, r=r, pos_bias_u=bu, pos_bias_v=bu) == (True, 0)
    assert _supports(b200, qq, kk, kk, r=r, pos_bias_u=bu)[1] == abi.E_NULL
    assert _supports(b200, qq, kk, kk, q_v=qq, r=r, pos_bias_u=bu, pos_bias_v=bu)[1] == abi.E_NULL
    assert _supports(b200, qq, kk, kk, pos_bias_u=bu, pos_bias_v=bu)[1] == abi.E_NULL        # no r
    assert _supports(b200, qq, kk, kk, r=r, pos_bias_u=bu, pos_bias_v=_desc((8, 64)))[1] == abi.E_TYPE
    assert _supports(b200, qq, kk, kk, r=r, pos_bias_u=bu, pos_bias_v=_desc((4, 64), torch.float32))[1] == abi.E_SHAPE
    assert b200.lib().b200_fattn_supports(None, None, None, None, None, None, None, None) == 0
    assert b"NULL" in b200.lib().b200_strerror(abi.E_NULL)


def test_plan_choices(b200):
    enc_q = _desc((1, 20, 1500, 64), torch.float32)
    enc_k = _desc((1, 20, 1500, 64))
    kern, ns = b200.plan(enc_q, enc_k, enc_k, scale=0.125)
    assert kern in (abi.KERNEL_PREFILL_TC5, abi.KERNEL_TILE_MMA) and ns == 1
    # whisper cross-attention decode: 5 beams share the cache -> split-KV; up to eight splits of a resident grid merge
    # inside thread-block clusters (no workspace), more splits go through the workspace and the merge kernel
    dq = _desc((1, 20, 5, 64), torch.float32)
    kern, ns = b200.plan(dq, enc_k, enc_k, scale=0.35)
    assert kern == abi.KERNEL_DECODE_SPLIT and 1 < ns <= 8
    assert b200.workspace_bytes(dq, enc_k, enc_k, scale=0.35) == 0
    assert b200.lib().b200_set_decode_splits(12) == 0
    try:
        assert b200.plan(dq, enc_k, enc_k, scale=0.35) == (abi.KERNEL_DECODE_SPLIT, 12)
        assert b200.workspace_bytes(dq, enc_k, enc_k, scale=0.35) >= 20 * 12 * 16 * 64 * 4
    finally:
        b200.lib().b200_set_decode_splits(0)
    # LLM decode, GQA 4, Q8_0
    kq = torch.zeros((8, 8, 663, 136), dtype=torch.uint8)
    kern, ns = b200.plan(_desc((8, 32, 1, 128), torch.float32), kq, kq, scale=0.088, kv_type=abi.Q8_0)
    assert kern == abi.KERNEL_DECODE_SPLIT and 1 < ns <= 8
    # ... whose few splits merge inside thread-block clusters: no workspace is asked for
    assert b200.workspace_bytes(_desc((8, 32, 1, 128), torch.float32), kq, kq, scale=0.088, kv_type=abi.Q8_0) == 0
    # the same streams over an F16 cache: the same form
    kf = _desc((8, 8, 663, 128))
    assert b200.workspace_bytes(_desc((8, 32, 1, 128), torch.float32), kf, kf, scale=0.088) == 0
    # explicit per-head mask or relpos -> general tile kernel unless the tcgen05 kernel takes it
    r = _desc((1, 20, 2999, 64))
    kern, _ = b200.plan(enc_q, enc_k, enc_k, scale=0.125, q_v=enc_q, r=r)
    assert kern in (abi.KERNEL_TILE_MMA, abi.KERNEL_PREFILL_TC5)
    assert b200.lib().b200_set_kernel_override(abi.KERNEL_TILE_MMA) == 0
    try:
        assert b200.plan(dq, enc_k, enc_k, scale=0.35)[0] == abi.KERNEL_TILE_MMA
    finally:
        b200.lib().b200_set_kernel_override(abi.KERNEL_NONE)
    assert b200.lib().b200_set_kernel_override(99) < 0


def test_launch_without_gpu_reports_no_device(b200):
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    q = _desc((1, 8, 10, 64), torch.float32)
    k = _desc((1, 8, 20, 64))
    with pytest.raises(b200.B200Error) as e:
        b200.flash_attn_ext_host(q, k, k, scale=1.0)
    assert e.value.code in (abi.E_NO_DEVICE, abi.E_CUDA)


def test_partition_covers_units_exactly(b200):
    for n, w in [(64, 8), (64, 3), (5, 8), (0, 4), (16, 1)]:
        seen = []
        for i in range(w):
            f, c = b200.SegmentScheduler.partition(n, w, i)
            seen += list(range(f, f + c))
        assert seen == list(range(n))
        sizes = [b200.SegmentScheduler.partition(n, w, i)[1] for i in range(w)]
        assert max(sizes) - min(sizes) <= 1


def test_scheduler_runs_every_unit_once(b200):
    s = b200.SegmentScheduler(n_host_workers=4)
    hits = np.zeros(100, np.int32)
    lock = threading.Lock()

    def unit(dev, u, stream):
        with lock:
            hits[u] += 1
        return 0
    failed, owners = s.run(100, unit)
    assert failed == 0 and (hits == 1).all() and all(0 <= o < 4 for o in owners)
    assert s.run(0, unit) == (0, [])
    s.close()


def test_scheduler_retries_failed_unit_on_another_worker(b200):
    """Host-side fault injection: unit 7 fails on its first worker (a raised exception) and must be retried
    elsewhere; unit 11 always fails and is reported, without stopping the other units."""
    s = b200.SegmentScheduler(n_host_workers=3)
    tried = {}
    lock = threading.Lock()

    def unit(dev, u, stream):
        me = threading.get_ident()
        with lock:
            tried.setdefault(u, []).append(me)
            n = len(tried[u])
        if u == 7 and n == 1:
            raise RuntimeError("injected")
        if u == 11:
            return 5
        return 0
    failed, owners = s.run(20, unit)
    assert failed == 1 and owners[11] == -1 and owners[7] >= 0
    assert len(tried[7]) == 2 and tried[7][0] != tried[7][1]
    assert len(tried[11]) == 2
    assert all(len(tried[u]) == 1 for u in range(20) if u not in (7, 11))
    s.close()


def test_scheduler_steals_from_slow_worker(b200):
    import time
    s = b200.SegmentScheduler(n_host_workers=2)
    first = {}

    def unit(dev, u, stream):
        first.setdefault(threading.get_ident(), u)
        if u < 8:            # worker 0's static range is slow
            time.sleep(0.01)
        return 0
    failed, owners = s.run(16, unit)
    assert failed == 0
    assert any(o == 1 for o in owners[:8]), "the idle worker never stole from the busy one"
    s.close()


def test_batched_scheduler_hands_out_contiguous_runs(b200):
    """b200_sched_run_batched: runs of consecutive units, never across the border of a worker's static share;
    max_batch >= share size gives each worker its share as one batch; without stealing every unit stays with its
    owner; a failing run is retried whole on another worker."""
    s = b200.SegmentScheduler(n_host_workers=4)
    calls = []
    lock = threading.Lock()

    def batch(dev, first, count, stream):
        with lock:
            calls.append((first, count))
        return 0
    failed, owners = s.run_batched(64, 64, batch, steal=False)
    assert failed == 0 and sorted(calls) == [(0, 16), (16, 16), (32, 16), (48, 16)]
    assert owners == [u // 16 for u in range(64)]
    calls.clear()
    failed, owners = s.run_batched(23, 4, batch, steal=True)
    assert failed == 0 and sorted(u for f, c in calls for u in range(f, f + c)) == list(range(23))
    borders = {b200.SegmentScheduler.partition(23, 4, w)[0] for w in range(4)}
    for f, c in calls:
        assert 1 <= c <= 4 and not any(f < b < f + c for b in borders), "a run crossed a share border"
    # a run that fails once is retried as a whole somewhere else; one that always fails is reported per unit
    tried = {}

    def flaky(dev, first, count, stream):
        me = threading.get_ident()
        with lock:
            tried.setdefault(first, []).append(me)
            n = len(tried[first])
        if first == 8 and n == 1:
            return 3
        return 7 if first == 12 else 0
    failed, owners = s.run_batched(16, 4, flaky, steal=True)
    assert failed == 4 and owners[12:16] == [-1] * 4 and all(o >= 0 for o in owners[:12])
    assert len(tried[8]) == 2 and tried[8][0] != tried[8][1]
    s.close()


def test_slice_packer_groups_units_of_similar_length(b200):
    """b200_batch_pack: every unit exactly once, launches of at most max_units, longest first, and inside a launch no
    unit below (1 - max_pad) of the longest, so padded buffers stay within 1 / (1 - max_pad) of the payload."""
    L = b200.lib()
    rng = np.random.default_rng(9)
    n = 57
    q = rng.integers(1, 1500, n).astype(np.int32)
    kv = (q + rng.integers(0, 200, n)).astype(np.int32)
    order, ends, ng = np.zeros(n, np.int32), np.zeros(n, np.int32), C.c_int(0)
    for max_units, max_pad in ((8, 0.25), (64, 0.1), (4, 1.0)):
        assert L.b200_batch_pack(q.ctypes.data, kv.ctypes.data, n, max_units, max_pad, order.ctypes.data, ends.ctypes.data, C.byref(ng)) == 0
        assert sorted(order.tolist()) == list(range(n))
        assert ends[ng.value - 1] == n and (np.diff(np.r_[0, ends[:ng.value]]) <= max_units).all()
        assert (np.diff(kv[order]) <= 0).all(), "longest first"
        start = 0
        for e in ends[:ng.value]:
            g = order[start:e]
            assert kv[g].min() >= (1 - max_pad) * kv[g].max() - 1e-6 and q[g].min() >= (1 - max_pad) * q[g].max() - 1e-6
            start = e
        if max_pad == 1.0:
            assert ng.value == -(-n // max_units)   # no length constraint: full launches
    assert L.b200_batch_pack(q.ctypes.data, kv.ctypes.data, 0, 4, 0.5, order.ctypes.data, ends.ctypes.data, C.byref(ng)) == 0 and ng.value == 0
    assert L.b200_batch_pack(q.ctypes.data, kv.ctypes.data, n, 0, 0.5, order.ctypes.data, ends.ctypes.data, C.byref(ng)) == abi.E_SHAPE


def test_slot_table_of_a_resident_batch(b200):
    """b200_batch: units take the lowest free slot, a freed slot inside the span stays in the launch with zero
    lengths, one decode step advances every resident stream."""
    L = b200.lib()
    h = C.c_void_p()
    assert L.b200_batch_create(4, C.byref(h)) == 0
    assert [L.b200_batch_add(h, 100 + i, 1, 400 + i) for i in range(4)] == [0, 1, 2, 3]
    assert L.b200_batch_add(h, 200, 1, 1) == abi.E_LIMIT
    span, act, mq, mk = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    assert L.b200_batch_span(h, C.byref(span), C.byref(act), C.byref(mq), C.byref(mk)) == 0
    assert (span.value, act.value, mq.value, mk.value) == (4, 4, 1, 403)
    assert L.b200_batch_remove(h, 1) == 0 and L.b200_batch_remove(h, 1) == abi.E_STATE
    assert L.b200_batch_advance(h, 1) == 0
    ql, kl = C.c_int(), C.c_int()
    assert L.b200_batch_lengths(h, 1, C.byref(ql), C.byref(kl)) == 0 and (ql.value, kl.value) == (0, 0)
    assert L.b200_batch_lengths(h, 2, C.byref(ql), C.byref(kl)) == 0 and (ql.value, kl.value) == (1, 403)
    assert L.b200_batch_unit(h, 1) == -1 and L.b200_batch_unit(h, 3) == 103
    assert L.b200_batch_add(h, 300, 1, 7) == 1                      # the hole is reused first
    assert L.b200_batch_remove(h, 3) == 0
    L.b200_batch_span(h, C.byref(span), C.byref(act), None, None)
    assert (span.value, act.value) == (3, 3)
    assert L.b200_batch_set(h, 3, 1, 1) == abi.E_STATE and L.b200_batch_set(h, 9, 1, 1) == abi.E_SHAPE
    if not torch.cuda.is_available():
        a, b_ = C.c_void_p(), C.c_void_p()
        assert L.b200_batch_tables(h, None, C.byref(a), C.byref(b_)) == abi.E_NO_DEVICE
    L.b200_batch_destroy(h)


def test_beam_cells_to_index_is_the_complement_of_the_mask_rule(b200, orc):
    """The index lists hold exactly the cells the reference's mask leaves at 0 (src/crispasr.cpp:3480-3488)."""
    L = b200.lib()
    rng = np.random.default_rng(10)
    n_cells, n_tok, stride = 300, 5, 256
    cell_pos = rng.integers(0, 60, n_cells).astype(np.int32)
    bits = rng.integers(0, 32, n_cells).astype(np.uint32)           # random subsets of 5 sequence ids; 0 = empty cell
    tok_seq, tok_pos = np.arange(n_tok, dtype=np.int32), rng.integers(20, 60, n_tok).astype(np.int32)
    idx, lens = np.full((n_tok, stride), -1, np.int32), np.zeros(n_tok, np.int32)
    rc = L.b200_beam_cells_to_index(cell_pos.ctypes.data, bits.ctypes.data, n_cells, tok_seq.ctypes.data, tok_pos.ctypes.data,
                                    n_tok, idx.ctypes.data, stride, lens.ctypes.data)
    assert rc == 0
    mask = orc.whisper_beam_mask(cell_pos, bits, tok_seq, tok_pos)   # (n_tok, n_cells) f16: 0 or -inf
    for j in range(n_tok):
        assert idx[j, :lens[j]].tolist() == np.flatnonzero(mask[j] == 0).tolist()
    assert L.b200_beam_cells_to_index(cell_pos.ctypes.data, bits.ctypes.data, n_cells, tok_seq.ctypes.data, tok_pos.ctypes.data,
                                      n_tok, idx.ctypes.data, 8, lens.ctypes.data) == abi.E_LIMIT


def test_mask_classify_recognises_the_masks_the_runtimes_build_on_the_host(b200, orc):
    """The causal prefill mask of src/voxtral.cpp:1187-1194 and a tail padding mask map to ext.causal / ext.kv_len;
    anything else stays an explicit mask."""
    L = b200.lib()

    def classify(m):
        m = np.ascontiguousarray(m, np.float16)
        kind, n_past, kv_len = np.zeros(1, np.int32), np.full(1, -7, np.int32), np.full(1, -7, np.int32)
        rc = L.b200_mask_classify(m.ctypes.data, m.shape[1], m.shape[0], m.strides[0] // 2, kind.ctypes.data, n_past.ctypes.data,
                                  kv_len.ctypes.data)
        assert rc == 0
        return int(kind[0]), int(n_past[0]), int(kv_len[0])

    for n_past, T in ((0, 7), (5, 3), (407, 1), (0, 300)):
        m = orc.causal_mask(n_past + T, T, n_past)            # (T, Lk), the reference's fill
        kind, got_past, _ = classify(m)
        if T == 1:
            assert kind == abi.MASK_NONE                      # a single row that sees every key
        else:
            assert (kind, got_past) == (abi.MASK_CAUSAL, n_past)
    assert classify(np.zeros((4, 64)))[0] == abi.MASK_NONE
    pad = np.zeros((6, 96), np.float16)
    pad[:, 70:] = -np.inf
    assert classify(pad) == (abi.MASK_TAIL, -7, 70)
    assert classify(-np.zeros((2, 8)))[0] == abi.MASK_NONE    # -0.0
    holes = pad.copy()
    holes[2, 10] = -np.inf
    assert classify(holes)[0] == abi.MASK_GENERAL
    bias = np.zeros((3, 16), np.float16)
    bias[1, 4] = -0.5
    assert classify(bias)[0] == abi.MASK_GENERAL
    shifted = orc.causal_mask(12, 4, 8).copy()
    shifted[3, :] = shifted[2, :]                             # not a step of one key per row
    assert classify(shifted)[0] == abi.MASK_GENERAL
    wide = np.zeros((5, 32 + 8), np.float16)[:, :32]          # a view with a row stride
    wide[:, 20:] = -np.inf
    m = np.ascontiguousarray(wide)
    assert classify(m) == (abi.MASK_TAIL, -7, 20)
    kind = np.zeros(1, np.int32)
    assert L.b200_mask_classify(None, 4, 4, 4, kind.ctypes.data, None, None) == abi.E_NULL
    assert L.b200_mask_classify(m.ctypes.data, 32, 5, 16, kind.ctypes.data, None, None) == abi.E_SHAPE


def test_beam_cells_to_union_lists_each_visible_cell_once(b200, orc):
    """The shared list holds every cell some token of the step can see, in pool order; the compact mask over the
    list's entries is the reference's mask (src/crispasr.cpp:3480-3488) restricted to those columns."""
    L = b200.lib()
    rng = np.random.default_rng(11)
    n_cells, n_tok, stride = 300, 5, 320
    cell_pos = rng.integers(0, 60, n_cells).astype(np.int32)
    bits = rng.integers(0, 32, n_cells).astype(np.uint32)
    tok_seq, tok_pos = np.arange(n_tok, dtype=np.int32), rng.integers(20, 60, n_tok).astype(np.int32)
    idx, n = np.full(stride, -1, np.int32), np.zeros(1, np.int32)
    cmask = np.zeros((n_tok, stride), np.uint16)
    args = (cell_pos.ctypes.data, bits.ctypes.data, n_cells, tok_seq.ctypes.data, tok_pos.ctypes.data, n_tok)
    assert L.b200_beam_cells_to_union(*args, idx.ctypes.data, stride, n.ctypes.data, cmask.ctypes.data) == 0
    mask = orc.whisper_beam_mask(cell_pos, bits, tok_seq, tok_pos)   # (n_tok, n_cells) f16: 0 or -inf
    seen = np.flatnonzero((mask == 0).any(axis=0))
    assert idx[:n[0]].tolist() == seen.tolist()
    got = cmask.view(np.float16)
    assert np.array_equal(got[:, :n[0]], mask[:, seen])
    assert np.all(np.isneginf(got[:, n[0]:])) and np.all(idx[n[0]:] == 0)   # the tail is masked out and points at a valid row
    assert L.b200_beam_cells_to_union(*args, idx.ctypes.data, 8, n.ctypes.data, cmask.ctypes.data) == abi.E_LIMIT
