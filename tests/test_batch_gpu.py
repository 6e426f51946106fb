"""Index lists instead of a dense beam mask, and batched launches over units of different lengths
(per-unit q_len / kv_len tables instead of a padding mask), through the C-ABI against the oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

from crispasr_b200 import abi
from tests.util import assert_close, errors, gpu_op, randn_f16

pytestmark = pytest.mark.gpu


def _beam_pool(rng, n_cells, n_beams, prefix, suffix, scatter):
    """A whisper-style cell pool: `prefix` cells shared by every beam (positions 0..prefix-1), then `suffix[j]`
    private cells per beam; `scatter` places them at random slots of the pool instead of packing them at the front.
    Returns cell_pos, cell_seq_bits, tok_seq, tok_pos."""
    cell_pos = np.full(n_cells, -1, np.int32)
    bits = np.zeros(n_cells, np.uint32)
    need = prefix + int(sum(suffix))
    slots = rng.permutation(n_cells)[:need] if scatter else np.arange(need)
    it = iter(slots)
    for p in range(prefix):
        c = next(it)
        cell_pos[c], bits[c] = p, (1 << n_beams) - 1
    for j in range(n_beams):
        for p in range(suffix[j]):
            c = next(it)
            cell_pos[c], bits[c] = prefix + p, 1 << j
    tok_pos = np.array([prefix + suffix[j] - 1 for j in range(n_beams)], np.int32)
    return cell_pos, bits, np.arange(n_beams, dtype=np.int32), tok_pos


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
@pytest.mark.parametrize("case", ["packed", "scattered", "one beam empty"])
def test_index_lists_equal_the_dense_mask_form(b200, orc, kv, case):
    """Decoder self-attention over a pooled beam cache (src/crispasr.cpp:3163-3222): the reference form gives every
    beam (query row) the whole pool and an F16 membership mask [n_kv, n_beams] (:3467-3499); the index form makes
    each beam a batch entry that gathers only its own cells.  Both are compared with the oracle run with the
    reference's mask, and with each other.  (They are equal within the parity tolerance, not bit for bit: compacting
    the keys changes which keys share an MMA step and a rescale, i.e. the fp32 summation order.)"""
    rng = np.random.default_rng({"packed": 1, "scattered": 2, "one beam empty": 3}[case])
    H, hd, n_beams, n_cells = 20 if kv == "f16" else 4, 64, 5, 640
    suffix = [70, 33, 1, 64, 12] if case != "one beam empty" else [70, 0, 1, 64, 12]
    prefix = 57 if case != "one beam empty" else 0
    cell_pos, bits, tok_seq, tok_pos = _beam_pool(rng, n_cells, n_beams, prefix, suffix, scatter=(case == "scattered"))
    if case == "one beam empty":
        tok_pos[1] = 0      # beam 1 owns no cell at all
    q = (rng.standard_normal((1, H, n_beams, hd)) * 0.5).astype(np.float16).astype(np.float32)
    kf = (rng.standard_normal((1, H, n_cells, hd)) * 0.5).astype(np.float32)
    vf = (rng.standard_normal((1, H, n_cells, hd)) * 0.5).astype(np.float32)
    kw = dict(scale=1.0)
    if kv == "q8_0":
        k, v = orc.quantize_q8_0(kf), orc.quantize_q8_0(vf)
        kw["kv_type"] = abi.Q8_0
    else:
        k, v = kf.astype(np.float16), vf.astype(np.float16)
    mask = orc.whisper_beam_mask(cell_pos, bits, tok_seq, tok_pos)[None, None]     # (1, 1, n_beams, n_cells)
    ref = orc.flash_attn_ext(q, k, v, mask, **kw)                                  # (1, n_beams, H, hd)
    dense = gpu_op(b200, q, k, v, mask, **kw)
    assert_close(dense, ref, "dense mask form")
    stride = 192
    idx, lens = np.zeros((n_beams, stride), np.int32), np.zeros(n_beams, np.int32)
    rc = b200.lib().b200_beam_cells_to_index(cell_pos.ctypes.data, bits.ctypes.data, n_cells, tok_seq.ctypes.data,
                                             tok_pos.ctypes.data, n_beams, idx.ctypes.data, stride, lens.ctypes.data)
    assert rc == 0 and lens.tolist() == [prefix + s for s in suffix]
    qb = np.ascontiguousarray(q.transpose(2, 1, 0, 3))                             # (n_beams, H, 1, hd): a beam = a batch entry
    got = gpu_op(b200, qb, k, v, kv_index=idx, kv_len=lens, **kw)                  # (n_beams, 1, H, hd)
    assert b200.lib().b200_last_kernel() == abi.KERNEL_DECODE_SPLIT
    got = got.reshape(1, n_beams, H, hd)
    assert_close(got, ref, "index form vs oracle")
    ma, rl = errors(got, dense)
    assert ma <= 2e-3 and rl <= 1e-3, f"index form vs dense form: {ma:.2e} / {rl:.2e}"
    if case == "one beam empty":
        assert not got[0, 1].any() and not dense[0, 1].any()
    if kv == "f16":
        # the shared form: one list with the union of the live cells, the beams as query rows, a compact mask over the
        # list's entries - every live cell read once for all beams
        ustride = 256
        uidx, ulen, umask = np.zeros(ustride, np.int32), np.zeros(1, np.int32), np.zeros((n_beams, ustride), np.uint16)
        rc = b200.lib().b200_beam_cells_to_union(cell_pos.ctypes.data, bits.ctypes.data, n_cells, tok_seq.ctypes.data,
                                                 tok_pos.ctypes.data, n_beams, uidx.ctypes.data, ustride, ulen.ctypes.data,
                                                 umask.ctypes.data)
        live = np.flatnonzero((mask[0, 0] == 0).any(axis=0))
        assert rc == 0 and ulen[0] == len(live) and uidx[:ulen[0]].tolist() == live.tolist()
        assert np.array_equal(umask.view(np.float16)[:, :ulen[0]], mask[0, 0][:, live])
        got_u = gpu_op(b200, q, k, v, umask.view(np.float16)[None, None], kv_index=uidx[None], kv_len=ulen, **kw)
        assert b200.lib().b200_last_kernel() == abi.KERNEL_DECODE_SPLIT
        assert_close(got_u, ref, "shared list + compact mask vs oracle")
    # every forced split count merges to the same result
    for ns in (1, 2, 3):
        assert b200.lib().b200_set_decode_splits(ns) == 0
        try:
            assert_close(gpu_op(b200, qb, k, v, kv_index=idx, kv_len=lens, **kw).reshape(1, n_beams, H, hd), ref, f"index form, {ns} splits")
        finally:
            b200.lib().b200_set_decode_splits(0)


def test_shared_lists_over_a_batch_of_segments(b200, orc):
    """Three segments in one launch, each with its own pool state: one shared list + compact mask per segment
    (list stride 200: not a multiple of the 64-key tile), lengths 0 (a segment whose beams see nothing yet), 37 and
    200 (a full list), every forced split count.  The oracle sees each segment's dense pool and the reference's mask."""
    rng = np.random.default_rng(12)
    S, H, hd, n_beams, n_cells, stride = 3, 4, 64, 5, 512, 200
    q = (rng.standard_normal((S, H, n_beams, hd)) * 0.5).astype(np.float16)
    k = (rng.standard_normal((S, H, n_cells, hd)) * 0.5).astype(np.float16)
    v = (rng.standard_normal((S, H, n_cells, hd)) * 0.5).astype(np.float16)
    uidx, ulen = np.zeros((S, stride), np.int32), np.zeros(S, np.int32)
    umask = np.zeros((S, 1, n_beams, stride), np.uint16)
    dense = np.full((S, 1, n_beams, n_cells), -np.inf, np.float16)
    pools = [(0, [0, 0, 0, 0, 0]), (12, [9, 3, 1, 7, 5]), (100, [20, 20, 20, 20, 20])]
    for s, (prefix, suffix) in enumerate(pools):
        cell_pos, bits, tok_seq, tok_pos = _beam_pool(rng, n_cells, n_beams, prefix, suffix, scatter=True)
        if s == 0:
            tok_pos[:] = -1     # nothing is at or before position -1: no beam sees any cell
        one = np.zeros(1, np.int32)
        rc = b200.lib().b200_beam_cells_to_union(cell_pos.ctypes.data, bits.ctypes.data, n_cells, tok_seq.ctypes.data,
                                                 tok_pos.ctypes.data, n_beams, uidx[s].ctypes.data, stride, one.ctypes.data,
                                                 umask[s, 0].ctypes.data)
        assert rc == 0
        ulen[s] = one[0]
        dense[s, 0] = orc.whisper_beam_mask(cell_pos, bits, tok_seq, tok_pos)
    assert ulen.tolist() == [0, 37, 200]
    ref = orc.flash_attn_ext(q, k, v, dense, scale=1.0)
    for ns in (0, 1, 2, 3):
        assert b200.lib().b200_set_decode_splits(ns) == 0
        try:
            got = gpu_op(b200, q, k, v, umask.view(np.float16), kv_index=uidx, kv_len=ulen, scale=1.0)
        finally:
            b200.lib().b200_set_decode_splits(0)
        assert b200.lib().b200_last_kernel() == abi.KERNEL_DECODE_SPLIT
        assert_close(got, ref, f"shared lists, {ns} splits")
        assert not got[0].any()


def test_index_lists_are_refused_where_no_kernel_has_them(b200):
    q = torch.zeros((2, 4, 300, 64), dtype=torch.float16, device="cuda")
    k = torch.zeros((1, 4, 512, 64), dtype=torch.float16, device="cuda")
    idx = torch.zeros((2, 64), dtype=torch.int32, device="cuda")
    lens = torch.zeros(2, dtype=torch.int32, device="cuda")
    with pytest.raises(b200.B200Error) as e:
        b200.flash_attn_ext(q, k, k, scale=1.0, kv_index=idx, kv_len=lens)       # prefill-sized: not the decode kernel
    assert e.value.code == abi.E_UNSUPPORTED
    qd = torch.zeros((2, 4, 1, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(b200.B200Error) as e:
        b200.flash_attn_ext(qd, k, k, scale=1.0, kv_index=idx)                   # lists need their lengths
    assert e.value.code == abi.E_NULL


def _ragged(rng, lens, Tmax, H, hd, garbage=7.0):
    """Padded (B, H, Tmax, hd) f16 with random live rows and finite garbage in the padding."""
    x = np.full((len(lens), H, Tmax, hd), garbage, np.float16)
    for b, n in enumerate(lens):
        x[b, :, :n] = randn_f16(rng, (H, n, hd))
    return x


@pytest.mark.parametrize("form", ["hd64", "hd128 gqa causal q8_0", "relpos", "tile kernel"])
def test_batched_units_of_different_lengths_equal_per_unit_launches(b200, orc, form):
    """One launch over units of different lengths (concatenated on ne[3], padded to the longest, lengths in
    ext->q_len / ext->kv_len) against the oracle run unit by unit on the unpadded operands, and against per-unit
    launches of the library itself; rows of the padding come back as zeros."""
    rng = np.random.default_rng(50)
    L = b200.lib()
    if form == "hd64":
        H, Hkv, hd, qlens, klens = 6, 6, 64, [300, 1, 129, 0, 256], [300, 77, 129, 50, 256]
        kw = dict(scale=0.125)
    elif form == "hd128 gqa causal q8_0":
        H, Hkv, hd, qlens, klens = 8, 2, 128, [200, 64, 131], [260, 64, 140]     # new tokens are the LAST q_len keys
        kw = dict(scale=128 ** -0.5, causal=True)
    elif form == "relpos":
        H, Hkv, hd, qlens = 4, 4, 128, [333, 130, 257]
        klens = qlens
        kw = dict(scale=128 ** -0.5)
    else:
        H, Hkv, hd, qlens, klens = 4, 2, 80, [100, 3, 64], [150, 90, 64]
        kw = dict(scale=0.11, softcap=4.0)
    B, Tq, Lk = len(qlens), max(qlens), max(klens)
    q = _ragged(rng, qlens, Tq, H, hd).astype(np.float32)
    kf, vf = _ragged(rng, klens, Lk, Hkv, hd), _ragged(rng, klens, Lk, Hkv, hd)
    extra = {}
    if form == "hd128 gqa causal q8_0":
        k, v = orc.quantize_q8_0(kf.astype(np.float32)), orc.quantize_q8_0(vf.astype(np.float32))
        kw["kv_type"] = abi.Q8_0
    else:
        k, v = kf, vf
    if form == "relpos":
        extra["q_v"] = _ragged(rng, qlens, Tq, H, hd).astype(np.float32)
        pe = orc.make_pos_enc(H * hd, Tq)
        w = (rng.standard_normal((H * hd, H * hd)) / 32.0).astype(np.float32)
        extra["r"] = np.ascontiguousarray((pe @ w).reshape(2 * Tq - 1, H, hd).transpose(1, 0, 2)[None]).astype(np.float16)
    if form == "tile kernel":
        L.b200_set_kernel_override(abi.KERNEL_TILE_MMA)
    try:
        got = gpu_op(b200, q, k, v, q_len=qlens, kv_len=klens, **kw, **extra)
        kern = L.b200_last_kernel()
        for b in range(B):
            nq, nk = qlens[b], klens[b]
            assert not got[b, nq:].any(), f"unit {b}: padding rows must be zero"
            if nq == 0:
                continue
            okw = {x: y for x, y in kw.items() if x != "causal"}
            if form == "relpos":
                # the unit alone, with the table of ITS length: the same relative positions
                r_b = extra["r"][:, :, Tq - nq: Tq - nq + 2 * nq - 1]
                okw.update(q_v=extra["q_v"][b:b + 1, :, :nq], r=np.ascontiguousarray(r_b))
            if kw.get("causal"):
                okw.update(causal=True, n_past=nk - nq)
            ref = orc.flash_attn_ext(q[b:b + 1, :, :nq], k[b:b + 1, :, :nk], v[b:b + 1, :, :nk], **okw)
            assert_close(got[b:b + 1, :nq], ref, f"{form}: unit {b} of the batched launch")
            alone = gpu_op(b200, np.ascontiguousarray(q[b:b + 1, :, :nq]), np.ascontiguousarray(k[b:b + 1, :, :nk]),
                           np.ascontiguousarray(v[b:b + 1, :, :nk]), **okw)
            ma, rl = errors(got[b:b + 1, :nq], alone)
            assert ma <= 2e-3 and rl <= 1e-3, f"{form}: unit {b} batched vs alone {ma:.2e} / {rl:.2e}"
    finally:
        L.b200_set_kernel_override(abi.KERNEL_NONE)
    if form in ("hd64", "hd128 gqa causal q8_0", "relpos"):
        assert kern == abi.KERNEL_PREFILL_TC5
    assert L.b200_device_status() == 0


def test_slot_table_drives_a_decode_batch(b200, orc):
    """b200_batch over a Q8_0 cache with 6 stream slots: streams join with different cache lengths, every step
    appends one row per resident stream and attends with the tables b200_batch_tables uploads; a stream that
    leaves frees its slot (zero rows, zero keys: zero output, no work) and a new one takes the hole."""
    rng = np.random.default_rng(51)
    L = b200.lib()
    S, H, Hkv, hd, ctx = 6, 16, 4, 128, 160
    scale = hd ** -0.5
    kvc = b200.KvCache(abi.Q8_0, hd, Hkv, n_layers=1, max_ctx=ctx, n_streams=S)
    h = C.c_void_p()
    assert L.b200_batch_create(S, C.byref(h)) == 0
    host_k = np.zeros((S, Hkv, ctx, hd), np.float32)
    host_v = np.zeros_like(host_k)
    st = torch.cuda.current_stream().cuda_stream

    def join(unit, n0):
        slot = L.b200_batch_add(h, unit, 1, n0)
        assert slot >= 0
        kk, vv = rng.standard_normal((Hkv, n0, hd)).astype(np.float32), rng.standard_normal((Hkv, n0, hd)).astype(np.float32)
        host_k[slot, :, :n0], host_v[slot, :, :n0] = kk, vv
        full_k, full_v = torch.zeros((S, Hkv, n0, hd), device="cuda"), torch.zeros((S, Hkv, n0, hd), device="cuda")
        full_k[slot], full_v[slot] = torch.from_numpy(kk).cuda(), torch.from_numpy(vv).cuda()
        pos = torch.full((S,), ctx + 5, dtype=torch.int32, device="cuda")   # out-of-range rows are dropped: only `slot` is written
        pos[slot] = 0
        kvc.append(0, full_k, full_v, pos=pos)
        return slot

    def step(check):
        """Append one token to every resident stream, attend, compare with the oracle."""
        span, act = C.c_int(), C.c_int()
        L.b200_batch_span(h, C.byref(span), C.byref(act), None, None)
        lens = np.zeros(S, np.int32)
        for s_ in range(S):
            ql, kl = C.c_int(), C.c_int()
            L.b200_batch_lengths(h, s_, C.byref(ql), C.byref(kl))
            lens[s_] = kl.value
        live = [s_ for s_ in range(S) if L.b200_batch_unit(h, s_) >= 0]
        kn, vn = rng.standard_normal((S, Hkv, 1, hd)).astype(np.float32), rng.standard_normal((S, Hkv, 1, hd)).astype(np.float32)
        pos = np.full(S, ctx + 5, np.int32)
        for s_ in live:
            host_k[s_, :, lens[s_]], host_v[s_, :, lens[s_]] = kn[s_, :, 0], vn[s_, :, 0]
            pos[s_] = lens[s_]
        kvc.append(0, torch.from_numpy(kn).cuda(), torch.from_numpy(vn).cuda(), pos=torch.from_numpy(pos).cuda())
        assert L.b200_batch_advance(h, 1) == 0
        qd, kd = C.c_void_p(), C.c_void_p()
        assert L.b200_batch_tables(h, st, C.byref(qd), C.byref(kd)) == 0
        n = span.value
        q = rng.standard_normal((S, H, 1, hd)).astype(np.float16).astype(np.float32)
        q_dev = torch.from_numpy(q[:n]).cuda()        # kept alive until the launch has run
        tq = abi.from_torch(q_dev)
        tk, tv = kvc.view(0, ctx)
        tk.ne[3] = tv.ne[3] = n                       # the launch covers the span only
        dst = torch.full((n, 1, H, hd), 9.0, dtype=torch.float32, device="cuda")
        td = abi.from_torch(dst)
        p, e = abi.Params(scale, 0.0, 0.0, 0), abi.Ext()
        e.q_len, e.kv_len = qd.value, kd.value
        nb = C.c_size_t(0)
        assert L.b200_fattn_workspace_bytes(C.byref(tq), C.byref(tk), C.byref(tv), None, C.byref(td), C.byref(p), C.byref(e), C.byref(nb)) == 0
        ws = torch.empty(max(nb.value, 256), dtype=torch.uint8, device="cuda")
        rc = L.b200_fattn_launch(C.byref(tq), C.byref(tk), C.byref(tv), None, C.byref(td), C.byref(p), C.byref(e), ws.data_ptr(), ws.numel(), st)
        assert rc == 0, L.b200_strerror(rc)
        torch.cuda.synchronize()
        out = dst.cpu().numpy()
        if check:
            for s_ in range(n):
                if s_ in live:
                    nk = int(lens[s_]) + 1
                    ref = orc.flash_attn_ext(q[s_:s_ + 1], orc.quantize_q8_0(host_k[s_:s_ + 1, :, :nk]),
                                             orc.quantize_q8_0(host_v[s_:s_ + 1, :, :nk]), scale=scale, kv_type=abi.Q8_0)
                    assert_close(out[s_:s_ + 1], ref, f"slot {s_}")
                else:
                    assert not out[s_].any(), f"free slot {s_} must give zeros"
        return n

    slots = [join(100 + i, n0) for i, n0 in enumerate([70, 1, 33, 64, 100])]
    assert slots == [0, 1, 2, 3, 4]
    assert step(True) == 5
    assert L.b200_batch_remove(h, 1) == 0 and L.b200_batch_remove(h, 4) == 0
    assert step(True) == 4                              # span shrinks to the highest live slot; slot 1 is a hole
    assert join(200, 17) == 1                           # the hole is reused, its old rows are overwritten from row 0
    for _ in range(3):
        step(False)
    assert step(True) == 4
    L.b200_batch_destroy(h)
    kvc.close()
