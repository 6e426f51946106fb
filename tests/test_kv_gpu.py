"""KV slab allocator and the append kernels (F32 -> F16 / Q8_0 on write)."""
import ctypes as C

import numpy as np
import pytest
import torch

from crispasr_b200 import abi
from tests.util import XorShift, assert_close

pytestmark = pytest.mark.gpu


def _read_slab(t: abi.Tensor, nbytes):
    buf = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    C.cdll.LoadLibrary("libcudart.so").cudaMemcpy(C.c_void_p(buf.data_ptr()), C.c_void_p(t.data), C.c_size_t(nbytes), 3)
    torch.cuda.synchronize()
    return buf.cpu().numpy()


@pytest.mark.parametrize("type_", [abi.F16, abi.Q8_0])
def test_append_matches_oracle_bits(b200, orc, type_):
    """Prefill rows then one appended decode row (tests/test-kv-quant-roundtrip.cpp second case), bit-exact
    against the oracle's quantiser, which is itself pinned to gguf-py."""
    hd, heads, streams, ctx = 128, 2, 3, 40
    kv = b200.KvCache(type_, hd, heads, n_layers=2, max_ctx=ctx, n_streams=streams)
    r = XorShift(0x371)
    pre = r.fill(streams * heads * 3 * hd).reshape(streams, heads, 3, hd)
    step = r.fill(streams * heads * hd).reshape(streams, heads, 1, hd)
    pre[0, 0, 0, :32] = 0.0
    tp, ts = torch.from_numpy(pre).cuda(), torch.from_numpy(step).cuda()
    kv.append(1, tp, tp * 0.5, pos0=0)
    pos = torch.tensor([3, 3, 3], dtype=torch.int32, device="cuda")
    kv.append(1, ts, ts * 0.5, pos=pos)
    torch.cuda.synchronize()
    k, v = kv.view(1, 4)
    assert k.data % 1024 == 0 and v.data % 1024 == 0 and k.nb[2] % 16 == 0
    row = k.nb[1]
    raw = _read_slab(k, k.nb[3] * streams).reshape(streams, heads, -1, row)[:, :, :4]
    want = np.concatenate([pre, step], 2)
    if type_ == abi.Q8_0:
        assert np.array_equal(raw, orc.quantize_q8_0(want))
        assert np.abs(orc.dequantize_q8_0(raw) - want).max() <= 0.02
    else:
        assert np.array_equal(raw.view(np.float16).reshape(want.shape), want.astype(np.float16))
    rawv = _read_slab(v, v.nb[3] * streams).reshape(streams, heads, -1, row)[:, :, :4]
    wantv = want * np.float32(0.5)
    if type_ == abi.Q8_0:
        assert np.array_equal(rawv, orc.quantize_q8_0(wantv))
    # layer 0 untouched (zero-cleared)
    k0, _ = kv.view(0, 4)
    assert not _read_slab(k0, k0.nb[3] * streams).any()
    kv.close()


@pytest.mark.parametrize("type_", [abi.F16, abi.Q8_0])
def test_decode_through_slab(b200, orc, type_):
    """append -> view -> attention launch, descriptors straight from the allocator."""
    rng = np.random.default_rng(21)
    hd, Hkv, H, S, L = 128, 8, 32, 4, 300
    kv = b200.KvCache(type_, hd, Hkv, n_layers=1, max_ctx=512, n_streams=S)
    kn = rng.standard_normal((S, Hkv, L, hd)).astype(np.float32)
    vn = rng.standard_normal((S, Hkv, L, hd)).astype(np.float32)
    kv.append(0, torch.from_numpy(kn).cuda(), torch.from_numpy(vn).cuda(), pos0=0)
    tk, tv = kv.view(0, L)
    q = torch.from_numpy(rng.standard_normal((S, H, 1, hd)).astype(np.float16).astype(np.float32)).cuda()
    dst = torch.empty((S, 1, H, hd), dtype=torch.float32, device="cuda")
    tq, td = abi.from_torch(q), abi.from_torch(dst)
    p = abi.Params(hd ** -0.5, 0.0, 0.0, 0)
    L_ = b200.lib()
    n = C.c_size_t(0)
    assert L_.b200_fattn_workspace_bytes(C.byref(tq), C.byref(tk), C.byref(tv), None, C.byref(td), C.byref(p), None, C.byref(n)) == 0
    ws = torch.empty(max(n.value, 1), dtype=torch.uint8, device="cuda")
    rc = L_.b200_fattn_launch(C.byref(tq), C.byref(tk), C.byref(tv), None, C.byref(td), C.byref(p), None,
                              ws.data_ptr(), n.value, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L_.b200_strerror(rc)
    torch.cuda.synchronize()
    if type_ == abi.Q8_0:
        kq, vq = orc.quantize_q8_0(kn), orc.quantize_q8_0(vn)
        ref = orc.flash_attn_ext(q.cpu().numpy(), kq, vq, scale=hd ** -0.5, kv_type=abi.Q8_0)
    else:
        ref = orc.flash_attn_ext(q.cpu().numpy(), kn.astype(np.float16), vn.astype(np.float16), scale=hd ** -0.5)
    assert_close(dst.cpu().numpy(), ref, "decode through slab")
    kv.close()


def _launch_on_views(b200, q, tk, tv, dst, scale, kv_len=None, causal=False):
    """b200_fattn_launch with K/V descriptors straight from the allocator."""
    tq, td = abi.from_torch(q), abi.from_torch(dst)
    p = abi.Params(scale, 0.0, 0.0, 0)
    e = abi.Ext()
    e.causal = int(causal)
    if kv_len is not None:
        e.kv_len = kv_len.data_ptr()
    L_ = b200.lib()
    n = C.c_size_t(0)
    assert L_.b200_fattn_workspace_bytes(C.byref(tq), C.byref(tk), C.byref(tv), None, C.byref(td), C.byref(p), C.byref(e), C.byref(n)) == 0
    ws = torch.empty(max(n.value, 256), dtype=torch.uint8, device="cuda")
    rc = L_.b200_fattn_launch(C.byref(tq), C.byref(tk), C.byref(tv), None, C.byref(td), C.byref(p), C.byref(e),
                              ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L_.b200_strerror(rc)
    return ws   # kept alive by the caller until the stream has been synchronised


def test_llm_decode_loop_on_one_slab(b200, orc):
    """The whole decode loop of the LLM runtimes on one Q8_0 cache (src/voxtral.cpp:1176-1224 around
    core_attn::kv_self_attn, src/core/attention.h:840-867): causal prefill of 375 audio + 32 text tokens into the
    cache, then 256 steps of (quantise-on-append at a DEVICE position per stream, single-token attention with a
    DEVICE kv_len per stream), 8 streams, GQA 32/8, head_dim 128, nothing synchronised between steps.  After the
    prefill the streams are cut to ragged lengths, so appends overwrite rows and every stream grows from its own
    length.  The prefill result and decode steps 1, 128 and 256 are compared with the oracle run on a cache that was
    quantised on the host."""
    rng = np.random.default_rng(3)
    S, H, Hkv, hd, T0, steps = 8, 32, 8, 128, 407, 256
    scale = hd ** -0.5
    kv = b200.KvCache(abi.Q8_0, hd, Hkv, n_layers=1, max_ctx=T0 + steps, n_streams=S)
    k_pre = rng.standard_normal((S, Hkv, T0, hd)).astype(np.float32)
    v_pre = rng.standard_normal((S, Hkv, T0, hd)).astype(np.float32)
    kv.append(0, torch.from_numpy(k_pre).cuda(), torch.from_numpy(v_pre).cuda(), pos0=0)
    # ---- prefill: every stream attends causally to its own 407 rows ----
    qp = torch.from_numpy(rng.standard_normal((S, H, T0, hd)).astype(np.float16).astype(np.float32)).cuda()
    out_p = torch.empty((S, T0, H, hd), dtype=torch.float32, device="cuda")
    tk, tv = kv.view(0, T0)
    keep = [_launch_on_views(b200, qp, tk, tv, out_p, scale, causal=True)]
    torch.cuda.synchronize()
    kq_pre, vq_pre = orc.quantize_q8_0(k_pre), orc.quantize_q8_0(v_pre)
    for s_ in (0, 5):
        ref = orc.flash_attn_ext(qp[s_:s_ + 1].cpu().numpy(), kq_pre[s_:s_ + 1], vq_pre[s_:s_ + 1], scale=scale,
                                 kv_type=abi.Q8_0, causal=True)
        assert_close(out_p[s_:s_ + 1].cpu().numpy(), ref, f"prefill, stream {s_}")
    # ---- decode: ragged starting lengths, device-side positions ----
    len0 = np.array([T0 - 5 * s_ for s_ in range(S)], np.int32)
    pos = torch.from_numpy(len0.copy()).cuda()            # row the next token of each stream is written to
    kv_len = pos + 1
    k_new = rng.standard_normal((steps, S, Hkv, 1, hd)).astype(np.float32)
    v_new = rng.standard_normal((steps, S, Hkv, 1, hd)).astype(np.float32)
    q_all = rng.standard_normal((steps, S, H, 1, hd)).astype(np.float16).astype(np.float32)
    dk, dv, dq = torch.from_numpy(k_new).cuda(), torch.from_numpy(v_new).cuda(), torch.from_numpy(q_all).cuda()
    outs = torch.empty((steps, S, 1, H, hd), dtype=torch.float32, device="cuda")
    tk, tv = kv.view(0, T0 + steps)
    for t in range(steps):
        kv.append(0, dk[t], dv[t], pos=pos)
        keep.append(_launch_on_views(b200, dq[t], tk, tv, outs[t], scale, kv_len=kv_len))
        pos += 1
        kv_len += 1
    torch.cuda.synchronize()
    assert b200.lib().b200_last_kernel() == abi.KERNEL_DECODE_SPLIT and b200.lib().b200_device_status() == 0
    for t in (0, 127, 255):
        kq = np.zeros((S, Hkv, T0 + steps, hd // 32 * 34), np.uint8)
        vq = np.zeros_like(kq)
        for s_ in range(S):
            L0 = int(len0[s_])
            kq[s_, :, :L0], vq[s_, :, :L0] = kq_pre[s_, :, :L0], vq_pre[s_, :, :L0]
            kq[s_, :, L0:L0 + t + 1] = orc.quantize_q8_0(k_new[:t + 1, s_, :, 0].transpose(1, 0, 2))
            vq[s_, :, L0:L0 + t + 1] = orc.quantize_q8_0(v_new[:t + 1, s_, :, 0].transpose(1, 0, 2))
        ref = orc.flash_attn_ext(q_all[t], kq, vq, scale=scale, kv_type=abi.Q8_0, kv_len=len0 + t + 1)
        assert_close(outs[t].cpu().numpy(), ref, f"decode step {t + 1}")
    kv.close()


def test_copy_stream_forks_a_beam(b200):
    """kv_snapshot_pool semantics: after the copy the destination stream reads the source's first n rows, other
    streams and rows beyond n are untouched."""
    hd, heads, streams = 64, 3, 4
    kv = b200.KvCache(abi.F16, hd, heads, n_layers=2, max_ctx=64, n_streams=streams)
    rng = np.random.default_rng(5)
    x = torch.from_numpy(rng.standard_normal((streams, heads, 40, hd)).astype(np.float32)).cuda()
    for layer in range(2):
        kv.append(layer, x + layer, x - layer, pos0=0)
    kv.copy_stream(dst_stream=2, src_stream=0, n_rows=25)
    torch.cuda.synchronize()
    for layer in range(2):
        k, _ = kv.view(layer, 40)
        raw = _read_slab(k, k.nb[3] * streams).view(np.float16).reshape(streams, heads, -1, hd)[:, :, :40]
        want = (x + layer).cpu().numpy().astype(np.float16)
        assert np.array_equal(raw[2, :, :25], want[0, :, :25])
        assert np.array_equal(raw[2, :, 25:], want[2, :, 25:])
        assert np.array_equal(raw[[0, 1, 3]], want[[0, 1, 3]])
    kv.close()


def test_scheduler_on_device(b200, orc):
    """Units processed by the per-GPU worker thread on its own stream."""
    rng = np.random.default_rng(7)
    n = 6
    qs = [torch.from_numpy(rng.standard_normal((1, 4, 100, 64)).astype(np.float16)).cuda() for _ in range(n)]
    outs = [None] * n

    def unit(dev, u, stream):
        outs[u] = b200.flash_attn_ext(qs[u], qs[u], qs[u], scale=0.125, stream=stream)
        return 0
    s = b200.SegmentScheduler(devices=[0])
    failed, owners = s.run(n, unit)
    assert failed == 0 and owners == [0] * n
    for u in range(n):
        x = qs[u].cpu().numpy()
        assert_close(outs[u].cpu().numpy(), orc.flash_attn_ext(x, x, x, scale=0.125), f"unit {u}")
    s.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_batched_scheduler_over_two_gpus_equals_one(b200, orc):
    """b200_sched_run_batched over two devices: each worker receives its static share as one batch on its own device
    and stream, unit_device covers both workers, and the outputs equal a one-GPU run of the same units bit for bit."""
    rng = np.random.default_rng(8)
    n, H, T, hd = 6, 4, 200, 64
    q = rng.standard_normal((n, H, T, hd)).astype(np.float16)
    ref_dev = b200.flash_attn_ext(*(torch.from_numpy(q).cuda(0),) * 3, scale=0.125)
    torch.cuda.synchronize(0)
    outs = {}

    def batch(dev, first, count, stream):
        with torch.cuda.device(dev):
            x = torch.from_numpy(q[first:first + count]).cuda(dev)
            outs[first] = (dev, b200.flash_attn_ext(x, x, x, scale=0.125, stream=stream))
            torch.cuda.current_stream(dev).synchronize()   # the upload ran on torch's stream
        return 0
    s = b200.SegmentScheduler(devices=[0, 1])
    failed, owners = s.run_batched(n, n, batch, steal=False)
    assert failed == 0 and owners == [0, 0, 0, 1, 1, 1]
    for first, (dev, out) in outs.items():
        torch.cuda.synchronize(dev)
        assert torch.equal(out.cpu(), ref_dev[first:first + out.shape[0]].cpu())
    s.close()
