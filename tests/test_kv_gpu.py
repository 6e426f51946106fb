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
