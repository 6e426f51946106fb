"""Python call surface over the C-ABI, shaped like ggml_flash_attn_ext(q, k, v, mask, scale, max_bias,
logit_softcap) (reference call sites: src/crispasr.cpp:2821, src/core/attention.h:992).

Tensors are torch tensors in torch order (slowest first): q (B,H,Tq,hd), k/v (Bk,Hkv,Lk,hd) or uint8
Q8_0 block rows (Bk,Hkv,Lk,hd/32*34), mask (1|B,1|H,Tq,Lk) f16; the result is (B,Tq,H,hd) f32, i.e.
ggml's dst [hd,H,Tq,B].  Any of them may be a strided view.
"""
from __future__ import annotations

import ctypes as C

from . import abi


def _lib():
    from . import lib
    return lib()


def _err(code, where):
    from . import B200Error
    return B200Error(code, where)


class _Call:
    """Descriptors of one op call; keeps every ctypes object alive for the duration of the call."""

    def __init__(self, q, k, v, mask, dst, scale, max_bias, softcap, kv_type, causal, n_past, kv_len, q_v, r,
                 relpos_bias_f32, conv, pos_bias_u=None, pos_bias_v=None, kv_index=None, q_len=None):
        self.q, self.k, self.v = conv(q), conv(k, kv_type), conv(v, kv_type)
        self.mask = conv(mask) if mask is not None else None
        self.dst = conv(dst)
        self.params = abi.Params(float(scale), float(max_bias), float(softcap), 0)
        self.ext = abi.Ext()
        if q_v is not None:
            self.qv = conv(q_v)
            self.ext.q_v = C.pointer(self.qv)
        if r is not None:
            self.r = conv(r)
            self.ext.r = C.pointer(self.r)
        if pos_bias_u is not None:  # (H, hd) f32: Q_u = Q + pos_bias_u formed inside the op
            self.bu = conv(pos_bias_u)
            self.ext.pos_bias_u = C.pointer(self.bu)
        if pos_bias_v is not None:
            self.bv = conv(pos_bias_v)
            self.ext.pos_bias_v = C.pointer(self.bv)
        self.ext.causal, self.ext.n_past = int(bool(causal)), int(n_past)
        self.kv_len = kv_len
        if kv_len is not None:
            self.ext.kv_len = kv_len.data_ptr() if hasattr(kv_len, "data_ptr") else kv_len.ctypes.data
        self.ext.relpos_bias_f32 = int(bool(relpos_bias_f32))
        self.kv_index, self.q_len = kv_index, q_len
        if kv_index is not None:   # int32 (B, stride): cache row of each logical key
            self.ext.kv_index = kv_index.data_ptr() if hasattr(kv_index, "data_ptr") else kv_index.ctypes.data
            self.ext.kv_index_stride = int(kv_index.shape[-1])
        if q_len is not None:      # int32 (B,): valid query rows per batch entry
            self.ext.q_len = q_len.data_ptr() if hasattr(q_len, "data_ptr") else q_len.ctypes.data

    def args(self):
        return (C.byref(self.q), C.byref(self.k), C.byref(self.v),
                C.byref(self.mask) if self.mask is not None else None, C.byref(self.dst), C.byref(self.params),
                C.byref(self.ext))


def _dst_like(q, device=None):
    import torch
    B, H, Tq, hd = q.shape
    return torch.empty((B, Tq, H, hd), dtype=torch.float32, device=device if device is not None else q.device)


def _make(q, k, v, mask, dst, kw, conv):
    return _Call(q, k, v, mask, dst, kw["scale"], kw.get("max_bias", 0.0), kw.get("softcap", 0.0),
                 kw.get("kv_type"), kw.get("causal", False), kw.get("n_past", 0), kw.get("kv_len"), kw.get("q_v"),
                 kw.get("r"), kw.get("relpos_bias_f32", False), conv, kw.get("pos_bias_u"), kw.get("pos_bias_v"),
                 kw.get("kv_index"), kw.get("q_len"))


def supports(q, k, v, mask=None, **kw) -> bool:
    """b200_fattn_supports: True when the launch would accept these operands (no device work)."""
    c = _make(q, k, v, mask, _dst_like(q), kw, abi.from_torch)
    why = C.c_int(0)
    return bool(_lib().b200_fattn_supports(*c.args(), C.byref(why)))


def plan(q, k, v, mask=None, **kw):
    """(kernel id, n_splits) the launch would use."""
    c = _make(q, k, v, mask, _dst_like(q), kw, abi.from_torch)
    kern, ns = C.c_int(0), C.c_int(0)
    rc = _lib().b200_fattn_plan(*c.args(), C.byref(kern), C.byref(ns))
    if rc:
        raise _err(rc, "b200_fattn_plan")
    return kern.value, ns.value


def workspace_bytes(q, k, v, mask=None, **kw) -> int:
    c = _make(q, k, v, mask, _dst_like(q), kw, abi.from_torch)
    n = C.c_size_t(0)
    rc = _lib().b200_fattn_workspace_bytes(*c.args(), C.byref(n))
    if rc:
        raise _err(rc, "b200_fattn_workspace_bytes")
    return n.value


def flash_attn_ext(q, k, v, mask=None, *, out=None, workspace=None, stream=None, **kw):
    """Device tensors in, device tensor out; asynchronous on `stream` (default: torch's current stream).
    `workspace` (uint8 device tensor) is allocated here when the launch needs one and none is given."""
    import torch
    if not q.is_cuda:
        raise ValueError("flash_attn_ext takes CUDA tensors; use flash_attn_ext_host for host buffers")
    dst = out if out is not None else _dst_like(q)
    c = _make(q, k, v, mask, dst, kw, abi.from_torch)
    L = _lib()
    n = C.c_size_t(0)
    rc = L.b200_fattn_workspace_bytes(*c.args(), C.byref(n))
    if rc:
        raise _err(rc, "b200_fattn_workspace_bytes")
    ws_ptr, ws_len = None, 0
    if n.value:
        if workspace is None or workspace.numel() < n.value:
            workspace = torch.empty(n.value, dtype=torch.uint8, device=q.device)
        ws_ptr, ws_len = workspace.data_ptr(), workspace.numel()
    st = stream if stream is not None else torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        rc = L.b200_fattn_launch(*c.args(), ws_ptr, ws_len, st)
    if rc:
        raise _err(rc, "b200_fattn_launch")
    return dst


def flash_attn_ext_host(q, k, v, mask=None, *, out=None, **kw):
    """Host (CPU, ideally pinned) tensors in, host tensor out: H2D, compute, D2H inside one C call."""
    dst = out if out is not None else _dst_like(q)
    c = _make(q, k, v, mask, dst, kw, abi.from_torch)
    rc = _lib().b200_fattn_forward_host(*c.args())
    if rc:
        raise _err(rc, "b200_fattn_forward_host")
    return dst


class KvCache:
    """KV-cache slabs (b200_kv_*): the cache tensors of core_attn (src/core/attention.h:593-595)."""

    def __init__(self, type_, head_dim, n_kv_heads, n_layers, max_ctx, n_streams=1):
        self.cfg = abi.KvConfig(type_, head_dim, n_kv_heads, n_layers, max_ctx, n_streams)
        self._h = C.c_void_p()
        rc = _lib().b200_kv_create(C.byref(self.cfg), C.byref(self._h))
        if rc:
            raise _err(rc, "b200_kv_create")

    def close(self):
        if self._h:
            _lib().b200_kv_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass

    @property
    def nbytes(self):
        return _lib().b200_kv_bytes(self._h)

    def view(self, layer, n_rows):
        k, v = abi.Tensor(), abi.Tensor()
        rc = _lib().b200_kv_view(self._h, layer, n_rows, C.byref(k), C.byref(v))
        if rc:
            raise _err(rc, "b200_kv_view")
        return k, v

    def append(self, layer, k_new, v_new, pos=None, pos0=0, stream=None):
        """k_new/v_new: float32 CUDA tensors (n_streams, n_kv, n_new, hd)."""
        import torch
        tk, tv = abi.from_torch(k_new), abi.from_torch(v_new)
        st = stream if stream is not None else torch.cuda.current_stream(k_new.device).cuda_stream
        rc = _lib().b200_kv_append(self._h, layer, C.byref(tk), C.byref(tv),
                                   pos.data_ptr() if pos is not None else None, int(pos0), st)
        if rc:
            raise _err(rc, "b200_kv_append")


    def copy_stream(self, dst_stream, src_stream, n_rows, stream=None):
        """Fork a hypothesis: rows [0, n_rows) of every layer/head from one stream to another (kv_snapshot_pool)."""
        import torch
        st = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        rc = _lib().b200_kv_copy_stream(self._h, int(dst_stream), int(src_stream), int(n_rows), st)
        if rc:
            raise _err(rc, "b200_kv_copy_stream")


class SegmentScheduler:
    """b200_sched_*: independent units over one worker thread per GPU (or host-only workers)."""

    def __init__(self, devices=None, n_host_workers=0):
        self._h = C.c_void_p()
        if devices:
            arr = (C.c_int * len(devices))(*devices)
            rc = _lib().b200_sched_create(arr, len(devices), 0, C.byref(self._h))
        else:
            rc = _lib().b200_sched_create(None, 0, n_host_workers, C.byref(self._h))
        if rc:
            raise _err(rc, "b200_sched_create")

    def close(self):
        if self._h:
            _lib().b200_sched_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass

    def run(self, n_units, fn):
        """fn(device, unit, stream) -> int (0 ok). Returns (n_failed, worker-per-unit list)."""
        def tramp(_user, device, unit, stream):
            try:
                return int(fn(device, unit, stream) or 0)
            except Exception:  # a raising unit is a failed unit, never an abort
                return 1
        cb = abi.UNIT_FN(tramp)
        owners = (C.c_int * max(n_units, 1))()
        rc = _lib().b200_sched_run(self._h, n_units, cb, None, owners)
        if rc < 0:
            raise _err(rc, "b200_sched_run")
        return rc, list(owners)[:n_units]

    def run_batched(self, n_units, max_batch, fn, steal=True):
        """fn(device, first_unit, n_units, stream) -> int (0 ok): runs of up to `max_batch` consecutive units per call.
        Returns (n_failed, worker-per-unit list)."""
        def tramp(_user, device, first, count, stream):
            try:
                return int(fn(device, first, count, stream) or 0)
            except Exception:  # a raising batch is a failed batch, never an abort
                return 1
        cb = abi.BATCH_FN(tramp)
        owners = (C.c_int * max(n_units, 1))()
        rc = _lib().b200_sched_run_batched(self._h, n_units, int(max_batch), int(bool(steal)), cb, None, owners)
        if rc < 0:
            raise _err(rc, "b200_sched_run_batched")
        return rc, list(owners)[:n_units]

    @staticmethod
    def partition(n_units, n_workers, w):
        f, c = C.c_int(0), C.c_int(0)
        _lib().b200_sched_partition(n_units, n_workers, w, C.byref(f), C.byref(c))
        return f.value, c.value
