"""ctypes mirror of include/b200_fattn.h.

Only declarations live here: the structs, the enum values and helpers that describe a numpy
array or a torch tensor as a ``b200_tensor`` with ggml ne/nb conventions (ne[0] fastest,
nb in bytes).  ggml lists dimensions fastest-first, numpy/torch slowest-first, so an array of
shape (B, H, T, hd) is the ggml tensor [hd, T, H, B].
"""
from __future__ import annotations

import ctypes as C

F32, F16, Q8_0 = 0, 1, 8
TYPE_NAMES = {F32: "f32", F16: "f16", Q8_0: "q8_0"}
QK8_0, Q8_0_BLOCK_BYTES = 32, 34

OK = 0
E_NULL, E_TYPE, E_SHAPE, E_STRIDE, E_ALIGN, E_UNSUPPORTED = -1, -2, -3, -4, -5, -6
E_WORKSPACE, E_CUDA, E_NO_DEVICE, E_LIMIT, E_STATE, E_DEVICE_WAIT = -7, -8, -9, -10, -11, -12

KERNEL_NONE, KERNEL_TILE_MMA, KERNEL_DECODE_SPLIT, KERNEL_PREFILL_TC5 = 0, 1, 2, 3
KERNEL_NAMES = {0: "none", 1: "tile_mma", 2: "decode_split", 3: "prefill_tc5"}


class Tensor(C.Structure):
    _fields_ = [
        ("data", C.c_void_p),
        ("type", C.c_int32),
        ("reserved", C.c_int32),
        ("ne", C.c_int64 * 4),
        ("nb", C.c_uint64 * 4),
    ]


class Params(C.Structure):
    _fields_ = [
        ("scale", C.c_float),
        ("max_bias", C.c_float),
        ("logit_softcap", C.c_float),
        ("prec_f32", C.c_int32),
    ]


class Ext(C.Structure):
    _fields_ = [
        ("q_v", C.POINTER(Tensor)),
        ("r", C.POINTER(Tensor)),
        ("pos_bias_u", C.POINTER(Tensor)),
        ("pos_bias_v", C.POINTER(Tensor)),
        ("causal", C.c_int32),
        ("n_past", C.c_int32),
        ("kv_len", C.c_void_p),
        ("relpos_bias_f32", C.c_int32),
        ("kv_index_stride", C.c_int32),
        ("kv_index", C.c_void_p),
        ("q_len", C.c_void_p),
    ]


class KvConfig(C.Structure):
    _fields_ = [
        ("type", C.c_int32),
        ("head_dim", C.c_int32),
        ("n_kv_heads", C.c_int32),
        ("n_layers", C.c_int32),
        ("max_ctx", C.c_int32),
        ("n_streams", C.c_int32),
    ]


class TraceRecord(C.Structure):
    _fields_ = [("kernel", C.c_int32), ("n_splits", C.c_int32), ("head_dim", C.c_int32), ("q_len", C.c_int32),
                ("kv_len", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("n_batch", C.c_int32),
                ("kv_type", C.c_int32), ("ms", C.c_float)]


UNIT_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p)
BATCH_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p)

TP = C.POINTER(Tensor)

# name -> (restype, argtypes); every symbol include/b200_fattn.h declares.
_OP_ARGS = [TP, TP, TP, TP, TP, C.POINTER(Params), C.POINTER(Ext)]
MASK_GENERAL, MASK_NONE, MASK_CAUSAL, MASK_TAIL = 0, 1, 2, 3

SYMBOLS = {
    "b200_set_kernel_override": (C.c_int, [C.c_int]),
    "b200_set_decode_splits": (C.c_int, [C.c_int]),
    "b200_strerror": (C.c_char_p, [C.c_int]),
    "b200_version": (C.c_char_p, []),
    "b200_last_cuda_error": (C.c_char_p, []),
    "b200_fattn_supports": (C.c_int, _OP_ARGS + [C.POINTER(C.c_int)]),
    "b200_fattn_plan": (C.c_int, _OP_ARGS + [C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "b200_fattn_workspace_bytes": (C.c_int, _OP_ARGS + [C.POINTER(C.c_size_t)]),
    "b200_fattn_launch": (C.c_int, _OP_ARGS + [C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_fattn_forward_host": (C.c_int, _OP_ARGS),
    "b200_host_arena_release": (None, []),
    "b200_fattn_launch_static": (C.c_int, _OP_ARGS + [C.c_void_p]),
    "b200_fattn_static_scratch_bytes": (C.c_size_t, []),
    "b200_last_kernel": (C.c_int, []),
    "b200_device_status": (C.c_int, []),
    "b200_device_status_reset": (C.c_int, []),
    "b200_trace_enable": (C.c_int, [C.c_int]),
    "b200_trace_read": (C.c_int, [C.POINTER(TraceRecord), C.c_int, C.POINTER(C.c_int)]),
    "b200_test_empty_launch": (C.c_int, [C.c_void_p]),
    "b200_test_bounded_wait": (C.c_int, [C.c_int, C.c_void_p]),
    "b200_kv_create": (C.c_int, [C.POINTER(KvConfig), C.POINTER(C.c_void_p)]),
    "b200_kv_destroy": (None, [C.c_void_p]),
    "b200_kv_bytes": (C.c_size_t, [C.c_void_p]),
    "b200_kv_view": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, TP, TP]),
    "b200_kv_append": (C.c_int, [C.c_void_p, C.c_int, TP, TP, C.c_void_p, C.c_int32, C.c_void_p]),
    "b200_kv_copy_stream": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_void_p]),
    "b200_beam_cells_to_index": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "b200_mask_classify": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200_beam_cells_to_union": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "b200_relpos_table": (C.c_int, [TP, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_relpos_cache_create": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "b200_relpos_cache_destroy": (None, [C.c_void_p]),
    "b200_relpos_cache_bytes": (C.c_size_t, [C.c_void_p]),
    "b200_relpos_cache_get": (C.c_int, [C.c_void_p, C.c_int, C.c_int, TP, C.c_int, C.c_void_p, TP, C.POINTER(C.c_int)]),
    "b200_batch_pack": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]),
    "b200_batch_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "b200_batch_destroy": (None, [C.c_void_p]),
    "b200_batch_add": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "b200_batch_set": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "b200_batch_advance": (C.c_int, [C.c_void_p, C.c_int]),
    "b200_batch_remove": (C.c_int, [C.c_void_p, C.c_int]),
    "b200_batch_span": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "b200_batch_unit": (C.c_int, [C.c_void_p, C.c_int]),
    "b200_batch_lengths": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "b200_batch_tables": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "b200_sched_create": (C.c_int, [C.POINTER(C.c_int), C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "b200_sched_destroy": (None, [C.c_void_p]),
    "b200_sched_run": (C.c_int, [C.c_void_p, C.c_int, UNIT_FN, C.c_void_p, C.POINTER(C.c_int)]),
    "b200_sched_run_batched": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, BATCH_FN, C.c_void_p, C.POINTER(C.c_int)]),
    "b200_sched_partition": (None, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
}


def bind(lib: C.CDLL, symbols=SYMBOLS) -> C.CDLL:
    """Attach restype/argtypes; raises AttributeError if the library lacks a symbol."""
    for name, (res, args) in symbols.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


def _elem_size(t: int) -> int:
    return {F32: 4, F16: 2, Q8_0: Q8_0_BLOCK_BYTES}[t]


def describe(ptr: int, type_: int, shape, strides_bytes) -> Tensor:
    """Build a descriptor from a slowest-first shape/byte-stride pair (numpy/torch order).

    For Q8_0 the caller passes the LOGICAL shape (elements) with strides of the block storage:
    the fastest stride must be 34 (one block) and the fastest extent counts elements.
    """
    nd = len(shape)
    if nd > 4:
        raise ValueError("at most 4 dimensions")
    t = Tensor()
    t.data = ptr
    t.type = type_
    ne = [1, 1, 1, 1]
    nb = [0, 0, 0, 0]
    for i in range(nd):
        ne[i] = int(shape[nd - 1 - i])
        nb[i] = int(strides_bytes[nd - 1 - i])
    nb[0] = _elem_size(type_) if nd == 0 else nb[0]
    # ggml fills strides of absent (size-1) trailing dimensions with the full extent
    for i in range(max(nd, 1), 4):
        prev_rows = ne[i - 1] if not (type_ == Q8_0 and i - 1 == 0) else ne[0] // QK8_0
        nb[i] = nb[i - 1] * prev_rows
    for i in range(4):
        t.ne[i] = ne[i]
        t.nb[i] = nb[i]
    return t


def from_numpy(a, type_: int | None = None, logical_last: int | None = None) -> Tensor:
    """Describe a numpy array. uint8 arrays with type_=Q8_0 hold blocks: the last axis is bytes
    (a multiple of 34) and ``logical_last`` (default bytes/34*32) is the element count."""
    import numpy as np

    if type_ is None:
        type_ = {np.dtype(np.float32): F32, np.dtype(np.float16): F16}[a.dtype]
    if type_ == Q8_0:
        if a.dtype != np.uint8 or a.strides[-1] != 1:
            raise ValueError("Q8_0 arrays are uint8 with a contiguous last axis")
        n = logical_last if logical_last is not None else a.shape[-1] // Q8_0_BLOCK_BYTES * QK8_0
        shape = list(a.shape[:-1]) + [n]
        strides = list(a.strides[:-1]) + [Q8_0_BLOCK_BYTES]
        return describe(a.ctypes.data, Q8_0, shape, strides)
    return describe(a.ctypes.data, type_, a.shape, a.strides)


def from_torch(x, type_: int | None = None) -> Tensor:
    """Describe a torch tensor (any device). uint8 tensors with type_=Q8_0 hold blocks."""
    import torch

    if type_ is None:
        type_ = {torch.float32: F32, torch.float16: F16}[x.dtype]
    es = x.element_size()
    strides = [s * es for s in x.stride()]
    if type_ == Q8_0:
        if x.dtype != torch.uint8 or x.stride(-1) != 1:
            raise ValueError("Q8_0 tensors are uint8 with a contiguous last axis")
        shape = list(x.shape[:-1]) + [x.shape[-1] // Q8_0_BLOCK_BYTES * QK8_0]
        strides = strides[:-1] + [Q8_0_BLOCK_BYTES]
        return describe(x.data_ptr(), Q8_0, shape, strides)
    return describe(x.data_ptr(), type_, x.shape, strides)
