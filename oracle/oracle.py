"""ctypes front end of the CPU oracle (oracle/fattn_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's
CPU-baseline legs as the checker.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import sys

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(_HERE))
from crispasr_b200 import abi  # noqa: E402  (struct declarations only)

_LIB = None


def build() -> str:
    subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return os.path.join(_HERE, "libfattn_oracle.so")


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libfattn_oracle.so")
        if not os.path.exists(path):
            build()
        try:
            _LIB = C.CDLL(path)
        except OSError:
            os.remove(path)
            build()
            _LIB = C.CDLL(path)
        L = _LIB
        L.orc_flash_attn_ext.restype = C.c_int
        L.orc_flash_attn_ext.argtypes = [abi.TP, abi.TP, abi.TP, abi.TP, abi.TP, C.POINTER(abi.Params),
                                         C.POINTER(abi.Ext), C.c_int, C.c_int, C.c_int]
        L.orc_flash_attn_ext_opt.restype = C.c_int
        L.orc_flash_attn_ext_opt.argtypes = [abi.TP, abi.TP, abi.TP, abi.TP, abi.TP, C.POINTER(abi.Params),
                                             C.POINTER(abi.Ext), C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.orc_relpos_mask.restype = C.c_int
        L.orc_relpos_mask.argtypes = [abi.TP, abi.TP, C.c_float, C.c_int, C.c_void_p]
        L.orc_max_threads.restype = C.c_int
    return _LIB


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def flash_attn_ext(q, k, v, mask=None, *, scale, max_bias=0.0, softcap=0.0, kv_type=None, causal=False, n_past=0,
                   kv_len=None, q_v=None, r=None, r_type=None, relpos_bias_f32=False, gold=False,
                   q_round_f16=True, n_threads=0, q_as_q8_0=False, acc_f16=False, rows=None):
    """Run the oracle on numpy arrays in numpy order: q (B,H,Tq,hd) f32|f16; k,v (Bk,Hkv,Lk,hd)
    f32|f16, or uint8 block rows (Bk,Hkv,Lk,hd/32*34) with kv_type=abi.Q8_0; mask (Bm,Hm,Tq,Lk) f16.
    Arrays may be strided views.  Returns (B,Tq,H,hd) float32 (= ggml dst [hd,H,Tq,B]).
    `rows`: only these query rows are computed (the result still has Tq rows; the others are zero).
    `q_as_q8_0`, `acc_f16`: diagnostic switches (see OrcOptions in fattn_oracle.cpp), never the oracle of record."""
    L = lib()
    tq = abi.from_numpy(q)
    tk = abi.from_numpy(k, kv_type)
    tv = abi.from_numpy(v, kv_type)
    B, H, Tq, hd = q.shape
    out = np.zeros((B, Tq, H, hd), np.float32) if rows is not None else np.empty((B, Tq, H, hd), np.float32)
    td = abi.from_numpy(out)
    tm = abi.from_numpy(mask) if mask is not None else None
    p = abi.Params(float(scale), float(max_bias), float(softcap), 0)
    e = abi.Ext()
    keep = []
    if q_v is not None:
        tqv, tr = abi.from_numpy(q_v), abi.from_numpy(r, r_type)
        keep += [tqv, tr]
        e.q_v, e.r = C.pointer(tqv), C.pointer(tr)
    e.causal, e.n_past = int(bool(causal)), int(n_past)
    if kv_len is not None:
        kl = np.ascontiguousarray(kv_len, np.int32)
        keep.append(kl)
        e.kv_len = kl.ctypes.data
    e.relpos_bias_f32 = int(bool(relpos_bias_f32))
    flags = int(bool(gold)) | (0 if q_round_f16 else 2) | (4 if q_as_q8_0 else 0) | (8 if acc_f16 else 0)
    rows_arr = np.ascontiguousarray(rows, np.int32) if rows is not None else None
    rc = L.orc_flash_attn_ext_opt(C.byref(tq), C.byref(tk), C.byref(tv), C.byref(tm) if tm is not None else None,
                                  C.byref(td), C.byref(p), C.byref(e), flags, int(n_threads),
                                  rows_arr.ctypes.data if rows_arr is not None else None,
                                  len(rows_arr) if rows_arr is not None else 0)
    if rc != 0:
        raise RuntimeError(f"oracle rejected the operands: code {rc}")
    return out


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """float32 (..., n) with n % 32 == 0 -> uint8 (..., n/32*34) block rows."""
    x = np.ascontiguousarray(x, np.float32)
    n = x.shape[-1]
    assert n % 32 == 0
    out = np.empty(x.shape[:-1] + (n // 32 * 34,), np.uint8)
    lib().orc_quantize_q8_0(_ptr(x), _ptr(out), C.c_int64(x.size))
    return out


def dequantize_q8_0(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, np.uint8)
    n = b.shape[-1] // 34 * 32
    out = np.empty(b.shape[:-1] + (n,), np.float32)
    lib().orc_dequantize_q8_0(_ptr(b), _ptr(out), C.c_int64(out.size))
    return out


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_f16(_ptr(x), _ptr(out), C.c_int64(x.size))
    return out


def make_pos_enc(d_model: int, T: int) -> np.ndarray:
    """(2T-1, d_model) float32, row p = position T-1-p."""
    out = np.empty((2 * T - 1, d_model), np.float32)
    lib().orc_make_pos_enc(C.c_int(d_model), C.c_int(T), _ptr(out))
    return out


def relpos_mask(q_v: np.ndarray, r: np.ndarray, scale: float, q_round_f16=True, r_type=None) -> np.ndarray:
    """q_v (1,H,T,hd), r (1,H,2T-1,hd) -> F16 mask (1,H,T,T) = f16(scale*rel_shift(q_v r^T))."""
    _, H, T, _ = q_v.shape
    out = np.empty((1, H, T, T), np.float16)
    tqv, tr = abi.from_numpy(q_v), abi.from_numpy(r, r_type)
    rc = lib().orc_relpos_mask(C.byref(tqv), C.byref(tr), C.c_float(scale), int(q_round_f16), _ptr(out))
    if rc != 0:
        raise RuntimeError(f"oracle rejected the operands: code {rc}")
    return out


def whisper_beam_mask(cell_pos, cell_seq_bits, tok_seq, tok_pos) -> np.ndarray:
    cell_pos = np.ascontiguousarray(cell_pos, np.int32)
    cell_seq_bits = np.ascontiguousarray(cell_seq_bits, np.uint32)
    tok_seq = np.ascontiguousarray(tok_seq, np.int32)
    tok_pos = np.ascontiguousarray(tok_pos, np.int32)
    out = np.empty((len(tok_seq), len(cell_pos)), np.float16)
    lib().orc_whisper_beam_mask(_ptr(cell_pos), _ptr(cell_seq_bits), C.c_int(len(cell_pos)), _ptr(tok_seq),
                                _ptr(tok_pos), C.c_int(len(tok_seq)), _ptr(out))
    return out


def causal_mask(Lk: int, T: int, n_past: int) -> np.ndarray:
    out = np.empty((T, Lk), np.float16)
    lib().orc_causal_mask(C.c_int(Lk), C.c_int(T), C.c_int(n_past), _ptr(out))
    return out


def max_threads() -> int:
    return int(lib().orc_max_threads())
