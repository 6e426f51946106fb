"""Generates tests/golden/*.npz.  Run in the build container (needs gguf-py and torch on CPU):

    python tests/golden/make_golden.py

Sources of truth:
  * q8_0.npz      — gguf-py 0.19.0 quants.quantize/dequantize(Q8_0), the library the reference's
                    converters call (models/convert-arkasr-to-gguf.py:304-305), on the xorshift rows of
                    tests/test-kv-quant-roundtrip.cpp (seeds 0x370, 0x371; hd 128, 2 KV heads, 3 rows)
                    and on N(0,1) rows.
  * sdpa.npz      — torch.nn.functional.scaled_dot_product_attention in float64 on CPU (an independent
                    implementation; a secondary cross-check, not the reference) for small cases of each
                    operand form.
  * crossattn.npz — inputs of tests/test-core-cross-attn.cpp (seed 0x5151) and the output of that test's
                    own plain-C++ reference algorithm, restated in numpy float32.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from tests.util import XorShift  # noqa: E402


def q8_0():
    from gguf import GGMLQuantizationType as QT
    from gguf import quants
    out = {}
    for name, seed in (("s370", 0x370), ("s371", 0x371)):
        x = XorShift(seed).fill(128 * 3 * 2).reshape(2, 3, 128)
        out[name + "_x"] = x
        out[name + "_blocks"] = quants.quantize(x, QT.Q8_0)
        out[name + "_deq"] = quants.dequantize(out[name + "_blocks"], QT.Q8_0)
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 16, 128)).astype(np.float32)
    x[0, 0, :32] = 0.0                      # an all-zero block (d == 0)
    x[0, 1, :32] = np.arange(32) - 15.5     # exact .5 ties after scaling
    out["n01_x"] = x
    out["n01_blocks"] = quants.quantize(x, QT.Q8_0)
    out["n01_deq"] = quants.dequantize(out["n01_blocks"], QT.Q8_0)
    np.savez_compressed(os.path.join(HERE, "q8_0.npz"), **out)


def sdpa():
    rng = np.random.default_rng(11)
    out = {}

    def case(name, B, H, Hkv, Tq, Lk, hd, scale, mask=None, causal_past=None):
        q = rng.standard_normal((B, H, Tq, hd)).astype(np.float16)
        k = rng.standard_normal((B, Hkv, Lk, hd)).astype(np.float16)
        v = rng.standard_normal((B, Hkv, Lk, hd)).astype(np.float16)
        m = None
        if mask == "rand":
            m = (rng.standard_normal((B, H, Tq, Lk)) * 0.5).astype(np.float16)
            m[rng.random((B, H, Tq, Lk)) < 0.2] = -np.inf
            m[..., 0] = 0  # keep every row alive
        if causal_past is not None:
            m = np.where(np.arange(Lk)[None, :] > causal_past + np.arange(Tq)[:, None], -np.inf, 0.0).astype(np.float16)
            m = np.broadcast_to(m, (1, 1, Tq, Lk)).copy()
        g = H // Hkv
        kk = torch.from_numpy(np.repeat(k, g, axis=1)).double()
        vv = torch.from_numpy(np.repeat(v, g, axis=1)).double()
        ref = torch.nn.functional.scaled_dot_product_attention(
            torch.from_numpy(q).double(), kk, vv, attn_mask=None if m is None else torch.from_numpy(m).double(),
            scale=scale).permute(0, 2, 1, 3).numpy().astype(np.float32)
        out[name + "_q"], out[name + "_k"], out[name + "_v"], out[name + "_out"] = q, k, v, ref
        out[name + "_scale"] = np.float32(scale)
        if m is not None:
            out[name + "_mask"] = m

    case("enc64", 1, 2, 2, 150, 150, 64, 0.125)
    case("gqa128_causal", 1, 4, 2, 37, 50, 128, 128 ** -0.5, causal_past=13)
    case("perhead_mask", 1, 2, 2, 40, 70, 64, 0.125, mask="rand")
    case("decode1", 2, 8, 2, 1, 200, 128, 128 ** -0.5)
    case("beams5", 1, 2, 2, 5, 200, 64, 1.0 / 8)
    np.savez_compressed(os.path.join(HERE, "sdpa.npz"), **out)


def crossattn():
    d_model, hd, H, T_enc = 8, 4, 2, 3
    qd = H * hd
    rng = XorShift(0x5151)
    dec = rng.fill(d_model)
    q_proj = rng.fill(d_model * qd).reshape(qd, d_model)     # qp[d,o] = q_proj[o*d_model+d]
    o_proj = rng.fill(qd * d_model).reshape(d_model, qd)     # op[i,dm] = o_proj[dm*qd+i]
    cK = rng.fill(hd * T_enc * H).reshape(H, T_enc, hd)
    cV = rng.fill(hd * T_enc * H).reshape(H, T_enc, hd)
    f = np.float32
    head_out = np.zeros(qd, f)
    for h in range(H):
        Q = np.array([sum(f(q_proj[h * hd + c, d] * dec[d]) for d in range(d_model)) for c in range(hd)], f)
        sc = np.array([sum(f(cK[h, te, c] * Q[c]) for c in range(hd)) for te in range(T_enc)], f)
        p = np.exp(sc - sc.max()).astype(f)
        p = (p / p.sum()).astype(f)
        for c in range(hd):
            head_out[h * hd + c] = sum(f(p[te] * cV[h, te, c]) for te in range(T_enc))
    ref = np.array([sum(f(o_proj[dm, i] * head_out[i]) for i in range(qd)) for dm in range(d_model)], f)
    np.savez_compressed(os.path.join(HERE, "crossattn.npz"), dec=dec, q_proj=q_proj, o_proj=o_proj, cK=cK, cV=cV,
                        head_out=head_out, out=ref)


if __name__ == "__main__":
    q8_0()
    sdpa()
    crossattn()
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
