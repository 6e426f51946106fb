"""Pins of the CPU oracle (no GPU): every known-answer the reference's own tests, in-tree code and
the gguf-py library offer for the neighbourhood of GGML_OP_FLASH_ATTN_EXT."""
import os

import numpy as np
import pytest

from crispasr_b200 import abi
from tests.util import XorShift, errors

G = os.path.join(os.path.dirname(__file__), "golden")


def test_f16_conversion_bit_exact(orc):
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(200000) * np.exp(rng.uniform(-30, 12, 200000))).astype(np.float32)
    x[:8] = [0.0, -0.0, 65504.0, 65520.0, 5.9604645e-8, 2.9802322e-8, 2.98023259e-8, 6.1035156e-5]
    with np.errstate(over="ignore"):
        assert np.array_equal(orc.f32_to_f16_bits(x), x.astype(np.float16).view(np.uint16))


@pytest.mark.parametrize("name", ["s370", "s371", "n01"])
def test_q8_0_matches_gguf_py(orc, name):
    """Bit-exact against blocks written by gguf-py (fixture made by tests/golden/make_golden.py)."""
    g = np.load(os.path.join(G, "q8_0.npz"))
    blocks = orc.quantize_q8_0(g[name + "_x"])
    assert np.array_equal(blocks, g[name + "_blocks"])
    assert np.array_equal(orc.dequantize_q8_0(blocks), g[name + "_deq"])


def test_q8_0_roundtrip_bound_of_reference_test(orc):
    """tests/test-kv-quant-roundtrip.cpp:192-195: |x - deq(quant(x))| <= 0.02 for x in [-1,1] (Q8_0),
    both for the bulk write (seed 0x370) and the prefill + one appended row (seed 0x371)."""
    hd, heads, rows = 128, 2, 3
    x = XorShift(0x370).fill(hd * rows * heads)
    assert np.abs(orc.dequantize_q8_0(orc.quantize_q8_0(x.reshape(-1, hd))).ravel() - x).max() <= 0.02
    r = XorShift(0x371)
    prefill, step = r.fill(hd * rows * heads).reshape(heads, rows, hd), r.fill(hd * heads).reshape(heads, 1, hd)
    cache = np.zeros((heads, 16, hd // 32 * 34), np.uint8)
    cache[:, :rows] = orc.quantize_q8_0(prefill)
    cache[:, rows:rows + 1] = orc.quantize_q8_0(step)
    got = orc.dequantize_q8_0(cache[:, :rows + 1])
    assert np.abs(got - np.concatenate([prefill, step], 1)).max() <= 0.02


def test_cross_attn_kat(orc):
    """tests/test-core-cross-attn.cpp: seed 0x5151, d_model 8, hd 4, 2 heads, T_enc 3, T_dec 1, unscaled,
    F32 K/V; the expected vector is that test's own plain-C++ algorithm (fixture), tolerance 1e-4."""
    g = np.load(os.path.join(G, "crossattn.npz"))
    hd, H = 4, 2
    Q = (g["q_proj"] @ g["dec"]).astype(np.float32).reshape(1, H, 1, hd)
    out = orc.flash_attn_ext(Q, g["cK"][None], g["cV"][None], scale=1.0, q_round_f16=False)
    assert np.abs(out.reshape(-1) - g["head_out"]).max() < 1e-4
    assert np.abs(g["o_proj"] @ out.reshape(-1) - g["out"]).max() < 1e-4


def _relpos_inputs(T=12, HD=4, NH=2):
    """Deterministic fills of tools/dev/tiledbd_parity.cpp:28,112-117: frand(i) = sin(0.37 i) * 0.9."""
    D = HD * NH
    fr = lambda n, s: (np.sin((np.arange(n) + s).astype(np.float32) * np.float32(0.37)) * np.float32(0.9)).astype(np.float32)
    Q = fr(D * T, 1).reshape(T, NH, HD)
    K = fr(D * T, 100).reshape(T, NH, HD)
    V = fr(D * T, 200).reshape(T, NH, HD)
    R = fr(D * (2 * T - 1), 300).reshape(2 * T - 1, NH, HD)
    pbu, pbv = fr(D, 400).reshape(NH, HD), fr(D, 500).reshape(NH, HD)
    tr = lambda x: np.ascontiguousarray(x.transpose(1, 0, 2))[None]  # (1,H,T,hd)
    return tr(Q + pbu), tr(Q + pbv), tr(K), tr(V), tr(R)


def _manual_relpos(Qu, Qv, K, V, R, scale):
    """The monolithic reference graph of tools/dev/tiledbd_parity.cpp:57-66 in float64."""
    _, H, T, hd = Qu.shape
    out = np.zeros((1, T, H, hd))
    for h in range(H):
        ac = Qu[0, h].astype(np.float64) @ K[0, h].astype(np.float64).T
        bd_raw = Qv[0, h].astype(np.float64) @ R[0, h].astype(np.float64).T        # [q, r]
        bd = np.array([[bd_raw[q, k - q + T - 1] for k in range(T)] for q in range(T)])
        s = (ac + bd) * scale
        p = np.exp(s - s.max(1, keepdims=True))
        out[0, :, h] = (p / p.sum(1, keepdims=True)) @ V[0, h].astype(np.float64)
    return out


@pytest.mark.parametrize("T", [12, 7, 33])
def test_rel_shift_parity(orc, T):
    """Fused rel-pos bias == the manual (2T-1 -> T,T) rel_shift attention, tolerance 1e-4 as in
    tools/dev/tiledbd_parity.cpp:123-126 (bias kept in fp32: the F16 cast is a separate rounding point)."""
    Qu, Qv, K, V, R = _relpos_inputs(T)
    scale = 1.0 / np.sqrt(4.0)
    ref = _manual_relpos(Qu, Qv, K, V, R, scale)
    got = orc.flash_attn_ext(Qu, K, V, scale=scale, q_v=Qv, r=R, relpos_bias_f32=True, q_round_f16=False)
    assert np.abs(got - ref).max() < 1e-4
    # materialised F16 mask (what src/core/fastconformer.h:880-918 feeds the op) == fused with F16 rounding
    m = orc.relpos_mask(Qv, R, scale, q_round_f16=False)
    a = orc.flash_attn_ext(Qu, K, V, m, scale=scale, q_round_f16=False)
    b = orc.flash_attn_ext(Qu, K, V, scale=scale, q_v=Qv, r=R, q_round_f16=False)
    assert np.array_equal(a, b)
    assert np.abs(a - ref).max() < 5e-3


def test_pos_enc_layout(orc):
    """src/core/fastconformer.h:118-130: row p is position T-1-p, sin in even columns, cos in odd."""
    d, T = 16, 5
    pe = orc.make_pos_enc(d, T)
    assert pe.shape == (2 * T - 1, d)
    div = np.exp(-np.log(10000.0) * np.arange(0, d, 2) / d)
    for p in range(2 * T - 1):
        pos = T - 1 - p
        assert np.allclose(pe[p, 0::2], np.sin(pos * div), atol=1e-6)
        assert np.allclose(pe[p, 1::2], np.cos(pos * div), atol=1e-6)
    assert np.allclose(pe[T - 1, 0::2], 0) and np.allclose(pe[T - 1, 1::2], 1)


def test_mask_rules(orc):
    """src/voxtral.cpp:1191-1193 (causal) and src/crispasr.cpp:3480-3488 (beam cells)."""
    m = orc.causal_mask(6, 3, 2)
    for q in range(3):
        for k in range(6):
            assert (m[q, k] == -np.inf) == (k > 2 + q)
    # 2 beams: cells 0-2 are a shared prefix (seqs 0 and 1), cell 3 belongs to seq 0, cell 4 to seq 1
    cell_pos = [0, 1, 2, 3, 3]
    bits = [3, 3, 3, 1, 2]
    bm = orc.whisper_beam_mask(cell_pos, bits, tok_seq=[0, 1], tok_pos=[4, 2])
    assert (bm[0] == 0).tolist() == [True, True, True, True, False]
    assert (bm[1] == 0).tolist() == [True, True, True, False, False]   # cell 4: pos 3 > 2


def test_implicit_equals_explicit_causal(orc):
    rng = np.random.default_rng(5)
    q = rng.standard_normal((1, 4, 9, 32)).astype(np.float16)
    k = rng.standard_normal((1, 2, 20, 32)).astype(np.float16)
    v = rng.standard_normal((1, 2, 20, 32)).astype(np.float16)
    m = orc.causal_mask(20, 9, 11)[None, None]
    a = orc.flash_attn_ext(q, k, v, m, scale=0.2)
    b = orc.flash_attn_ext(q, k, v, scale=0.2, causal=True, n_past=11)
    assert np.array_equal(a, b)
    # kv_len == masking the tail
    m2 = np.zeros((1, 1, 9, 20), np.float16)
    m2[..., 13:] = -np.inf
    assert np.array_equal(orc.flash_attn_ext(q, k, v, m2, scale=0.2), orc.flash_attn_ext(q, k, v, scale=0.2, kv_len=[13]))


@pytest.mark.parametrize("name", ["enc64", "gqa128_causal", "perhead_mask", "decode1", "beams5"])
def test_against_sdpa_fixture(orc, name):
    """Secondary cross-check: float64 torch SDPA outputs committed as fixtures."""
    g = np.load(os.path.join(G, "sdpa.npz"))
    mask = g[name + "_mask"] if name + "_mask" in g else None
    out = orc.flash_attn_ext(g[name + "_q"], g[name + "_k"], g[name + "_v"], mask, scale=float(g[name + "_scale"]))
    ma, rl = errors(out, g[name + "_out"])
    assert ma < 2e-5 and rl < 1e-5


def test_fp32_vs_fp64_accumulation(orc):
    rng = np.random.default_rng(9)
    q = rng.standard_normal((1, 2, 64, 128)).astype(np.float16)
    k = rng.standard_normal((1, 2, 700, 128)).astype(np.float16)
    v = rng.standard_normal((1, 2, 700, 128)).astype(np.float16)
    ma, rl = errors(orc.flash_attn_ext(q, k, v, scale=0.088), orc.flash_attn_ext(q, k, v, scale=0.088, gold=True))
    assert ma < 2e-5 and rl < 1e-5


def test_edge_cases(orc):
    rng = np.random.default_rng(2)
    q = rng.standard_normal((1, 1, 3, 32)).astype(np.float16)
    k = rng.standard_normal((1, 1, 5, 32)).astype(np.float16)
    # a fully masked row yields zeros; the other rows are unaffected
    m = np.zeros((1, 1, 3, 5), np.float16)
    m[0, 0, 1, :] = -np.inf
    out = orc.flash_attn_ext(q, k, k, m, scale=1.0)
    assert np.all(out[0, 1] == 0) and np.isfinite(out).all() and np.abs(out[0, 0]).max() > 0
    # kv_len 0 -> zeros
    assert np.all(orc.flash_attn_ext(q, k, k, scale=1.0, kv_len=[0]) == 0)
    # single key: output is that V row
    out = orc.flash_attn_ext(q, k[:, :, :1], k[:, :, :1], scale=1.0)
    assert np.allclose(out[0, :, 0], k[0, 0, 0].astype(np.float32)[None].repeat(3, 0))
    # Q8_0 through a strided view (rows of a wider cache)
    cache = orc.quantize_q8_0(rng.standard_normal((1, 1, 16, 32)).astype(np.float32))
    a = orc.flash_attn_ext(q, cache[:, :, :5], cache[:, :, :5], scale=1.0, kv_type=abi.Q8_0)
    b = orc.flash_attn_ext(q, orc.dequantize_q8_0(cache[:, :, :5]), orc.dequantize_q8_0(cache[:, :, :5]), scale=1.0)
    assert np.array_equal(a, b)


def test_softcap_and_alibi(orc):
    rng = np.random.default_rng(4)
    B, H, T, L, hd = 1, 6, 4, 9, 32
    q = rng.standard_normal((B, H, T, hd)).astype(np.float16)
    k = rng.standard_normal((B, H, L, hd)).astype(np.float16)
    v = rng.standard_normal((B, H, L, hd)).astype(np.float16)
    m = (rng.standard_normal((1, 1, T, L))).astype(np.float16)
    out = orc.flash_attn_ext(q, k, v, m, scale=0.3, max_bias=8.0, softcap=5.0)
    n2 = 4
    m0, m1 = 2.0 ** (-8.0 / n2), 2.0 ** (-4.0 / n2)
    ref = np.zeros_like(out, dtype=np.float64)
    for h in range(H):
        slope = m0 ** (h + 1) if h < n2 else m1 ** (2 * (h - n2) + 1)
        s = q[0, h].astype(np.float64) @ k[0, h].astype(np.float64).T * 0.3
        s = 5.0 * np.tanh(s / 5.0) + slope * m[0, 0].astype(np.float64)
        p = np.exp(s - s.max(1, keepdims=True))
        ref[0, :, h] = (p / p.sum(1, keepdims=True)) @ v[0, h].astype(np.float64)
    assert np.abs(out - ref).max() < 1e-5


def test_row_subset_equals_full_run(orc):
    rng = np.random.default_rng(15)
    q, k, v = (rng.standard_normal((1, 2, 50, 32)).astype(np.float16) for _ in range(3))
    full = orc.flash_attn_ext(q, k, v, scale=0.2, causal=True)
    rows = [0, 7, 49]
    part = orc.flash_attn_ext(q, k, v, scale=0.2, causal=True, rows=rows)
    assert np.array_equal(part[:, rows], full[:, rows])
    assert not part[:, [1, 2, 48]].any()


def test_diagnostic_switches_size_the_unverified_gap(orc, capsys):
    """How far two things the upstream CPU kernel is believed to do (its source is absent, so neither can be
    checked) would move a result away from the oracle of record: the query re-quantised to Q8_0 against a Q8_0 K,
    and an F16 output accumulator with F16 V.  Both move results by MORE than the parity tolerance of the CUDA
    path (max-abs 2e-3 / rel-L2 1e-3), which is why they are recorded as unverified instead of being adopted;
    the fp32 oracle itself sits within 1e-6 of fp64."""
    from crispasr_b200 import abi
    rng = np.random.default_rng(3)
    S, H, Hkv, hd, Lk = 2, 32, 8, 128, 535
    q = rng.standard_normal((S, H, 1, hd)).astype(np.float16)
    k = orc.quantize_q8_0(rng.standard_normal((S, Hkv, Lk, hd)).astype(np.float32))
    v = orc.quantize_q8_0(rng.standard_normal((S, Hkv, Lk, hd)).astype(np.float32))
    kw = dict(scale=hd ** -0.5, kv_type=abi.Q8_0)
    rec = orc.flash_attn_ext(q, k, v, **kw)
    _, rl_gold = errors(rec, orc.flash_attn_ext(q, k, v, gold=True, **kw))
    ma_q8, rl_q8 = errors(orc.flash_attn_ext(q, k, v, q_as_q8_0=True, **kw), rec)
    rng = np.random.default_rng(1)
    q2 = (rng.standard_normal((1, 20, 5, 64)) * 0.5).astype(np.float16)
    k2, v2 = ((rng.standard_normal((1, 20, 1500, 64)) * 0.5).astype(np.float16) for _ in range(2))
    rec2 = orc.flash_attn_ext(q2, k2, v2, scale=64 ** -0.25)
    ma_16, rl_16 = errors(orc.flash_attn_ext(q2, k2, v2, scale=64 ** -0.25, acc_f16=True), rec2)
    with capsys.disabled():
        print(f"\n  oracle fp32 vs fp64 (Q8_0 decode): rel-L2 {rl_gold:.2e}")
        print(f"  q_as_q8_0 vs oracle of record (Q8_0 decode, 535 keys): max-abs {ma_q8:.2e} rel-L2 {rl_q8:.2e}")
        print(f"  acc_f16 vs oracle of record (F16 cross-attention, 1500 keys): max-abs {ma_16:.2e} rel-L2 {rl_16:.2e}")
    assert rl_gold < 5e-6
    assert 1e-3 < rl_q8 < 2e-2 and 1e-3 < rl_16 < 2e-2
    # the switches are inert where they do not apply
    assert np.array_equal(orc.flash_attn_ext(q2, k2, v2, scale=0.3, q_as_q8_0=True), orc.flash_attn_ext(q2, k2, v2, scale=0.3))
    assert np.array_equal(orc.flash_attn_ext(q, k, v, acc_f16=True, **kw), rec)
