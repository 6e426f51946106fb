"""Host-side checks of bench.py's accounting and of the switches the documentation names (no GPU)."""
import os
import re
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_algorithmic_work_of_the_named_configurations():
    enc = bench.algorithmic_work(bench.WORKLOADS["whisper_large_v3_encoder"], 64)
    assert enc["bound"] == "tensor" and enc["amount"] == 4.0 * 1500 * 1500 * 64 * 20 * 64      # 737.28 GFLOP per launch
    assert enc["bytes"] == 64 * (20 * 1500 * 64 * (2 + 4) + 2 * 20 * 1500 * 128)               # Q f16 + O f32 + K,V f16
    cross = bench.algorithmic_work(bench.WORKLOADS["whisper_large_v3_decode_cross"], 64)
    assert cross["bound"] == "hbm" and cross["amount"] == 64 * (2.0 * 1500 * 20 * 128 + 20 * 5 * 64 * 6)
    q8 = bench.algorithmic_work(bench.WORKLOADS["voxtral_decode_q8_0"], 8)
    assert q8["amount"] == 8 * (2.0 * 535 * 8 * 136 + 32 * 1 * 128 * 6)                        # 34-byte blocks: 136 B per row
    union = bench.algorithmic_work(bench.WORKLOADS["whisper_large_v3_decode_self_pool_union"], 1)
    dense = bench.algorithmic_work(bench.WORKLOADS["whisper_large_v3_decode_self_pool_dense"], 1)
    assert union["amount"] == dense["amount"]                                                  # live cells, whatever the call form
    causal = bench.algorithmic_work(bench.WORKLOADS["voxtral_prefill_q8_0"], 8)
    assert causal["amount"] == 2.0 * 407 * 408 * 128 * 32 * 8                                  # lower triangle


def test_roofline_reports_the_longer_floor():
    class DW:
        kernel_id, n_splits = 3, 1

    class ABI:
        KERNEL_NAMES = {3: "prefill_tc5"}

    pk = {"tensor": 1376.4, "hbm": 6446.6, "src": "measured"}
    w = bench.WORKLOADS["voxtral_prefill_q8_0"]
    r = bench.roofline_of(ABI, w, "voxtral_prefill_q8_0", 8, DW, [48.0e-3 * w["layers"]], pk, {})
    assert r["bound"] == "hbm" and r["floors_us"]["hbm"] > r["floors_us"]["tensor"]
    assert abs(r["frac"] - r["floors_us"]["hbm"] / 48.0) < 1e-6                               # 48 us per launch
    w = bench.WORKLOADS["whisper_large_v3_encoder"]
    r = bench.roofline_of(ABI, w, "whisper_large_v3_encoder", 64, DW, [1.3 * w["layers"]], pk, {})
    assert r["bound"] == "tensor" and abs(r["achieved"] - 737.28e9 / 1.3e-3 / 1e12) < 1e-6


def test_documented_switches_exist_in_the_sources():
    """Every B200_* environment variable README.md names is read somewhere in the library, and the other way round."""
    readme = open(os.path.join(ROOT, "README.md")).read()
    named = set(re.findall(r"`(B200_[A-Z0-9_]+)", readme))
    read = set()
    csrc = os.path.join(ROOT, "crispasr_b200", "csrc")
    for f in os.listdir(csrc):
        read |= set(re.findall(r'getenv\("(B200_[A-Z0-9_]+)"\)', open(os.path.join(csrc, f)).read()))
    assert named, "README lists the switches"
    assert named <= read, f"documented but not read: {sorted(named - read)}"
    assert read <= named, f"read but not documented: {sorted(read - named)}"
