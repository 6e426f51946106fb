"""One encoder-shaped and one causal GQA prefill through the C-ABI against the oracle, in a process of its own so
that an opt-in kernel variant (selected by an environment variable read once per process) can be exercised.
Run by tests/test_fattn_gpu.py::test_opt_in_prefill_variants; prints OK <max-abs> <rel-L2> per case."""
import sys

import numpy as np

sys.path.insert(0, __file__.rsplit("/tests/", 1)[0])
import crispasr_b200 as b200  # noqa: E402
from crispasr_b200 import abi  # noqa: E402
from oracle import oracle as orc  # noqa: E402
from tests.util import errors, gpu_op, randn_f16  # noqa: E402


def main():
    rng = np.random.default_rng(77)
    # Whisper encoder shape (ragged last tiles: 1500 = 11 * 128 + 92), two segments of different length
    S, H, T, hd = 2, 4, 1500, 64
    q, k, v = (randn_f16(rng, (S, H, T, hd)) for _ in range(3))
    q[0, 1] *= 6.0   # one head with peaked rows: the reference maximum moves while the tiles go by
    lens = np.array([1500, 700], np.int32)
    ref = orc.flash_attn_ext(q, k, v, scale=0.125, kv_len=lens)
    got = gpu_op(b200, q, k, v, scale=0.125, kv_len=lens)
    assert b200.lib().b200_last_kernel() == abi.KERNEL_PREFILL_TC5
    e = errors(got, ref)
    assert e[0] <= 2e-3 and e[1] <= 1e-3, e
    print("OK encoder %.2e %.2e" % e)
    # causal prefill with a past, grouped heads
    B, H, Hkv, Tq, Lk = 1, 4, 2, 300, 520
    q = randn_f16(rng, (B, H, Tq, hd))
    k, v = (randn_f16(rng, (B, Hkv, Lk, hd)) for _ in range(2))
    ref = orc.flash_attn_ext(q, k, v, scale=0.125, causal=True, n_past=Lk - Tq)
    got = gpu_op(b200, q, k, v, scale=0.125, causal=True, n_past=Lk - Tq)
    e = errors(got, ref)
    assert e[0] <= 2e-3 and e[1] <= 1e-3, e
    print("OK causal %.2e %.2e" % e)
    assert b200.lib().b200_device_status() == 0


if __name__ == "__main__":
    main()
