"""Generates tests/golden/*.npz -- small input/output vectors for the quantized path.

Run in a checkout that has the reference mounted and oracle/_ref built
(``make -C oracle``):  ``python tests/golden/make_golden.py``.

Each case stores seeded inputs, the packed bytes produced by the CPU
restatement of the reference packer (oracle/smith_oracle.c), and the matmul
output of the REFERENCE's own shader source compiled as C++
(oracle/_ref/libsmith_ref.so).  The fixtures travel with the repository so the
checks can run where the reference checkout is not available.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as O  # noqa: E402


def weights(rng, K, N, dist):
    if dist == "uniform":
        return rng.random((K, N), dtype=np.float32)
    if dist == "normal02":
        return (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    raise ValueError(dist)


def quirks(rng, K, N):
    """Constant groups, zeros, a min of +0, negative-only columns, NaN and Inf entries."""
    w = (rng.standard_normal((K, N)) * 0.5).astype(np.float32)
    w[:32, 0] = 0.25                  # constant group -> scale 1, zero 8
    w[:32, 1] = 0.0                   # all zero
    w[:32, 2] = np.abs(w[:32, 2]); w[3, 2] = 0.0     # min == +0 -> zero stored as -0.0
    w[:32, 3] = -np.abs(w[:32, 3]) - 0.1             # all negative
    w[5, 4] = np.nan                  # NaN is skipped by min/max, encodes as 0
    w[:32, 5] = np.nan                # all NaN -> scale 1, zero 8
    w[7, 6] = np.inf                  # infinite range
    w[:32, 7] = np.float32(1e-30)     # tiny constant
    w[0, 8] = -0.0; w[1:32, 8] = np.abs(w[1:32, 8])  # min == -0
    return w


CASES = [
    # name, K, N, M, weight dist, activation
    ("ref_test_k64_n32", 64, 32, 1, "uniform", "ones"),     # tests/inference.test.js:94-123
    ("ref_ratio_k256_n256", 256, 256, 2, "uniform", "normal"),  # tests/inference.test.js:125-135
    ("ragged_k100_n40", 100, 40, 3, "normal02", "normal"),
    ("tiny_k1_n1", 1, 1, 1, "normal02", "normal"),
    ("odd_n_k96_n7", 96, 7, 5, "normal02", "normal"),
    ("skinny_k512_n64", 512, 64, 16, "normal02", "normal"),
    ("rows_k128_n96", 128, 96, 70, "normal02", "normal"),
    ("quirks_k64_n16", 64, 16, 2, "quirks", "normal"),
]


def main():
    assert O.have_ref(), "build oracle/_ref first (make -C oracle) with the reference mounted"
    for i, (name, K, N, M, dist, act) in enumerate(CASES):
        rng = np.random.default_rng(1000 + i)
        w = quirks(rng, K, N) if dist == "quirks" else weights(rng, K, N, dist)
        a = np.ones((M, K), np.float32) if act == "ones" else rng.standard_normal((M, K)).astype(np.float32)
        out = {"w": w, "a": a}
        for kind in ("q4", "q8"):
            packed = O.quantize_q4(w) if kind == "q4" else O.quantize_q8(w)
            with np.errstate(all="ignore"):
                c = O.ref_matmul(a, packed, K, N, kind)
            out[f"packed_{kind}"] = packed
            out[f"c_{kind}"] = c
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
