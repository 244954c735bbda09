"""Shared helpers for the test-suite (CPU side only; imports the oracle)."""
import glob
import math
import os

import numpy as np

from oracle import oracle as O

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_cases():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load_golden(name):
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def bits_equal(a, b):
    """Bit-for-bit equality of two f32 arrays (NaN payloads and signed zeros included)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def within_tolerance(c, c_ref, a, packed, K, N, kind, rel=1e-3):
    """max |delta_mn| <= rel * ||a_m||_2 * ||w_deq[:,n]||_2 wherever the reference output is finite.

    Returns (ok, worst ratio err/bound)."""
    w = O.dequant(packed, K, N, kind)
    with np.errstate(all="ignore"):
        bound = O.tolerance_bound(a, w, rel)
        err = np.abs(c.astype(np.float64) - c_ref.astype(np.float64))
    finite = np.isfinite(c_ref) & np.isfinite(bound)
    same_nonfinite = np.all(np.isnan(c[~finite]) == np.isnan(c_ref[~finite]))
    if not finite.any():
        return bool(same_nonfinite), 0.0
    ratio = err[finite] / np.maximum(bound[finite], 1e-300)
    ok = bool(np.all(err[finite] <= bound[finite] + 1e-30)) and bool(same_nonfinite)
    return ok, float(ratio.max())


# ---- an independent, line-by-line Python reading of the reference packer ----
# Python floats are IEEE f64 like JS Numbers, so this is a second statement of
# src/ops/quantize.js:14-68 that shares no code with the C oracle.

def _js_round(x):
    if x != x:
        return x
    f = math.floor(x)
    return f + 1 if x - f >= 0.5 else f


def py_quantize_q4(w):
    w = np.asarray(w, dtype=np.float32)
    K, N = w.shape
    groups = -(-K // 32)
    packed = np.zeros(groups * N * 24, dtype=np.uint8)
    for g in range(groups):
        k0, k1 = g * 32, min(g * 32 + 32, K)
        for col in range(N):
            mn, mx = math.inf, -math.inf
            for k in range(k0, k1):
                v = float(w[k, col])
                if v < mn:
                    mn = v
                if v > mx:
                    mx = v
            rng = mx - mn
            scale = rng / 15 if rng > 0 else 1.0
            zero = (-mn) / scale if rng > 0 else 8.0
            off = (g * N + col) * 24
            for k in range(32):
                v = float(w[k0 + k, col]) if k < k1 - k0 else 0.0
                with np.errstate(all="ignore"):
                    t = float(np.float64(v) / np.float64(scale)) + zero
                if t == t:
                    t = max(0.0, t) if t > 0 else 0.0
                    t = min(15.0, t)
                q = _js_round(t)
                q = 0 if q != q else int(q)
                if k & 1:
                    packed[off + (k >> 1)] |= (q << 4) & 0xFF
                else:
                    packed[off + (k >> 1)] = q
            with np.errstate(all="ignore"):
                packed[off + 16:off + 20] = np.frombuffer(np.float32(scale).tobytes(), np.uint8)
                packed[off + 20:off + 24] = np.frombuffer(np.float32(zero).tobytes(), np.uint8)
    return packed
