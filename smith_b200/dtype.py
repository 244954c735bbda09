"""Element types and the f16 codec -- the role of src/dtype.js in the reference.

``toFloat16`` deliberately keeps the reference encoder's behaviour
(src/dtype.js:29-58): the mantissa is truncated, not rounded, and values below
the smallest normal half end as a signed zero.  The Q8 scale stored by
``quantizeQ8`` is defined through this encoder, so it has to match bit for bit.
"""
import struct

import numpy as np

_BYTES = {"f32": 4, "f16": 2, "i32": 4, "u32": 4, "u8": 1, "i8": 1}
_ARRAY = {"f32": np.float32, "f16": np.uint16, "i32": np.int32, "u32": np.uint32, "u8": np.uint8, "i8": np.int8}


def dtypeBytes(dtype):
    try:
        return _BYTES[dtype]
    except KeyError:
        raise ValueError(f"Unknown dtype: {dtype}")


def dtypeArray(dtype):
    try:
        return _ARRAY[dtype]
    except KeyError:
        raise ValueError(f"Unknown dtype: {dtype}")


def toFloat16(val):
    """f64 -> half bits, as src/dtype.js:29-58."""
    bits = struct.unpack("<I", struct.pack("<f", _to_f32(val)))[0]
    sign = (bits >> 31) & 1
    exp = (bits >> 23) & 0xFF
    frac = bits & 0x7FFFFF
    if exp == 0xFF:
        return (sign << 15) | 0x7C00 | (0x200 if frac else 0)
    exp -= 127
    if exp > 15:
        return (sign << 15) | 0x7C00
    if exp < -14:
        if exp < -24:
            return sign << 15
        frac |= 0x800000
        frac >>= (-1 - exp)
        return (sign << 15) | (frac >> 13)
    return (sign << 15) | ((exp + 15) << 10) | (frac >> 13)


def _to_f32(val):
    val = float(val)
    try:
        return struct.unpack("<f", struct.pack("<f", val))[0]
    except OverflowError:  # beyond f32 range: the typed-array store gives +-Infinity
        return float("inf") if val > 0 else float("-inf")


def fromFloat16(h):
    """half bits -> f64, as src/dtype.js:60-79."""
    sign = (h >> 15) & 1
    exp = (h >> 10) & 0x1F
    frac = h & 0x3FF
    if exp == 0:
        if frac == 0:
            return -0.0 if sign else 0.0
        val = 2.0 ** -14 * (frac / 1024)
        return -val if sign else val
    if exp == 31:
        if frac:
            return float("nan")
        return float("-inf") if sign else float("inf")
    val = 2.0 ** (exp - 15) * (1 + frac / 1024)
    return -val if sign else val
