"""Specification of the weight-only INT8 format, on nested Python lists.

Same functions, argument meaning and errors as the reference's llm/quantization.py:1-56
(`fp32`, `fp16`, `validate_matrix`, `quantize`, `dequantize`): matrices are [input, output];
one symmetric scale per OUTPUT channel (column); values are first rounded to binary16;
scale = fp32(max|column| / 127) or 1.0 for an all-zero column; q = round-half-even(w / scale)
clipped to [-127, 127] (never -128, no zero point); dequantisation multiplies in binary32 and
rounds once to binary16.  Pure stdlib so it can arbitrate between implementations.
"""
import math
import struct

_F32 = struct.Struct("<f")
_F16 = struct.Struct("<e")


def fp32(value):
    """Round a Python float to the nearest binary32 value."""
    return _F32.unpack(_F32.pack(value))[0]


def fp16(value):
    """Round a Python float to the nearest binary16 value (OverflowError past 65504)."""
    return _F16.unpack(_F16.pack(value))[0]


def validate_matrix(rows):
    """Returns (height, width) of a rectangular, non-empty matrix of finite reals."""
    if not rows or not rows[0]:
        raise ValueError("matrix must be nonempty")
    width = len(rows[0])
    for row in rows:
        if len(row) != width:
            raise ValueError("ragged matrix")
        for value in row:
            if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
                raise ValueError("weights must be finite real numbers")
    return len(rows), width


def quantize(rows):
    """[in, out] reals -> (q [in][out] ints in [-127, 127], scales [out] as binary32 values)."""
    height, width = validate_matrix(rows)
    half = [[fp16(float(v)) for v in row] for row in rows]
    scales = []
    for j in range(width):
        top = max(abs(half[i][j]) for i in range(height))
        scales.append(fp32(top / 127.0) if top != 0 else 1.0)
    if any(s <= 0 or not math.isfinite(s) for s in scales):
        raise ValueError("scale underflow/overflow")
    # round() on a float is round-half-to-even; the division is binary64 on exact operands.
    q = [[min(127, max(-127, round(half[i][j] / scales[j]))) for j in range(width)] for i in range(height)]
    return q, scales


def dequantize(q, scales, *, to_fp16=True):
    """q [in][out] ints, scales [out] -> values fp32(q * fp32(scale)), rounded to binary16 by default."""
    _, width = validate_matrix(q)
    if len(scales) != width:
        raise ValueError("positive finite output-channel scales required")
    for s in scales:
        if isinstance(s, bool) or not isinstance(s, (int, float)) or not math.isfinite(s) or s <= 0:
            raise ValueError("positive finite output-channel scales required")
    for row in q:
        for v in row:
            if type(v) is not int or not -127 <= v <= 127:
                raise ValueError("q must contain symmetric INT8 integers")
    narrow = fp16 if to_fp16 else float
    return [[narrow(fp32(v * fp32(scales[j]))) for j, v in enumerate(row)] for row in q]
