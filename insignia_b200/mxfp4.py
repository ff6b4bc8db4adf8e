"""Host-side MXFP4 helpers: quantise fp32 to the MLX checkpoint layout and back.

Layout (reference: include/insignia_layout.cuh:47-48, src/mxfp4.cu:50-52): a
matrix of ``rows x cols`` values is stored as ``U32[rows][cols/8]`` where nibble
``j`` of word ``i`` is element ``8*i+j`` (E2M1 code, bit 3 = sign), plus one E8M0
byte per 32 consecutive elements of a row, ``U8[rows][cols/32]``.  A weight is
``lut[code] * 2**(scale-127)``.

The reference ships no quantiser (its checkpoint comes pre-quantised), so the
one here follows the OCP Microscaling v1.0 recipe: the shared exponent is
``floor(log2(max|v|)) - 2`` (2 = largest E2M1 exponent) and elements are rounded
to nearest, ties to even, saturating at +-6.  Scale bytes are clamped to 1..254
because the reference decodes 0 as 0.0 and 255 as +Inf (src/mxfp4.cu:52).

These are utilities for building synthetic checkpoints and for tests; they do no
GPU work and are not on the decode path.
"""
from __future__ import annotations

import numpy as np

E2M1_LUT = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
# a magnitude maps to code c when it exceeds the first c midpoints; ties go to the even code
_MID = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
_TIE_UP = np.array([False, True, False, True, False, True, False])  # midpoint itself rounds up?


def quantize_rows(values: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """fp32 ``[rows, cols]`` -> (``uint32[rows, cols/8]``, ``uint8[rows, cols/32]``)."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    rows, cols = v.shape
    if cols % 32:
        raise ValueError("cols must be a multiple of 32")
    g = v.reshape(rows, cols // 32, 32)
    amax = np.abs(g).max(axis=2)
    # floor(log2(amax)) straight from the exponent field (exact, no libm)
    ebits = (amax.view(np.uint32) >> 23).astype(np.int32) & 0xFF
    scale = np.clip(ebits - 2, 1, 254).astype(np.uint8)
    scale[amax == 0] = 127
    inv = ((254 - scale.astype(np.uint32)) << 23).view(np.float32)  # 2**-(scale-127), exact
    a = np.abs(g) * inv[:, :, None]
    code = np.zeros(a.shape, np.uint8)
    for mid, up in zip(_MID, _TIE_UP):
        code += (a >= mid) if up else (a > mid)
    code |= (np.signbit(g).astype(np.uint8) << 3)
    code = code.reshape(rows, cols // 8, 8).astype(np.uint32)
    packed = np.zeros((rows, cols // 8), np.uint32)
    for j in range(8):
        packed |= code[:, :, j] << np.uint32(4 * j)
    return packed, scale


def unpack_codes(weight: np.ndarray) -> np.ndarray:
    """``uint32[rows, cols/8]`` -> ``uint8[rows, cols]`` of E2M1 codes."""
    w = np.ascontiguousarray(weight, dtype=np.uint32)
    sh = (np.arange(8, dtype=np.uint32) * 4)
    return ((w[:, :, None] >> sh) & 15).astype(np.uint8).reshape(w.shape[0], -1)


def dequantize(weight: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """Exact fp32 dequantisation (``scale << 23`` semantics of src/mxfp4.cu:52)."""
    codes = unpack_codes(weight)
    s = (np.ascontiguousarray(scales, dtype=np.uint8).astype(np.uint32) << 23).view(np.float32)
    return E2M1_LUT[codes] * np.repeat(s, 32, axis=1)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
