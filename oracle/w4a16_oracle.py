"""CPU oracle for the W4A16 linear path -- TEST INFRASTRUCTURE, not product code.

A numpy restatement of the reference's packing format, quantiser, dequantiser
and linear layer.  Only the test-suite, the smoke check and the CPU-baseline leg
of the benchmark may import this module; the shipped package never does.

Parity status: PINNED.  Every function here is checked (tests/test_oracle.py)
against the reference's own known-answer vectors and against fixtures under
tests/golden/ that were produced by importing the reference's Python modules
(tests/golden/make_golden.py).

Reference locations restated here (paths inside the reference project):
  pack_int4            w4a16/quantization.py:4-28
  unpack_int4          w4a16/quantization.py:31-63
  quantize_groupwise   w4a16/quantization.py:65-102
  quantize_and_pack    w4a16/quantization.py:105-113
  dequantize_weights   w4a16/reference.py:6-46
  linear_reference     w4a16/reference.py:49-80
"""
from __future__ import annotations

import numpy as np

__all__ = [
    "pack_int4",
    "unpack_int4",
    "quantize_groupwise",
    "quantize_and_pack_weights",
    "dequantize_weights",
    "linear_reference",
    "linear_fp64",
    "error_bound",
]


def pack_int4(codes: np.ndarray) -> np.ndarray:
    """int8 [N, K] codes in [-7, 7] -> uint8 [N, K/2].

    Byte j of a row holds code 2j in bits 0-3 and code 2j+1 in bits 4-7, both as
    4-bit two's complement (reference w4a16/quantization.py:17-26).
    """
    codes = np.asarray(codes)
    if codes.dtype != np.int8:
        raise TypeError("codes must be int8")
    if codes.ndim != 2:
        raise ValueError("codes must be [N, K]")
    if codes.shape[1] % 2:
        raise ValueError("K must be even")
    if codes.size and (codes.min() < -7 or codes.max() > 7):
        raise ValueError("codes must lie in [-7, 7]")
    nib = codes.view(np.uint8) & np.uint8(0x0F)
    return (nib[:, 0::2] | (nib[:, 1::2] << np.uint8(4))).astype(np.uint8)


def unpack_int4(packed: np.ndarray) -> np.ndarray:
    """uint8 [N, K/2] -> int8 [N, K]; every nibble value 0..15 maps to -8..7
    (reference w4a16/quantization.py:38-61, which also decodes 0x8 as -8)."""
    packed = np.asarray(packed)
    if packed.dtype != np.uint8:
        raise TypeError("packed must be uint8")
    if packed.ndim != 2:
        raise ValueError("packed must be [N, K/2]")
    out = np.empty((packed.shape[0], packed.shape[1] * 2), dtype=np.int8)
    lo = (packed & np.uint8(0x0F)).astype(np.int16)
    hi = (packed >> np.uint8(4)).astype(np.int16)
    out[:, 0::2] = np.where(lo >= 8, lo - 16, lo)
    out[:, 1::2] = np.where(hi >= 8, hi - 16, hi)
    return out


def quantize_groupwise(weights: np.ndarray, group_size: int = 128):
    """fp16/fp32 [N, K] -> (int8 codes [N, K], fp16 scales [N, K/group]).

    Symmetric absmax round-to-nearest-even: per group the FP32 scale is amax/7
    (1.0 for an all-zero group), codes are round(w / scale_fp32) clamped to
    [-7, 7], and only afterwards is the scale rounded to FP16
    (reference w4a16/quantization.py:76-102).
    """
    weights = np.asarray(weights)
    if weights.dtype not in (np.float16, np.float32):
        raise TypeError("weights must be float16 or float32")
    if weights.ndim != 2:
        raise ValueError("weights must be [N, K]")
    if group_size <= 0:
        raise ValueError("group_size must be positive")
    n, k = weights.shape
    if k % group_size:
        raise ValueError("K must be divisible by group_size")
    w32 = weights.astype(np.float32).reshape(n, k // group_size, group_size)
    amax = np.abs(w32).max(axis=2) if w32.size else np.zeros((n, k // group_size), np.float32)
    s32 = (amax / np.float32(7.0)).astype(np.float32)
    s32 = np.where(amax == 0, np.float32(1.0), s32).astype(np.float32)
    q = np.rint(w32 / s32[:, :, None]).clip(-7, 7)
    return q.astype(np.int8).reshape(n, k), s32.astype(np.float16)


def quantize_and_pack_weights(weights: np.ndarray, group_size: int = 128):
    """quantize_groupwise followed by pack_int4 (reference w4a16/quantization.py:105-113)."""
    codes, scales = quantize_groupwise(weights, group_size)
    return pack_int4(codes), scales


def dequantize_weights(packed: np.ndarray, scales: np.ndarray, group_size: int = 128) -> np.ndarray:
    """packed uint8 [N, K/2] + fp16 scales [N, K/group] -> fp32 [N, K] = code * scale
    (reference w4a16/reference.py:25-46).  The product of a 4-bit integer and an
    FP16 value is exact in FP32."""
    packed = np.asarray(packed)
    scales = np.asarray(scales)
    if packed.dtype != np.uint8:
        raise TypeError("packed must be uint8")
    if scales.dtype != np.float16:
        raise TypeError("scales must be float16")
    if packed.ndim != 2 or scales.ndim != 2:
        raise ValueError("packed must be [N, K/2] and scales [N, K/group]")
    if group_size <= 0:
        raise ValueError("group_size must be positive")
    codes = unpack_int4(packed)
    n, k = codes.shape
    if k % group_size:
        raise ValueError("K must be divisible by group_size")
    if scales.shape != (n, k // group_size):
        raise ValueError(f"scales must have shape {(n, k // group_size)}, got {scales.shape}")
    w = codes.astype(np.float32).reshape(n, k // group_size, group_size)
    w = w * scales.astype(np.float32)[:, :, None]
    return w.reshape(n, k)


def linear_reference(x: np.ndarray, packed: np.ndarray, scales: np.ndarray, group_size: int = 128) -> np.ndarray:
    """fp16 x [M, K] -> fp16 y [M, N] = half(float(x) @ dequant(W)^T), FP32 matmul
    and one final rounding to FP16 (reference w4a16/reference.py:75-80)."""
    x = np.asarray(x)
    if x.dtype != np.float16:
        raise TypeError("x must be float16")
    if x.ndim != 2:
        raise ValueError("x must be [M, K]")
    w = dequantize_weights(packed, scales, group_size)
    if x.shape[1] != w.shape[1]:
        raise ValueError("x and weights disagree on K")
    return (x.astype(np.float32) @ w.T).astype(np.float16)


def linear_fp64(x: np.ndarray, packed: np.ndarray, scales: np.ndarray, group_size: int = 128) -> np.ndarray:
    """The same product accumulated in FP64 and left unrounded: the yardstick for
    the absolute-error bound (no rounding noise of its own)."""
    w = dequantize_weights(packed, scales, group_size).astype(np.float64)
    return np.asarray(x).astype(np.float64) @ w.T


def error_bound(x: np.ndarray, packed: np.ndarray, scales: np.ndarray, group_size: int = 128) -> np.ndarray:
    """Per-row allowance 1e-2 * ||x_m||_2 * max|w| on |y - dequantize-then-matmul|,
    the acceptance criterion stated for this path; returned with shape [M, 1]."""
    w = dequantize_weights(packed, scales, group_size)
    wmax = float(np.abs(w).max()) if w.size else 0.0
    norms = np.linalg.norm(np.asarray(x).astype(np.float64), axis=1, keepdims=True)
    return 1e-2 * norms * wmax
