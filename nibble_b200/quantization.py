"""Owner of the packed W4A16 weight format (offline, host side, any torch device).

Layout, identical to the reference so checkpoints interchange
(reference w4a16/quantization.py:4-113):

* ``packed_weights``: uint8 ``[N, K/2]`` row-major.  Byte ``j`` of row ``n``
  stores code ``(n, 2j)`` in bits 0-3 and code ``(n, 2j+1)`` in bits 4-7, each a
  4-bit two's-complement integer.  Read as little-endian 32-bit words, word ``w``
  of a row holds k = 8w .. 8w+7 with weight ``j`` in nibble ``j``.
* ``scales``: float16 ``[N, K/group_size]``; one absmax/7 scale per
  ``group_size`` consecutive k of one output row.
* codes are symmetric round-to-nearest-even in ``[-7, 7]``; they are computed
  with the FP32 scale and the scale is rounded to FP16 only afterwards.
"""
from __future__ import annotations

import torch

_NIBBLE = 0x0F


def _require_2d(tensor: torch.Tensor, what: str) -> None:
    if tensor.ndim != 2:
        raise ValueError(f"{what} must be a 2-D tensor")


def pack_int4(quantized_weights: torch.Tensor) -> torch.Tensor:
    """int8 ``[N, K]`` codes in ``[-7, 7]`` -> uint8 ``[N, K/2]`` (even k in the low nibble)."""
    if quantized_weights.dtype != torch.int8:
        raise TypeError("quantized_weights must have dtype torch.int8")
    _require_2d(quantized_weights, "quantized_weights")
    if quantized_weights.shape[1] % 2:
        raise ValueError("K must be even: one byte carries two weights")
    if quantized_weights.numel():
        low, high = torch.aminmax(quantized_weights)
        if int(low) < -7 or int(high) > 7:
            raise ValueError("quantized_weights must lie in [-7, 7]")
    pairs = quantized_weights.reshape(quantized_weights.shape[0], quantized_weights.shape[1] // 2, 2)
    nibbles = (pairs & _NIBBLE).to(torch.uint8)
    return nibbles[..., 0] | (nibbles[..., 1] << 4)


def unpack_int4(packed_weights: torch.Tensor) -> torch.Tensor:
    """uint8 ``[N, K/2]`` -> int8 ``[N, K]``.  All 16 nibble values decode (0x8 -> -8)."""
    if packed_weights.dtype != torch.uint8:
        raise TypeError("packed_weights must have dtype torch.uint8")
    _require_2d(packed_weights, "packed_weights")
    both = torch.stack((packed_weights & _NIBBLE, packed_weights >> 4), dim=2)
    # Sign-extend a 4-bit two's-complement value: flip the sign bit, subtract its weight.
    signed = (both.to(torch.int8) ^ 8) - 8
    return signed.reshape(packed_weights.shape[0], packed_weights.shape[1] * 2)


def quantize_groupwise(
    weights: torch.Tensor,
    group_size: int = 128,
) -> tuple[torch.Tensor, torch.Tensor]:
    """FP16/FP32 ``[N, K]`` -> (int8 codes ``[N, K]``, FP16 scales ``[N, K/group_size]``).

    Per group: ``s = amax/7`` in FP32 (``1`` for an all-zero group),
    ``code = clamp(round_half_even(w / s), -7, 7)``, ``scale = half(s)``.
    """
    if weights.dtype not in (torch.float16, torch.float32):
        raise TypeError("weights must have dtype torch.float16 or torch.float32")
    if weights.ndim != 2:
        raise ValueError("weights must have shape [N, K]")
    if group_size <= 0:
        raise ValueError("group_size must be greater than zero")
    rows, cols = weights.shape
    if cols % group_size:
        raise ValueError("K must be divisible by group_size")

    grouped = weights.float().reshape(rows, cols // group_size, group_size)
    amax = grouped.abs().amax(dim=2, keepdim=True)
    step = amax / 7.0
    step = torch.where(amax == 0, torch.ones_like(step), step)
    codes = torch.round(grouped / step).clamp_(-7, 7).to(torch.int8)
    return codes.reshape(rows, cols), step.squeeze(2).to(torch.float16)


def quantize_and_pack_weights(
    weights: torch.Tensor,
    group_size: int = 128,
) -> tuple[torch.Tensor, torch.Tensor]:
    """``quantize_groupwise`` then ``pack_int4``: (uint8 ``[N, K/2]``, FP16 ``[N, K/group_size]``).

    CUDA weights with an even ``group_size`` go through the one-pass device kernel (same bits) when the
    extension is built; everything else runs the torch operators below on the tensor's device.
    """
    if weights.is_cuda and weights.ndim == 2 and weights.dtype in (torch.float16, torch.float32) \
            and group_size > 0 and group_size % 2 == 0 and weights.shape[1] % group_size == 0:
        from . import cuda as _cuda   # late: this module must import without the extension

        if _cuda.cuda_extension_available():
            return _cuda.quantize_and_pack_cuda(weights, group_size)
    codes, scales = quantize_groupwise(weights, group_size)
    return pack_int4(codes), scales
