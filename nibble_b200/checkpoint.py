"""Single-matrix checkpoint in the reference's on-disk format (w4a16/checkpoint.py:6-94).

The file is a ``torch.save`` of a plain dict
``{"format": "w4a16-linear", "version": 1, "packed_weights", "scales", "group_size",
"original_shape": (N, K)}`` with CPU tensors, so files written by either project load in the other.
"""
from __future__ import annotations

import os

import torch

FORMAT_NAME = "w4a16-linear"
FORMAT_VERSION = 1


def _check_pair(packed_weights: torch.Tensor, scales: torch.Tensor, group_size: int) -> tuple[int, int]:
    """Validate a (packed, scales, group_size) triple and return the logical weight shape (N, K)."""
    if packed_weights.dtype != torch.uint8 or packed_weights.ndim != 2:
        raise ValueError("packed_weights must be a uint8 tensor shaped [N, K / 2]")
    if scales.dtype != torch.float16 or scales.ndim != 2:
        raise ValueError("scales must be a float16 tensor shaped [N, K / group_size]")
    if packed_weights.device != scales.device:
        raise ValueError("packed_weights and scales must share a device")
    if group_size <= 0:
        raise ValueError("group_size must be greater than zero")
    n, k = packed_weights.shape[0], 2 * packed_weights.shape[1]
    if k % group_size:
        raise ValueError("K must be divisible by group_size")
    if tuple(scales.shape) != (n, k // group_size):
        raise ValueError(f"scales must have shape {(n, k // group_size)}")
    return n, k


def save_quantized_weight_checkpoint(
    path: str | os.PathLike,
    packed_weights: torch.Tensor,
    scales: torch.Tensor,
    group_size: int = 128,
) -> None:
    """Write one packed matrix with its format metadata."""
    shape = _check_pair(packed_weights, scales, group_size)
    torch.save(
        {
            "format": FORMAT_NAME,
            "version": FORMAT_VERSION,
            "packed_weights": packed_weights.detach().cpu(),
            "scales": scales.detach().cpu(),
            "group_size": group_size,
            "original_shape": shape,
        },
        os.fspath(path),
    )


def load_quantized_weight_checkpoint(
    path: str | os.PathLike,
    map_location: str | torch.device = "cpu",
) -> tuple[torch.Tensor, torch.Tensor, int]:
    """Read and re-validate one packed matrix: ``(packed_weights, scales, group_size)``."""
    blob = torch.load(os.fspath(path), map_location=map_location, weights_only=True)
    if not isinstance(blob, dict):
        raise ValueError("checkpoint must contain a dictionary")
    if blob.get("format") != FORMAT_NAME:
        raise ValueError("checkpoint has an unsupported format")
    if blob.get("version") != FORMAT_VERSION:
        raise ValueError("checkpoint has an unsupported version")
    packed_weights, scales, group_size = (blob.get(key) for key in ("packed_weights", "scales", "group_size"))
    if not isinstance(packed_weights, torch.Tensor):
        raise ValueError("checkpoint is missing packed_weights")
    if not isinstance(scales, torch.Tensor):
        raise ValueError("checkpoint is missing scales")
    if not isinstance(group_size, int):
        raise ValueError("checkpoint is missing group_size")
    shape = _check_pair(packed_weights, scales, group_size)
    if tuple(blob.get("original_shape", ())) != shape:
        raise ValueError("checkpoint original_shape does not match its tensors")
    return packed_weights, scales, group_size
