"""Timed CPU baseline -- TEST/BENCH INFRASTRUCTURE, not product code.

The reference's CPU path for this layer is a short chain of PyTorch CPU tensor operations
(w4a16/reference.py:25-80 on top of w4a16/quantization.py:38-61): split bytes into nibbles,
sign-extend, widen to FP32, multiply by the per-group scale, FP32 matmul, round to FP16.  This file
restates that chain with the same operator granularity so that timing it on the host cores (all
intra-op threads) is a fair stand-in for timing the reference itself, which cannot travel to the
GPU machine.  The numpy oracle (w4a16_oracle.py) stays the checker; tests assert that both agree.

Parity status: pinned through tests/test_oracle.py::test_torch_port_matches_numpy_oracle.
"""
from __future__ import annotations

import torch


def unpack_codes(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [N, K/2] -> int8 [N, K] (even k from the low nibble)."""
    low = (packed & 0x0F).to(torch.int8)
    high = (packed >> 4).to(torch.int8)
    low = torch.where(low >= 8, low - 16, low)
    high = torch.where(high >= 8, high - 16, high)
    codes = torch.empty((packed.shape[0], packed.shape[1] * 2), dtype=torch.int8)
    codes[:, 0::2] = low
    codes[:, 1::2] = high
    return codes


def dequantize(packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """FP32 [N, K] = code * scale, group-wise."""
    codes = unpack_codes(packed)
    n, k = codes.shape
    grouped = codes.to(torch.float32).reshape(n, k // group_size, group_size)
    return (grouped * scales.to(torch.float32).unsqueeze(2)).reshape(n, k)


def linear(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """FP16 [M, N] = half(float(x) @ dequantize(...)^T)."""
    weights = dequantize(packed, scales, group_size)
    return torch.matmul(x.to(torch.float32), weights.t()).to(torch.float16)
