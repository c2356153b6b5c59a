"""``QuantizedLinear``: inference-only ``nn.Module`` over packed INT4 weights.

Same constructor, class methods, buffers and ``state_dict`` keys (``packed_weights``, ``scales``,
``bias``) as the reference's w4a16/linear.py:12-200, so checkpoints and model-surgery code carry
over.  What differs is what runs underneath: every CUDA call goes to this package's sm_100a
kernels, and tensors that are not on a CUDA device are refused -- the reference evaluates those
with its PyTorch CPU routine (w4a16/linear.py:188-194); this package ships no CPU arithmetic.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .cuda import dequantize_cuda, linear_cuda
from .quantization import quantize_and_pack_weights

# Largest flattened batch M sent to the streaming (mma.sync) fused kernel.  The reference stops at 8
# and dequantises to FP16 + cuBLAS above that (w4a16/linear.py:9,179-187).
FUSED_MAX_ROWS = 64
# Above FUSED_MAX_ROWS the operator runs the tcgen05 kernel that dequantises inside the GEMM.  It beats
# dequantise-then-cuBLAS while the FP16 weight matrix's round trip through HBM is a large share of the
# cuBLAS time (batches up to about a thousand rows) and there are enough 128-channel weight tiles to
# occupy the GPU; outside that window the module does what the reference does.
PREFILL_FUSED_MAX_ROWS = 1024
PREFILL_MIN_WEIGHT_TILES = 40


def uses_fused_kernel(rows: int, out_features: int, group_size: int) -> bool:
    """Whether ``forward`` sends a flattened batch of ``rows`` to the fused operator."""
    if rows <= FUSED_MAX_ROWS:
        return True
    if group_size % 32:
        return True  # the dequantise operator needs group_size % 32 == 0; the fused one does not
    if group_size != 128:
        return False  # the tcgen05 kernel is built for 128-wide groups
    return rows <= PREFILL_FUSED_MAX_ROWS and -(-out_features // 128) >= PREFILL_MIN_WEIGHT_TILES


def _run_fused(flat, packed_weights, scales, group_size):
    return linear_cuda(flat, packed_weights, scales, group_size)


def _run_dequant_matmul(flat, packed_weights, scales, group_size):
    weight = dequantize_cuda(packed_weights, scales, group_size)
    return F.linear(flat, weight)


def _require_cuda(tensor: torch.Tensor) -> None:
    if not tensor.is_cuda:
        raise RuntimeError(
            "QuantizedLinear computes on CUDA devices only: this build has no CPU implementation "
            f"(got a tensor on '{tensor.device}')"
        )


class QuantizedLinear(torch.nn.Module):
    """``y = x @ dequant(packed_weights, scales).T (+ bias)`` for FP16 ``x[..., K]``."""

    def __init__(
        self,
        packed_weights: torch.Tensor,
        scales: torch.Tensor,
        group_size: int = 128,
        bias: torch.Tensor | None = None,
        fused: bool = True,
    ) -> None:
        super().__init__()
        if packed_weights.dtype != torch.uint8 or packed_weights.ndim != 2:
            raise ValueError("packed_weights must be uint8 with shape [N, K / 2]")
        if scales.dtype != torch.float16 or scales.ndim != 2:
            raise ValueError("scales must be float16 with shape [N, K / group_size]")
        if packed_weights.device != scales.device:
            raise ValueError("packed_weights and scales must share a device")
        if group_size <= 0:
            raise ValueError("group_size must be greater than zero")

        self.out_features = packed_weights.shape[0]
        self.in_features = 2 * packed_weights.shape[1]
        self.group_size = group_size
        if self.in_features % group_size:
            raise ValueError("K must be divisible by group_size")
        wanted = (self.out_features, self.in_features // group_size)
        if tuple(scales.shape) != wanted:
            raise ValueError(f"scales must have shape {wanted}")
        if bias is not None:
            if bias.dtype != torch.float16 or tuple(bias.shape) != (self.out_features,):
                raise ValueError("bias must be float16 with shape [N]")
            if bias.device != packed_weights.device:
                raise ValueError("bias and packed_weights must share a device")

        self.register_buffer("packed_weights", packed_weights.detach())
        self.register_buffer("scales", scales.detach())
        self.register_buffer("bias", bias.detach() if bias is not None else None)
        self.fused = fused

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_float(cls, layer: torch.nn.Linear, group_size: int = 128, fused: bool = True) -> "QuantizedLinear":
        """Quantise a floating-point ``nn.Linear`` (weights FP16 or FP32; bias cast to FP16)."""
        if not isinstance(layer, torch.nn.Linear):
            raise TypeError("layer must be an instance of torch.nn.Linear")
        packed_weights, scales = quantize_and_pack_weights(layer.weight.detach(), group_size)
        bias = layer.bias.detach().to(torch.float16) if layer.bias is not None else None
        return cls(packed_weights, scales, group_size=group_size, bias=bias, fused=fused)

    @classmethod
    def empty(
        cls,
        out_features: int,
        in_features: int,
        group_size: int = 128,
        bias: bool = False,
        fused: bool = True,
        device: torch.device | str | None = None,
    ) -> "QuantizedLinear":
        """Packed storage of the right shapes with undefined contents; no FP16 weights involved."""
        if out_features <= 0 or in_features <= 0:
            raise ValueError("out_features and in_features must be greater than zero")
        if in_features % 2:
            raise ValueError("in_features must be even")
        if group_size <= 0:
            raise ValueError("group_size must be greater than zero")
        if in_features % group_size:
            raise ValueError("K must be divisible by group_size")
        device = torch.device("cpu") if device is None else device
        return cls(
            torch.empty((out_features, in_features // 2), dtype=torch.uint8, device=device),
            torch.empty((out_features, in_features // group_size), dtype=torch.float16, device=device),
            group_size=group_size,
            bias=torch.empty((out_features,), dtype=torch.float16, device=device) if bias else None,
            fused=fused,
        )

    # ------------------------------------------------------------------ forward
    def forward(self, activations: torch.Tensor) -> torch.Tensor:
        if activations.ndim < 1:
            raise ValueError("activations must have at least one dimension")
        if activations.shape[-1] != self.in_features:
            raise ValueError("activations last dimension must equal in_features")
        if activations.dtype != torch.float16:
            raise TypeError("activations must have dtype torch.float16")
        if activations.requires_grad:
            raise RuntimeError("activations must not require grad")
        if activations.device != self.packed_weights.device:
            raise ValueError("activations and packed_weights must share a device")
        _require_cuda(activations)
        if not self.packed_weights.is_contiguous():
            raise ValueError("packed_weights must be contiguous")
        if not self.scales.is_contiguous():
            raise ValueError("scales must be contiguous")

        # The operator wants a dense [M, K]; views handed over by generation loops often are not.
        flat = activations.contiguous().reshape(-1, self.in_features)
        use_fused = (self.fused or self.group_size % 32 != 0) and uses_fused_kernel(
            flat.shape[0], self.out_features, self.group_size)
        run = _run_fused if use_fused else _run_dequant_matmul
        flat_out = run(flat, self.packed_weights, self.scales, self.group_size)
        out = flat_out.reshape(*activations.shape[:-1], self.out_features)
        return out if self.bias is None else out + self.bias

    def extra_repr(self) -> str:
        return (
            f"in_features={self.in_features}, out_features={self.out_features}, "
            f"group_size={self.group_size}, bias={self.bias is not None}, fused={self.fused}"
        )


# The module is also known by this name.
Int4Linear = QuantizedLinear
