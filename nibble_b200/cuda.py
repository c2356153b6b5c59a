"""Python entry points of the CUDA operators (same surface as the reference's w4a16/cuda.py:1-83).

``torch.ops.w4a16.linear`` and ``torch.ops.w4a16.dequantize`` are registered by the native shim
``_C.so``; this module loads it, registers the shape-only fake kernels ``torch.compile`` needs, and
exposes ``linear_cuda`` / ``dequantize_cuda`` / ``cuda_extension_available``.  There is no
non-CUDA implementation behind these functions: without the built extension they raise.
"""
from __future__ import annotations

import torch

from . import _native

def _register_fakes() -> None:
    """Shape-only kernels so ``torch.compile`` can trace through the native operators."""

    @torch.library.register_fake("w4a16::linear")
    def _linear_fake(activations, packed_weights, scales, group_size):
        # [M, K] x [N, K/2] -> [M, N], dtype of the activations
        return activations.new_empty((activations.shape[0], packed_weights.shape[0]))

    @torch.library.register_fake("w4a16::linear_partial")
    def _linear_partial_fake(activations, packed_weights, scales, group_size):
        return activations.new_empty((activations.shape[0], packed_weights.shape[0]), dtype=torch.float32)

    @torch.library.register_fake("w4a16::dequantize")
    def _dequantize_fake(packed_weights, scales, group_size):
        # [N, K/2] -> FP16 [N, K]
        return packed_weights.new_empty(
            (packed_weights.shape[0], packed_weights.shape[1] * 2), dtype=torch.float16
        )

    @torch.library.register_fake("w4a16::quantize_pack")
    def _quantize_pack_fake(weights, group_size):
        rows, cols = weights.shape
        return (weights.new_empty((rows, cols // 2), dtype=torch.uint8),
                weights.new_empty((rows, cols // group_size), dtype=torch.float16))


try:
    _native.load_torch_ops()
    _register_fakes()
except (ImportError, OSError, RuntimeError) as error:  # not built, stale, or built against another torch
    _EXTENSION_LOAD_ERROR: Exception | None = error
else:
    _EXTENSION_LOAD_ERROR = None


def set_programmatic_launch(enabled: bool) -> None:
    """Turn programmatic dependent launch of the fused kernel on or off for this process.

    With it on, a fused-linear kernel may start and prefetch packed weights and scales while the
    previous kernel of the stream is still finishing; it waits for that kernel before reading its
    activations or writing its output.  Only valid while no kernel that may still be running writes
    the weights or scales, i.e. for inference with weights already in place.  Off by default.
    """
    import os

    if enabled:
        os.environ["W4A16_PDL"] = "1"
    else:
        os.environ.pop("W4A16_PDL", None)


def programmatic_launch_enabled() -> bool:
    import os

    return os.environ.get("W4A16_PDL") == "1"


def check_device_status() -> None:
    """Raise if a bounded wait inside the prefill (tcgen05) kernel gave up since the last check.

    The kernel never hangs: a barrier wait that exceeds its poll limit records a code in a device word and the
    kernel still runs to the end of its clean-up -- with an unfinished result.  Callers of the prefill route
    (``torch.ops.w4a16.linear`` with 65 rows or more) should call this where they synchronise anyway, e.g. after a
    prompt has been processed.  Synchronises the device; clears the word.
    """
    import ctypes

    _require_extension()
    value = ctypes.c_uint32(0)
    status = _native.core().w4a16_device_status(ctypes.byref(value))
    if status != 0:
        raise RuntimeError(f"w4a16_device_status failed: {_native.status_string(status)}")
    if value.value:
        raise RuntimeError(f"a W4A16 prefill kernel gave up waiting on a barrier (code 0x{value.value:x}); "
                           "its output is incomplete")


def cuda_extension_available() -> bool:
    """True when the compiled operator library loaded."""
    return _EXTENSION_LOAD_ERROR is None


def _require_extension() -> None:
    if _EXTENSION_LOAD_ERROR is not None:
        raise RuntimeError(
            "The W4A16 CUDA extension is not built. Build it with `python nibble_b200/_build.py`."
        ) from _EXTENSION_LOAD_ERROR


def linear_cuda(
    activations: torch.Tensor,
    packed_weights: torch.Tensor,
    scales: torch.Tensor,
    group_size: int = 128,
) -> torch.Tensor:
    """FP16 ``[M, K]`` x packed INT4 ``[N, K/2]`` -> FP16 ``[M, N]`` on the current CUDA stream.

    ``group_size == 128`` with 16-byte aligned activations and weights runs the fused tensor-core
    kernel for every M; other even group sizes or misaligned tensors run the generic kernel.
    Invalid arguments raise ``RuntimeError``.
    """
    _require_extension()
    return torch.ops.w4a16.linear(activations, packed_weights, scales, group_size)


def dequantize_cuda(
    packed_weights: torch.Tensor,
    scales: torch.Tensor,
    group_size: int = 128,
) -> torch.Tensor:
    """Packed INT4 ``[N, K/2]`` -> FP16 ``[N, K]``, bit-identical to ``half(float(code) * float(scale))``.

    Needs ``group_size`` to be a positive multiple of 32 and 16-byte aligned packed weights.
    """
    _require_extension()
    return torch.ops.w4a16.dequantize(packed_weights, scales, group_size)


def linear_partial_cuda(
    activations: torch.Tensor,
    packed_weights: torch.Tensor,
    scales: torch.Tensor,
    group_size: int = 128,
) -> torch.Tensor:
    """``linear_cuda`` without the final rounding: FP32 ``[M, N]`` sums.

    Not part of the reference's surface; used for layers sharded along K, whose per-device partial
    results are added across devices before the single rounding to FP16.
    """
    _require_extension()
    return torch.ops.w4a16.linear_partial(activations, packed_weights, scales, group_size)


def quantize_and_pack_cuda(weights: torch.Tensor, group_size: int = 128) -> tuple[torch.Tensor, torch.Tensor]:
    """FP16/FP32 CUDA weights ``[N, K]`` -> (packed uint8 ``[N, K/2]``, FP16 scales ``[N, K/group_size]``)
    in one kernel, bit-identical to ``quantize_and_pack_weights`` (the reference's host routine,
    w4a16/quantization.py:65-113).  Not part of the reference's surface."""
    _require_extension()
    return torch.ops.w4a16.quantize_pack(weights, group_size)
