"""ctypes wrappers the GPU tests use to call the C ABI directly with torch CUDA tensors."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from nibble_b200 import _native
from oracle import w4a16_oracle as oracle


_CANARY = 512            # FP16 elements either side of an output (a multiple of 8 keeps the output 16-byte aligned)
_CANARY_VALUE = -1234.0


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def new_workspace(m: int, n: int, k: int, splits: int = 8) -> torch.Tensor:
    """Zero-filled scratch large enough for `splits` K-splits (counters + FP32 partials)."""
    counters = (max(((n + 15) // 16) * ((m + 7) // 8), 65536) * 4 + 255) // 256 * 256      # fixed 256 KB prefix
    return torch.zeros(counters + splits * m * n * 4 + 256, dtype=torch.uint8, device="cuda")


def capi_linear(x, packed, scales, group_size=128, *, workspace=None, flags=0, config=None, expect=0):
    m, k = x.shape
    n = packed.shape[0]
    # The output sits between two canary zones (this pool has no compute-sanitizer): a kernel that writes outside
    # [M, N] disturbs them, one that skips an element leaves its NaN in place.
    guarded = torch.full((2 * _CANARY + m * n,), float("nan"), dtype=torch.float16, device=x.device)
    guarded[:_CANARY] = _CANARY_VALUE
    guarded[_CANARY + m * n:] = _CANARY_VALUE
    y = guarded[_CANARY:_CANARY + m * n].view(m, n)
    ws_ptr = ctypes.c_void_p(workspace.data_ptr()) if workspace is not None else None
    ws_bytes = workspace.numel() if workspace is not None else 0
    args = [
        ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(packed.data_ptr()), ctypes.c_void_p(scales.data_ptr()),
        ctypes.c_void_p(y.data_ptr()), m, n, k, group_size, ws_ptr, ws_bytes, flags,
    ]
    lib = _native.core()
    if config is None:
        status = lib.w4a16_linear_f16(*args, _stream())
    else:
        cfg = _native.LinearConfig(*config)
        status = lib.w4a16_linear_f16_config(*args, ctypes.byref(cfg), _stream())
    assert status == expect, f"status {status}: {_native.status_string(status)}"
    assert bool((guarded[:_CANARY] == _CANARY_VALUE).all()) and bool((guarded[_CANARY + m * n:] == _CANARY_VALUE).all()), \
        "the kernel wrote outside its output"
    return y


def capi_dequantize(packed, scales, group_size=128, expect=0):
    n, k = packed.shape[0], packed.shape[1] * 2
    w = torch.empty((n, k), dtype=torch.float16, device=packed.device)
    status = _native.core().w4a16_dequantize_f16(
        ctypes.c_void_p(packed.data_ptr()), ctypes.c_void_p(scales.data_ptr()), ctypes.c_void_p(w.data_ptr()),
        n, k, group_size, _stream(),
    )
    assert status == expect, f"status {status}: {_native.status_string(status)}"
    return w


def check_against_oracle(y: torch.Tensor, x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor,
                         group_size: int = 128, rows=None, fp16_weights: bool = False) -> float:
    """Both acceptance criteria for the fused linear, on the same packed codes:

    * ``|y - fp64(dequantize-then-matmul)| <= 1e-2 * ||x_m||_2 * max|w|`` for every output, and
    * ``assert_close(rtol=1e-2, atol=1e-2)`` against the oracle's FP16 result (the tolerance the
      reference's CUDA tests use).

    ``rows`` restricts the check to a subset of output rows (outputs are independent per row).
    ``fp16_weights`` makes the second comparison against the product with the dequantised weights
    rounded to FP16 first, which is what the reference computes for batches above its fused limit
    (dequantise, then ``F.linear``; w4a16/linear.py:132-190) and what the prefill kernel computes.
    Returns the largest error as a fraction of the bound.
    """
    xs = x.cpu().numpy()
    p = packed.cpu().numpy()
    s = scales.cpu().numpy()
    got = y.cpu()
    if rows is not None:
        rows = np.asarray(rows)
        p, s, got = p[rows], s[rows], got[:, torch.from_numpy(rows)]
    assert not torch.isnan(got).any(), "output holds values the kernel never wrote"
    exact = oracle.linear_fp64(xs, p, s, group_size)
    bound = oracle.error_bound(xs, p, s, group_size)
    err = np.abs(got.numpy().astype(np.float64) - exact)
    worst = float((err / np.maximum(bound, 1e-30)).max()) if err.size else 0.0
    assert (err <= bound).all(), f"max error {err.max():.4g} exceeds bound (ratio {worst:.3f})"
    if fp16_weights:
        w16 = oracle.dequantize_weights(p, s, group_size).astype(np.float16).astype(np.float32)
        expected = torch.from_numpy((xs.astype(np.float32) @ w16.T).astype(np.float16))
    else:
        expected = torch.from_numpy(oracle.linear_reference(xs, p, s, group_size))
    torch.testing.assert_close(got, expected, rtol=1e-2, atol=1e-2)
    return worst
