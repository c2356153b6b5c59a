"""Loaders for the two native libraries built by ``nibble_b200._build``.

``core()`` returns a ``ctypes.CDLL`` for ``libw4a16_b200.so`` with argument types set for every
function declared in ``include/w4a16_b200.h``; ``load_torch_ops()`` loads ``_C.so`` so that
``torch.ops.w4a16.*`` exist.  Neither builds anything and neither has a fallback: a missing
library is an error the caller sees.
"""
from __future__ import annotations

import ctypes
import functools
import pathlib

PKG = pathlib.Path(__file__).resolve().parent
CORE_LIB = PKG / "libw4a16_b200.so"
CHECKED_LIB = PKG / "libw4a16_b200_checked.so"     # the same library built with -DW4A16_BOUNDS_CHECK
TORCH_LIB = PKG / "_C.so"


class LinearConfig(ctypes.Structure):
    """Mirror of ``w4a16_linear_config``; zero fields mean "library's choice"."""

    _fields_ = [
        ("row_tiles", ctypes.c_int32),
        ("k_warps", ctypes.c_int32),
        ("k_splits", ctypes.c_int32),
        ("unroll", ctypes.c_int32),
        ("stages", ctypes.c_int32),
    ]


class PeerTarget(ctypes.Structure):
    """Mirror of ``w4a16_peer_target``: where a sharded layer's result goes on every rank."""

    _fields_ = [
        ("outputs", ctypes.c_void_p),
        ("consumed", ctypes.c_void_p),
        ("done_counter", ctypes.c_void_p),
        ("send_epoch", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
        ("buffer_stride", ctypes.c_int64),
        ("ld", ctypes.c_int64),
        ("column_offset", ctypes.c_int64),
        ("max_polls", ctypes.c_int64),
        ("rank", ctypes.c_int32),
        ("world", ctypes.c_int32),
    ]


class PeerSource(ctypes.Structure):
    """Mirror of ``w4a16_peer_source``: how a kernel reads another sharded layer's published result."""

    _fields_ = [
        ("epoch", ctypes.c_void_p),
        ("consumed", ctypes.c_void_p),
        ("staged_counter", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
        ("buffer_stride", ctypes.c_int64),
        ("max_polls", ctypes.c_int64),
        ("first_column", ctypes.c_int64),
        ("columns_per_rank", ctypes.c_int64),
        ("rank", ctypes.c_int32),
        ("world", ctypes.c_int32),
    ]


class DecodeLayer(ctypes.Structure):
    """``w4a16_decode_layer``: device pointers of one decoder block."""

    _fields_ = [(name, ctypes.c_void_p) for name in (
        "norm1", "qkv_packed", "qkv_scales", "o_packed", "o_scales", "norm2", "gate_up_packed", "gate_up_scales",
        "down_packed", "down_scales", "k_cache", "v_cache")]


class DecodeModel(ctypes.Structure):
    """``w4a16_decode_model``."""

    _fields_ = [(name, ctypes.c_int32) for name in (
        "layers", "hidden", "q_heads", "kv_heads", "head_dim", "intermediate", "vocab", "max_len")] + [
        ("eps", ctypes.c_float), ("rope_scale", ctypes.c_float), ("softmax_scale", ctypes.c_float),
        ("embed", ctypes.c_void_p), ("final_norm", ctypes.c_void_p), ("lm_head_packed", ctypes.c_void_p),
        ("lm_head_scales", ctypes.c_void_p), ("inv_freq", ctypes.c_void_p), ("layer", ctypes.POINTER(DecodeLayer))]


class DecodePlanInfo(ctypes.Structure):
    """``w4a16_decode_plan_info``."""

    _fields_ = [("logits", ctypes.c_void_p), ("status", ctypes.c_void_p), ("operations", ctypes.c_int32),
                ("grid", ctypes.c_int32), ("head_dim", ctypes.c_int32), ("smem_bytes", ctypes.c_uint32)]


_P = ctypes.c_void_p
_I = ctypes.c_int64

# name -> (restype, argtypes): the complete exported surface of include/w4a16_b200.h
C_API = {
    "w4a16_linear_f16": (ctypes.c_int, [_P, _P, _P, _P, _I, _I, _I, _I, _P, ctypes.c_size_t, ctypes.c_uint32, _P]),
    "w4a16_linear_f16_config": (
        ctypes.c_int,
        [_P, _P, _P, _P, _I, _I, _I, _I, _P, ctypes.c_size_t, ctypes.c_uint32, ctypes.POINTER(LinearConfig), _P],
    ),
    "w4a16_linear_workspace_bytes": (ctypes.c_size_t, [_I, _I, _I]),
    "w4a16_linear_workspace_bytes_flags": (ctypes.c_size_t, [_I, _I, _I, ctypes.c_uint32]),
    "w4a16_linear_f16_static_scratch": (ctypes.c_int, [_P, _P, _P, _P, _I, _I, _I, _I, ctypes.c_uint32, _P]),
    "w4a16_static_scratch_bytes": (ctypes.c_size_t, []),
    "w4a16_linear_f16_peers": (
        ctypes.c_int,
        [_P, _I, _P, _P, _P, _I, _I, _I, _I, _P, ctypes.c_size_t, ctypes.c_uint32, ctypes.POINTER(PeerTarget),
         ctypes.POINTER(PeerSource), _P],
    ),
    "w4a16_wait_peers": (ctypes.c_int, [ctypes.POINTER(PeerSource), _P, _P, _I, ctypes.c_uint32, _P]),
    "w4a16_sum_partials_f16": (ctypes.c_int, [_P, _P, _I, ctypes.c_int32, ctypes.POINTER(PeerSource), ctypes.c_uint32, _P]),
    "w4a16_dequantize_f16": (ctypes.c_int, [_P, _P, _P, _I, _I, _I, _P]),
    "w4a16_quantize_pack_f16": (ctypes.c_int, [_P, _P, _P, _I, _I, _I, _P]),
    "w4a16_quantize_pack_f32": (ctypes.c_int, [_P, _P, _P, _I, _I, _I, _P]),
    "w4a16_linear_f16_input": (ctypes.c_int, [_P, _P, _P, _P, _I, _I, _I, _I, _P, ctypes.c_size_t, ctypes.c_uint32, _P, _P]),
    "w4a16_add_rmsnorm_f16": (ctypes.c_int, [_P, _P, _P, _P, _P, _I, ctypes.c_float, ctypes.c_uint32, _P]),
    "w4a16_silu_mul_f16": (ctypes.c_int, [_P, _P, _I, ctypes.c_uint32, _P]),
    "w4a16_argmax_advance_f16": (ctypes.c_int, [_P, _I, _P, _P, ctypes.c_uint32, _P]),
    "w4a16_attention_decode_f16": (
        ctypes.c_int,
        [_P, _P, _P, _P, _P, _P, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_float,
         ctypes.c_float, _P, ctypes.c_uint32, _P],
    ),
    "w4a16_decode_plan_bytes": (ctypes.c_size_t, [ctypes.POINTER(DecodeModel)]),
    "w4a16_decode_plan_build": (ctypes.c_int, [ctypes.POINTER(DecodeModel), _P, ctypes.c_size_t, _P, _P,
                                               ctypes.POINTER(DecodePlanInfo), _P]),
    "w4a16_decode_step_f16": (ctypes.c_int, [_P, ctypes.POINTER(DecodePlanInfo), _P]),
    "w4a16_device_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_uint32)]),
    "w4a16_bounds_check_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint32)]),
    "w4a16_launch_count": (ctypes.c_uint64, []),
    "w4a16_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "w4a16_abi_version": (ctypes.c_int, []),
}

INPUT_PLAIN, INPUT_SILU_MUL, INPUT_ADD_RMSNORM = 0, 1, 2


class InputTransform(ctypes.Structure):
    """``w4a16_input_transform`` of include/w4a16_b200.h."""

    _fields_ = [("kind", ctypes.c_int32), ("second", ctypes.c_void_p), ("norm_weight", ctypes.c_void_p),
                ("stream_out", ctypes.c_void_p), ("eps", ctypes.c_float)]


FLAG_PROGRAMMATIC_LAUNCH = 1 << 0
FLAG_FORCE_GENERIC = 1 << 1
FLAG_OUTPUT_F32 = 1 << 2
FLAG_NO_TCGEN05 = 1 << 3
FLAG_FORCE_TCGEN05 = 1 << 4


@functools.lru_cache(maxsize=None)
def core() -> ctypes.CDLL:
    import os

    path = CORE_LIB
    if os.environ.get("W4A16_CHECKED_LIB") == "1":     # tests: the bounds-checking build, C ABI calls only
        path = CHECKED_LIB
    if not path.exists():
        raise RuntimeError(
            f"{path.name} is not built; run `python nibble_b200/_build.py` (needs nvcc)"
        )
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in C_API.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def status_string(status: int) -> str:
    return core().w4a16_status_string(status).decode()


@functools.lru_cache(maxsize=None)
def load_torch_ops() -> None:
    if not TORCH_LIB.exists():
        raise ImportError(f"{TORCH_LIB.name} is not built; run `python nibble_b200/_build.py`")
    import torch

    torch.ops.load_library(str(TORCH_LIB))
