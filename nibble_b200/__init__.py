"""B200-native W4A16 linear path with the reference project's Python surface."""
from .checkpoint import (load_packed_model, load_quantized_model_checkpoint, load_quantized_weight_checkpoint,
                         save_quantized_model_checkpoint, save_quantized_weight_checkpoint)
from .cuda import (check_device_status, cuda_extension_available, dequantize_cuda, linear_cuda,
                   quantize_and_pack_cuda)
from .fusion import FusedQuantizedLinear, FusedSlice, fuse_parallel_linears
from .integration import load_packed_state_dict, replace_linear_layers
from .linear import Int4Linear, QuantizedLinear
from .quantization import pack_int4, quantize_and_pack_weights, quantize_groupwise, unpack_int4

__all__ = [
    "QuantizedLinear",
    "Int4Linear",
    "pack_int4",
    "unpack_int4",
    "quantize_groupwise",
    "quantize_and_pack_weights",
    "save_quantized_weight_checkpoint",
    "load_quantized_weight_checkpoint",
    "save_quantized_model_checkpoint",
    "load_quantized_model_checkpoint",
    "load_packed_model",
    "replace_linear_layers",
    "load_packed_state_dict",
    "fuse_parallel_linears",
    "FusedQuantizedLinear",
    "FusedSlice",
    "linear_cuda",
    "dequantize_cuda",
    "quantize_and_pack_cuda",
    "cuda_extension_available",
    "check_device_status",
]
