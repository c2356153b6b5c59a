"""Model surgery: swap ``nn.Linear`` layers for ``QuantizedLinear`` and load packed state dicts.

API-compatible with the reference's w4a16/integration.py:8-119 (``replace_linear_layers``,
``load_packed_state_dict``): same arguments, same return value (number of layers replaced), same
warning for layers whose ``in_features`` the group size does not divide.
"""
from __future__ import annotations

import warnings

import torch

from .linear import QuantizedLinear


def replace_linear_layers(
    module: torch.nn.Module,
    group_size: int = 128,
    prefix: str = "",
    fused: bool = True,
    packed_only: bool = False,
    fuse_siblings: bool | None = None,
) -> int:
    """Recursively replace every compatible ``nn.Linear`` below ``module``; returns how many.

    ``packed_only=True`` only looks at layer shapes and allocates empty packed storage (works on
    the meta device); the packed tensors are expected to arrive through ``load_state_dict``.

    ``fuse_siblings`` (not in the reference): afterwards, sibling projections that read the same activations
    (``q_proj``/``k_proj``/``v_proj``; ``gate_proj``/``up_proj``) are served by one launch over their
    concatenated rows (``nibble_b200.fusion.fuse_parallel_linears``).  Module names, outputs and state-dict keys
    stay what they were.  Default: on, unless the environment variable ``W4A16_FUSE_SIBLINGS`` is ``0``.
    """
    if group_size <= 0:
        raise ValueError("group_size must be greater than zero")

    replaced = 0
    for name, child in list(module.named_children()):
        path = f"{prefix}.{name}" if prefix else name
        if isinstance(child, QuantizedLinear):
            continue
        if not isinstance(child, torch.nn.Linear):
            replaced += replace_linear_layers(child, group_size, prefix=path, fused=fused, packed_only=packed_only,
                                              fuse_siblings=False)
            continue
        if child.in_features % group_size:
            warnings.warn(
                f"Skipping linear layer '{path}' because in_features={child.in_features} "
                f"is not divisible by group_size={group_size}",
                UserWarning,
                stacklevel=2,
            )
            continue
        if packed_only:
            new = QuantizedLinear.empty(
                child.out_features,
                child.in_features,
                group_size=group_size,
                bias=child.bias is not None,
                fused=fused,
                device=child.weight.device,
            )
        else:
            new = QuantizedLinear.from_float(child, group_size=group_size, fused=fused)
        new.train(child.training)
        setattr(module, name, new)
        replaced += 1
    if not prefix:   # the outermost call: every replacement below is done
        if fuse_siblings is None:
            import os

            fuse_siblings = os.environ.get("W4A16_FUSE_SIBLINGS", "1") != "0"
        if fuse_siblings:
            from .fusion import fuse_parallel_linears

            fuse_parallel_linears(module)
    return replaced


def _restore_computed_buffers(module: torch.nn.Module) -> None:
    """Recompute non-persistent buffers that ``to_empty`` leaves uninitialised.

    Rotary embeddings of HuggingFace models keep ``inv_freq`` out of the state dict; modules that
    expose ``compute_default_rope_parameters`` and a ``config`` get it rebuilt from the config.
    """
    for sub in module.modules():
        compute = getattr(sub, "compute_default_rope_parameters", None)
        target = getattr(sub, "inv_freq", None)
        if compute is None or target is None or not hasattr(sub, "config"):
            continue
        inv_freq, attention_scaling = compute(sub.config)
        target.copy_(inv_freq.to(device=target.device, dtype=target.dtype))
        original = getattr(sub, "original_inv_freq", None)
        if original is not None:
            original.copy_(inv_freq.to(device=original.device, dtype=original.dtype))
        sub.attention_scaling = attention_scaling


def load_packed_state_dict(
    module: torch.nn.Module,
    state_dict: dict,
    group_size: int = 128,
    device: str | torch.device = "cpu",
    fused: bool = True,
) -> int:
    """Turn a (possibly meta-device) model into its packed form and fill it from ``state_dict``.

    FP16 linear weights are never allocated: linears become empty packed modules first, then the
    whole model is materialised on ``device`` and loaded.
    """
    replaced = replace_linear_layers(module, group_size=group_size, fused=fused, packed_only=True)
    module.to_empty(device=device)
    module.load_state_dict(state_dict)
    _restore_computed_buffers(module)
    return replaced
