"""Launch-count fusion: sibling ``QuantizedLinear`` layers that read the same activations
(q/k/v projections; gate/up projections) become ONE operator launch.

The packed layout is row-major per output channel, so concatenating layers along dim 0 of
``packed_weights`` and ``scales`` is the fused layer: no repacking.  The model code is not touched:
each original child is replaced by a ``FusedSlice`` that returns its columns of the shared output,
and the first slice that sees a new activation tensor triggers the single launch.

The reference has no counterpart; its loader quantises each ``nn.Linear`` separately
(w4a16/integration.py:8-69).  This is the caller-side step that removes launches once the kernels sit
at the launch floor.
"""
from __future__ import annotations

from typing import Iterable, Sequence

import torch

from .linear import QuantizedLinear

DEFAULT_GROUPS: tuple[tuple[str, ...], ...] = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"))


def _version_of(tensor: torch.Tensor) -> int:
    """In-place-write counter of a tensor; tensors made under ``torch.inference_mode`` keep none
    (for those the cache can only go by identity, shape and address)."""
    try:
        return tensor._version
    except RuntimeError:
        return -1


class FusedQuantizedLinear(QuantizedLinear):
    """A ``QuantizedLinear`` over the concatenated rows of several layers, plus a one-entry cache
    keyed on the identity and version of the activation tensor."""

    def __init__(self, parts: Sequence[QuantizedLinear]):
        first = parts[0]
        for part in parts:
            if (part.in_features, part.group_size, part.fused) != (first.in_features, first.group_size, first.fused):
                raise ValueError("fused layers must share in_features, group_size and the fused flag")
            if part.packed_weights.device != first.packed_weights.device:
                raise ValueError("fused layers must live on one device")
            if (part.bias is None) != (first.bias is None):
                raise ValueError("fused layers must all have a bias or none")
        packed = torch.cat([part.packed_weights for part in parts], dim=0).contiguous()
        scales = torch.cat([part.scales for part in parts], dim=0).contiguous()
        bias = None if first.bias is None else torch.cat([part.bias for part in parts], dim=0).contiguous()
        super().__init__(packed, scales, first.group_size, bias=bias, fused=first.fused)
        # The fused tensors stay out of state dicts: every FusedSlice saves and loads its own rows under the
        # name its layer always had, so checkpoints do not depend on whether siblings were fused.
        for name in ("packed_weights", "scales", "bias"):
            self._non_persistent_buffers_set.add(name)
        self.split_sizes = [part.out_features for part in parts]
        self._offsets = [0]
        for size in self.split_sizes:
            self._offsets.append(self._offsets[-1] + size)
        self._key: tuple | None = None
        self._input: torch.Tensor | None = None
        self._output: torch.Tensor | None = None
        self._served = 0
        self.launches = 0

    def _columns(self, activations: torch.Tensor, index: int) -> torch.Tensor:
        key = (activations.data_ptr(), _version_of(activations), tuple(activations.shape), tuple(activations.stride()))
        # The cached input is held by reference, so its storage cannot have been handed to another
        # tensor; the version counter catches in-place writes.
        if self._output is None or self._input is not activations or self._key != key:
            self._output = self.forward(activations)
            self._input, self._key, self._served = activations, key, 0
            self.launches += 1
        out = self._output[..., self._offsets[index]:self._offsets[index + 1]]
        self._served += 1
        if self._served >= len(self.split_sizes):   # every sibling has its columns: drop the references
            self._input = self._output = self._key = None
        return out

    def extra_repr(self) -> str:
        return super().extra_repr() + f", split_sizes={self.split_sizes}"


class FusedSlice(torch.nn.Module):
    """Stands where one of the fused layers stood; ``forward`` returns that layer's columns."""

    def __init__(self, owner: FusedQuantizedLinear, index: int):
        super().__init__()
        object.__setattr__(self, "_owner", owner)      # not a registered child: the parent registers the owner once
        self.index = index
        self.in_features = owner.in_features
        self.out_features = owner.split_sizes[index]

    @property
    def packed_weights(self) -> torch.Tensor:
        owner = self._owner
        return owner.packed_weights[owner._offsets[self.index]:owner._offsets[self.index + 1]]

    @property
    def scales(self) -> torch.Tensor:
        owner = self._owner
        return owner.scales[owner._offsets[self.index]:owner._offsets[self.index + 1]]

    @property
    def bias(self):
        owner = self._owner
        return None if owner.bias is None else owner.bias[owner._offsets[self.index]:owner._offsets[self.index + 1]]

    def forward(self, activations: torch.Tensor) -> torch.Tensor:
        return self._owner._columns(activations, self.index)

    # ---- state dict: this layer's rows under this layer's name, exactly as before fusion -------------
    def _tensors(self) -> dict:
        named = {"packed_weights": self.packed_weights, "scales": self.scales}
        if self._owner.bias is not None:
            named["bias"] = self.bias
        return named

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        for name, view in self._tensors().items():
            destination[prefix + name] = view if keep_vars else view.detach()

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        for name, view in self._tensors().items():
            key = prefix + name
            if key not in state_dict:
                if strict:
                    missing_keys.append(key)
                continue
            value = state_dict[key]
            if tuple(value.shape) != tuple(view.shape) or value.dtype != view.dtype:
                error_msgs.append(f"size mismatch for {key}: copying a param with shape {tuple(value.shape)} "
                                  f"and dtype {value.dtype}, the layer holds {tuple(view.shape)} {view.dtype}")
                continue
            with torch.no_grad():
                view.copy_(value)
        if strict:
            unexpected_keys.extend(key for key in state_dict
                                   if key.startswith(prefix) and key[len(prefix):] not in self._tensors())

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, slice={self.index} of a fused launch"


def fuse_parallel_linears(module: torch.nn.Module, groups: Iterable[Sequence[str]] = DEFAULT_GROUPS) -> int:
    """Below ``module``, wherever one parent holds every name of a group as ``QuantizedLinear``
    children with equal ``in_features``, replace them by slices of one fused layer (registered on
    the parent as ``"<a>__<b>..."``).  Returns the number of fused launches created.

    The children must be called with the very same activation tensor (as HuggingFace attention and
    MLP blocks do); a child called with anything else simply triggers its own fused launch.
    """
    fused_count = 0
    groups = [tuple(group) for group in groups]
    for parent in list(module.modules()):
        children = dict(parent.named_children())
        for group in groups:
            parts = [children.get(name) for name in group]
            if len(parts) < 2 or any(type(part) is not QuantizedLinear for part in parts):
                continue
            if len({(p.in_features, p.group_size, p.fused, p.bias is None, p.packed_weights.device) for p in parts}) != 1:
                continue
            owner = FusedQuantizedLinear(parts)
            owner.train(parts[0].training)
            setattr(parent, "__".join(group), owner)
            for index, name in enumerate(group):
                setattr(parent, name, FusedSlice(owner, index))
            fused_count += 1
    return fused_count
