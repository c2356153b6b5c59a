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


# ----------------------------------------------------------------------------- whole models
# The reference writes a quantised model as one ``torch.save`` dict (scripts/quantize_tinyllama.py:71-83)
# and reads it back into an empty model (scripts/generate.py:214-257).  Same keys here, so files interchange.
MODEL_FORMAT_NAME = "w4a16-tinyllama"
MODEL_FORMAT_VERSION = 1


def save_quantized_model_checkpoint(path: str | os.PathLike, model: torch.nn.Module, group_size: int = 128,
                                    source_model: str = "") -> None:
    """Write the state dict of a model whose linears are already ``QuantizedLinear`` (CPU tensors, the
    reference's keys ``format``, ``version``, ``source_model``, ``group_size``, ``state_dict``).

    Layers fused by ``fuse_parallel_linears`` appear under their original names (each slice saves its own
    rows), so the file does not depend on whether fusion was applied.
    """
    # FusedSlice modules save their own rows under their own names, so the model's state dict already is the file's
    state = {key: tensor.detach().cpu().clone() for key, tensor in model.state_dict().items()}
    os.makedirs(os.path.dirname(os.path.abspath(os.fspath(path))), exist_ok=True)
    torch.save({"format": MODEL_FORMAT_NAME, "version": MODEL_FORMAT_VERSION, "source_model": source_model,
                "group_size": int(group_size), "state_dict": state}, os.fspath(path))


def load_quantized_model_checkpoint(path: str | os.PathLike) -> dict:
    """Read and validate a model checkpoint; tensors stay on the CPU (errors as in the reference)."""
    checkpoint = torch.load(os.fspath(path), map_location="cpu", weights_only=True)
    if not isinstance(checkpoint, dict):
        raise ValueError("checkpoint must contain a dictionary")
    if checkpoint.get("format") != MODEL_FORMAT_NAME:
        raise ValueError("checkpoint has an unsupported format")
    if checkpoint.get("version") != MODEL_FORMAT_VERSION:
        raise ValueError("checkpoint has an unsupported version")
    if not isinstance(checkpoint.get("group_size"), int):
        raise ValueError("checkpoint is missing group_size")
    if not isinstance(checkpoint.get("state_dict"), dict):
        raise ValueError("checkpoint is missing state_dict")
    return checkpoint


def load_packed_model(model: torch.nn.Module, path: str | os.PathLike, device: str | torch.device = "cuda",
                      fused: bool = True, *, plan: dict[str, str] | None = None, rank: int | None = None,
                      world: int | None = None, process_group=None, exchange: str = "nccl", max_rows: int = 8) -> int:
    """Fill ``model`` (typically built on the meta device from a config) from a model checkpoint:
    its linears become packed modules, everything is materialised directly on ``device`` -- FP16
    linear weights never exist -- and the packed tensors are copied in.  Returns the number of
    linears replaced (the reference's ``load_packed_model``, scripts/generate.py:230-257, without the
    hub download).

    With ``plan`` the loader also partitions layers across the ``world`` ranks of a tensor-parallel group
    while it reads them: ``plan`` maps the last component of a layer's name to ``"column"`` (this rank
    keeps rows ``[rank*N/world, (rank+1)*N/world)`` of the packed matrix -- a contiguous slab -- and the
    layer gathers its output) or ``"row"`` (this rank keeps a K slice of every row and the layer sums the
    partial results), e.g. ``{"q_proj": "column", ..., "down_proj": "row"}`` for a LLaMA block.  Only this
    rank's shard of a planned layer is ever copied to ``device``.  ``exchange`` picks the modules of
    ``nibble_b200.sharded`` that do the collectives: ``"nccl"`` (``torch.distributed``; also gloo on CPU
    ranks) or ``"peer"`` (the kernels' own exchange over peer-mapped memory, batches up to ``max_rows``).
    ``rank`` / ``world`` default to those of ``process_group``.
    """
    from .integration import _restore_computed_buffers, load_packed_state_dict, replace_linear_layers
    from .linear import QuantizedLinear

    checkpoint = load_quantized_model_checkpoint(path)
    group_size = checkpoint["group_size"]
    if not plan:
        return load_packed_state_dict(model, checkpoint["state_dict"], group_size=group_size, device=device, fused=fused)

    import torch.distributed as dist

    from . import sharded

    if exchange not in ("nccl", "peer"):
        raise ValueError("exchange must be 'nccl' or 'peer'")
    if any(cut not in ("column", "row") for cut in plan.values()):
        raise ValueError("plan values must be 'column' or 'row'")
    if rank is None:
        rank = dist.get_rank(process_group)
    if world is None:
        world = dist.get_world_size(process_group)
    state = dict(checkpoint["state_dict"])
    replaced = replace_linear_layers(model, group_size=group_size, fused=fused, packed_only=True, fuse_siblings=False)

    # Take the planned layers out of the tree before it is materialised, so that their full-size packed
    # storage is never allocated on the device; remember where they sat.
    planned = []
    for name, module in list(model.named_modules()):
        leaf = name.rsplit(".", 1)[-1]
        if isinstance(module, QuantizedLinear) and leaf in plan:
            parent = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
            planned.append((name, leaf, parent, plan[leaf]))
            setattr(parent, leaf, torch.nn.Identity())
    shards = {}
    for name, leaf, parent, cut in planned:
        packed, scales = state.pop(f"{name}.packed_weights"), state.pop(f"{name}.scales")
        bias = state.pop(f"{name}.bias", None)
        _check_pair(packed, scales, group_size)
        cutter = sharded.shard_rows if cut == "column" else sharded.shard_k
        extra = () if cut == "column" else (group_size,)
        shards[name] = tuple(t.to(device) for t in cutter(packed, scales, rank, world, *extra)) + (
            None if bias is None else bias.to(device),)
    model.to_empty(device=device)
    model.load_state_dict(state)
    _restore_computed_buffers(model)
    for name, leaf, parent, cut in planned:
        packed, scales, bias = shards.pop(name)
        if exchange == "peer":
            cls = sharded.PeerColumnParallelQuantizedLinear if cut == "column" else sharded.PeerRowParallelQuantizedLinear
            if bias is not None:
                raise ValueError(f"layer '{name}' has a bias: the peer exchange modules carry none")
            layer = cls(packed, scales, group_size, process_group=process_group, max_rows=max_rows)
            if cut == "row":
                layer = sharded.SliceInput(layer, rank)
        elif cut == "column":
            layer = sharded.ColumnParallelQuantizedLinear(packed, scales, group_size, bias=bias, process_group=process_group)
        else:
            layer = sharded.RowParallelQuantizedLinear(packed, scales, group_size, bias=bias, process_group=process_group)
        setattr(parent, leaf, layer)
    return replaced
