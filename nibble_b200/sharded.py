"""One W4A16 layer partitioned across the GPUs of a node (one process per GPU).

The reference project is single-GPU; this module adds the two classic tensor-parallel cuts for
layers too large or too slow for one device (Llama-70B shapes):

* **column parallel** (split the output rows N): rank r owns rows ``[r*N/G, (r+1)*N/G)``.  The
  packed layout is row-major per output row, so a shard is a contiguous slab of ``packed_weights``
  and ``scales`` -- no repacking.  Every rank computes ``y[:, its rows]`` from the full ``x``; an
  all-gather assembles ``y``.
* **row parallel** (split K, used for ``down_proj``): rank r owns a K-slice of every row (made
  contiguous once at load time) and the matching slice of ``x``.  Every rank produces an FP32
  partial ``[M, N]``; an all-reduce adds them and the sum is rounded to FP16 once.

Collectives go through ``torch.distributed`` (NCCL on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import cuda as _cuda
from .linear import QuantizedLinear, _require_cuda


def _run_fused(flat, packed_weights, scales, group_size):
    return _cuda.linear_cuda(flat, packed_weights, scales, group_size)


def _run_partial_f32(flat, packed_weights, scales, group_size):
    return _cuda.linear_partial_cuda(flat, packed_weights, scales, group_size)


def shard_rows(packed_weights: torch.Tensor, scales: torch.Tensor, rank: int, world: int):
    """Column-parallel shard: contiguous views of rows ``[rank*N/world, (rank+1)*N/world)``."""
    n = packed_weights.shape[0]
    if n % world:
        raise ValueError(f"N={n} is not divisible by the number of ranks ({world})")
    per = n // world
    return packed_weights[rank * per:(rank + 1) * per], scales[rank * per:(rank + 1) * per]


def shard_k(packed_weights: torch.Tensor, scales: torch.Tensor, rank: int, world: int, group_size: int = 128):
    """Row-parallel shard: contiguous copies of the K-slice ``[rank*K/world, (rank+1)*K/world)``."""
    k = 2 * packed_weights.shape[1]
    if k % (world * group_size):
        raise ValueError(f"K={k} must be divisible by ranks*group_size = {world * group_size}")
    per = k // world
    cols = slice(rank * per // 2, (rank + 1) * per // 2)
    groups = slice(rank * per // group_size, (rank + 1) * per // group_size)
    return packed_weights[:, cols].contiguous(), scales[:, groups].contiguous()


class ColumnParallelQuantizedLinear(torch.nn.Module):
    """``y = all_gather_N( x @ dequant(W[rows of this rank]).T )``; bias (full length) added after."""

    def __init__(self, packed_shard, scales_shard, group_size=128, bias=None, process_group=None,
                 gather_output=True):
        super().__init__()
        self.local = QuantizedLinear(packed_shard, scales_shard, group_size)
        self.register_buffer("bias", bias.detach() if bias is not None else None)
        self.process_group = process_group
        self.gather_output = gather_output

    @classmethod
    def from_full(cls, packed_weights, scales, group_size=128, bias=None, process_group=None, gather_output=True):
        rank, world = dist.get_rank(process_group), dist.get_world_size(process_group)
        packed_shard, scales_shard = shard_rows(packed_weights, scales, rank, world)
        return cls(packed_shard, scales_shard, group_size, bias, process_group, gather_output)

    def forward(self, activations: torch.Tensor) -> torch.Tensor:
        layer = self.local
        if activations.dtype != torch.float16:
            raise TypeError("activations must have dtype torch.float16")
        if activations.shape[-1] != layer.in_features:
            raise ValueError("activations last dimension must equal in_features")
        _require_cuda(activations)
        flat = activations.contiguous().reshape(-1, layer.in_features)
        local = _run_fused(flat, layer.packed_weights, layer.scales, layer.group_size)   # [M, N/G]
        if not self.gather_output:
            return local.reshape(*activations.shape[:-1], layer.out_features)
        world = dist.get_world_size(self.process_group)
        rows = flat.shape[0]
        gathered = local.new_empty((world * rows, layer.out_features))          # rank-major concatenation
        dist.all_gather_into_tensor(gathered, local, group=self.process_group)
        full = gathered.view(world, rows, layer.out_features).permute(1, 0, 2).reshape(rows, -1)
        out = full.reshape(*activations.shape[:-1], world * layer.out_features)
        return out if self.bias is None else out + self.bias


class RowParallelQuantizedLinear(torch.nn.Module):
    """``y = half( all_reduce_sum( x[:, K-slice] @ dequant(W[:, K-slice]).T ) )``; bias added after.

    ``input_is_parallel=True`` means the caller already passes this rank's K-slice of x.
    """

    def __init__(self, packed_shard, scales_shard, group_size=128, bias=None, process_group=None,
                 input_is_parallel=False):
        super().__init__()
        self.local = QuantizedLinear(packed_shard, scales_shard, group_size)
        self.register_buffer("bias", bias.detach() if bias is not None else None)
        self.process_group = process_group
        self.input_is_parallel = input_is_parallel

    @classmethod
    def from_full(cls, packed_weights, scales, group_size=128, bias=None, process_group=None,
                  input_is_parallel=False):
        rank, world = dist.get_rank(process_group), dist.get_world_size(process_group)
        packed_shard, scales_shard = shard_k(packed_weights, scales, rank, world, group_size)
        return cls(packed_shard, scales_shard, group_size, bias, process_group, input_is_parallel)

    def forward(self, activations: torch.Tensor) -> torch.Tensor:
        layer = self.local
        if activations.dtype != torch.float16:
            raise TypeError("activations must have dtype torch.float16")
        _require_cuda(activations)
        k_local = layer.in_features
        if self.input_is_parallel:
            mine = activations
        else:
            rank = dist.get_rank(self.process_group)
            world = dist.get_world_size(self.process_group)
            if activations.shape[-1] != k_local * world:
                raise ValueError("activations last dimension must equal the full in_features")
            mine = activations[..., rank * k_local:(rank + 1) * k_local]
        if mine.shape[-1] != k_local:
            raise ValueError("activations last dimension must equal this rank's K slice")
        flat = mine.contiguous().reshape(-1, k_local)
        partial = _run_partial_f32(flat, layer.packed_weights, layer.scales, layer.group_size)   # FP32 [M, N]
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.process_group)
        out = partial.to(torch.float16).reshape(*mine.shape[:-1], layer.out_features)
        return out if self.bias is None else out + self.bias
