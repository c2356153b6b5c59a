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


# ---------------------------------------------------------------------------------------------
# Exchange fused into the kernel epilogue: results are stored straight into every rank's buffer
# over NVLink (peer-mapped memory), followed by a flag; no collective-library call per layer.
# ---------------------------------------------------------------------------------------------
import ctypes

from . import _native

_MAX_POLLS = 2_000_000   # bounded device-side wait: roughly a second before a missing rank is reported


def _stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class _PeerRegion:
    """One symmetric allocation per layer: [result bytes | 256 bytes of arrival flags], mapped on
    every rank of the group, plus this rank's private counters (done, send epoch, wait epoch, status)."""

    def __init__(self, result_bytes: int, process_group) -> None:
        import torch.distributed._symmetric_memory as symm

        self.group = process_group if process_group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.result_bytes = (result_bytes + 255) // 256 * 256
        device = torch.device("cuda", torch.cuda.current_device())
        self.buffer = symm.empty((self.result_bytes + 256,), dtype=torch.uint8, device=device)
        self.buffer.zero_()
        self.handle = symm.rendezvous(self.buffer, self.group)
        self.peer_base = [int(p) for p in self.handle.buffer_ptrs]
        self.flag_table = torch.tensor([p + self.result_bytes for p in self.peer_base], dtype=torch.int64, device=device)
        self.counters = torch.zeros(4, dtype=torch.int32, device=device)   # done, send epoch, wait epoch, status
        torch.cuda.synchronize()
        dist.barrier(group=self.group)   # every rank's flags are zero before anyone publishes

    def table(self, byte_offset_for_rank) -> torch.Tensor:
        """Device array of per-rank destinations: peer base + byte_offset_for_rank(r)."""
        return torch.tensor([p + byte_offset_for_rank(r) for r, p in enumerate(self.peer_base)],
                            dtype=torch.int64, device=self.buffer.device)

    def target(self, out_table: torch.Tensor, ld: int, column_offset: int, wait: bool) -> _native.PeerTarget:
        c = self.counters.data_ptr()
        return _native.PeerTarget(out_table.data_ptr(), self.flag_table.data_ptr(), c, c + 4, c + 12, ld, column_offset,
                                  _MAX_POLLS if wait else 0, self.rank, self.world)

    def wait(self) -> None:
        c = self.counters.data_ptr()
        status = _native.core().w4a16_wait_peers(self.buffer.data_ptr() + self.result_bytes, c + 8, self.world, c + 12,
                                                 _MAX_POLLS, _stream_ptr())
        if status != 0:
            raise RuntimeError(f"w4a16_wait_peers failed: {_native.status_string(status)}")

    def check(self) -> None:
        """Host-side health check (synchronises): raises if a wait gave up on some rank."""
        missing = int(self.counters[3].item())
        if missing:
            raise RuntimeError(f"rank {missing - 1} never published its part of a sharded layer")


def _workspace(m: int, n: int, k: int, device) -> torch.Tensor | None:
    need = _native.core().w4a16_linear_workspace_bytes(m, n, k)
    return torch.zeros(need, dtype=torch.uint8, device=device) if need else None


class PeerColumnParallelQuantizedLinear(torch.nn.Module):
    """Column-parallel layer whose all-gather is the kernel's own epilogue.

    Every rank's kernel stores its ``[M, N/G]`` slice into the ``[M, N]`` result buffer of every
    rank and then raises a flag there; ``forward`` returns this rank's buffer after a bounded wait
    for all flags.  ``max_rows`` fixes the largest batch the buffers are sized for.  The returned
    tensor is reused by the next call of this layer.
    """

    def __init__(self, packed_shard, scales_shard, group_size=128, process_group=None, max_rows=8):
        super().__init__()
        if group_size != 128:
            raise ValueError("the peer-store path needs group_size == 128")
        self.local = QuantizedLinear(packed_shard, scales_shard, group_size)
        n_local = self.local.out_features
        self.region = _PeerRegion(max_rows * n_local * dist.get_world_size(process_group) * 2, process_group)
        self.max_rows = max_rows
        self.out_features = n_local * self.region.world
        self._out_table = self.region.table(lambda r: 0)
        self._workspace = {}

    def forward(self, activations: torch.Tensor) -> torch.Tensor:
        layer, region = self.local, self.region
        if activations.dtype != torch.float16:
            raise TypeError("activations must have dtype torch.float16")
        _require_cuda(activations)
        flat = activations.contiguous().reshape(-1, layer.in_features)
        m = flat.shape[0]
        if m > self.max_rows:
            raise ValueError(f"batch of {m} rows exceeds max_rows={self.max_rows}")
        if m not in self._workspace:
            self._workspace[m] = _workspace(m, layer.out_features, layer.in_features, flat.device)
        ws = self._workspace[m]
        # wait=True: the launch returns to the stream only when every rank's slice has landed here
        target = region.target(self._out_table, self.out_features, region.rank * layer.out_features, wait=True)
        flags = _native.FLAG_PROGRAMMATIC_LAUNCH if _cuda.programmatic_launch_enabled() else 0
        status = _native.core().w4a16_linear_f16_peers(
            flat.data_ptr(), layer.packed_weights.data_ptr(), layer.scales.data_ptr(), m, layer.out_features,
            layer.in_features, 128, ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            flags, ctypes.byref(target), _stream_ptr())
        if status != 0:
            raise RuntimeError(f"w4a16_linear_f16_peers failed: {_native.status_string(status)}")
        full = region.buffer[: m * self.out_features * 2].view(torch.float16).view(m, self.out_features)
        return full.reshape(*activations.shape[:-1], self.out_features)


class PeerRowParallelQuantizedLinear(torch.nn.Module):
    """Row-parallel layer (K split) with a one-shot all-reduce built from peer stores.

    Each rank's kernel writes its FP32 partial ``[M, N]`` into slot ``rank`` of the staging buffer on
    every rank and raises a flag; after a bounded wait each rank sums the ``G`` partials in rank order
    (identical bits everywhere) and rounds once to FP16.  Takes this rank's K-slice of x.
    """

    def __init__(self, packed_shard, scales_shard, group_size=128, process_group=None, max_rows=8):
        super().__init__()
        if group_size != 128:
            raise ValueError("the peer-store path needs group_size == 128")
        self.local = QuantizedLinear(packed_shard, scales_shard, group_size)
        world = dist.get_world_size(process_group)
        self.region = _PeerRegion(world * max_rows * self.local.out_features * 4, process_group)
        self.max_rows = max_rows
        self._tables = {}
        self._workspace = {}

    def forward(self, activations: torch.Tensor) -> torch.Tensor:
        layer, region = self.local, self.region
        if activations.dtype != torch.float16:
            raise TypeError("activations must have dtype torch.float16")
        _require_cuda(activations)
        flat = activations.contiguous().reshape(-1, layer.in_features)
        m, n = flat.shape[0], layer.out_features
        if m > self.max_rows:
            raise ValueError(f"batch of {m} rows exceeds max_rows={self.max_rows}")
        if m not in self._tables:
            self._tables[m] = region.table(lambda r: region.rank * m * n * 4)   # my slot on every rank
            self._workspace[m] = _workspace(m, n, layer.in_features, flat.device)
        ws = self._workspace[m]
        target = region.target(self._tables[m], n, 0, wait=False)   # the summing kernel does the waiting
        flags = _native.FLAG_OUTPUT_F32 | (_native.FLAG_PROGRAMMATIC_LAUNCH if _cuda.programmatic_launch_enabled() else 0)
        lib = _native.core()
        status = lib.w4a16_linear_f16_peers(
            flat.data_ptr(), layer.packed_weights.data_ptr(), layer.scales.data_ptr(), m, n, layer.in_features, 128,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, flags,
            ctypes.byref(target), _stream_ptr())
        if status != 0:
            raise RuntimeError(f"w4a16_linear_f16_peers failed: {_native.status_string(status)}")
        out = torch.empty((m, n), dtype=torch.float16, device=flat.device)
        counters = region.counters.data_ptr()
        status = lib.w4a16_sum_partials_f16(region.buffer.data_ptr(), out.data_ptr(), m * n, region.world,
                                            region.buffer.data_ptr() + region.result_bytes, counters + 4, counters + 12,
                                            _MAX_POLLS, _stream_ptr())
        if status != 0:
            raise RuntimeError(f"w4a16_sum_partials_f16 failed: {_native.status_string(status)}")
        return out.reshape(*activations.shape[:-1], n)
