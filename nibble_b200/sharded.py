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
# Exchange fused into the kernels: a sender's epilogue stores its result straight into a buffer on
# every rank over NVLink (peer-mapped memory), every element together with a tag naming the
# publication it belongs to; the kernel that consumes the result re-reads, while it stages its
# activations and with its weight prefetch already in flight, whatever has not arrived yet, and gives
# the buffer back through a set of flags.  No fence, no flag round trip, no collective-library call.
# The protocol is described beside w4a16_peer_target / w4a16_peer_source in include/w4a16_b200.h.
# ---------------------------------------------------------------------------------------------
import ctypes

from . import _native

_MAX_POLLS = 1_000_000   # bounded device-side wait: about a second before a missing rank is reported
_FLAG_BYTES = 256        # consumed[world]
_HALF_ELEMENT = 4        # bytes of a tagged FP16 element in a result buffer
_FLOAT_ELEMENT = 8       # bytes of a tagged FP32 element


def _stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _launch_flags() -> int:
    return _native.FLAG_PROGRAMMATIC_LAUNCH if _cuda.programmatic_launch_enabled() else 0


class LocalRanks:
    """Stand-in for a process group when all ``world`` ranks of a sharded layer live in ONE process on
    ONE GPU (tests, single-GPU bring-up): the "peer" buffers are ordinary device tensors.  The ranks'
    kernels then run one after the other on a stream, so every rank's senders must be launched before
    any rank's readers."""

    def __init__(self, world: int):
        self.world = world
        self._regions: dict = {}

    def buffers(self, key, nbytes: int, device) -> list[torch.Tensor]:
        """The ``world`` regions of the layer called ``key`` (created at the first rank's request)."""
        if key not in self._regions:
            self._regions[key] = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(self.world)]
        return self._regions[key]


class PeerRegion:
    """Memory of one sharded layer on this rank: ``[result buffer 0 | result buffer 1 | consumed[world]]``
    in memory every rank can write (torch symmetric memory, or plain tensors with
    ``LocalRanks``), plus this rank's private words (done, send epoch, staged, status)."""

    def __init__(self, result_bytes: int, process_group=None, *, local: LocalRanks | None = None, rank: int | None = None,
                 key=None, max_polls: int = _MAX_POLLS) -> None:
        self.result_bytes = (result_bytes + 255) // 256 * 256
        self.max_polls = int(max_polls)
        device = torch.device("cuda", torch.cuda.current_device())
        total = 2 * self.result_bytes + _FLAG_BYTES
        if local is not None:
            self.rank, self.world = int(rank), local.world
            buffers = local.buffers(key, total, device)
            self.buffer = buffers[self.rank]
            self.peer_base = [int(b.data_ptr()) for b in buffers]
            self._keep = buffers
        else:
            import torch.distributed._symmetric_memory as symm

            group = process_group if process_group is not None else dist.group.WORLD
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
            self.buffer = symm.empty((total,), dtype=torch.uint8, device=device)
            self.buffer.zero_()
            handle = symm.rendezvous(self.buffer, group)
            self.peer_base = [int(p) for p in handle.buffer_ptrs]
            self._keep = handle
            torch.cuda.synchronize()
            dist.barrier(group=group)   # every rank's flags are zero before anyone publishes
        if self.world > 32:
            raise ValueError("at most 32 ranks")
        flags0 = 2 * self.result_bytes
        i64 = dict(dtype=torch.int64, device=device)
        self._consumed_table = torch.tensor([p + flags0 for p in self.peer_base], **i64)
        self.counters = torch.zeros(4, dtype=torch.int32, device=device)   # done, send epoch, staged, status
        self._tables: dict = {}

    # addresses on this rank
    @property
    def base(self) -> int:
        return self.buffer.data_ptr()

    def _counter(self, index: int) -> int:
        return self.counters.data_ptr() + 4 * index

    def out_table(self, byte_offset: int) -> torch.Tensor:
        """Device array of every rank's result buffer 0 plus ``byte_offset``."""
        if byte_offset not in self._tables:
            self._tables[byte_offset] = torch.tensor([p + byte_offset for p in self.peer_base], dtype=torch.int64,
                                                     device=self.buffer.device)
        return self._tables[byte_offset]

    def target(self, byte_offset: int, ld: int, column_offset: int) -> _native.PeerTarget:
        return _native.PeerTarget(self.out_table(byte_offset).data_ptr(), self.base + 2 * self.result_bytes,
                                  self._counter(0), self._counter(1), self._counter(3), self.result_bytes, ld,
                                  column_offset, self.max_polls, self.rank, self.world)

    def source(self, first_column: int = 0, columns_per_rank: int = 0) -> _native.PeerSource:
        return _native.PeerSource(self._counter(1), self._consumed_table.data_ptr(), self._counter(2), self._counter(3),
                                  self.result_bytes, self.max_polls, first_column, columns_per_rank, self.rank, self.world)

    def check(self) -> None:
        """Host-side health check (synchronises): raises if a bounded wait gave up on some rank."""
        code = int(self.counters[3].item())
        if code > 32:
            raise RuntimeError(f"rank {code - 33} never released a result buffer of a sharded layer")
        if code:
            raise RuntimeError(f"rank {code - 1} never published its part of a sharded layer")


class PeerView:
    """The gathered ``[rows, columns]`` FP16 result of a peer layer's latest launch, still in its result
    buffer and possibly still arriving.  Hand it to another peer layer's ``launch`` (that kernel then does the
    waiting, in its prologue) or call ``materialize()`` (a small kernel waits and copies it out).  Every
    launch's view must be consumed exactly once on every rank before the layer is launched a third time."""

    def __init__(self, region: PeerRegion, rows: int, ld: int, column0: int = 0, columns: int | None = None):
        self.region, self.rows, self.ld, self.column0 = region, rows, ld, column0
        self.columns = ld if columns is None else columns

    def narrow(self, column0: int, columns: int) -> "PeerView":
        if column0 < 0 or column0 + columns > self.columns or column0 % 8:
            raise ValueError("column slice out of range or not a multiple of 8")
        return PeerView(self.region, self.rows, self.ld, self.column0 + column0, columns)

    @property
    def data_ptr(self) -> int:
        return self.region.base + _HALF_ELEMENT * self.column0

    def source(self) -> _native.PeerSource:
        return self.region.source(self.column0, self.ld // self.region.world)

    def materialize(self) -> torch.Tensor:
        if self.column0 or self.columns != self.ld:
            raise ValueError("materialize() copies whole rows: call it on the un-narrowed view")
        if (self.rows * self.ld) % 8:
            raise ValueError("rows * columns must be a multiple of 8")
        out = torch.empty((self.rows, self.ld), dtype=torch.float16, device=self.region.buffer.device)
        source = self.source()
        status = _native.core().w4a16_wait_peers(ctypes.byref(source), self.region.base, out.data_ptr(),
                                                 out.numel(), _launch_flags(), _stream_ptr())
        if status != 0:
            raise RuntimeError(f"w4a16_wait_peers failed: {_native.status_string(status)}")
        return out


def _workspace(m: int, n: int, k: int, device) -> torch.Tensor | None:
    need = _native.core().w4a16_linear_workspace_bytes(m, n, k)
    return torch.zeros(need, dtype=torch.uint8, device=device) if need else None


def _launch_peer_linear(layer: QuantizedLinear, x, m: int, workspaces: dict, target, out_f32: bool, y=None) -> None:
    """One fused linear whose input is a tensor or a ``PeerView`` and whose output goes to ``target`` (or ``y``)."""
    if isinstance(x, PeerView):
        if x.columns != layer.in_features or x.rows != m:
            raise ValueError("the view's shape does not match the layer")
        x_ptr, x_ld, source = x.data_ptr, x.ld, x.source()
        device = x.region.buffer.device
    else:
        if x.dtype != torch.float16 or x.ndim != 2 or x.shape[1] != layer.in_features or x.stride(1) != 1:
            raise ValueError("activations must be FP16 [M, K] with unit stride along K")
        _require_cuda(x)
        x_ptr, x_ld, source, device = x.data_ptr(), x.stride(0) if m > 1 else layer.in_features, None, x.device
    if m not in workspaces:
        workspaces[m] = _workspace(m, layer.out_features, layer.in_features, device)
    ws = workspaces[m]
    flags = _launch_flags() | (_native.FLAG_OUTPUT_F32 if out_f32 else 0)
    status = _native.core().w4a16_linear_f16_peers(
        x_ptr, x_ld, layer.packed_weights.data_ptr(), layer.scales.data_ptr(), None if y is None else y.data_ptr(), m,
        layer.out_features, layer.in_features, 128, ws.data_ptr() if ws is not None else None,
        ws.numel() if ws is not None else 0, flags, None if target is None else ctypes.byref(target),
        None if source is None else ctypes.byref(source), _stream_ptr())
    if status != 0:
        raise RuntimeError(f"w4a16_linear_f16_peers failed: {_native.status_string(status)}")


class PeerColumnParallelQuantizedLinear(torch.nn.Module):
    """Column-parallel layer whose all-gather is done by the kernels themselves.

    ``launch(x)`` runs this rank's slice and stores the ``[M, N/G]`` result into the ``[M, N]`` result buffer
    of every rank; it returns a ``PeerView`` and does not wait.  ``forward(x)`` is ``launch(x).materialize()``.
    ``x`` may itself be a ``PeerView`` (of a column slice) of another peer layer.  ``max_rows`` fixes the
    largest batch the buffers are sized for.
    """

    def __init__(self, packed_shard, scales_shard, group_size=128, process_group=None, max_rows=8, *,
                 local: LocalRanks | None = None, rank: int | None = None, name: str | None = None,
                 max_polls: int = _MAX_POLLS):
        super().__init__()
        if local is not None and (rank is None or name is None):
            raise ValueError("with LocalRanks, give this rank's index and a name shared by the layer's ranks")
        if group_size != 128:
            raise ValueError("the peer-store path needs group_size == 128")
        self.local = QuantizedLinear(packed_shard, scales_shard, group_size)
        n_local = self.local.out_features
        world = local.world if local is not None else dist.get_world_size(process_group)
        self.region = PeerRegion(max_rows * n_local * world * _HALF_ELEMENT, process_group, local=local, rank=rank, key=name,
                                 max_polls=max_polls)
        self.max_rows = max_rows
        self.in_features = self.local.in_features
        self.out_features = n_local * self.region.world
        self._workspace: dict = {}

    def launch(self, x) -> PeerView:
        m = x.rows if isinstance(x, PeerView) else x.shape[0]
        if m > self.max_rows:
            raise ValueError(f"batch of {m} rows exceeds max_rows={self.max_rows}")
        region = self.region
        target = region.target(0, self.out_features, region.rank * self.local.out_features)
        _launch_peer_linear(self.local, x, m, self._workspace, target, out_f32=False)
        return PeerView(region, m, self.out_features)

    def forward(self, activations: torch.Tensor) -> torch.Tensor:
        if activations.dtype != torch.float16:
            raise TypeError("activations must have dtype torch.float16")
        _require_cuda(activations)
        flat = activations.contiguous().reshape(-1, self.in_features)
        return self.launch(flat).materialize().reshape(*activations.shape[:-1], self.out_features)


class PeerRowParallelQuantizedLinear(torch.nn.Module):
    """Row-parallel layer (K split) with a one-shot all-reduce built from peer stores.

    ``launch(x)``: this rank's kernel writes its FP32 partial ``[M, N]`` into slot ``rank`` of the staging
    buffer on every rank and raises a flag.  ``finish(m)``: one small kernel waits (bounded) for every rank's
    partial, sums the ``G`` partials in rank order (identical bits everywhere), rounds once to FP16 and gives the
    staging buffer back.  ``forward`` is both.  Takes this rank's K-slice of x (a tensor or a ``PeerView``).
    """

    def __init__(self, packed_shard, scales_shard, group_size=128, process_group=None, max_rows=8, *,
                 local: LocalRanks | None = None, rank: int | None = None, name: str | None = None,
                 max_polls: int = _MAX_POLLS):
        super().__init__()
        if local is not None and (rank is None or name is None):
            raise ValueError("with LocalRanks, give this rank's index and a name shared by the layer's ranks")
        if group_size != 128:
            raise ValueError("the peer-store path needs group_size == 128")
        self.local = QuantizedLinear(packed_shard, scales_shard, group_size)
        world = local.world if local is not None else dist.get_world_size(process_group)
        n = self.local.out_features
        self.region = PeerRegion(world * max_rows * n * _FLOAT_ELEMENT, process_group, local=local, rank=rank, key=name,
                                 max_polls=max_polls)
        self.max_rows = max_rows
        self.in_features = self.local.in_features
        self.out_features = n
        self._workspace: dict = {}

    def launch(self, x) -> int:
        m = x.rows if isinstance(x, PeerView) else x.shape[0]
        if m > self.max_rows:
            raise ValueError(f"batch of {m} rows exceeds max_rows={self.max_rows}")
        region, n = self.region, self.out_features
        target = region.target(region.rank * m * n * _FLOAT_ELEMENT, n, 0)   # my slot on every rank
        _launch_peer_linear(self.local, x, m, self._workspace, target, out_f32=True)
        return m

    def finish(self, m: int, out: torch.Tensor | None = None) -> torch.Tensor:
        region, n = self.region, self.out_features
        if out is None:
            out = torch.empty((m, n), dtype=torch.float16, device=region.buffer.device)
        source = region.source()
        status = _native.core().w4a16_sum_partials_f16(region.base, out.data_ptr(), m * n, region.world,
                                                       ctypes.byref(source), _launch_flags(), _stream_ptr())
        if status != 0:
            raise RuntimeError(f"w4a16_sum_partials_f16 failed: {_native.status_string(status)}")
        return out

    def forward(self, activations: torch.Tensor) -> torch.Tensor:
        if activations.dtype != torch.float16:
            raise TypeError("activations must have dtype torch.float16")
        _require_cuda(activations)
        flat = activations.contiguous().reshape(-1, self.in_features)
        return self.finish(self.launch(flat)).reshape(*activations.shape[:-1], self.out_features)


class SliceInput(torch.nn.Module):
    """Feeds a row-parallel layer that wants this rank's K slice from the full activations."""

    def __init__(self, layer: torch.nn.Module, rank: int):
        super().__init__()
        self.layer, self.rank = layer, rank

    def forward(self, activations: torch.Tensor) -> torch.Tensor:
        k = self.layer.in_features
        return self.layer(activations[..., self.rank * k:(self.rank + 1) * k])
