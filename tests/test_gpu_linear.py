"""-m gpu: the fused linear through the C ABI and the torch op against the oracle on identical
packed codes.  Shapes and edge cases follow the reference's tests/test_cuda.py:11-478."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from capi_helpers import capi_linear, check_against_oracle, new_workspace
from conftest import LLAMA70B_LAYERS, TINYLLAMA_LAYERS, seeded_activations, seeded_weights
from nibble_b200 import _native, linear_cuda, quantize_and_pack_weights

pytestmark = pytest.mark.gpu


def _random_case(m, k, n, gs=128, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn((n, k), generator=g) * std).half()
    x = torch.randn((m, k), generator=g).half()
    packed, scales = quantize_and_pack_weights(w, gs)
    return x.cuda(), packed.cuda(), scales.cuda()


# ---------------------------------------------------------------- golden, full size, M = 1
@pytest.mark.parametrize(("name", "k", "n"), TINYLLAMA_LAYERS)
def test_tinyllama_layers_m1_against_reference_outputs(golden, name, k, n):
    data = golden("tinyllama_m1.npz")
    index = [layer[0] for layer in TINYLLAMA_LAYERS].index(name)
    packed, scales = quantize_and_pack_weights(seeded_weights(n, k, seed=index), 128)
    x = seeded_activations(1, k, seed=1000 + index)
    y = capi_linear(x.cuda(), packed.cuda(), scales.cuda())
    torch.testing.assert_close(y.cpu(), torch.from_numpy(data[f"{name}/y"]), rtol=1e-2, atol=1e-2)
    bound = 1e-2 * float(x.float().norm()) * float(data[f"{name}/wmax"])
    assert float((y.cpu().float() - torch.from_numpy(data[f"{name}/y"]).float()).abs().max()) <= bound
    check_against_oracle(y, x, packed, scales)


def test_config1_m8_against_reference_outputs(golden):
    data = golden("config1_m8.npz")
    packed, scales = quantize_and_pack_weights(seeded_weights(2048, 2048, seed=0), 128)
    x = torch.from_numpy(data["x"])
    y = capi_linear(x.cuda(), packed.cuda(), scales.cuda())
    torch.testing.assert_close(y.cpu(), torch.from_numpy(data["y"]), rtol=1e-2, atol=1e-2)
    check_against_oracle(y, x, packed, scales)


@pytest.mark.parametrize("m", [2, 4, 8])
@pytest.mark.parametrize(("name", "k", "n"), TINYLLAMA_LAYERS)
def test_tinyllama_layers_small_batch_against_reference_outputs(golden, name, k, n, m):
    """The small-batch sweep at full size: M in {2, 4, 8} over all five TinyLlama-shaped layers, against
    outputs of the reference's CPU path on the same seeds (reference cases tests/test_cuda.py:397-451)."""
    data = golden("tinyllama_small_batch.npz")
    index = [layer[0] for layer in TINYLLAMA_LAYERS].index(name)
    packed, scales = quantize_and_pack_weights(seeded_weights(n, k, seed=index), 128)
    x = seeded_activations(m, k, seed=2000 + 10 * index + m)
    y = capi_linear(x.cuda(), packed.cuda(), scales.cuda())
    columns = torch.from_numpy(data[f"{name}/columns"])
    torch.testing.assert_close(y.cpu()[:, columns], torch.from_numpy(data[f"{name}/m{m}/y"]), rtol=1e-2, atol=1e-2)
    rows = None if n <= 8192 else data[f"{name}/columns"]
    check_against_oracle(y, x, packed, scales, rows=rows)
    assert torch.equal(linear_cuda(x.cuda(), packed.cuda(), scales.cuda(), 128), y)


@pytest.mark.parametrize("tag", ["n8_k256_g128_m4", "n7_k256_g128_m1", "n13_k384_g64_m3", "n16_k128_g32_m2",
                                 "n5_k64_g4_m9", "n33_k1024_g128_m8"])
def test_small_golden_cases(golden, tag):
    data = golden("small_cases.npz")
    gs = int(data[f"{tag}/group_size"])
    x, packed, scales = (torch.from_numpy(data[f"{tag}/{key}"]).cuda() for key in ("x", "packed", "scales"))
    y = capi_linear(x, packed, scales, gs)
    torch.testing.assert_close(y.cpu(), torch.from_numpy(data[f"{tag}/y"]), rtol=1e-2, atol=1e-2)
    check_against_oracle(y, x, packed, scales, gs)


def test_all_nibble_values(golden):
    data = golden("all_nibbles.npz")
    x, packed, scales = (torch.from_numpy(data[key]).cuda() for key in ("x", "packed", "scales"))
    for rows in (1, 3, 8):
        y = capi_linear(x[:rows].contiguous(), packed, scales)
        torch.testing.assert_close(y.cpu(), torch.from_numpy(data["y"][:rows]), rtol=1e-2, atol=1e-2)
        check_against_oracle(y, x[:rows], packed, scales)


# ---------------------------------------------------------------- batch sizes and ragged shapes
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 6, 7, 8, 9, 15, 16, 17, 24, 32, 33, 70])
def test_batch_sizes_on_2048_square(m):
    x, packed, scales = _random_case(m, 2048, 2048, seed=m)
    # from 65 rows on the tensor-core kernel runs: its weights are rounded to FP16 before the product,
    # as in the reference's route for large batches
    check_against_oracle(capi_linear(x, packed, scales), x, packed, scales, fp16_weights=m >= 65)


@pytest.mark.parametrize("m", [1, 2, 8, 12])
@pytest.mark.parametrize(("k", "n"), [(128, 1), (256, 7), (384, 13), (5632, 33), (1024, 17), (2048, 250)])
def test_ragged_shapes(m, k, n):
    x, packed, scales = _random_case(m, k, n, seed=k + n)
    check_against_oracle(capi_linear(x, packed, scales), x, packed, scales)


@pytest.mark.parametrize("m", [1, 8, 20])
@pytest.mark.parametrize("row_tiles", [1, 2])
@pytest.mark.parametrize("k_warps", [1, 2, 4, 8])
@pytest.mark.parametrize("k_splits", [1, 2, 3, 8])
@pytest.mark.parametrize(("unroll", "stages"), [(1, 0), (1, 3), (2, 0), (2, 3), (2, 4), (2, 5)])
def test_every_launch_shape(m, row_tiles, k_warps, k_splits, unroll, stages):
    k, n = 5632, 77   # 44 chunks: ragged against most k_warps * unroll * k_splits combinations
    x, packed, scales = _random_case(m, k, n, seed=3)
    ws = new_workspace(m, n, k)
    per_split = -(-(-(-44 // k_splits)) // unroll) * unroll
    buildable = not (m > 16 and row_tiles == 2)          # 32-row batches come with one row tile only
    valid = buildable and (k_splits - 1) * per_split < 44  # no K split may be empty
    if stages not in (0, 3, 4) or (unroll == 1 and (row_tiles != 1 or stages == 4)):
        valid = False
    # the activation slice of a CTA plus a minimal copy ring must fit in shared memory
    nt = 1 if m <= 8 else (2 if m <= 16 else 4)
    x_rows = 1 if m == 1 else 8 * nt
    stage_bytes = 256 * 2 * row_tiles * unroll * 16 + (8 * 16 * row_tiles * 4 if unroll == 2 else 0)
    red_bytes = 0 if k_warps == 1 else 2 * 8 * row_tiles * nt * 4 * 32 * 4
    fixed = 128 + x_rows * per_split * 256 + red_bytes
    half_sm, budget = 113 * 1024, 220 * 1024
    two_with_four, two_with_three = fixed + 4 * stage_bytes <= half_sm, fixed + 3 * stage_bytes <= half_sm
    automatic = 3 if unroll == 1 or (not two_with_four and (two_with_three or fixed + 4 * stage_bytes > budget)) else 4
    depth = stages or automatic
    fits = fixed + depth * stage_bytes <= 220 * 1024
    y = capi_linear(x, packed, scales, workspace=ws, config=(row_tiles, k_warps, k_splits, unroll, stages),
                    expect=(0 if fits else -5) if valid else -6)
    valid = valid and fits
    if valid:
        check_against_oracle(y, x, packed, scales)
        assert int(ws[:256].sum()) == 0, "arrival counters must be back at zero"


def test_split_k_workspace_is_reusable_and_deterministic():
    x, packed, scales = _random_case(4, 8192, 1024, seed=9, std=0.02)
    ws = new_workspace(4, 1024, 8192)
    first = capi_linear(x, packed, scales, workspace=ws)
    second = capi_linear(x, packed, scales, workspace=ws)
    third = capi_linear(x, packed, scales, workspace=ws, config=(1, 8, 4, 2, 0))
    assert torch.equal(first, second)
    check_against_oracle(first, x, packed, scales)
    check_against_oracle(third, x, packed, scales)
    too_small = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    capi_linear(x, packed, scales, workspace=too_small, config=(1, 8, 4, 2, 0), expect=-5)
    # without a workspace the library simply does not split
    check_against_oracle(capi_linear(x, packed, scales), x, packed, scales)


def test_one_workspace_serves_calls_of_different_shapes():
    """Split-K calls of different N share one workspace back to back (as the torch operator's per-stream workspace
    does): the partial sums of one call must never end up where the next call keeps its arrival counters.  N = 2048
    followed by N = 2560 at K = 8192 used to leave tiles 128.. of the second call unwritten."""
    lib = _native.core()
    ws = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
    torch.manual_seed(3)
    x = torch.randn((1, 8192), device="cuda").half()
    cases = []
    for n in (2048, 2560, 1024, 4096, 2560, 256, 2048):
        packed = torch.randint(0, 256, (n, 4096), dtype=torch.uint8, device="cuda")
        scales = (torch.rand((n, 64), device="cuda") * 0.002 + 0.001).half()
        assert lib.w4a16_linear_workspace_bytes(1, n, 8192) > 0 or n >= 4096, "these shapes split K"
        cases.append((packed, scales, capi_linear(x, packed, scales, workspace=ws)))     # no synchronisation in between
    torch.cuda.synchronize()
    for packed, scales, y in cases:
        assert not torch.isnan(y).any()
        rows = np.unique(np.concatenate([np.arange(0, packed.shape[0], 37), np.arange(packed.shape[0] - 40, packed.shape[0])]))
        check_against_oracle(y, x, packed, scales, rows=rows)
    assert int(ws[: 256 * 1024].sum()) == 0, "arrival counters must be back at zero"
    # the operator's own per-stream workspace, same sequence
    for packed, scales, y in cases:
        assert torch.equal(linear_cuda(x, packed, scales, 128), y)


def test_programmatic_launch_flag_gives_identical_results():
    x, packed, scales = _random_case(1, 2048, 5632, seed=4, std=0.02)
    plain = capi_linear(x, packed, scales)
    chained = [capi_linear(x, packed, scales, flags=_native.FLAG_PROGRAMMATIC_LAUNCH) for _ in range(4)]
    for y in chained:
        assert torch.equal(y, plain)


# ---------------------------------------------------------------- generic kernel
def test_misaligned_activations_take_the_generic_kernel():
    torch.manual_seed(0)
    x = torch.randn((1, 2049), dtype=torch.float16, device="cuda")[:, 1:]
    assert x.is_contiguous() and x.data_ptr() % 16 != 0
    _, packed, scales = _random_case(1, 2048, 64, seed=1)
    check_against_oracle(capi_linear(x, packed, scales), x, packed, scales)
    check_against_oracle(linear_cuda(x, packed, scales, 128), x, packed, scales)


@pytest.mark.parametrize(("gs", "m"), [(2, 1), (4, 9), (32, 3), (64, 8), (256, 2), (128, 5)])
def test_generic_kernel_group_sizes(gs, m):
    x, packed, scales = _random_case(m, 512, 21, gs=gs, seed=gs)
    y = capi_linear(x, packed, scales, gs, flags=_native.FLAG_FORCE_GENERIC)
    check_against_oracle(y, x, packed, scales, gs)


# ---------------------------------------------------------------- 70B-shaped layers, row sampling
@pytest.mark.parametrize("m", [1, 8])
@pytest.mark.parametrize(("name", "k", "n"), LLAMA70B_LAYERS)
def test_llama70b_shapes_by_row_sampling(name, k, n, m):
    """Full-size launch; outputs are independent per row, so the oracle checks a row sample."""
    torch.manual_seed(k + n + m)
    packed = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda")
    scales = (torch.rand((n, k // 128), device="cuda") * 0.01 + 1e-3).half()
    x = torch.randn((m, k), device="cuda").half()
    ws = new_workspace(m, n, k)
    y = capi_linear(x, packed, scales, workspace=ws)
    rows = np.unique(np.concatenate([np.arange(40), np.random.default_rng(0).integers(0, n, 200), np.arange(n - 40, n)]))
    check_against_oracle(y, x, packed, scales, rows=rows)
    assert not torch.isnan(y).any()
    # linearity in x: f(2x) == 2 f(x) exactly (power-of-two scaling commutes with every rounding)
    # (FP16-subnormal outputs excepted: there doubling and rounding do not commute.)
    y2 = capi_linear((x * 2).contiguous(), packed, scales, workspace=ws)
    normal = y.abs() >= 1e-3
    assert torch.equal(y2[normal], (y * 2)[normal])
    assert float((y2.float() - 2 * y.float()).abs().max()) <= 2.0 ** -22


# ---------------------------------------------------------------- torch operator behaviour
def test_op_matches_capi_and_handles_empty():
    x, packed, scales = _random_case(3, 1024, 40, seed=2)
    assert torch.equal(linear_cuda(x, packed, scales, 128), capi_linear(x, packed, scales))
    assert linear_cuda(x[:0], packed, scales, 128).shape == (0, 40)
    assert linear_cuda(x, packed[:0], scales[:0], 128).shape == (3, 0)


def test_op_argument_errors_are_runtime_errors():
    x, packed, scales = _random_case(2, 256, 8)
    with pytest.raises(RuntimeError):
        linear_cuda(x.float(), packed, scales, 128)
    with pytest.raises(RuntimeError):
        linear_cuda(torch.randn((2, 512), device="cuda").half()[:, ::2], packed, scales, 128)
    with pytest.raises(RuntimeError):
        linear_cuda(x.cpu(), packed.cpu(), scales.cpu(), 128)
    with pytest.raises(RuntimeError):
        linear_cuda(x[:, :128].contiguous(), packed, scales, 128)
    with pytest.raises(RuntimeError):
        linear_cuda(x, packed, scales, 127)
    with pytest.raises(RuntimeError):
        linear_cuda(x, packed, scales[:, :1], 128)


def test_rows_per_warp_env(monkeypatch):
    x, packed, scales = _random_case(1, 2048, 100, seed=6)
    expected = capi_linear(x, packed, scales)
    for value in ("1", "2", "4"):
        monkeypatch.setenv("W4A16_ROWS_PER_WARP", value)
        check_against_oracle(linear_cuda(x, packed, scales, 128), x, packed, scales)
    monkeypatch.setenv("W4A16_ROWS_PER_WARP", "3")
    with pytest.raises(RuntimeError):
        linear_cuda(x, packed, scales, 128)
    monkeypatch.delenv("W4A16_ROWS_PER_WARP")
    for value in ("v1", "v4", "generic"):
        monkeypatch.setenv("W4A16_DECODE", value)
        torch.testing.assert_close(linear_cuda(x, packed, scales, 128), expected, rtol=1e-2, atol=1e-2)


def test_launch_counter_counts_kernels():
    lib = _native.core()
    x, packed, scales = _random_case(1, 256, 8)
    before = lib.w4a16_launch_count()
    capi_linear(x, packed, scales)
    capi_linear(x, packed, scales, flags=_native.FLAG_FORCE_GENERIC)
    assert lib.w4a16_launch_count() == before + 2


def test_graph_capture_and_replay():
    x, packed, scales = _random_case(1, 2048, 2048, seed=8, std=0.02)
    eager = linear_cuda(x, packed, scales, 128)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        linear_cuda(x, packed, scales, 128)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = linear_cuda(x, packed, scales, 128)
    x.mul_(0.5)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager * 0.5)
