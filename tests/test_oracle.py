"""Pins the CPU oracle: the reference's known-answer vectors and the golden fixtures
generated from the reference's own code (tests/golden/make_golden.py)."""
from __future__ import annotations

import hashlib

import numpy as np
import pytest

from oracle import w4a16_oracle as oracle

SMALL_TAGS = [
    "n8_k256_g128_m4",
    "n7_k256_g128_m1",
    "n13_k384_g64_m3",
    "n16_k128_g32_m2",
    "n5_k64_g4_m9",
    "n33_k1024_g128_m8",
]


# ---- known answers stated in the reference's unit tests --------------------------------
def test_pack_known_bytes():
    # reference tests/test_quantization.py:11-22
    codes = np.array([[2, -3, 7, 1]], dtype=np.int8)
    assert oracle.pack_int4(codes).tolist() == [[0xD2, 0x17]]


def test_unpack_known_bytes():
    # reference tests/test_quantization.py:25-36
    packed = np.array([[0xD2, 0x17]], dtype=np.uint8)
    assert oracle.unpack_int4(packed).tolist() == [[2, -3, 7, 1]]


def test_quantize_known_values_zero_group_scale_is_one():
    # reference tests/test_quantization.py:51-69
    w = np.array([[0.25, -0.375, 0.875, -0.125, 0, 0, 0, 0]], dtype=np.float16)
    codes, scales = oracle.quantize_groupwise(w, 4)
    assert codes.tolist() == [[2, -3, 7, -1, 0, 0, 0, 0]]
    assert scales.tolist() == [[0.125, 1.0]]
    assert scales.dtype == np.float16


def test_quantize_and_pack_known_values():
    # reference tests/test_quantization.py:72-90
    w = np.array([[0.25, -0.375, 0.875, -0.125]], dtype=np.float16)
    packed, scales = oracle.quantize_and_pack_weights(w, 4)
    assert packed.tolist() == [[0xD2, 0xF7]]
    assert scales.tolist() == [[0.125]]


def test_dequantize_known_values():
    # reference tests/test_reference.py:7-28
    packed = oracle.pack_int4(np.array([[2, -3, 7, -1, 0, 0, 0, 0]], dtype=np.int8))
    scales = np.array([[0.125, 1.0]], dtype=np.float16)
    out = oracle.dequantize_weights(packed, scales, 4)
    assert out.dtype == np.float32
    assert out.tolist() == [[0.25, -0.375, 0.875, -0.125, 0, 0, 0, 0]]


def test_linear_known_values():
    # reference tests/test_reference.py:31-69
    x = np.array([[1, 2, 3, 4], [-1, 0, 2, 0.5]], dtype=np.float16)
    packed = oracle.pack_int4(np.array([[2, -3, 7, -1], [1, 2, -1, 4]], dtype=np.int8))
    scales = np.array([[0.125], [0.25]], dtype=np.float16)
    y = oracle.linear_reference(x, packed, scales, 4)
    assert y.dtype == np.float16
    assert y.tolist() == [[1.625, 4.5], [1.4375, -0.25]]


def test_all_sixteen_nibbles_decode():
    packed = np.arange(256, dtype=np.uint8).reshape(1, 256)
    codes = oracle.unpack_int4(packed)
    lo, hi = codes[0, 0::2], codes[0, 1::2]
    expect = np.array([v if v < 8 else v - 16 for v in range(16)], dtype=np.int8)
    assert np.array_equal(lo, np.tile(expect, 16))
    assert np.array_equal(hi, np.repeat(expect, 16))


def test_rejects_bad_inputs():
    with pytest.raises(TypeError):
        oracle.pack_int4(np.zeros((1, 2), dtype=np.int32))
    with pytest.raises(ValueError):
        oracle.pack_int4(np.array([[8, 0]], dtype=np.int8))
    with pytest.raises(ValueError):
        oracle.pack_int4(np.zeros((1, 3), dtype=np.int8))
    with pytest.raises(ValueError):
        oracle.quantize_groupwise(np.zeros((1, 6), dtype=np.float32), 4)
    with pytest.raises(ValueError):
        oracle.dequantize_weights(np.zeros((2, 2), np.uint8), np.zeros((2, 2), np.float16), 4)


# ---- fixtures produced by the reference's code ------------------------------------------
@pytest.mark.parametrize("tag", SMALL_TAGS)
def test_small_cases_bit_exact(golden, tag):
    data = golden("small_cases.npz")
    gs = int(data[f"{tag}/group_size"])
    codes, scales = oracle.quantize_groupwise(data[f"{tag}/weights"], gs)
    assert np.array_equal(codes, data[f"{tag}/codes"])
    assert np.array_equal(scales.view(np.uint16), data[f"{tag}/scales"].view(np.uint16))
    packed = oracle.pack_int4(codes)
    assert np.array_equal(packed, data[f"{tag}/packed"])
    assert np.array_equal(oracle.unpack_int4(packed), codes)
    deq = oracle.dequantize_weights(packed, scales, gs)
    assert np.array_equal(deq.view(np.uint32), data[f"{tag}/dequant"].view(np.uint32))
    y = oracle.linear_reference(data[f"{tag}/x"], packed, scales, gs)
    _assert_within_one_half_ulp_step(y, data[f"{tag}/y"])


def test_all_nibbles_fixture(golden):
    data = golden("all_nibbles.npz")
    assert np.array_equal(oracle.unpack_int4(data["packed"]), data["codes"])
    assert int(data["codes"].min()) == -8 and int(data["codes"].max()) == 7
    deq = oracle.dequantize_weights(data["packed"], data["scales"], 128)
    assert np.array_equal(deq.view(np.uint32), data["dequant"].view(np.uint32))
    y = oracle.linear_reference(data["x"], data["packed"], data["scales"], 128)
    _assert_within_one_half_ulp_step(y, data["y"])


def test_config1_m1_full_size(golden):
    """K=N=2048, M=1 -- the reference's CPU-runnable configuration, from the seeds."""
    from conftest import seeded_activations, seeded_weights

    data = golden("tinyllama_m1.npz")
    w = seeded_weights(2048, 2048, seed=0).numpy()
    x = seeded_activations(1, 2048, seed=1000).numpy()
    packed, scales = oracle.quantize_and_pack_weights(w, 128)
    assert hashlib.sha256(packed.tobytes()).hexdigest() == str(data["qo_proj/packed_sha256"])
    assert hashlib.sha256(scales.tobytes()).hexdigest() == str(data["qo_proj/scales_sha256"])
    deq16 = oracle.dequantize_weights(packed, scales, 128).astype(np.float16)
    assert hashlib.sha256(deq16.tobytes()).hexdigest() == str(data["qo_proj/dequant_fp16_sha256"])
    y = oracle.linear_reference(x, packed, scales, 128)
    _assert_within_one_half_ulp_step(y, data["qo_proj/y"])
    # and inside the stated acceptance bound against an FP64 product
    err = np.abs(y.astype(np.float64) - oracle.linear_fp64(x, packed, scales, 128))
    assert (err <= oracle.error_bound(x, packed, scales, 128)).all()


@pytest.mark.parametrize("name", ["qo_proj", "kv_proj", "gate_up_proj", "down_proj"])
def test_small_batch_sweep_full_size(golden, name):
    """M = 2, 4, 8 on the full-size TinyLlama-shaped layers (the small-batch sweep), from the seeds."""
    from conftest import TINYLLAMA_LAYERS, seeded_activations, seeded_weights

    data = golden("tinyllama_small_batch.npz")
    index = [layer[0] for layer in TINYLLAMA_LAYERS].index(name)
    _, k, n = TINYLLAMA_LAYERS[index]
    packed, scales = oracle.quantize_and_pack_weights(seeded_weights(n, k, seed=index).numpy(), 128)
    columns = data[f"{name}/columns"]
    for m in (2, 4, 8):
        x = seeded_activations(m, k, seed=2000 + 10 * index + m).numpy()
        assert hashlib.sha256(x.tobytes()).hexdigest() == str(data[f"{name}/m{m}/x_sha256"])
        y = oracle.linear_reference(x, packed, scales, 128)
        _assert_within_one_half_ulp_step(np.ascontiguousarray(y[:, columns]), data[f"{name}/m{m}/y"])


def _assert_within_one_half_ulp_step(mine: np.ndarray, theirs: np.ndarray) -> None:
    """Both sides round an FP32 matmul to FP16; BLAS summation order may move a value
    sitting on a rounding boundary by one FP16 step, never more -- except for outputs that cancel
    to almost nothing, where the FP32 summation noise itself (a few 1e-6 on sums of terms of order
    0.1) spans several of the much finer FP16 steps near zero."""
    assert mine.shape == theirs.shape and mine.dtype == theirs.dtype == np.float16
    a = mine.view(np.int16).astype(np.int32)
    b = theirs.view(np.int16).astype(np.int32)
    # map sign-magnitude FP16 bit patterns to a monotone integer line
    a = np.where(a < 0, -(a & 0x7FFF), a)
    b = np.where(b < 0, -(b & 0x7FFF), b)
    steps = np.abs(a - b)
    noise = np.abs(mine.astype(np.float32) - theirs.astype(np.float32)) <= 4e-6
    assert np.where(noise, 0, steps).max(initial=0) <= 1, f"max FP16 step distance {steps.max()}"
    assert (steps > 0).mean() < 0.02


def test_torch_port_matches_numpy_oracle(golden):
    """The torch restatement that the benchmark times on the host cores computes the same thing."""
    import torch

    from oracle import torch_cpu_port as port

    data = golden("all_nibbles.npz")
    packed, scales, x = (torch.from_numpy(data[key]) for key in ("packed", "scales", "x"))
    assert np.array_equal(port.unpack_codes(packed).numpy(), data["codes"])
    assert np.array_equal(port.dequantize(packed, scales, 128).numpy().view(np.uint32), data["dequant"].view(np.uint32))
    _assert_within_one_half_ulp_step(port.linear(x, packed, scales, 128).numpy(), data["y"])


def test_oracle_against_the_compiled_reference_modules(tmp_path):
    """Where oracle/_ref holds the reference's own CPU modules (oracle/build_ref.py), run them in a child
    interpreter on seeded data and compare with the numpy oracle: codes, scales and dequantised weights bit for
    bit, the linear output to within one FP16 step."""
    import pathlib
    import subprocess
    import sys

    root = pathlib.Path(__file__).resolve().parent.parent
    if not (root / "oracle" / "_ref" / "w4a16" / "reference.bin").is_file():
        pytest.skip("oracle/_ref is not built (no checkout of the reference on this machine)")
    out = tmp_path / "ref.npz"
    script = f"""
import sys
sys.path.insert(0, {str(root / "oracle")!r})
import numpy as np, torch
import build_ref
q, r = build_ref.load()
assert 'nibble_b200' not in sys.modules
g = torch.Generator().manual_seed(42)
w = torch.randn((96, 640), generator=g) * 0.02
x = torch.randn((5, 640), generator=g).half()
packed, scales = q.quantize_and_pack_weights(w, 128)
np.savez({str(out)!r}, w=w.numpy(), x=x.numpy(), packed=packed.numpy(), scales=scales.numpy(),
         dequant=r.dequantize_weights(packed, scales, 128).numpy(), y=r.linear_reference(x, packed, scales, 128).numpy())
"""
    subprocess.run([sys.executable, "-c", script], check=True, cwd=str(tmp_path), timeout=300)
    data = np.load(out)
    packed, scales = oracle.quantize_and_pack_weights(data["w"], 128)
    assert np.array_equal(packed, data["packed"])
    assert np.array_equal(scales.view(np.uint16), data["scales"].view(np.uint16))
    deq = oracle.dequantize_weights(packed, scales, 128)
    assert np.array_equal(deq.view(np.uint32), data["dequant"].view(np.uint32))
    _assert_within_one_half_ulp_step(oracle.linear_reference(data["x"], packed, scales, 128), data["y"])
