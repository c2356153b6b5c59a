"""The shipped quantiser / packer against the reference's known answers, the golden fixtures made
from the reference's code, and the oracle."""
from __future__ import annotations

import hashlib

import numpy as np
import pytest
import torch

from conftest import seeded_weights
from nibble_b200.quantization import pack_int4, quantize_and_pack_weights, quantize_groupwise, unpack_int4
from oracle import w4a16_oracle as oracle
from test_oracle import SMALL_TAGS


def test_pack_known_bytes():
    # reference tests/test_quantization.py:11-22
    out = pack_int4(torch.tensor([[2, -3, 7, 1]], dtype=torch.int8))
    assert out.dtype == torch.uint8 and out.tolist() == [[0xD2, 0x17]]


def test_unpack_known_bytes():
    # reference tests/test_quantization.py:25-36
    out = unpack_int4(torch.tensor([[0xD2, 0x17]], dtype=torch.uint8))
    assert out.dtype == torch.int8 and out.tolist() == [[2, -3, 7, 1]]


def test_round_trip_random_codes():
    g = torch.Generator().manual_seed(3)
    codes = torch.randint(-7, 8, (4, 128), dtype=torch.int8, generator=g)
    assert torch.equal(unpack_int4(pack_int4(codes)), codes)


def test_unpack_every_byte_value():
    packed = torch.arange(256, dtype=torch.uint8).reshape(1, 256)
    assert np.array_equal(unpack_int4(packed).numpy(), oracle.unpack_int4(packed.numpy()))


def test_quantize_known_values():
    # reference tests/test_quantization.py:51-69 (zero group -> scale 1.0)
    w = torch.tensor([[0.25, -0.375, 0.875, -0.125, 0, 0, 0, 0]], dtype=torch.float16)
    codes, scales = quantize_groupwise(w, group_size=4)
    assert codes.tolist() == [[2, -3, 7, -1, 0, 0, 0, 0]] and codes.dtype == torch.int8
    assert scales.tolist() == [[0.125, 1.0]] and scales.dtype == torch.float16


def test_quantize_and_pack_known_values():
    # reference tests/test_quantization.py:72-90
    w = torch.tensor([[0.25, -0.375, 0.875, -0.125]], dtype=torch.float16)
    packed, scales = quantize_and_pack_weights(w, group_size=4)
    assert packed.tolist() == [[0xD2, 0xF7]]
    assert scales.tolist() == [[0.125]]


@pytest.mark.parametrize("tag", SMALL_TAGS)
def test_small_cases_match_reference_bits(golden, tag):
    data = golden("small_cases.npz")
    gs = int(data[f"{tag}/group_size"])
    w = torch.from_numpy(data[f"{tag}/weights"])
    codes, scales = quantize_groupwise(w, gs)
    assert np.array_equal(codes.numpy(), data[f"{tag}/codes"])
    assert np.array_equal(scales.numpy().view(np.uint16), data[f"{tag}/scales"].view(np.uint16))
    assert np.array_equal(pack_int4(codes).numpy(), data[f"{tag}/packed"])
    assert np.array_equal(unpack_int4(torch.from_numpy(data[f"{tag}/packed"])).numpy(), data[f"{tag}/codes"])


def test_full_size_layer_matches_reference_digest(golden):
    data = golden("tinyllama_m1.npz")
    packed, scales = quantize_and_pack_weights(seeded_weights(2048, 2048, seed=0), 128)
    assert hashlib.sha256(packed.numpy().tobytes()).hexdigest() == str(data["qo_proj/packed_sha256"])
    assert hashlib.sha256(scales.numpy().tobytes()).hexdigest() == str(data["qo_proj/scales_sha256"])


def test_matches_oracle_on_fp16_weights():
    g = torch.Generator().manual_seed(11)
    w = torch.randn((24, 512), generator=g).half()
    packed, scales = quantize_and_pack_weights(w, 64)
    o_packed, o_scales = oracle.quantize_and_pack_weights(w.numpy(), 64)
    assert np.array_equal(packed.numpy(), o_packed)
    assert np.array_equal(scales.numpy().view(np.uint16), o_scales.view(np.uint16))


@pytest.mark.parametrize(
    ("call", "error"),
    [
        (lambda: pack_int4(torch.zeros((1, 2), dtype=torch.int32)), TypeError),
        (lambda: pack_int4(torch.zeros((2,), dtype=torch.int8)), ValueError),
        (lambda: pack_int4(torch.zeros((1, 3), dtype=torch.int8)), ValueError),
        (lambda: pack_int4(torch.tensor([[8, 0]], dtype=torch.int8)), ValueError),
        (lambda: pack_int4(torch.tensor([[-8, 0]], dtype=torch.int8)), ValueError),
        (lambda: unpack_int4(torch.zeros((1, 2), dtype=torch.int8)), TypeError),
        (lambda: unpack_int4(torch.zeros((2,), dtype=torch.uint8)), ValueError),
        (lambda: quantize_groupwise(torch.zeros((1, 4), dtype=torch.float64), 4), TypeError),
        (lambda: quantize_groupwise(torch.zeros((4,), dtype=torch.float32), 4), ValueError),
        (lambda: quantize_groupwise(torch.zeros((1, 4), dtype=torch.float32), 0), ValueError),
        (lambda: quantize_groupwise(torch.zeros((1, 6), dtype=torch.float32), 4), ValueError),
    ],
)
def test_argument_errors(call, error):
    with pytest.raises(error):
        call()


def test_empty_matrix():
    packed, scales = quantize_and_pack_weights(torch.zeros((0, 128), dtype=torch.float32), 128)
    assert packed.shape == (0, 64) and scales.shape == (0, 1)
