"""Whole-model checkpoint in the reference's dict format: round trip, fused layers, validation."""
from __future__ import annotations

import pytest
import torch

from nibble_b200 import (fuse_parallel_linears, load_packed_model, load_quantized_model_checkpoint,
                         replace_linear_layers, save_quantized_model_checkpoint)
from nibble_b200.checkpoint import MODEL_FORMAT_NAME, MODEL_FORMAT_VERSION
from test_fusion_host_logic import Block


def _quantised(seed=0, bias=False):
    torch.manual_seed(seed)
    block = Block(bias=bias).half()
    replace_linear_layers(block, group_size=128)
    return block


def test_round_trip_into_a_meta_model(tmp_path, oracle_backend):
    source = _quantised(bias=True)
    path = tmp_path / "sub" / "model.pt"
    save_quantized_model_checkpoint(path, source, group_size=128, source_model="unit-test")
    checkpoint = load_quantized_model_checkpoint(path)
    assert checkpoint["format"] == MODEL_FORMAT_NAME == "w4a16-tinyllama" and checkpoint["version"] == MODEL_FORMAT_VERSION == 1
    assert checkpoint["source_model"] == "unit-test" and checkpoint["group_size"] == 128
    assert set(checkpoint["state_dict"]) == set(source.state_dict())
    assert all(t.device.type == "cpu" for t in checkpoint["state_dict"].values())
    with torch.device("meta"):
        target = Block(bias=True).half()
    assert load_packed_model(target, path, device="cpu") == 7
    for key, tensor in source.state_dict().items():
        assert torch.equal(target.state_dict()[key], tensor), key
    x = torch.randn((2, 128)).half()
    assert torch.equal(target(x), source(x))


def test_fused_models_are_written_under_the_original_names(tmp_path):
    plain = _quantised(seed=2)
    want = {k: v.clone() for k, v in plain.state_dict().items()}
    fuse_parallel_linears(plain)
    path = tmp_path / "fused.pt"
    save_quantized_model_checkpoint(path, plain)
    state = load_quantized_model_checkpoint(path)["state_dict"]
    assert set(state) == set(want)
    for key in want:
        assert torch.equal(state[key], want[key]), key


def test_validation_messages(tmp_path):
    good = {"format": MODEL_FORMAT_NAME, "version": 1, "source_model": "", "group_size": 128, "state_dict": {}}
    cases = [
        ([1, 2], "checkpoint must contain a dictionary"),
        ({**good, "format": "other"}, "checkpoint has an unsupported format"),
        ({**good, "version": 2}, "checkpoint has an unsupported version"),
        ({**good, "group_size": "128"}, "checkpoint is missing group_size"),
        ({**good, "state_dict": None}, "checkpoint is missing state_dict"),
    ]
    for index, (payload, message) in enumerate(cases):
        path = tmp_path / f"bad{index}.pt"
        torch.save(payload, path)
        with pytest.raises(ValueError, match=message):
            load_quantized_model_checkpoint(path)
    path = tmp_path / "good.pt"
    torch.save(good, path)
    assert load_quantized_model_checkpoint(path)["group_size"] == 128
