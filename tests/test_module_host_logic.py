"""Host-side behaviour of QuantizedLinear / integration / checkpoint without a GPU.

Device arithmetic is supplied by the ``oracle_backend`` fixture; these tests pin the known answers
of the reference's module tests (tests/test_linear.py:11-129, tests/test_integration.py:34-154,
tests/test_checkpoint.py:10-30) and the one intended difference: CPU tensors are refused.
"""
from __future__ import annotations

import pytest
import torch

import nibble_b200
import w4a16
from nibble_b200 import (
    Int4Linear,
    QuantizedLinear,
    load_packed_state_dict,
    load_quantized_weight_checkpoint,
    quantize_and_pack_weights,
    replace_linear_layers,
    save_quantized_weight_checkpoint,
)
from nibble_b200.linear import FUSED_MAX_ROWS

WEIGHTS = torch.tensor([[0.25, -0.375, 0.875, -0.125], [0.25, 0.5, -0.25, 1.75]], dtype=torch.float16)
ACTIVATIONS = torch.tensor([[1.0, 2.0, 3.0, 4.0], [-1.0, 0.0, 2.0, 0.5]], dtype=torch.float16)


def _layer(**kwargs):
    packed, scales = quantize_and_pack_weights(WEIGHTS, group_size=4)
    return QuantizedLinear(packed, scales, group_size=4, **kwargs)


def test_package_surface_matches_reference_names():
    for name in [
        "QuantizedLinear", "pack_int4", "unpack_int4", "quantize_groupwise", "quantize_and_pack_weights",
        "save_quantized_weight_checkpoint", "load_quantized_weight_checkpoint", "replace_linear_layers",
        "load_packed_state_dict", "linear_cuda", "dequantize_cuda", "cuda_extension_available",
    ]:
        assert getattr(w4a16, name) is getattr(nibble_b200, name)
    assert Int4Linear is QuantizedLinear
    import importlib

    for sub in ["cuda", "linear", "quantization", "integration", "checkpoint"]:
        alias = importlib.import_module(f"w4a16.{sub}")
        real = importlib.import_module(f"nibble_b200.{sub}")
        public = [k for k in vars(real) if not k.startswith("_")]
        assert public and all(getattr(alias, k) is getattr(real, k) for k in public)
    assert importlib.import_module("w4a16.linear").FUSED_MAX_ROWS == FUSED_MAX_ROWS


def test_cpu_tensors_are_refused_loudly():
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        _layer()(ACTIVATIONS)


def test_known_values_3d_input(oracle_backend):
    layer = _layer()
    out = layer(ACTIVATIONS.unsqueeze(0))
    assert torch.equal(out, torch.tensor([[[1.625, 7.5], [1.4375, 0.125]]], dtype=torch.float16))
    assert set(layer.state_dict()) == {"packed_weights", "scales"}
    assert oracle_backend == ["fused"]


def test_bias_is_a_buffer_and_is_added(oracle_backend):
    bias = torch.tensor([0.5, -0.25], dtype=torch.float16)
    layer = _layer(bias=bias)
    assert set(layer.state_dict()) == {"packed_weights", "scales", "bias"}
    assert torch.equal(layer(ACTIVATIONS), torch.tensor([[2.125, 7.25], [1.9375, -0.125]], dtype=torch.float16))


def test_routing_by_rows_and_fused_flag(oracle_backend):
    packed, scales = quantize_and_pack_weights(torch.randn(8, 128).half(), 128)
    layer = QuantizedLinear(packed, scales, 128)
    layer(torch.zeros((FUSED_MAX_ROWS, 128), dtype=torch.float16))
    layer(torch.zeros((FUSED_MAX_ROWS + 1, 128), dtype=torch.float16))
    layer(torch.zeros((2, FUSED_MAX_ROWS, 128), dtype=torch.float16))
    QuantizedLinear(packed, scales, 128, fused=False)(torch.zeros((1, 128), dtype=torch.float16))
    assert oracle_backend == ["fused", "dequant", "dequant", "dequant"]


def test_prefill_window_routes_wide_layers_to_the_fused_operator(oracle_backend):
    from nibble_b200.linear import PREFILL_FUSED_MAX_ROWS, PREFILL_MIN_WEIGHT_TILES, uses_fused_kernel

    wide = 128 * PREFILL_MIN_WEIGHT_TILES
    assert uses_fused_kernel(FUSED_MAX_ROWS + 1, wide, 128)
    assert uses_fused_kernel(PREFILL_FUSED_MAX_ROWS, wide, 128)
    assert not uses_fused_kernel(PREFILL_FUSED_MAX_ROWS + 1, wide, 128)
    assert not uses_fused_kernel(FUSED_MAX_ROWS + 1, wide - 128, 128)     # too few weight tiles to fill the GPU
    assert not uses_fused_kernel(FUSED_MAX_ROWS + 1, wide, 64)            # tensor-core kernel is for 128-wide groups
    assert uses_fused_kernel(10_000, 8, 4)                                # no dequantise operator for this group size
    packed, scales = quantize_and_pack_weights(torch.randn(wide, 128).half(), 128)
    layer = QuantizedLinear(packed, scales, 128)
    layer(torch.zeros((FUSED_MAX_ROWS + 1, 128), dtype=torch.float16))
    layer(torch.zeros((4, PREFILL_FUSED_MAX_ROWS // 4 + 1, 128), dtype=torch.float16))
    layer.fused = False
    layer(torch.zeros((FUSED_MAX_ROWS + 1, 128), dtype=torch.float16))
    assert oracle_backend == ["fused", "dequant", "dequant"]


def test_group_size_without_dequantize_kernel_stays_fused(oracle_backend):
    layer = _layer(fused=False)  # group_size 4 is not a multiple of 32
    layer(ACTIVATIONS)
    assert oracle_backend == ["fused"]


def test_noncontiguous_activations_are_accepted(oracle_backend):
    layer = _layer()
    wide = torch.zeros((2, 8), dtype=torch.float16)
    wide[:, :4] = ACTIVATIONS
    view = wide[:, :4]
    assert not view.is_contiguous()
    assert torch.equal(layer(view), layer(ACTIVATIONS))


def test_empty_shapes():
    layer = QuantizedLinear.empty(out_features=2, in_features=4, group_size=4, bias=True, fused=False)
    assert layer.packed_weights.shape == (2, 2) and layer.packed_weights.dtype == torch.uint8
    assert layer.scales.shape == (2, 1) and layer.scales.dtype == torch.float16
    assert layer.bias is not None and layer.bias.shape == (2,)
    assert layer.fused is False


def test_from_float_equals_fp16_linear_on_representable_weights(oracle_backend):
    fp = torch.nn.Linear(4, 2, bias=True, dtype=torch.float16)
    with torch.no_grad():
        fp.weight.copy_(WEIGHTS)
        fp.bias.copy_(torch.tensor([0.5, -0.25], dtype=torch.float16))
    q = QuantizedLinear.from_float(fp, group_size=4)
    assert torch.equal(q(ACTIVATIONS), fp(ACTIVATIONS))
    assert torch.equal(q.bias, fp.bias)


@pytest.mark.parametrize(
    ("build", "error", "match"),
    [
        (lambda: QuantizedLinear.empty(2, 6, group_size=4), ValueError, "K must be divisible by group_size"),
        (lambda: QuantizedLinear.empty(0, 4, group_size=4), ValueError, "greater than zero"),
        (lambda: QuantizedLinear.empty(2, 4, group_size=0), ValueError, "group_size"),
        (lambda: QuantizedLinear(torch.zeros((2, 2), dtype=torch.int8), torch.zeros((2, 1), dtype=torch.float16), 4),
         ValueError, "packed_weights must be uint8"),
        (lambda: QuantizedLinear(torch.zeros((2, 2), dtype=torch.uint8), torch.zeros((2, 1), dtype=torch.float32), 4),
         ValueError, "scales must be float16"),
        (lambda: QuantizedLinear(torch.zeros((2, 2), dtype=torch.uint8), torch.zeros((2, 2), dtype=torch.float16), 4),
         ValueError, "scales must have shape"),
        (lambda: _layer(bias=torch.zeros(3, dtype=torch.float16)), ValueError, "bias must be float16"),
        (lambda: QuantizedLinear.from_float(torch.nn.ReLU()), TypeError, "torch.nn.Linear"),
    ],
)
def test_constructor_errors(build, error, match):
    with pytest.raises(error, match=match):
        build()


def test_forward_errors(oracle_backend):
    layer = _layer()
    with pytest.raises(TypeError, match="activations must have dtype torch.float16"):
        layer(torch.ones((2, 4), dtype=torch.float32))
    with pytest.raises(RuntimeError, match="activations must not require grad"):
        layer(torch.ones((2, 4), dtype=torch.float16, requires_grad=True))
    with pytest.raises(ValueError, match="last dimension"):
        layer(torch.ones((2, 6), dtype=torch.float16))
    with pytest.raises(ValueError, match="at least one dimension"):
        layer(torch.tensor(1.0, dtype=torch.float16))


# ---------------------------------------------------------------- model surgery
class Toy(torch.nn.Module):
    def __init__(self, fill: bool = True):
        super().__init__()
        self.direct = torch.nn.Linear(4, 2, bias=True, dtype=torch.float16)
        self.nested = torch.nn.Sequential(torch.nn.Linear(4, 2, bias=False, dtype=torch.float16))
        if fill:
            with torch.no_grad():
                self.direct.weight.copy_(WEIGHTS)
                self.direct.bias.copy_(torch.tensor([0.5, -0.25], dtype=torch.float16))
                self.nested[0].weight.copy_(WEIGHTS)

    def forward(self, x):
        return self.direct(x) + self.nested(x)


def test_replace_linear_layers_preserves_outputs(oracle_backend):
    model = Toy()
    expected = model(ACTIVATIONS)
    assert replace_linear_layers(model, group_size=4) == 2
    assert isinstance(model.direct, QuantizedLinear) and isinstance(model.nested[0], QuantizedLinear)
    assert torch.equal(model(ACTIVATIONS), expected)
    assert replace_linear_layers(model, group_size=4) == 0  # already replaced


def test_replace_warns_and_skips_unaligned():
    class Mixed(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.aligned = torch.nn.Linear(4, 2, dtype=torch.float16)
            self.nested = torch.nn.Sequential(torch.nn.Linear(6, 2, bias=False, dtype=torch.float16))

    model = Mixed()
    with pytest.warns(UserWarning, match=r"nested\.0"):
        assert replace_linear_layers(model, group_size=4) == 1
    assert isinstance(model.aligned, QuantizedLinear)
    assert isinstance(model.nested[0], torch.nn.Linear)


def test_replace_propagates_fused_flag_and_training_mode():
    model = Toy().eval()
    assert replace_linear_layers(model, group_size=4, fused=False) == 2
    assert model.direct.fused is False and model.nested[0].fused is False
    assert model.direct.training is False
    with pytest.raises(ValueError):
        replace_linear_layers(Toy(), group_size=0)


def test_packed_only_round_trip(oracle_backend):
    source = Toy()
    replace_linear_layers(source, group_size=4)
    expected = source(ACTIVATIONS)
    state = {k: v.clone() for k, v in source.state_dict().items()}
    target = Toy(fill=False)
    assert replace_linear_layers(target, group_size=4, packed_only=True) == 2
    target.load_state_dict(state)
    assert torch.equal(target(ACTIVATIONS), expected)


def test_load_packed_state_dict_from_meta(oracle_backend):
    source = Toy()
    replace_linear_layers(source, group_size=4, fused=False)
    expected = source(ACTIVATIONS)
    state = {k: v.clone() for k, v in source.state_dict().items()}
    with torch.device("meta"):
        target = Toy(fill=False)
    assert load_packed_state_dict(target, state, group_size=4, device="cpu", fused=False) == 2
    assert target.direct.packed_weights.device.type == "cpu"
    assert "weight" not in target.direct.state_dict()
    assert target.direct.fused is False
    assert torch.equal(target(ACTIVATIONS), expected)


def test_tiny_llama_round_trip(oracle_backend):
    transformers = pytest.importorskip("transformers")
    config = transformers.LlamaConfig(
        vocab_size=32, hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
        num_key_value_heads=2, max_position_embeddings=32, rms_norm_eps=1e-5, tie_word_embeddings=False,
    )
    torch.manual_seed(0)
    source = transformers.AutoModelForCausalLM.from_config(config, dtype=torch.float16).eval()
    replaced = replace_linear_layers(source, group_size=64, fused=False)
    assert replaced == 8  # q, k, v, o, gate, up, down, lm_head
    state = {k: v.detach().clone() for k, v in source.state_dict().items()}
    ids = torch.randint(0, 32, (1, 4))
    with torch.device("meta"):
        target = transformers.AutoModelForCausalLM.from_config(config, dtype=torch.float16)
    assert load_packed_state_dict(target, state, group_size=64, device="cpu", fused=False) == 8
    target.eval()
    with torch.inference_mode():
        expected = source(input_ids=ids).logits
        result = target(input_ids=ids).logits
    assert not any(isinstance(m, torch.nn.Linear) for m in target.modules())
    assert torch.equal(source.model.rotary_emb.inv_freq, target.model.rotary_emb.inv_freq)
    assert torch.equal(result, expected)


# ---------------------------------------------------------------- checkpoint
def test_checkpoint_round_trip(tmp_path):
    packed, scales = quantize_and_pack_weights(WEIGHTS[:1], group_size=4)
    path = tmp_path / "w.pt"
    save_quantized_weight_checkpoint(path, packed, scales, group_size=4)
    got_packed, got_scales, got_group = load_quantized_weight_checkpoint(path)
    assert torch.equal(got_packed, packed) and torch.equal(got_scales, scales) and got_group == 4
    blob = torch.load(path, weights_only=True)
    assert blob["format"] == "w4a16-linear" and blob["version"] == 1
    assert tuple(blob["original_shape"]) == (1, 4)


def test_checkpoint_rejects_foreign_or_inconsistent_files(tmp_path):
    packed, scales = quantize_and_pack_weights(WEIGHTS, group_size=4)
    good = {"format": "w4a16-linear", "version": 1, "packed_weights": packed, "scales": scales,
            "group_size": 4, "original_shape": (2, 4)}
    for key, value in [("format", "other"), ("version", 2), ("group_size", "4"), ("original_shape", (4, 2)),
                       ("scales", None), ("packed_weights", None)]:
        bad = dict(good)
        bad[key] = value
        torch.save(bad, tmp_path / "bad.pt")
        with pytest.raises(ValueError):
            load_quantized_weight_checkpoint(tmp_path / "bad.pt")
    torch.save([1, 2], tmp_path / "list.pt")
    with pytest.raises(ValueError):
        load_quantized_weight_checkpoint(tmp_path / "list.pt")
    with pytest.raises(ValueError):
        save_quantized_weight_checkpoint(tmp_path / "x.pt", packed, scales[:, :0], group_size=4)
