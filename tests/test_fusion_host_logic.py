"""Launch fusion of sibling layers: host logic on CPU with the oracle standing in for the kernels."""
from __future__ import annotations

import torch

from nibble_b200 import QuantizedLinear, fuse_parallel_linears, quantize_and_pack_weights, replace_linear_layers
from nibble_b200.fusion import FusedQuantizedLinear, FusedSlice


class Block(torch.nn.Module):
    """The shape of a LLaMA decoder block's linears: q/k/v and gate/up share their input."""

    def __init__(self, hidden=128, kv=32, inter=256, bias=False):
        super().__init__()
        self.q_proj = torch.nn.Linear(hidden, hidden, bias=bias)
        self.k_proj = torch.nn.Linear(hidden, kv, bias=bias)
        self.v_proj = torch.nn.Linear(hidden, kv, bias=bias)
        self.o_proj = torch.nn.Linear(hidden, hidden, bias=bias)
        self.gate_proj = torch.nn.Linear(hidden, inter, bias=bias)
        self.up_proj = torch.nn.Linear(hidden, inter, bias=bias)
        self.down_proj = torch.nn.Linear(inter, hidden, bias=bias)

    def forward(self, x):
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        h = self.o_proj(q + torch.cat([k, v, k, v], dim=-1))
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(h)) * self.up_proj(h))


def _quantised_block(bias=False, seed=0):
    torch.manual_seed(seed)
    block = Block(bias=bias).half()
    assert replace_linear_layers(block, group_size=128, fuse_siblings=False) == 7
    return block


def test_fused_block_matches_unfused_block_with_three_fewer_launches(oracle_backend):
    block = _quantised_block()
    x = torch.randn((3, 128), generator=torch.Generator().manual_seed(1)).half()
    expected = block(x)
    calls_unfused = len(oracle_backend)
    assert calls_unfused == 7
    assert fuse_parallel_linears(block) == 2
    assert isinstance(block.q_proj, FusedSlice) and isinstance(block.up_proj, FusedSlice)
    assert isinstance(block.q_proj__k_proj__v_proj, FusedQuantizedLinear)
    assert block.q_proj__k_proj__v_proj.split_sizes == [128, 32, 32]
    assert type(block.o_proj) is QuantizedLinear
    del oracle_backend[:]
    got = block(x)
    assert len(oracle_backend) == 4          # qkv, o, gate+up, down
    assert torch.equal(got, expected)        # rows are independent: same arithmetic per output channel
    assert block.q_proj__k_proj__v_proj.launches == 1 and block.gate_proj__up_proj.launches == 1
    assert fuse_parallel_linears(block) == 0  # nothing left to fuse


def test_slices_expose_the_original_layers_tensors_and_bias_is_carried():
    block = _quantised_block(bias=True, seed=3)
    k_packed, k_scales, k_bias = block.k_proj.packed_weights.clone(), block.k_proj.scales.clone(), block.k_proj.bias.clone()
    fuse_parallel_linears(block)
    assert torch.equal(block.k_proj.packed_weights, k_packed)
    assert torch.equal(block.k_proj.scales, k_scales)
    assert torch.equal(block.k_proj.bias, k_bias)
    keys = set(block.state_dict())
    # the state dict keeps the layers' own names; the concatenated tensors are not saved a second time
    assert {"q_proj.packed_weights", "k_proj.scales", "v_proj.bias", "up_proj.packed_weights"} <= keys
    assert not any(key.startswith("q_proj__k_proj__v_proj.") for key in keys)


def test_cache_follows_tensor_identity_and_version(oracle_backend):
    block = _quantised_block()
    fuse_parallel_linears(block)
    owner = block.gate_proj__up_proj
    x = torch.ones((2, 128), dtype=torch.float16)
    first = block.gate_proj(x)
    x.mul_(2)                                # in-place write between the siblings' calls: no stale columns
    second = block.up_proj(x)
    assert owner.launches == 2
    assert torch.equal(second, owner(x)[..., 256:])
    assert not torch.equal(first, owner(x)[..., :256])
    y = x.clone()                            # equal values, different tensor: its own launch
    block.gate_proj(y)
    assert owner.launches == 3
    block.up_proj(y)
    assert owner.launches == 3 and owner._input is None   # both siblings served: references dropped


def test_groups_that_do_not_qualify_are_left_alone():
    block = _quantised_block()
    packed, scales = quantize_and_pack_weights(torch.randn(32, 256).half(), 128)
    block.k_proj = QuantizedLinear(packed, scales, 128)      # different in_features
    assert fuse_parallel_linears(block) == 1                 # only gate/up
    assert type(block.q_proj) is QuantizedLinear
    plain = Block().half()
    assert fuse_parallel_linears(plain) == 0                 # nn.Linear children are not touched


def test_inference_mode_tensors_are_cached_by_identity(oracle_backend):
    block = _quantised_block()
    fuse_parallel_linears(block)
    with torch.inference_mode():
        x = torch.ones((1, 128), dtype=torch.float16)
        block.gate_proj(x)
        block.up_proj(x)
    assert block.gate_proj__up_proj.launches == 1


def test_replacement_fuses_siblings_by_default_and_keeps_names_and_state_dict(oracle_backend, monkeypatch):
    torch.manual_seed(5)
    plain = Block(bias=True).half()
    fused = Block(bias=True).half()
    fused.load_state_dict(plain.state_dict())
    assert replace_linear_layers(plain, group_size=128, fuse_siblings=False) == 7
    assert replace_linear_layers(fused, group_size=128) == 7          # default: siblings share a launch
    assert isinstance(fused.q_proj, FusedSlice) and isinstance(fused.gate_proj, FusedSlice)
    assert type(fused.o_proj) is QuantizedLinear and type(plain.q_proj) is QuantizedLinear
    want, got = plain.state_dict(), fused.state_dict()
    assert list(got) == list(want)                                    # same keys, same order
    for key in want:
        assert torch.equal(got[key], want[key]), key
    x = torch.randn((2, 128), generator=torch.Generator().manual_seed(1)).half()
    del oracle_backend[:]
    assert torch.equal(fused(x), plain(x))
    assert len(oracle_backend) == 4 + 7
    # a state dict written by either loads into the other
    other = Block(bias=True).half()
    replace_linear_layers(other, group_size=128)
    other.load_state_dict(want)
    assert torch.equal(other(x), plain(x))
    plain.load_state_dict(other.state_dict())
    with __import__("pytest").raises(RuntimeError, match="size mismatch"):
        other.load_state_dict({**want, "k_proj.scales": want["k_proj.scales"][:1]})
    monkeypatch.setenv("W4A16_FUSE_SIBLINGS", "0")
    unfused = Block().half()
    replace_linear_layers(unfused, group_size=128)
    assert type(unfused.q_proj) is QuantizedLinear
