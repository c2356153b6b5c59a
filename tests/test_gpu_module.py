"""-m gpu: QuantizedLinear and the model-surgery helpers on a CUDA device
(reference tests/test_linear.py:130-243, tests/test_integration.py:157-204, tests/test_cuda.py:535-556)."""
from __future__ import annotations

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from capi_helpers import check_against_oracle
from nibble_b200 import QuantizedLinear, load_packed_state_dict, quantize_and_pack_weights, replace_linear_layers
from nibble_b200.linear import FUSED_MAX_ROWS
from oracle import w4a16_oracle as oracle

pytestmark = pytest.mark.gpu


def _layer(n=8, k=128, bias=False, fused=True, seed=0):
    torch.manual_seed(seed)
    w = torch.randn((n, k), dtype=torch.float16, device="cuda")
    packed, scales = quantize_and_pack_weights(w, 128)
    b = torch.randn((n,), dtype=torch.float16, device="cuda") if bias else None
    return QuantizedLinear(packed, scales, 128, bias=b, fused=fused)


def _oracle_out(layer, x):
    y = oracle.linear_reference(x.reshape(-1, layer.in_features).cpu().numpy(), layer.packed_weights.cpu().numpy(),
                                layer.scales.cpu().numpy(), layer.group_size)
    y = torch.from_numpy(y).reshape(*x.shape[:-1], layer.out_features)
    return y if layer.bias is None else y + layer.bias.cpu()


@pytest.mark.parametrize("rows", [1, 2, 16])
def test_module_matches_oracle_with_bias(rows):
    layer = _layer(bias=True)
    x = torch.randn((rows, 128), dtype=torch.float16, device="cuda")
    torch.testing.assert_close(layer(x).cpu(), _oracle_out(layer, x), rtol=1e-2, atol=1e-2)


def test_module_accepts_noncontiguous_and_3d():
    layer = _layer()
    x = torch.randn((2, 3, 256), dtype=torch.float16, device="cuda")[..., :128]
    assert not x.is_contiguous()
    out = layer(x)
    assert out.shape == (2, 3, 8)
    torch.testing.assert_close(out.cpu(), _oracle_out(layer, x.contiguous()), rtol=1e-2, atol=1e-2)


def test_large_batch_and_unfused_mode_match_fp16_matmul_of_dequantised_weights():
    layer = _layer(n=64, k=512, seed=2)
    w16 = torch.from_numpy(
        oracle.dequantize_weights(layer.packed_weights.cpu().numpy(), layer.scales.cpu().numpy(), 128).astype(np.float16)
    ).cuda()
    big = torch.randn((FUSED_MAX_ROWS + 5, 512), dtype=torch.float16, device="cuda")
    torch.testing.assert_close(layer(big), F.linear(big, w16), rtol=1e-3, atol=1e-3)
    layer.fused = False
    one = torch.randn((1, 512), dtype=torch.float16, device="cuda")
    torch.testing.assert_close(layer(one), F.linear(one, w16), rtol=1e-3, atol=1e-3)


def test_prefill_batch_on_a_wide_layer_takes_the_tensor_core_kernel():
    from nibble_b200 import _native
    from nibble_b200.linear import PREFILL_MIN_WEIGHT_TILES, uses_fused_kernel

    n = 128 * PREFILL_MIN_WEIGHT_TILES
    layer = _layer(n=n, k=1024, seed=3)
    w16 = torch.from_numpy(
        oracle.dequantize_weights(layer.packed_weights.cpu().numpy(), layer.scales.cpu().numpy(), 128).astype(np.float16)
    ).cuda()
    x = torch.randn((3, 100, 1024), dtype=torch.float16, device="cuda")
    assert uses_fused_kernel(300, n, 128)
    before = _native.core().w4a16_launch_count()
    out = layer(x)
    assert _native.core().w4a16_launch_count() == before + 1      # one fused launch, no dequantise pass
    torch.testing.assert_close(out, F.linear(x, w16), rtol=2e-3, atol=2e-3)


def test_replace_linear_layers_on_cuda_model():
    torch.manual_seed(1)
    model = torch.nn.Sequential(
        torch.nn.Linear(256, 512, bias=True), torch.nn.SiLU(), torch.nn.Linear(512, 128, bias=False)
    ).half().cuda()
    x = torch.randn((4, 256), dtype=torch.float16, device="cuda")
    assert replace_linear_layers(model, group_size=128) == 2
    first = model[0]
    check_against_oracle(first(x) - first.bias, x, first.packed_weights, first.scales)
    assert model(x).shape == (4, 128)


def test_packed_load_never_materialises_fp16_weights():
    n = k = 2048
    source = torch.nn.Linear(k, n, bias=False, dtype=torch.float16)
    q = QuantizedLinear.from_float(source, group_size=128)
    state = {"layer.packed_weights": q.packed_weights.clone(), "layer.scales": q.scales.clone()}

    class Wrapper(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layer = torch.nn.Linear(k, n, bias=False, dtype=torch.float16)

    with torch.device("meta"):
        model = Wrapper()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    before = torch.cuda.memory_allocated()
    assert load_packed_state_dict(model, state, group_size=128, device="cuda") == 1
    delta = torch.cuda.memory_allocated() - before
    packed_bytes = q.packed_weights.numel() + 2 * q.scales.numel()
    assert model.layer.packed_weights.is_cuda
    assert packed_bytes <= delta < 2 * n * k
    x = torch.randn((1, k), dtype=torch.float16, device="cuda")
    check_against_oracle(model.layer(x), x, model.layer.packed_weights, model.layer.scales)


@pytest.mark.parametrize("rows", [1, 4, 24])
def test_traces_under_torch_compile_aot_eager(rows):
    layer = _layer(n=16, k=256, seed=3)
    x = torch.randn((rows, 256), dtype=torch.float16, device="cuda")
    compiled = torch.compile(layer, backend="aot_eager", fullgraph=True)
    assert torch.equal(compiled(x), layer(x))


def test_fused_siblings_one_launch_same_numbers():
    from nibble_b200 import _native, fuse_parallel_linears

    class Attn(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = torch.nn.Linear(2048, 2048, bias=False)
            self.k_proj = torch.nn.Linear(2048, 256, bias=False)
            self.v_proj = torch.nn.Linear(2048, 256, bias=False)

        def forward(self, x):
            return self.q_proj(x), self.k_proj(x), self.v_proj(x)

    torch.manual_seed(4)
    attn = Attn().half().cuda()
    assert replace_linear_layers(attn, group_size=128, fuse_siblings=False) == 3
    x = torch.randn((1, 1, 2048), dtype=torch.float16, device="cuda")
    separate = [t.clone() for t in attn(x)]
    packed = [m.packed_weights.clone() for m in (attn.q_proj, attn.k_proj, attn.v_proj)]
    scales = [m.scales.clone() for m in (attn.q_proj, attn.k_proj, attn.v_proj)]
    assert fuse_parallel_linears(attn) == 1
    before = _native.core().w4a16_launch_count()
    fused = attn(x)
    assert _native.core().w4a16_launch_count() == before + 1
    for got, ref, p, s in zip(fused, separate, packed, scales):
        assert got.shape == ref.shape
        torch.testing.assert_close(got, ref, rtol=1e-2, atol=1e-2)
        check_against_oracle(got.reshape(1, -1), x.reshape(1, -1), p, s)


def test_model_checkpoint_loads_straight_onto_the_device(tmp_path):
    """A file in the reference's model-checkpoint format (scripts/generate.py:214-257) into a meta-device model:
    packed tensors go straight to the GPU, FP16 linear weights never exist, the block computes what the source
    block computes."""
    from nibble_b200 import load_packed_model, save_quantized_model_checkpoint
    from test_fusion_host_logic import Block

    torch.manual_seed(6)
    source = Block(hidden=1024, kv=256, inter=2048, bias=True).half()
    assert replace_linear_layers(source, group_size=128) == 7        # quantised on the host
    path = tmp_path / "model.pt"
    save_quantized_model_checkpoint(path, source, group_size=128, source_model="gpu-test")
    with torch.device("meta"):
        target = Block(hidden=1024, kv=256, inter=2048, bias=True).half()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    before = torch.cuda.memory_allocated()
    assert load_packed_model(target, path, device="cuda") == 7
    delta = torch.cuda.memory_allocated() - before
    packed_bytes = sum(t.numel() * t.element_size() for t in source.state_dict().values())
    fp16_bytes = 2 * sum(m.in_features * m.out_features for m in source.modules() if isinstance(m, QuantizedLinear))
    assert packed_bytes <= delta < fp16_bytes / 2
    for key, tensor in source.state_dict().items():
        got = target.state_dict()[key]
        assert got.is_cuda and torch.equal(got.cpu(), tensor), key
    x = torch.randn((2, 1024), dtype=torch.float16, device="cuda")
    q = target.q_proj
    check_against_oracle(q(x) - q.bias, x, q.packed_weights, q.scales)
    assert target(x).shape == (2, 1024) and not torch.isnan(target(x)).any()
