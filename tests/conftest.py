"""Shared fixtures.  ``gpu`` marks tests that need a CUDA device and the built library."""
from __future__ import annotations

import pathlib
import sys

import numpy as np
import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"

# name, K, N of the TinyLlama-1.1B-shaped linears; order fixes the weight seeds.
TINYLLAMA_LAYERS = [
    ("qo_proj", 2048, 2048),
    ("kv_proj", 2048, 256),
    ("gate_up_proj", 2048, 5632),
    ("down_proj", 5632, 2048),
    ("lm_head", 2048, 32000),
]
# Llama-3-70B-shaped linears (K, N).
LLAMA70B_LAYERS = [
    ("qo_proj", 8192, 8192),
    ("kv_proj", 8192, 1024),
    ("gate_up_proj", 8192, 28672),
    ("down_proj", 28672, 8192),
]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device and the built CUDA library")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def seeded_weights(n: int, k: int, seed: int = 0) -> torch.Tensor:
    """FP32 N(0, 0.02) weights from a CPU generator (stand-in for checkpoint weights)."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn((n, k), dtype=torch.float32, generator=g) * 0.02


def seeded_activations(m: int, k: int, seed: int = 1) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn((m, k), dtype=torch.float32, generator=g).half()


@pytest.fixture(scope="session")
def golden():
    def load(name: str):
        return np.load(GOLDEN / name)
    return load


@pytest.fixture
def oracle_backend(monkeypatch):
    """Lets the host-side module logic run without a GPU.

    The two device routines ``QuantizedLinear`` calls are replaced by the CPU oracle and the
    CUDA-only guard is lifted; everything else (validation, flattening, routing, bias, reshape)
    is the shipped code.  ``calls`` records which routine each forward used.
    """
    import nibble_b200.linear as linear_module
    from oracle import w4a16_oracle as oracle

    calls: list[str] = []

    def fused(flat, packed, scales, group_size):
        calls.append("fused")
        y = oracle.linear_reference(flat.numpy(), packed.numpy(), scales.numpy(), group_size)
        return torch.from_numpy(y)

    def dequant_matmul(flat, packed, scales, group_size):
        calls.append("dequant")
        w = oracle.dequantize_weights(packed.numpy(), scales.numpy(), group_size).astype(np.float16)
        y = flat.numpy().astype(np.float32) @ w.astype(np.float32).T
        return torch.from_numpy(y.astype(np.float16))

    monkeypatch.setattr(linear_module, "_run_fused", fused)
    monkeypatch.setattr(linear_module, "_run_dequant_matmul", dequant_matmul)
    monkeypatch.setattr(linear_module, "_require_cuda", lambda tensor: None)
    return calls
