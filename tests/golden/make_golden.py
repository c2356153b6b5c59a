"""Regenerate the golden fixtures in this folder from the reference's own Python code.

Run by hand where a checkout of the reference project is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's ``w4a16.quantization`` / ``w4a16.reference`` (pure
PyTorch, CPU) from that path, feeds them seeded inputs and stores inputs and
outputs as ``.npz`` files next to this script.  The test-suite only reads the
``.npz`` files; it never needs the reference checkout.

Fixtures written:
  small_cases.npz     ragged / odd-shaped cases with every intermediate tensor
  all_nibbles.npz     random bytes (all 16 codes incl. -8) through dequantize + linear
  tinyllama_m1.npz    the five TinyLlama-shaped layers at M=1: reference outputs and
                      SHA-256 digests of the packed codes and scales (inputs are
                      re-derived from the seeds by the tests)
  config1_m8.npz      K=N=2048 at M=8, same seeds
  tinyllama_small_batch.npz
                      the five TinyLlama-shaped layers at M = 2, 4 and 8 (the small-batch sweep of
                      the reference's tests/test_cuda.py:397-451, at full size): reference outputs
                      only; lm_head outputs are kept for a fixed column sample to bound the file
"""
from __future__ import annotations

import hashlib
import importlib
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent

# name, K, N -- TinyLlama-1.1B linear shapes (hidden 2048, 4 KV heads x 64, MLP 5632, vocab 32000)
TINYLLAMA_LAYERS = [
    ("qo_proj", 2048, 2048),
    ("kv_proj", 2048, 256),
    ("gate_up_proj", 2048, 5632),
    ("down_proj", 5632, 2048),
    ("lm_head", 2048, 32000),
]


def seeded_weights(n: int, k: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn((n, k), dtype=torch.float32, generator=g) * 0.02


def seeded_activations(m: int, k: int, seed: int = 1) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn((m, k), dtype=torch.float32, generator=g).half()


def small_batch_columns(n: int) -> np.ndarray:
    """Output columns kept in tinyllama_small_batch.npz: all of them up to 8192, else both ends and every 16th."""
    if n <= 8192:
        return np.arange(n, dtype=np.int64)
    return np.unique(np.concatenate([np.arange(256), np.arange(0, n, 16), np.arange(n - 256, n)])).astype(np.int64)


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    quant = importlib.import_module("w4a16.quantization")
    ref = importlib.import_module("w4a16.reference")
    assert pathlib.Path(quant.__file__).resolve().is_relative_to(pathlib.Path(reference_root).resolve())
    torch.set_num_threads(1)  # fixed summation order for the stored FP32 matmul results

    # ---- small, odd-shaped cases: keep every tensor --------------------------------
    small = {}
    cases = [  # tag, N, K, group, M, weight dtype, weight std
        ("n8_k256_g128_m4", 8, 256, 128, 4, torch.float16, 1.0),
        ("n7_k256_g128_m1", 7, 256, 128, 1, torch.float16, 1.0),
        ("n13_k384_g64_m3", 13, 384, 64, 3, torch.float32, 0.02),
        ("n16_k128_g32_m2", 16, 128, 32, 2, torch.float32, 0.02),
        ("n5_k64_g4_m9", 5, 64, 4, 9, torch.float16, 1.0),
        ("n33_k1024_g128_m8", 33, 1024, 128, 8, torch.float32, 0.02),
    ]
    for index, (tag, n, k, gs, m, dtype, std) in enumerate(cases):
        g = torch.Generator().manual_seed(100 + index)
        w = (torch.randn((n, k), dtype=torch.float32, generator=g) * std).to(dtype)
        if index == 2:
            w[3, 64:128] = 0  # an all-zero group: its scale must become 1.0
        x = torch.randn((m, k), dtype=torch.float32, generator=g).half()
        codes, scales = quant.quantize_groupwise(w, gs)
        packed = quant.pack_int4(codes)
        assert torch.equal(quant.unpack_int4(packed), codes)
        small[f"{tag}/group_size"] = np.int64(gs)
        small[f"{tag}/weights"] = w.numpy()
        small[f"{tag}/x"] = x.numpy()
        small[f"{tag}/codes"] = codes.numpy()
        small[f"{tag}/scales"] = scales.numpy()
        small[f"{tag}/packed"] = packed.numpy()
        small[f"{tag}/dequant"] = ref.dequantize_weights(packed, scales, gs).numpy()
        small[f"{tag}/y"] = ref.linear_reference(x, packed, scales, gs).numpy()
    np.savez_compressed(HERE / "small_cases.npz", **small)

    # ---- all 16 nibble values, both positions ---------------------------------------
    g = torch.Generator().manual_seed(7)
    packed = torch.randint(0, 256, (64, 512), dtype=torch.uint8, generator=g)
    scales = torch.rand((64, 8), generator=g).add(0.01).half()
    x = torch.randn((8, 1024), dtype=torch.float32, generator=g).half()
    np.savez_compressed(
        HERE / "all_nibbles.npz",
        packed=packed.numpy(),
        scales=scales.numpy(),
        x=x.numpy(),
        codes=quant.unpack_int4(packed).numpy(),
        dequant=ref.dequantize_weights(packed, scales, 128).numpy(),
        y=ref.linear_reference(x, packed, scales, 128).numpy(),
    )

    # ---- full-size TinyLlama-shaped layers, M=1 -------------------------------------
    tiny = {}
    for index, (name, k, n) in enumerate(TINYLLAMA_LAYERS):
        w = seeded_weights(n, k, seed=index)
        x = seeded_activations(1, k, seed=1000 + index)
        packed, scales = quant.quantize_and_pack_weights(w, 128)
        tiny[f"{name}/shape_kn"] = np.array([k, n], dtype=np.int64)
        tiny[f"{name}/packed_sha256"] = np.array(sha(packed))
        tiny[f"{name}/scales_sha256"] = np.array(sha(scales))
        tiny[f"{name}/x_sha256"] = np.array(sha(x))
        tiny[f"{name}/y"] = ref.linear_reference(x, packed, scales, 128).numpy()
        deq = ref.dequantize_weights(packed, scales, 128)
        tiny[f"{name}/dequant_fp16_sha256"] = np.array(sha(deq.half()))
        tiny[f"{name}/wmax"] = np.float64(deq.abs().max().item())
    np.savez_compressed(HERE / "tinyllama_m1.npz", **tiny)

    # ---- the reference's CPU-runnable configuration (K=N=2048), at M=8 ---------------
    w = seeded_weights(2048, 2048, seed=0)
    x = seeded_activations(8, 2048, seed=1)
    packed, scales = quant.quantize_and_pack_weights(w, 128)
    np.savez_compressed(
        HERE / "config1_m8.npz",
        packed_sha256=np.array(sha(packed)),
        scales_sha256=np.array(sha(scales)),
        x=x.numpy(),
        y=ref.linear_reference(x, packed, scales, 128).numpy(),
    )
    # ---- the small-batch sweep: every TinyLlama-shaped layer at M = 2, 4, 8 -----------
    batch = {}
    for index, (name, k, n) in enumerate(TINYLLAMA_LAYERS):
        w = seeded_weights(n, k, seed=index)
        packed, scales = quant.quantize_and_pack_weights(w, 128)
        columns = small_batch_columns(n)
        batch[f"{name}/columns"] = columns
        for m in (2, 4, 8):
            x = seeded_activations(m, k, seed=2000 + 10 * index + m)
            y = ref.linear_reference(x, packed, scales, 128).numpy()
            batch[f"{name}/m{m}/x_sha256"] = np.array(sha(x))
            batch[f"{name}/m{m}/y"] = y[:, columns]
    np.savez_compressed(HERE / "tinyllama_small_batch.npz", **batch)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
