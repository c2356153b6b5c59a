#!/usr/bin/env python
"""Benchmark of the W4A16 linear path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl product|reference]

One JSON line on stdout; progress on stderr.

Workload (``config.workload = "tinyllama_decode_linears_m1"``): the 155 W4A16 linears one
TinyLlama-1.1B decode token passes through (22 blocks x {q,k,v,o,gate,up,down} + lm_head), M=1,
group 128, every layer instance with its own seeded N(0, 0.02) weights quantised by the package's
quantiser -- 535 MB of packed weights and scales, four times the L2, so every step streams from
DRAM.  One *step* is one pass over the 155 layers.  Metric: algorithmic bytes moved per second
(``N*K/2 + N*K/128*2 + M*K*2 + M*N*2`` per layer -- the payload the reference's profiler counts,
scripts/profile_kernel.py:310-323).

* ``value``  -- steps replayed from a CUDA graph of ``torch.ops.w4a16.linear`` calls, activations
  resident in HBM; CUDA events around exactly K replays, max over ranks.
* ``e2e``    -- the same linears, but every step's activations are copied from pinned host memory
  and every step's outputs are gathered and copied back to pinned host memory, all inside the
  timed region.  Two input/output slots and two copy streams let the copies of steps i+1 and i-1
  run under the kernels of step i; ``one_stream_*`` is the same work serialised on one stream.
* ``roofline`` -- the fused kernel's bytes per launch over its mean launch duration inside the
  timed region, against the measured HBM copy bandwidth.
* ``cpu_baseline`` -- the reference's PyTorch CPU path on the host cores (the reference arm as a child process).
* ``layers`` -- per-shape latency of isolated launches over rotating weight copies (> 2x L2 per
  graph replay), M=1, 2, 4 and 8, next to cuBLAS FP16 on the dequantised weights.
* ``fused_siblings``, ``prefill``, ``quantize``, ``decode`` -- the token with q/k/v and gate/up as
  single launches; prefill-sized batches on the tcgen05 kernel; the device quantiser and
  dequantiser; decode tokens/s of the TinyLlama-shaped model (framework path and this package's
  decode runner).

With N > 1 (torchrun) every rank runs an independent replica of the same workload on its own GPU
(layers this small are not worth sharding); the job value is the sum.  The same line then carries a
``sharded`` object: one Llama-3-70B-shaped decoder block (layers that ARE worth sharding) cut across
the N GPUs -- column-parallel q/k/v, o, gate/up and row-parallel down -- at M = 1 and 8, with the
exchange done by the kernels themselves, by NCCL, with the two-exchange pairing, without any exchange,
and unsharded on one GPU (``sharded_block_bench``).

``--impl reference`` times the reference's own CPU code (``oracle/_ref``, built by oracle/build_ref.py where a
checkout of the reference exists; else the restatement in oracle/torch_cpu_port.py), one decoder block per step.
"""
from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

GROUP = 128
TINYLLAMA = {  # name: (K, N)
    "qo_proj": (2048, 2048),
    "kv_proj": (2048, 256),
    "gate_up_proj": (2048, 5632),
    "down_proj": (5632, 2048),
    "lm_head": (2048, 32000),
}
LLAMA70B = {
    "qo_proj": (8192, 8192),
    "kv_proj": (8192, 1024),
    "gate_up_proj": (8192, 28672),
    "down_proj": (28672, 8192),
}
# Mean DRAM bytes (read + write) per launch of the fused kernel over this workload, from one ncu capture of
# the timed region (algorithmic: 3,451,728), and the digest of the kernel sources that capture ran: the line
# reports the figure only while the sources are still those, otherwise null.
NCU_DRAM_BYTES_PER_LAUNCH = 3519756
NCU_CAPTURE_SOURCES = ("nibble_b200/csrc/linear_mma.cu", "nibble_b200/csrc/linear_mma_body.cuh", "nibble_b200/csrc/unpack.cuh")
NCU_CAPTURE_SOURCES_SHA16 = "fd6284de1045daff"


def kernel_sources_sha16() -> str:
    import hashlib

    digest = hashlib.sha256()
    for name in NCU_CAPTURE_SOURCES:
        digest.update((ROOT / name).read_bytes())
    return digest.hexdigest()[:16]


def measured_traffic_per_launch():
    return NCU_DRAM_BYTES_PER_LAUNCH if kernel_sources_sha16() == NCU_CAPTURE_SOURCES_SHA16 else None
BLOCK_ORDER = ["qo_proj", "kv_proj", "kv_proj", "qo_proj", "gate_up_proj", "gate_up_proj", "down_proj"]
N_BLOCKS = 22


def log(*parts) -> None:
    print(*parts, file=sys.stderr, flush=True)


class nvtx_range:
    """NVTX range around a profiled region (the reference's profiler marks each operator the same way,
    scripts/profile_kernel.py:346-354); a no-op where torch's NVTX bindings are not usable."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        try:
            import torch

            torch.cuda.nvtx.range_push(self.name)
            self.pushed = True
        except Exception:
            self.pushed = False
        return self

    def __exit__(self, *exc):
        if self.pushed:
            import torch

            torch.cuda.nvtx.range_pop()
        return False


def algorithmic_bytes(m: int, k: int, n: int) -> int:
    return n * k // 2 + n * (k // GROUP) * 2 + m * k * 2 + m * n * 2


def decode_token_layers() -> list[tuple[str, int, int]]:
    layers = []
    for _ in range(N_BLOCKS):
        layers += [(name, *TINYLLAMA[name]) for name in BLOCK_ORDER]
    layers.append(("lm_head", *TINYLLAMA["lm_head"]))
    return layers


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ----------------------------------------------------------------------------- clocks
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while ``active`` is set."""

    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, index: int, period_s: float = 0.05):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples: list[tuple[int, int]] = []
        self.max_mhz = None
        self.active = threading.Event()
        self.stop = threading.Event()
        self.error = None

    def run(self) -> None:
        try:
            import pynvml

            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            while not self.stop.is_set():
                if self.active.is_set():
                    mhz = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                    try:
                        reasons = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                    except Exception:
                        reasons = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                    self.samples.append((mhz, reasons))
                time.sleep(self.period)
        except Exception as error:  # NVML missing: report, never fail the bench
            self.error = repr(error)

    def summary(self, window: str) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0,
                    "window": window, "error": self.error}
        mask = 0
        for _, reasons in self.samples:
            mask |= reasons
        names = sorted(name for bit, name in self.REASONS.items() if mask & bit and name != "gpu_idle")
        return {"sm_mhz": statistics.median(mhz for mhz, _ in self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": names, "samples": len(self.samples), "window": window}


# ----------------------------------------------------------------------------- product arm
def make_layer(torch, k: int, n: int, seed: int, device):
    from nibble_b200 import quantize_and_pack_weights

    g = torch.Generator(device=device).manual_seed(seed)
    w = torch.randn((n, k), dtype=torch.float32, device=device, generator=g) * 0.02
    return quantize_and_pack_weights(w, GROUP)


def capture(torch, fn):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    torch.cuda.synchronize()
    return graph


def time_replays(torch, graph, replays: int) -> float:
    """Milliseconds for `replays` back-to-back replays, CUDA events on the current stream."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(replays):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end)


def per_shape_table(torch, shapes: dict, m: int, device, l2_bytes: int, with_cublas: bool) -> dict:
    """Reference method (scripts/profile_kernel.py:334-339,463-551): a graph of back-to-back calls,
    each on a different weight copy, one replay touching more than twice the L2; median of 20."""
    from nibble_b200 import dequantize_cuda, linear_cuda

    out = {}
    peak, _ = measured_peaks()
    for index, (name, (k, n)) in enumerate(shapes.items()):
        packed, scales = make_layer(torch, k, n, seed=index, device=device)
        w_bytes = packed.numel() + scales.numel() * 2
        copies = max(2, -(-2 * l2_bytes // w_bytes))
        calls = max(100, copies)
        pk = packed.unsqueeze(0).repeat(copies, 1, 1)
        sc = scales.unsqueeze(0).repeat(copies, 1, 1)
        x = torch.randn((m, k), device=device).half()

        def ours():
            for i in range(calls):
                linear_cuda(x, pk[i % copies], sc[i % copies], GROUP)

        graph = capture(torch, ours)
        us = statistics.median(time_replays(torch, graph, 1) * 1000.0 / calls for _ in range(20))
        payload = algorithmic_bytes(m, k, n)
        row = {"us": round(us, 3), "gbs": round(payload / us / 1e3, 1),
               "frac_measured": round(payload / us / 1e3 / peak, 3), "frac_8tbs": round(payload / us / 1e3 / 8000, 3)}
        del graph
        if with_cublas:
            w16 = dequantize_cuda(packed, scales, GROUP)
            c16 = max(2, -(-2 * l2_bytes // (w16.numel() * 2)))
            w16 = w16.unsqueeze(0).repeat(c16, 1, 1)
            calls16 = max(50, c16)

            def cublas():
                for i in range(calls16):
                    torch.nn.functional.linear(x, w16[i % c16])

            graph = capture(torch, cublas)
            us16 = statistics.median(time_replays(torch, graph, 1) * 1000.0 / calls16 for _ in range(10))
            row["cublas_fp16_us"] = round(us16, 3)
            row["speedup_vs_cublas_fp16"] = round(us16 / us, 2)
            del graph, w16
        out[name] = row
        del pk, sc
        torch.cuda.empty_cache()
        log(f"  M={m} {name} K={k} N={n}: {row}")
    return out


def prefill_table(torch, device) -> dict:
    """Prefill-sized batches: the tcgen05 kernel with fused dequantisation against the reference's route
    (dequantise to FP16, then cuBLAS; w4a16/linear.py:132-152) and against cuBLAS alone on FP16 weights
    that already exist.  Eager launches on one weight copy, median of 7 CUDA-event timings of 5 calls."""
    from nibble_b200 import dequantize_cuda, linear_cuda

    def timed(fn) -> float:
        for _ in range(2):
            fn()
        samples = []
        for _ in range(7):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(5):
                fn()
            end.record()
            torch.cuda.synchronize()
            samples.append(start.elapsed_time(end) * 1000.0 / 5)
        return statistics.median(samples)

    peaks_path = ROOT / "MEASURED_PEAKS.json"
    tensor_peak = json.loads(peaks_path.read_text()).get("bf16_tflops") if peaks_path.exists() else 1590.0
    out = {}
    shapes = {"tinyllama_gate_up": TINYLLAMA["gate_up_proj"], "llama70b_q_o": LLAMA70B["qo_proj"],
              "llama70b_gate_up": LLAMA70B["gate_up_proj"]}
    for index, (name, (k, n)) in enumerate(shapes.items()):
        packed, scales = make_layer(torch, k, n, seed=50 + index, device=device)
        w16 = dequantize_cuda(packed, scales, GROUP)
        for m in (128, 512, 2048):
            x = torch.randn((m, k), device=device).half()
            fused = timed(lambda: linear_cuda(x, packed, scales, GROUP))
            two_pass = timed(lambda: torch.nn.functional.linear(x, dequantize_cuda(packed, scales, GROUP)))
            cublas = timed(lambda: torch.nn.functional.linear(x, w16))
            exact = bool(torch.equal(linear_cuda(x, packed, scales, GROUP), torch.nn.functional.linear(x, w16)))
            tflops = 2.0 * m * n * k / fused / 1e6
            row = {"fused_us": round(fused, 1), "tflops": round(tflops, 1),
                   "dequant_then_cublas_us": round(two_pass, 1), "speedup_vs_dequant_then_cublas": round(two_pass / fused, 2),
                   "cublas_fp16_only_us": round(cublas, 1), "equals_cublas_on_fp16_weights": exact}
            row["frac_of_bf16_peak"] = round(tflops / tensor_peak, 3)   # measured cuBLAS burst figure (fallback 1590)
            out[f"{name}_m{m}"] = row
            log(f"  prefill {name} K={k} N={n} M={m}: {row}")
        del packed, scales, w16
        torch.cuda.empty_cache()
    from nibble_b200 import check_device_status

    check_device_status()      # no bounded wait of the tcgen05 kernel may have given up
    return out


def quantize_table(torch, device) -> dict:
    """Device quantise+pack and dequantise of one Llama-70B gate/up matrix (28672 x 8192) through the C ABI into
    preallocated outputs: microseconds and algorithmic GB/s (2.5 bytes per weight with FP16 weights), median of 7
    CUDA-event timings of 20 back-to-back calls each (470 MB per call, so nothing is served from L2)."""
    import ctypes

    from nibble_b200 import _native

    lib = _native.core()
    k, n = LLAMA70B["gate_up_proj"]
    weights = (torch.randn((n, k), device=device) * 0.02).half()
    packed = torch.empty((n, k // 2), dtype=torch.uint8, device=device)
    scales = torch.empty((n, k // GROUP), dtype=torch.float16, device=device)
    restored = torch.empty_like(weights)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def quantise():
        assert lib.w4a16_quantize_pack_f16(weights.data_ptr(), packed.data_ptr(), scales.data_ptr(), n, k, GROUP, stream) == 0

    def dequantise():
        assert lib.w4a16_dequantize_f16(packed.data_ptr(), scales.data_ptr(), restored.data_ptr(), n, k, GROUP, stream) == 0

    def timed(fn) -> float:
        for _ in range(3):
            fn()
        samples = []
        for _ in range(7):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(20):
                fn()
            end.record()
            torch.cuda.synchronize()
            samples.append(start.elapsed_time(end) * 1000.0 / 20)
        return statistics.median(samples)

    payload = n * k * 2.5 + n * (k // GROUP) * 2
    peak, _ = measured_peaks()
    out = {}
    for name, fn in (("quantize_pack_f16", quantise), ("dequantize_f16", dequantise)):
        us = timed(fn)
        out[name] = {"us": round(us, 1), "gbs": round(payload / us / 1e3, 1), "frac_measured": round(payload / us / 1e3 / peak, 3)}
    out["how"] = "C ABI, preallocated outputs, 20 calls per CUDA-event sample, median of 7"
    log(f"  quantise / dequantise 28672 x 8192: {out}")
    return out


def cpu_baseline_leg(blocks: int, repeats: int) -> dict:
    """The CPU baseline of the product line: this script's own reference arm, run as a child process (so that
    the reference's modules are imported in an interpreter that has not loaded this package) on a bounded
    sample of the workload -- `blocks` decoder blocks per pass, `repeats` timed passes."""
    import subprocess

    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", str(repeats), "--warmup", "3",
           "--cpu-blocks", str(blocks)]
    env = {key: value for key, value in os.environ.items() if key not in ("RANK", "LOCAL_RANK", "WORLD_SIZE")}
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    if proc.returncode != 0 or not proc.stdout.strip():
        return {"value": None, "unit": "GB/s", "cores": None, "kind": "unavailable", "sample": proc.stderr[-300:]}
    return json.loads(proc.stdout.strip().splitlines()[-1])["cpu_baseline"]


def decode_bench(torch, device, runners_only: bool = False) -> dict:
    """Decode tokens/s of a TinyLlama-1.1B-shaped model (random weights), FP16 cuBLAS vs W4A16.

    Protocol of the reference's scripts/generate.py:307-365: batch 1, 16-token prompt of seeded
    random ids, 32 greedy new tokens, static KV cache, the decode step replayed from a CUDA graph;
    decode tok/s = (new - 1) / (total - prefill); one warm-up, median of five.  No tokenizer and no
    checkpoint are involved (neither is available offline): the architecture and sizes are real,
    the weights are random, so only speed -- not text -- is meaningful.
    """
    import transformers
    from transformers import StaticCache

    from nibble_b200 import replace_linear_layers

    cfg = transformers.LlamaConfig(
        vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22,
        num_attention_heads=32, num_key_value_heads=4, max_position_embeddings=2048, rms_norm_eps=1e-5,
        tie_word_embeddings=False,
    )
    torch.manual_seed(0)
    with torch.device(device):
        model = transformers.AutoModelForCausalLM.from_config(cfg, dtype=torch.float16)
    model.eval()
    prompt_len, new_tokens = 16, 32
    prompt = torch.randint(0, 32000, (1, prompt_len), generator=torch.Generator().manual_seed(0)).to(device)
    positions = torch.arange(prompt_len, device=device)

    def measure(label: str) -> dict:
        cache = StaticCache(config=cfg, max_cache_len=prompt_len + new_tokens + 8)
        tok = torch.zeros((1, 1), dtype=torch.long, device=device)
        pos = torch.zeros((1,), dtype=torch.long, device=device)

        def prefill():
            cache.reset()
            out = model(input_ids=prompt, past_key_values=cache, cache_position=positions, use_cache=True)
            return out.logits[:, -1].argmax(-1, keepdim=True)

        def step():
            out = model(input_ids=tok, past_key_values=cache, cache_position=pos, use_cache=True)
            return out.logits[:, -1].argmax(-1, keepdim=True)

        with torch.inference_mode():
            tok.copy_(prefill())
            pos.fill_(prompt_len)
            for _ in range(3):   # lazy cache allocation, workspace allocation, autotuning
                step()
            torch.cuda.synchronize()
            mode = "cuda_graph"
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    next_tok = step()
                replay = graph.replay
            except Exception as error:   # a host sync inside the model: time eager launches instead
                torch.cuda.synchronize()
                mode = f"eager ({type(error).__name__})"
                holder = [None]

                def replay():
                    holder[0] = step()

                replay()
                next_tok = holder[0]

            def generate():
                e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
                e0.record()
                first = prefill()
                e1.record()
                tok.copy_(first)
                pos.fill_(prompt_len)
                for _ in range(new_tokens - 1):
                    replay()
                    tok.copy_(next_tok if mode == "cuda_graph" else holder[0])
                    pos.add_(1)
                e2.record()
                torch.cuda.synchronize()
                return e0.elapsed_time(e1), e0.elapsed_time(e2)

            generate()
            runs = [generate() for _ in range(5)]
        prefill_ms = statistics.median(r[0] for r in runs)
        total_ms = statistics.median(r[1] for r in runs)
        decode_ms = total_ms - prefill_ms
        row = {"decode_tok_s": round((new_tokens - 1) / decode_ms * 1e3, 1), "prefill_ms": round(prefill_ms, 3),
               "ms_per_token": round(decode_ms / (new_tokens - 1), 4), "e2e_tok_s": round(new_tokens / total_ms * 1e3, 1),
               "mode": mode, "peak_mib": round(torch.cuda.max_memory_allocated(device) / 2**20)}
        log(f"  decode {label}: {row}")
        return row

    out = {"model": "TinyLlama-1.1B architecture, random weights", "prompt_tokens": prompt_len, "new_tokens": new_tokens}
    saved_pdl = os.environ.pop("W4A16_PDL", None)
    torch.cuda.reset_peak_memory_stats(device)
    if not runners_only:
        out["fp16_cublas"] = measure("fp16")
    replaced = replace_linear_layers(model, group_size=GROUP, fuse_siblings=False)   # fused further down, to show both
    out["linears_replaced"] = replaced
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats(device)
    from nibble_b200 import fuse_parallel_linears

    if not runners_only:
        out["w4a16"] = measure("w4a16")
        os.environ["W4A16_PDL"] = "1"
        out["w4a16_programmatic_launch"] = measure("w4a16+pdl")
    out["launches_fused"] = fuse_parallel_linears(model)     # q/k/v -> one launch, gate/up -> one launch per block
    torch.cuda.empty_cache()
    if not runners_only:
        # with every fused launch sitting between two torch kernels there is no chain of our own kernels left
        # for programmatic launch to overlap, and the attribute costs time: measured both ways
        out["w4a16_programmatic_launch_fused_qkv_gate_up"] = measure("w4a16+pdl+fused q/k/v, gate/up")
        os.environ.pop("W4A16_PDL", None)
        out["w4a16_fused_qkv_gate_up"] = measure("w4a16+fused q/k/v, gate/up")
    os.environ.pop("W4A16_PDL", None)

    # this package's own decode step (nibble_b200/decode.py): same protocol, the prompt is consumed one
    # token per step, so "prefill" here is 16 decode steps
    from nibble_b200.decode import LlamaDecodeRunner

    def measure_runner(label: str, fuse_inputs: bool = True, persistent: bool = False) -> dict:
        runner = LlamaDecodeRunner(model, max_len=prompt_len + new_tokens + 8, fuse_inputs=fuse_inputs, persistent=persistent)
        ids = prompt.reshape(-1)

        def generate():
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            runner.reset()
            e0.record()
            for i in range(prompt_len):
                runner.token.copy_(ids[i:i + 1])
                runner.step()
            e1.record()
            for _ in range(new_tokens - 1):
                runner.step()
            e2.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1), e0.elapsed_time(e2)

        generate()
        runs = [generate() for _ in range(5)]
        prefill_ms = statistics.median(r[0] for r in runs)
        total_ms = statistics.median(r[1] for r in runs)
        decode_ms = total_ms - prefill_ms
        row = {"decode_tok_s": round((new_tokens - 1) / decode_ms * 1e3, 1), "prefill_ms": round(prefill_ms, 3),
               "ms_per_token": round(decode_ms / (new_tokens - 1), 4), "e2e_tok_s": round(new_tokens / total_ms * 1e3, 1),
               "mode": "one cooperative launch per token" if persistent else "cuda_graph, own decode step",
               "kernels_per_token": runner.launches_per_step + (0 if persistent else 1),
               "cache_overrun": int(runner.status.item()),
               "step_status": int(runner.step_status.item()) if persistent else 0}
        log(f"  decode {label}: {row}")
        return row

    try:
        if not runners_only:
            out["w4a16_decode_runner_separate_norm_and_silu_kernels"] = measure_runner("w4a16 decode runner, separate norm/silu kernels", False)
            out["w4a16_decode_runner"] = measure_runner("w4a16 decode runner")
        os.environ["W4A16_PDL"] = "1"
        out["w4a16_decode_runner_programmatic_launch"] = measure_runner("w4a16 decode runner+pdl")
        os.environ.pop("W4A16_PDL", None)
        out["w4a16_decode_runner_persistent"] = measure_runner("w4a16 decode runner, one persistent launch", persistent=True)
    except Exception as error:
        os.environ.pop("W4A16_PDL", None)
        out["w4a16_decode_runner"] = {"error": repr(error)[:300]}
    if saved_pdl is not None:
        os.environ["W4A16_PDL"] = saved_pdl
    del model
    torch.cuda.empty_cache()
    return out


def run_single_layer(args) -> dict:
    """A few launches of one layer shape over three weight copies: the small case profilers capture.

    `--single-layer K N M`; every call goes through ``torch.ops.w4a16.linear``.
    """
    import torch

    from nibble_b200 import linear_cuda

    k, n, m = args.single_layer
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    packed, scales = make_layer(torch, k, n, seed=0, device=device)
    copies = 3
    pk = packed.unsqueeze(0).repeat(copies, 1, 1)
    sc = scales.unsqueeze(0).repeat(copies, 1, 1)
    x = torch.randn((m, k), device=device).half()
    for i in range(4):
        linear_cuda(x, pk[i % copies], sc[i % copies], GROUP)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()
    start.record()
    with nvtx_range(f"w4a16.linear M={m} K={k} N={n}"):
        for i in range(args.steps):
            linear_cuda(x, pk[i % copies], sc[i % copies], GROUP)
    end.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    us = start.elapsed_time(end) * 1e3 / args.steps
    payload = algorithmic_bytes(m, k, n)
    peak, kind = measured_peaks()
    return {"single_layer": {"K": k, "N": n, "M": m}, "launches": args.steps, "us_per_launch_eager": round(us, 2),
            "gbs": round(payload / us / 1e3, 1), "peak": peak, "peak_kind": kind, "bytes_per_launch": payload}


def run_decode_step(args) -> dict:
    """`--workload decode_step`: the decode runner of nibble_b200/decode.py on the TinyLlama-1.1B-shaped model
    (random weights), `--steps` tokens after a 16-token prompt, eager launches (no graph) between
    cudaProfilerStart/Stop so that a profiler lists every kernel of a token."""
    import torch
    import transformers

    from nibble_b200 import _native, replace_linear_layers
    from nibble_b200.decode import LlamaDecodeRunner

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    if args.pdl:
        os.environ["W4A16_PDL"] = "1"
    cfg = transformers.LlamaConfig(
        vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22,
        num_attention_heads=32, num_key_value_heads=4, max_position_embeddings=2048, rms_norm_eps=1e-5,
        tie_word_embeddings=False)
    torch.manual_seed(0)
    with torch.device(device):
        model = transformers.AutoModelForCausalLM.from_config(cfg, dtype=torch.float16)
    model.eval()
    replace_linear_layers(model, group_size=GROUP)
    runner = LlamaDecodeRunner(model, max_len=16 + args.steps + 8, persistent=args.persistent)
    if args.persistent:
        runner._enqueue_step = runner._persistent_step      # one cooperative launch per token
    prompt = torch.randint(0, 32000, (16,), generator=torch.Generator().manual_seed(0)).to(device)
    with torch.inference_mode():
        for i in range(16):
            runner.token.copy_(prompt[i:i + 1])
            runner._enqueue_step()
        torch.cuda.synchronize()
        before = _native.core().w4a16_launch_count()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.profiler.start()
        start.record()
        for index in range(args.steps):
            with nvtx_range(f"w4a16.decode_step {index}"):
                runner._enqueue_step()
        end.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    ms = start.elapsed_time(end) / args.steps
    return {"workload": "decode_step", "tokens": args.steps, "ms_per_token_eager": round(ms, 4),
            "our_kernels_per_token": (_native.core().w4a16_launch_count() - before) // args.steps,
            "cache_overrun": int(runner.status.item())}


# ----------------------------------------------------------------------------- sharded Llama-70B block
TP_BLOCK = [  # name, K, N of one Llama-3-70B decoder block with q/k/v and gate/up as single layers
    ("qkv_proj", 8192, 8192 + 1024 + 1024),
    ("o_proj", 8192, 8192),
    ("gate_up_proj", 8192, 2 * 28672),
    ("down_proj", 28672, 8192),
]


def tp_block_bytes(m: int) -> int:
    return sum(algorithmic_bytes(m, k, n) for _, k, n in TP_BLOCK)


def sharded_block_bench(torch, dist, device, rank: int, world: int, m: int, steps: int, warmup: int,
                        modes=("peer", "nccl", "paired", "kernels_only", "one_gpu")) -> dict:
    """Milliseconds per Llama-3-70B-shaped decoder block (its linears only, chained: every layer's input is the
    previous layer's output), the block sharded over the `world` ranks of this job.

    peer          q/k/v, o, gate/up column-parallel and down row-parallel (the cut BASELINE's config names), the
                  exchange done by the kernels: peer stores in the epilogue, the wait in the next kernel's prologue
    nccl          the same cut with all_gather_into_tensor / all_reduce after every layer
    paired        q/k/v column-parallel feeding o row-parallel, gate/up column-parallel feeding down row-parallel
                  (two exchanges per block instead of four), kernels' own exchange
    kernels_only  every rank's shard of every layer with no exchange at all
    one_gpu       the unsharded block on this rank's GPU alone
    Three sets of weights per graph replay so that a replay never finds its weights in L2; CUDA events around
    `steps` replays; max over ranks.
    """
    import ctypes

    from nibble_b200.cuda import linear_cuda, linear_partial_cuda
    from nibble_b200.linear import QuantizedLinear
    from nibble_b200.sharded import (PeerColumnParallelQuantizedLinear, PeerRowParallelQuantizedLinear, PeerView,
                                     _launch_peer_linear)

    sets = 3
    gen = torch.Generator(device=device).manual_seed(77 + rank)

    def random_layer(n: int, k: int, full_k: int | None = None):
        # codes uniform in [-7, 7] (zero mean, so that a chain of layers keeps no common-mode growth)
        low = torch.randint(-7, 8, (n, k // 2), dtype=torch.int8, device=device, generator=gen)
        high = torch.randint(-7, 8, (n, k // 2), dtype=torch.int8, device=device, generator=gen)
        packed = ((low & 15) | ((high & 15) << 4)).to(torch.uint8)
        gain = 1.0 / (4.32 * (full_k or k) ** 0.5)      # keeps the chained activations at unit scale
        scales = ((torch.rand((n, k // GROUP), device=device, generator=gen) * 0.5 + 0.75) * gain).half()
        return packed, scales

    def time_chain(step_fn) -> float:
        with torch.inference_mode():
            graph = capture(torch, step_fn)
            for _ in range(max(warmup, 3)):
                graph.replay()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
                torch.cuda.synchronize()
            ms = time_replays(torch, graph, steps)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        del graph
        return ms / steps / sets

    x0 = torch.randn((m, 8192), device=device, generator=torch.Generator(device=device).manual_seed(5)).half()
    out = {}

    def plain(layer, x, y, workspaces):
        _launch_peer_linear(layer, x, m, workspaces, None, out_f32=False, y=y)

    def local_chain(div: int, exchange_free: bool):
        """The block's four layers with N (or K for down) divided by `div`, no exchange: inputs of o and down are
        column slices of the previous local output when they fit, else of a fixed tensor."""
        blocks = []
        for _ in range(sets):
            (_, k1, n1), (_, k2, n2), (_, k3, n3), (_, k4, n4) = TP_BLOCK
            layers = [QuantizedLinear(*random_layer(n1 // div, k1)), QuantizedLinear(*random_layer(n2 // div, k2)),
                      QuantizedLinear(*random_layer(n3 // div, k3)), QuantizedLinear(*random_layer(n4, k4 // div, k4))]
            outs = [torch.empty((m, layer.out_features), dtype=torch.float16, device=device) for layer in layers]
            blocks.append((layers, outs, [{} for _ in layers]))
        filler = torch.randn((m, 57344), device=device).half()

        def step():
            x = x0
            for layers, outs, ws in blocks:
                plain(layers[0], x, outs[0], ws[0])
                src = outs[0] if outs[0].shape[1] >= 8192 else filler
                plain(layers[1], src[:, :8192], outs[1], ws[1])
                src = outs[1] if outs[1].shape[1] >= 8192 else filler
                plain(layers[2], src[:, :8192], outs[2], ws[2])
                plain(layers[3], outs[2][:, :layers[3].in_features], outs[3], ws[3])
                x = outs[3] if div == 1 else x0
            return x
        return step

    if "one_gpu" in modes:
        out["one_gpu"] = time_chain(local_chain(1, False))
        torch.cuda.empty_cache()
    if "kernels_only" in modes and world > 1:
        out["kernels_only"] = time_chain(local_chain(world, True))
        torch.cuda.empty_cache()

    def shard_sets():
        """Per set: this rank's shards of the four layers (rows of qkv, o, gate/up; a K slice of down)."""
        result = []
        for _ in range(sets):
            (_, k1, n1), (_, k2, n2), (_, k3, n3), (_, k4, n4) = TP_BLOCK
            result.append([random_layer(n1 // world, k1), random_layer(n2 // world, k2), random_layer(n3 // world, k3),
                           random_layer(n4, k4 // world, k4)])
        return result

    if world > 1 and ("peer" in modes or "nccl" in modes or "paired" in modes):
        shards = shard_sets()
        k_down = 28672 // world
        finals = {}

        if "peer" in modes:
            blocks = []
            for qkv, o, gate_up, down in shards:
                blocks.append((PeerColumnParallelQuantizedLinear(*qkv, GROUP, max_rows=m),
                               PeerColumnParallelQuantizedLinear(*o, GROUP, max_rows=m),
                               PeerColumnParallelQuantizedLinear(*gate_up, GROUP, max_rows=m),
                               PeerRowParallelQuantizedLinear(*down, GROUP, max_rows=m),
                               torch.empty((m, 8192), dtype=torch.float16, device=device)))

            def peer_step():
                x = x0
                for qkv, o, gate_up, down, y in blocks:
                    view = qkv.launch(x)
                    view = o.launch(view.narrow(0, 8192))
                    view = gate_up.launch(view)
                    down.launch(view.narrow(rank * k_down, k_down))
                    x = down.finish(m, out=y)
                return x

            out["peer"] = time_chain(peer_step)
            torch.cuda.synchronize()
            finals["peer"] = blocks[-1][4].clone()
            for block in blocks:
                for layer in block[:4]:
                    layer.region.check()
            del blocks
            torch.cuda.empty_cache()

        if "nccl" in modes:
            def nccl_step():
                x = x0
                for qkv, o, gate_up, down in shards:
                    def gathered(x_in, shard):
                        local = linear_cuda(x_in, shard[0], shard[1], GROUP)
                        full = local.new_empty((world * m, local.shape[1]))
                        dist.all_gather_into_tensor(full, local)
                        return full.view(world, m, -1).permute(1, 0, 2).reshape(m, -1) if m > 1 else full.view(1, -1)
                    a = gathered(x, qkv)
                    b = gathered(a[:, :8192].contiguous(), o)
                    c = gathered(b, gate_up)
                    partial = linear_partial_cuda(c[:, rank * k_down:(rank + 1) * k_down].contiguous(), down[0], down[1], GROUP)
                    dist.all_reduce(partial)
                    x = partial.half()
                return x

            out["nccl"] = time_chain(nccl_step)
            with torch.inference_mode():
                finals["nccl"] = nccl_step()      # once more, eagerly: the chain's result for the comparison below
            torch.cuda.empty_cache()

        if "peer" in finals and "nccl" in finals:
            # same weights, same chain: the two exchanges must agree up to the order of FP32 sums
            torch.cuda.synchronize()
            a, b = finals["peer"].float(), finals["nccl"].float()
            scale = float(b.abs().max())
            diff = (a - b).abs()
            bad = diff > 0.05 * scale + 1e-3
            log(f"  [rank {rank}] peer vs nccl, M={m}: max|nccl| {scale:.4g}, max diff {float(diff.max()):.4g}, "
                f"{int(bad.sum())} of {bad.numel()} outside tolerance, nan {int(torch.isnan(a).sum())}/{int(torch.isnan(b).sum())}, "
                f"first bad columns {bad.nonzero()[:8, -1].tolist()}")
            out["peer_vs_nccl_max_rel_diff"] = round(float(diff.max()) / max(scale, 1e-30), 5)
            out["peer_equals_nccl"] = not bool(bad.any())
            if bad.any() or os.environ.get("W4A16_BENCH_CHECK_UNSHARDED", "1") == "1":
                # Parity gate of the sharded record: rebuild the unsharded layers from every rank's shards, run the same
                # chain on this GPU alone and compare both exchanges with it.
                def all_ranks(t, dim):
                    parts = [torch.empty_like(t) for _ in range(world)]
                    dist.all_gather(parts, t.contiguous())
                    return torch.cat(parts, dim).contiguous()

                with torch.inference_mode():
                    x = x0
                    for qkv, o, gate_up, down in shards:
                        t = linear_cuda(x, all_ranks(qkv[0], 0), all_ranks(qkv[1], 0), GROUP)
                        t = linear_cuda(t[:, :8192].contiguous(), all_ranks(o[0], 0), all_ranks(o[1], 0), GROUP)
                        t = linear_cuda(t, all_ranks(gate_up[0], 0), all_ranks(gate_up[1], 0), GROUP)
                        x = linear_cuda(t[:, :28672].contiguous(), all_ranks(down[0], 1), all_ranks(down[1], 1), GROUP)
                truth = x.float()
                out["peer_vs_unsharded_max_rel_diff"] = round(float((a - truth).abs().max()) / max(scale, 1e-30), 5)
                out["nccl_vs_unsharded_max_rel_diff"] = round(float((b - truth).abs().max()) / max(scale, 1e-30), 5)
                log(f"  [rank {rank}] against the unsharded chain: peer {out['peer_vs_unsharded_max_rel_diff']}, "
                    f"nccl {out['nccl_vs_unsharded_max_rel_diff']}")

        if "paired" in modes:
            blocks = []
            for qkv, o, gate_up, down in shards:
                # o_proj as a row-parallel layer: this rank's K slice of a [8192, 8192] matrix
                o_row = random_layer(8192, 8192 // world, 8192)
                blocks.append((QuantizedLinear(*qkv), PeerRowParallelQuantizedLinear(*o_row, GROUP, max_rows=m),
                               QuantizedLinear(*gate_up), PeerRowParallelQuantizedLinear(*down, GROUP, max_rows=m),
                               [torch.empty((m, n), dtype=torch.float16, device=device)
                                for n in (qkv[0].shape[0], 8192, gate_up[0].shape[0], 8192)], [{}, {}]))

            def paired_step():
                x = x0
                for qkv, o, gate_up, down, ys, ws in blocks:
                    plain(qkv, x, ys[0], ws[0])
                    o.launch(ys[0][:, :8192 // world])
                    x = o.finish(m, out=ys[1])
                    plain(gate_up, x, ys[2], ws[1])
                    down.launch(ys[2][:, :k_down])
                    x = down.finish(m, out=ys[3])
                return x

            out["paired"] = time_chain(paired_step)
            torch.cuda.synchronize()
            for block in blocks:
                block[1].region.check()
                block[3].region.check()
            del blocks
            torch.cuda.empty_cache()
        del shards
        torch.cuda.empty_cache()
    return {key: (round(value, 5) if isinstance(value, float) else value) for key, value in out.items()}


def sharded_record(torch, dist, device, rank: int, world: int, steps: int, warmup: int, pdl: bool = True) -> dict:
    """The `sharded` object of the JSON line: the Llama-70B block at M = 1 and 8 on this job's GPUs."""
    peak, peak_kind = measured_peaks()
    saved_pdl = os.environ.get("W4A16_PDL")
    os.environ["W4A16_PDL"] = "1" if pdl else "0"
    record = {"workload": "llama70b_block_tp", "layers_per_block": [name for name, _, _ in TP_BLOCK], "n_gpus": world,
              "unit": "ms per decoder block (linears only, chained), max over ranks", "programmatic_launch": pdl,
              "l2_policy": "three weight sets per graph replay"}
    for m in (1, 8):
        times = sharded_block_bench(torch, dist, device, rank, world, m, steps, warmup)
        row = dict(times)
        row["bytes_per_block"] = tp_block_bytes(m)
        best = min(times[key] for key in ("peer", "nccl", "paired") if key in times) if world > 1 else times["one_gpu"]
        row["speedup_vs_one_gpu"] = round(times["one_gpu"] / best, 3)
        basis = times.get("kernels_only", times["one_gpu"])
        row["roofline_frac_per_gpu_kernels_only"] = round(tp_block_bytes(m) / world / (basis * 1e-3) / 1e9 / peak, 4)
        row["roofline_frac_per_gpu_with_exchange"] = round(tp_block_bytes(m) / world / (best * 1e-3) / 1e9 / peak, 4)
        record[f"m{m}"] = row
        log(f"  sharded 70B block, {world} GPUs, M={m}: {row}")
    record["peak_kind"] = peak_kind
    if saved_pdl is None:
        os.environ.pop("W4A16_PDL", None)
    else:
        os.environ["W4A16_PDL"] = saved_pdl
    return record


def run_tensor_parallel(args) -> dict:
    """`--workload llama70b_tp`: the linears of one Llama-3-70B decoder block, sharded over the N ranks of this
    job (see sharded_block_bench).  Total work is fixed, so this is strong scaling; the value is the block's
    algorithmic bytes over the best sharded block time (max over ranks)."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    record = sharded_record(torch, dist, device, rank, world, args.steps, args.warmup, pdl=args.pdl)
    row = record[f"m{args.batch}" if args.batch in (1, 8) else "m1"]
    best = min(row[key] for key in ("peer", "nccl", "paired", "one_gpu") if key in row)
    peak, peak_kind = measured_peaks()
    result = {
        "metric": "w4a16_linear_hbm_gbs_tp", "value": round(row["bytes_per_block"] / (best * 1e-3) / 1e9, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": best,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate",
        "data": "synthetic (random codes and scales)",
        "config": {"workload": "llama70b_block_tp", "M": args.batch, "bytes_per_step": row["bytes_per_block"],
                   "parallelism": f"tp{world}", "l2_policy": "three weight sets per graph replay"},
        "sharded": record,
        "roofline": {"bound": "hbm", "achieved": round(row["bytes_per_block"] / world / (best * 1e-3) / 1e9, 1), "peak": peak,
                     "unit": "GB/s per GPU", "peak_kind": peak_kind, "frac": row["roofline_frac_per_gpu_with_exchange"],
                     "traffic": None},
        "gpu_launches": args.steps * 3 * 5,
    }
    if world > 1:
        dist.destroy_process_group()
    return result if rank == 0 else {}


def run_product(args) -> dict:
    import torch
    import torch.distributed as dist

    from nibble_b200 import _native, cuda_extension_available, linear_cuda

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this package has no CPU path")
    if not cuda_extension_available():
        raise SystemExit("the CUDA extension is not built: run `python -m nibble_b200._build`")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if args.pdl:
        os.environ["W4A16_PDL"] = "1"

    sampler = ClockSampler(local)
    sampler.start()

    layers = decode_token_layers()
    log(f"[rank {rank}] building {len(layers)} quantised layers on {torch.cuda.get_device_name(device)}")
    weights = [make_layer(torch, k, n, seed=1000 * rank + i, device=device) for i, (_, k, n) in enumerate(layers)]
    # All activations of a step live in one pinned host buffer and one device buffer; the layers read
    # 256-byte aligned views of the device buffer, so one copy brings a whole step's inputs in.
    g = torch.Generator().manual_seed(1)
    x_all_host = torch.cat([torch.randn((k,), dtype=torch.float32, generator=g).half() for _, k, _ in layers]).pin_memory()
    x_all_dev = x_all_host.to(device)
    x_host, x_dev, offset = [], [], 0
    for _, k, _ in layers:
        x_host.append(x_all_host[offset:offset + k].view(1, k))
        x_dev.append(x_all_dev[offset:offset + k].view(1, k))
        offset += k
    step_bytes = sum(algorithmic_bytes(1, k, n) for _, k, n in layers)
    outs: list = [None] * len(layers)

    def step():
        for i, (packed, scales) in enumerate(weights):
            outs[i] = linear_cuda(x_dev[i], packed, scales, GROUP)

    lib = _native.core()
    graph = capture(torch, step)
    # ---- parity gate before any timing: first, a ragged middle one and the last layer vs the oracle
    from oracle import w4a16_oracle as oracle

    graph.replay()
    torch.cuda.synchronize()
    for i in (0, 6, len(layers) - 1):
        packed, scales = weights[i]
        rows = slice(0, 512)
        exact = oracle.linear_fp64(x_host[i].numpy(), packed[rows].cpu().numpy(), scales[rows].cpu().numpy(), GROUP)
        bound = oracle.error_bound(x_host[i].numpy(), packed[rows].cpu().numpy(), scales[rows].cpu().numpy(), GROUP)
        err = abs(outs[i][:, rows].double().cpu().numpy() - exact)
        assert (err <= bound).all(), f"parity gate failed on layer {i}"

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- value: K graph replays, inputs resident
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    barrier()
    sampler.active.set()
    launches_before = lib.w4a16_launch_count()
    torch.cuda.profiler.start()   # `ncu --profile-from-start off` captures exactly the timed region
    with nvtx_range("w4a16.timed_region tinyllama_decode_linears_m1"):
        ms = time_replays(torch, graph, args.steps)
    torch.cuda.profiler.stop()
    barrier()
    ms = max_over_ranks(ms)
    ms_per_step = ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    kernel_us = ms_per_step * 1e3 / len(layers)

    if args.kernel_only:   # for profiler runs: nothing but the timed region
        sampler.stop.set()
        peak, peak_kind = measured_peaks()
        achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
        if world > 1:
            dist.destroy_process_group()
        return {"metric": "w4a16_linear_hbm_gbs_m1", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "ms_per_step": round(ms_per_step, 5), "kernel_only": True,
                "roofline": {"achieved": round(achieved, 1), "peak": peak, "frac": round(achieved / peak, 4)}} if rank == 0 else {}

    # ---- the same K replays with plain stream-ordered launches, for comparison
    plain = None
    if args.pdl:
        os.environ.pop("W4A16_PDL", None)
        plain_graph = capture(torch, step)
        for _ in range(3):
            plain_graph.replay()
        barrier()
        plain_ms = max_over_ranks(time_replays(torch, plain_graph, args.steps)) / args.steps
        plain = {"value": round(world * step_bytes / (plain_ms * 1e-3) / 1e9, 1), "ms_per_step": round(plain_ms, 5)}
        del plain_graph
        os.environ["W4A16_PDL"] = "1"
        graph = capture(torch, step)   # `outs` point at this graph's outputs again

    # ---- the same token with q/k/v and gate/up concatenated along N (what fuse_parallel_linears does to a
    # model): 89 launches instead of 155 over the same packed bytes; reported beside the headline, not as it
    fused_siblings = None
    if world == 1 and not args.quick:
        fused_layers = []
        for b in range(N_BLOCKS):
            base = b * len(BLOCK_ORDER)
            for members in ((0, 1, 2), (3,), (4, 5), (6,)):
                packed = torch.cat([weights[base + m][0] for m in members]).contiguous()
                scales = torch.cat([weights[base + m][1] for m in members]).contiguous()
                fused_layers.append((x_dev[base + members[0]], packed, scales))
        fused_layers.append((x_dev[-1], *weights[-1]))
        fused_outs: list = [None] * len(fused_layers)

        def fused_step():
            for i, (x, packed, scales) in enumerate(fused_layers):
                fused_outs[i] = linear_cuda(x, packed, scales, GROUP)

        fused_graph = capture(torch, fused_step)
        for _ in range(3):
            fused_graph.replay()
        barrier()
        fused_ms = time_replays(torch, fused_graph, args.steps) / args.steps
        fused_bytes = sum(algorithmic_bytes(1, x.shape[1], packed.shape[0]) for x, packed, _ in fused_layers)
        fused_value = fused_bytes / (fused_ms * 1e-3) / 1e9
        fused_siblings = {"launches_per_step": len(fused_layers), "ms_per_step": round(fused_ms, 5),
                          "value": round(fused_value, 1), "bytes_per_step": fused_bytes,
                          "roofline_frac": round(fused_value / measured_peaks()[0], 4),
                          "what": "the same token as replace_linear_layers serves it by default: q/k/v and gate/up as one launch each"}
        log(f"  q/k/v and gate/up as single launches: {fused_siblings}")
        del fused_graph, fused_layers, fused_outs
        torch.cuda.empty_cache()

    # ---- e2e: host activations in, host outputs back, every step
    y_all_host = torch.empty((sum(n for _, _, n in layers),), dtype=torch.float16).pin_memory()
    h2d = x_all_host.numel() * 2
    d2h = y_all_host.numel() * 2

    def e2e_step():
        x_all_dev.copy_(x_all_host, non_blocking=True)                 # one host -> device copy
        graph.replay()                                                  # 155 linears through the public op
        y_all_host.copy_(torch.cat([o.view(-1) for o in outs]), non_blocking=True)   # gather + one copy back

    for _ in range(3):
        e2e_step()
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        e2e_step()
    end.record()
    barrier()
    serial_ms = max_over_ranks(start.elapsed_time(end)) / args.steps

    # The same per-step work (every step's activations come from pinned host memory, every step's outputs go
    # back to it) with two input/output slots, so that the copies of steps i+1 and i-1 run on their own streams
    # under the kernels of step i.
    total_n = sum(n for _, _, n in layers)
    main_stream = torch.cuda.current_stream()
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    slots = []
    for _ in range(2):
        slot_x = x_all_host.to(device)
        views, offset = [], 0
        for _, k, _ in layers:
            views.append(slot_x[offset:offset + k].view(1, k))
            offset += k
        slot_outs: list = [None] * len(layers)

        def slot_step(views=views, slot_outs=slot_outs):
            for i, (packed, scales) in enumerate(weights):
                slot_outs[i] = linear_cuda(views[i], packed, scales, GROUP)

        slots.append({"x": slot_x, "outs": slot_outs, "graph": capture(torch, slot_step),
                      "gathered": torch.empty((total_n,), dtype=torch.float16, device=device),
                      "y_host": torch.empty((total_n,), dtype=torch.float16).pin_memory(),
                      "in_ready": torch.cuda.Event(), "computed": torch.cuda.Event(), "out_done": torch.cuda.Event()})

    def pipelined(steps: int) -> None:
        for i in range(steps):
            slot = slots[i % 2]
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(slot["computed"])                   # the step that last read this input slot
                slot["x"].copy_(x_all_host, non_blocking=True)
                slot["in_ready"].record(copy_in)
            main_stream.wait_event(slot["in_ready"])
            main_stream.wait_event(slot["out_done"])                   # its outputs have been copied away
            slot["graph"].replay()
            slot["computed"].record(main_stream)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(slot["computed"])
                torch.cat([o.view(-1) for o in slot["outs"]], out=slot["gathered"])
                slot["y_host"].copy_(slot["gathered"], non_blocking=True)
                slot["out_done"].record(copy_out)
        for slot in slots:
            main_stream.wait_event(slot["out_done"])

    pipelined(4)
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    pipelined(args.steps)
    end.record()
    barrier()
    e2e_ms = max_over_ranks(start.elapsed_time(end)) / args.steps
    e2e_value = world * step_bytes / (e2e_ms * 1e-3) / 1e9
    assert torch.equal(slots[0]["y_host"], y_all_host) and torch.equal(slots[1]["y_host"], y_all_host)
    del slots

    # keep the GPU under the same load long enough for the clock sampler when K is small
    window = "timed region"
    if ms + e2e_ms * args.steps < 1500.0:
        window = "timed region + identical load loop"
        deadline = time.perf_counter() + 1.5
        while time.perf_counter() < deadline:
            for _ in range(50):
                graph.replay()
            torch.cuda.synchronize()
    sampler.active.clear()
    clocks = sampler.summary(window)

    peak, peak_kind = measured_peaks()
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    result = {
        "metric": "w4a16_linear_hbm_gbs_m1", "value": round(value, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic (seeded N(0,0.02) weights, N(0,1) activations)",
        "config": {"workload": "tinyllama_decode_linears_m1", "layers_per_step": len(layers), "M": 1,
                   "group_size": GROUP, "bytes_per_step": step_bytes, "l2_policy": "inputs larger than L2 (535 MB per step)",
                   "parallelism": "replicas" if world > 1 else "single", "programmatic_launch": bool(args.pdl)},
        "decode_tok_s_linears_only": round(world * 1e3 / ms_per_step, 1),
        "plain_launch": plain,
        "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": round(e2e_ms, 5), "how": "two slots: copies of neighbouring steps overlap the kernels",
                "one_stream_ms_per_step": round(serial_ms, 5),
                "one_stream_value": round(world * step_bytes / (serial_ms * 1e-3) / 1e9, 1)},
        "gpu_launches": args.steps * len(layers),
        "fused_siblings": fused_siblings,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "peak_kind": peak_kind, "frac_of_8tbs": round(achieved / 8000, 4),
                     "traffic": measured_traffic_per_launch(), "kernel": "linear_mma_kernel", "mean_launch_us": round(kernel_us, 3),
                     "bytes_per_launch": step_bytes // len(layers)},
        "clocks": clocks,
    }
    assert lib.w4a16_launch_count() >= launches_before  # replays re-run captured nodes; capture itself counted

    if rank == 0 and world == 1 and not args.quick:
        l2 = torch.cuda.get_device_properties(device).L2_cache_size
        del graph
        weights.clear()
        torch.cuda.empty_cache()
        log("per-shape latency, rotating weight copies (TinyLlama shapes)")
        result["layers"] = {
            "tinyllama_m1": per_shape_table(torch, TINYLLAMA, 1, device, l2, with_cublas=True),
            "tinyllama_m2": per_shape_table(torch, TINYLLAMA, 2, device, l2, with_cublas=True),
            "tinyllama_m4": per_shape_table(torch, TINYLLAMA, 4, device, l2, with_cublas=True),
            "tinyllama_m8": per_shape_table(torch, TINYLLAMA, 8, device, l2, with_cublas=True),
            "llama70b_m1": per_shape_table(torch, LLAMA70B, 1, device, l2, with_cublas=False),
            "llama70b_m8": per_shape_table(torch, LLAMA70B, 8, device, l2, with_cublas=True),
        }
        short = {"qo_proj": "qo", "kv_proj": "kv", "gate_up_proj": "gate_up", "down_proj": "down", "lm_head": "lm_head"}
        result["roofline"]["per_layer_frac_m1"] = {
            **{f"tl_{short[name]}": row["frac_measured"] for name, row in result["layers"]["tinyllama_m1"].items()},
            **{f"70b_{short[name]}": row["frac_measured"] for name, row in result["layers"]["llama70b_m1"].items()}}
        result["roofline"]["per_layer_us_m1"] = {
            **{f"tl_{short[name]}": row["us"] for name, row in result["layers"]["tinyllama_m1"].items()},
            **{f"70b_{short[name]}": row["us"] for name, row in result["layers"]["llama70b_m1"].items()}}
        result["roofline"]["m8_vs_cublas_fp16"] = {
            **{f"tl_{short[name]}": row["speedup_vs_cublas_fp16"] for name, row in result["layers"]["tinyllama_m8"].items()},
            **{f"70b_{short[name]}": row["speedup_vs_cublas_fp16"] for name, row in result["layers"]["llama70b_m8"].items()}}
        log("prefill-sized batches (tcgen05 kernel)")
        result["prefill"] = prefill_table(torch, device)
        result["quantize"] = quantize_table(torch, device)
    if rank == 0 and world == 1 and not args.quick:
        log("decode tokens/s, TinyLlama-1.1B-shaped model")
        try:
            result["decode"] = decode_bench(torch, device)
        except Exception as error:   # transformers API drift must not cost the headline line
            result["decode"] = {"error": repr(error)[:300]}
    if rank == 0 and world == 1:
        result["cpu_baseline"] = cpu_baseline_leg(blocks=4, repeats=5)
    if world > 1:
        # the layers that ARE worth sharding: one Llama-3-70B-shaped decoder block over this job's GPUs
        del graph
        weights.clear()
        torch.cuda.empty_cache()
        try:
            result["sharded"] = sharded_record(torch, dist, device, rank, world, steps=30, warmup=5)
        except Exception as error:   # must not cost the headline line
            result["sharded"] = {"error": repr(error)[:400]}
    sampler.stop.set()
    if world > 1:
        dist.destroy_process_group()
    return result if rank == 0 else {}


# ----------------------------------------------------------------------------- reference arm
def run_reference(args) -> dict:
    """The reference's own CPU implementation of the path on the host cores, all threads.

    Where ``oracle/_ref`` holds the reference's compiled modules (oracle/build_ref.py) those are what runs:
    ``w4a16.quantization.quantize_and_pack_weights`` makes the packed weights and ``w4a16.reference.linear_reference``
    is timed (kind "reference").  Otherwise the restatement in oracle/torch_cpu_port.py is timed (kind "port").
    Nothing of this package is imported either way.  One step = `--cpu-blocks` decoder blocks of the workload.
    """
    if int(os.environ.get("RANK", "0")) != 0:
        return {}
    import importlib.util

    spec = importlib.util.spec_from_file_location("_w4a16_build_ref", ROOT / "oracle" / "build_ref.py")
    ref_recipe = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref_recipe)
    use_ref = ref_recipe.available()
    import torch

    torch.set_num_threads(os.cpu_count() or 1)
    if use_ref:
        ref_quant, ref_linear = ref_recipe.load()     # the reference's own modules, compiled

        assert "nibble_b200" not in sys.modules
        kind = "reference"

        def quantise(w):
            return ref_quant.quantize_and_pack_weights(w, GROUP)

        linear = ref_linear.linear_reference
    else:
        from oracle import torch_cpu_port as port, w4a16_oracle as oracle

        kind = "port"

        def quantise(w):
            packed, scales = oracle.quantize_and_pack_weights(w.numpy(), GROUP)
            return torch.from_numpy(packed), torch.from_numpy(scales)

        linear = port.linear
    block = [(name, *TINYLLAMA[name]) for name in BLOCK_ORDER] * max(1, args.cpu_blocks)
    data = []
    for index, (_, k, n) in enumerate(block):
        g = torch.Generator().manual_seed(index)
        packed, scales = quantise(torch.randn((n, k), generator=g) * 0.02)
        data.append((torch.randn((1, k), generator=g).half(), packed, scales))
    step_bytes = sum(algorithmic_bytes(1, k, n) for _, k, n in block)

    def step():
        for x, packed, scales in data:
            linear(x, packed, scales, GROUP)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    ms_per_step = sum(times) * 1e3 / args.steps
    value = step_bytes / (ms_per_step * 1e-3) / 1e9
    sample = (f"{max(1, args.cpu_blocks)} decoder block(s) of the workload ({len(block)} linears, "
              f"{step_bytes / 1e6:.1f} MB) per step, M=1, on the host cores")
    return {
        "impl": "reference", "metric": "w4a16_linear_hbm_gbs_m1", "value": round(value, 3), "unit": "GB/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 (torch CPU)", "data": "synthetic (seeded N(0,0.02) weights, N(0,1) activations)",
        "config": {"workload": "tinyllama_decode_linears_m1", "M": 1, "group_size": GROUP, "sample": sample},
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": sample, "seconds_per_sample": round(statistics.median(times), 4)},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", choices=["product", "reference"], default="product")
    parser.add_argument("--no-pdl", dest="pdl", action="store_false",
                        help="plain stream-ordered launches instead of programmatic dependent launch")
    parser.set_defaults(pdl=True)
    parser.add_argument("--quick", action="store_true", help="skip the per-shape tables")
    parser.add_argument("--kernel-only", action="store_true",
                        help="only the timed region (bracketed by cudaProfilerStart/Stop), for profiler runs")
    parser.add_argument("--workload", choices=["tinyllama_decode_linears_m1", "llama70b_tp", "decode_step", "decode"],
                        default="tinyllama_decode_linears_m1")
    parser.add_argument("--batch", type=int, default=1, help="M for --workload llama70b_tp")
    parser.add_argument("--persistent", action="store_true",
                        help="--workload decode_step: the step as one cooperative launch instead of a chain of kernels")
    parser.add_argument("--cpu-blocks", type=int, default=1,
                        help="--impl reference: decoder blocks (7 linears each) per step")
    parser.add_argument("--collective", choices=["p2p", "nccl"], default="p2p",
                        help="llama70b_tp: exchange fused into the kernel epilogue (peer stores) or NCCL calls")
    parser.add_argument("--single-layer", type=int, nargs=3, metavar=("K", "N", "M"),
                        help="run --steps launches of one layer shape only (profiling target)")
    args = parser.parse_args()
    if args.single_layer:
        result = run_single_layer(args)
    elif args.workload == "decode_step" and args.impl == "product":
        result = run_decode_step(args)
    elif args.workload == "decode" and args.impl == "product":
        import torch

        torch.cuda.set_device(0)
        result = {"workload": "decode", "decode": decode_bench(torch, torch.device("cuda", 0), runners_only=args.quick)}
    elif args.workload == "llama70b_tp" and args.impl == "product":
        result = run_tensor_parallel(args)
    else:
        result = run_reference(args) if args.impl == "reference" else run_product(args)
    if result:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
