"""Batch-1 decode runner for LLaMA-architecture models whose linears are ``QuantizedLinear``.

Replaces, for the decode step, what the reference gets from HuggingFace ``model.generate`` with a
static cache (scripts/generate.py:260-365): one token is ``8 * layers + 4`` kernel launches without input fusion, ``5 * layers + 3`` with it --
per block four W4A16 linears (q/k/v fused, o, gate/up fused, down) and one attention kernel that also
applies RoPE and appends to the cache; the two add+RMSNorm and the SiLU*up of a block are computed
inside the linears that consume them, while those stage their activations (``fuse_inputs``; without
it they are three more small kernels per block).  The step is captured once in a CUDA graph and
replayed with the token and the position living in device memory.

The arithmetic follows transformers' LlamaDecoderLayer rounding by rounding (FP16 residual sums,
FP32 RMSNorm statistics, FP16 rotary products, FP32 softmax), so logits agree with the framework's
eager forward up to summation order.  Short prompts are consumed one token per step; longer ones go
through the model's own batched forward once (its linears then run the prefill kernels) and the
resulting keys and values are copied into the runner's caches, which use the same layout.
"""
from __future__ import annotations

import ctypes

import torch

from . import _native
from .fusion import FusedQuantizedLinear, FusedSlice, fuse_parallel_linears
from .linear import QuantizedLinear


def _ptr(tensor: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())


def _flags() -> int:
    from .cuda import programmatic_launch_enabled

    return _native.FLAG_PROGRAMMATIC_LAUNCH if programmatic_launch_enabled() else 0


def _check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed: {_native.status_string(status)}")


def add_rmsnorm(stream: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                normed: torch.Tensor) -> None:
    """``stream += delta`` (FP16, in place; skipped when ``delta`` is None) and
    ``normed = weight * half(stream * rsqrt(mean(stream^2) + eps))`` for one row."""
    lib = _native.core()
    _check(lib.w4a16_add_rmsnorm_f16(_ptr(stream), _ptr(delta), _ptr(weight), _ptr(stream), _ptr(normed),
                                     stream.numel(), ctypes.c_float(eps), _flags(),
                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "add_rmsnorm")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """``out = half(silu(gate)) * up`` for ``gate_up = [gate | up]``."""
    lib = _native.core()
    _check(lib.w4a16_silu_mul_f16(_ptr(gate_up), _ptr(out), out.numel(), _flags(),
                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "silu_mul")


def attention_decode(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                     position: torch.Tensor, inv_freq: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int,
                     rope_scale: float, status: torch.Tensor) -> None:
    """RoPE + cache append + attention of one token over ``[0, position]``; caches are ``[kv_heads, max_len, d]``."""
    lib = _native.core()
    _check(lib.w4a16_attention_decode_f16(
        _ptr(qkv), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(position), _ptr(inv_freq), q_heads, kv_heads, head_dim,
        k_cache.shape[-2], ctypes.c_float(rope_scale), ctypes.c_float(head_dim ** -0.5), _ptr(status), _flags(),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "attention_decode")


def linear_with_input(layer: QuantizedLinear, x: torch.Tensor, out: torch.Tensor, workspace: torch.Tensor,
                      transform: "_native.InputTransform | None") -> None:
    """``out = layer(x')`` through the C ABI, ``x'`` being ``x`` or what ``transform`` derives from it
    on chip (see ``w4a16_linear_f16_input``).  ``layer`` must have 128-wide groups and no bias."""
    lib = _native.core()
    rows = out.shape[0]
    _check(lib.w4a16_linear_f16_input(
        _ptr(x), _ptr(layer.packed_weights), _ptr(layer.scales), _ptr(out), rows, layer.out_features, layer.in_features,
        layer.group_size, _ptr(workspace), workspace.numel(), _flags(),
        None if transform is None else ctypes.byref(transform),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "linear_with_input")


def argmax_advance(logits: torch.Tensor, token: torch.Tensor, position: torch.Tensor | None) -> None:
    """``token[0] = argmax(logits)`` (first maximum) and ``position[0] += 1`` in one launch."""
    lib = _native.core()
    _check(lib.w4a16_argmax_advance_f16(_ptr(logits), logits.numel(), _ptr(token), _ptr(position), _flags(),
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "argmax_advance")


def _owner_of(parent: torch.nn.Module, names: tuple[str, ...]) -> QuantizedLinear:
    """The fused layer behind sibling slices (they must all come from one fused launch, in order)."""
    slices = [getattr(parent, name) for name in names]
    if not all(isinstance(s, FusedSlice) for s in slices):
        raise TypeError(f"{names} must be fused QuantizedLinear siblings (run fuse_parallel_linears first)")
    owner = slices[0]._owner
    if any(s._owner is not owner for s in slices) or [s.index for s in slices] != list(range(len(slices))):
        raise ValueError(f"{names} are not the consecutive slices of one fused layer")
    if len(owner.split_sizes) != len(names):
        raise ValueError(f"the fused layer behind {names} has other members too")
    return owner


class LlamaDecodeRunner:
    """Greedy batch-1 generation for a ``LlamaForCausalLM``-shaped model with W4A16 linears.

    ``model`` keeps ownership of the weights; the runner fuses q/k/v and gate/up (if not fused yet),
    allocates its own KV caches ``[layers, kv_heads, max_len, head_dim]`` and work buffers, and
    captures the step in a CUDA graph at the first ``step``.
    """

    def __init__(self, model: torch.nn.Module, max_len: int, fuse_inputs: bool | None = None, persistent: bool = False):
        config = model.config
        self.model = model
        self.hidden = config.hidden_size
        self.q_heads = config.num_attention_heads
        self.kv_heads = config.num_key_value_heads
        self.head_dim = getattr(config, "head_dim", None) or self.hidden // self.q_heads
        self.eps = float(config.rms_norm_eps)
        self.max_len = int(max_len)
        if self.head_dim not in (64, 128):
            raise ValueError("the attention kernel supports head_dim 64 and 128")
        body = model.model
        fuse_parallel_linears(model)
        self.embed = body.embed_tokens.weight
        device = self.embed.device
        if device.type != "cuda" or self.embed.dtype != torch.float16:
            raise ValueError("the model must be an FP16 model on a CUDA device")
        self.layers = []
        for layer in body.layers:
            attn, mlp = layer.self_attn, layer.mlp
            entry = {
                "norm1": layer.input_layernorm.weight, "qkv": _owner_of(attn, ("q_proj", "k_proj", "v_proj")),
                "o": attn.o_proj, "norm2": layer.post_attention_layernorm.weight,
                "gate_up": _owner_of(mlp, ("gate_proj", "up_proj")), "down": mlp.down_proj,
            }
            for key in ("o", "down"):
                if not isinstance(entry[key], QuantizedLinear):
                    raise TypeError("o_proj and down_proj must be QuantizedLinear layers")
            self.layers.append(entry)
        self.final_norm = body.norm.weight
        self.lm_head = model.lm_head
        rotary = body.rotary_emb
        self.inv_freq = rotary.inv_freq.detach().to(device=device, dtype=torch.float32).contiguous()
        self.rope_scale = float(getattr(rotary, "attention_scaling", 1.0))
        self.inter = self.layers[0]["gate_up"].out_features // 2
        n_layers = len(self.layers)
        half = dict(dtype=torch.float16, device=device)
        self.k_cache = torch.zeros((n_layers, self.kv_heads, self.max_len, self.head_dim), **half)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.token = torch.zeros((1,), dtype=torch.long, device=device)
        self.position = torch.zeros((1,), dtype=torch.long, device=device)
        self.status = torch.zeros((1,), dtype=torch.int32, device=device)
        self.stream = torch.zeros((1, self.hidden), **half)
        self.normed = torch.zeros((1, self.hidden), **half)
        self.attn_out = torch.zeros((1, self.q_heads * self.head_dim), **half)
        self.act = torch.zeros((1, self.inter), **half)
        self.logits = None
        self._graph = None
        self.launches_per_step = 0
        linears = [entry[key] for entry in self.layers for key in ("qkv", "o", "gate_up", "down")] + [self.lm_head]
        can_fuse = all(isinstance(m, QuantizedLinear) and m.group_size == 128 and m.bias is None for m in linears)
        if fuse_inputs and not can_fuse:
            raise ValueError("fuse_inputs needs every linear to be a bias-free QuantizedLinear with group_size 128")
        self.fuse_inputs = can_fuse if fuse_inputs is None else bool(fuse_inputs)
        if self.fuse_inputs:
            self.stream_b = torch.zeros_like(self.stream)
            self.qkv_out = torch.zeros((1, self.layers[0]["qkv"].out_features), **half)
            self.o_out = torch.zeros((1, self.hidden), **half)
            self.gate_up_out = torch.zeros((1, 2 * self.inter), **half)
            self.down_out = torch.zeros((1, self.hidden), **half)
            self.logits = torch.zeros((1, self.lm_head.out_features), **half)
            self.workspace = torch.zeros((8 << 20,), dtype=torch.uint8, device=device)   # split-K scratch; kernels leave it zeroed
        self.persistent = bool(persistent)
        if self.persistent:
            if not self.fuse_inputs:
                raise ValueError("the persistent step needs bias-free QuantizedLinear layers with group_size 128")
            self._build_plan()

    # ------------------------------------------------------------------ the whole step as one cooperative launch
    def _build_plan(self) -> None:
        lib = _native.core()
        layers = (_native.DecodeLayer * len(self.layers))()
        for index, entry in enumerate(self.layers):
            layers[index] = _native.DecodeLayer(
                entry["norm1"].data_ptr(), entry["qkv"].packed_weights.data_ptr(), entry["qkv"].scales.data_ptr(),
                entry["o"].packed_weights.data_ptr(), entry["o"].scales.data_ptr(), entry["norm2"].data_ptr(),
                entry["gate_up"].packed_weights.data_ptr(), entry["gate_up"].scales.data_ptr(),
                entry["down"].packed_weights.data_ptr(), entry["down"].scales.data_ptr(),
                self.k_cache[index].data_ptr(), self.v_cache[index].data_ptr())
        model = _native.DecodeModel(
            len(self.layers), self.hidden, self.q_heads, self.kv_heads, self.head_dim, self.inter, self.lm_head.out_features,
            self.max_len, self.eps, self.rope_scale, self.head_dim ** -0.5, self.embed.data_ptr(), self.final_norm.data_ptr(),
            self.lm_head.packed_weights.data_ptr(), self.lm_head.scales.data_ptr(), self.inv_freq.data_ptr(), layers)
        need = lib.w4a16_decode_plan_bytes(ctypes.byref(model))
        if need == 0:
            raise ValueError("this model's shape does not fit the persistent decode step")
        self._plan = torch.zeros((need,), dtype=torch.uint8, device=self.embed.device)
        self._plan_info = _native.DecodePlanInfo()
        _check(lib.w4a16_decode_plan_build(ctypes.byref(model), self._plan.data_ptr(), need, self.token.data_ptr(),
                                           self.position.data_ptr(), ctypes.byref(self._plan_info),
                                           ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "decode_plan_build")
        base = self._plan.data_ptr()
        vocab = self.lm_head.out_features
        offset = self._plan_info.logits - base
        self.logits = self._plan[offset:offset + 2 * vocab].view(torch.float16).view(1, vocab)
        offset = self._plan_info.status - base
        self.step_status = self._plan[offset:offset + 4].view(torch.int32)
        self.launches_per_step = 1

    def _persistent_step(self) -> None:
        _check(_native.core().w4a16_decode_step_f16(self._plan.data_ptr(), ctypes.byref(self._plan_info),
                                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "decode_step")

    # ------------------------------------------------------------------ one token
    def _norm_into(self, source: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor,
                   target: torch.Tensor | None) -> "_native.InputTransform":
        return _native.InputTransform(_native.INPUT_ADD_RMSNORM, 0 if delta is None else delta.data_ptr(), weight.data_ptr(),
                                      0 if target is None else target.data_ptr(), self.eps)

    def _enqueue_fused_step(self) -> None:
        a, b, ws = self.stream, self.stream_b, self.workspace
        silu = _native.InputTransform(_native.INPUT_SILU_MUL, 0, 0, 0, 0.0)
        torch.index_select(self.embed, 0, self.token, out=a)
        delta = None
        for index, layer in enumerate(self.layers):
            linear_with_input(layer["qkv"], a, self.qkv_out, ws, self._norm_into(a, delta, layer["norm1"], b))
            attention_decode(self.qkv_out, self.k_cache[index], self.v_cache[index], self.attn_out, self.position,
                             self.inv_freq, self.q_heads, self.kv_heads, self.head_dim, self.rope_scale, self.status)
            linear_with_input(layer["o"], self.attn_out, self.o_out, ws, None)
            linear_with_input(layer["gate_up"], b, self.gate_up_out, ws, self._norm_into(b, self.o_out, layer["norm2"], a))
            linear_with_input(layer["down"], self.gate_up_out, self.down_out, ws, silu)
            delta = self.down_out
        linear_with_input(self.lm_head, a, self.logits, ws, self._norm_into(a, delta, self.final_norm, None))
        argmax_advance(self.logits, self.token, self.position)

    def _enqueue_step(self) -> None:
        if self.fuse_inputs:
            self._enqueue_fused_step()
            return
        torch.index_select(self.embed, 0, self.token, out=self.stream)
        delta = None
        for index, layer in enumerate(self.layers):
            add_rmsnorm(self.stream, delta, layer["norm1"], self.eps, self.normed)
            qkv = layer["qkv"](self.normed)
            attention_decode(qkv, self.k_cache[index], self.v_cache[index], self.attn_out, self.position, self.inv_freq,
                             self.q_heads, self.kv_heads, self.head_dim, self.rope_scale, self.status)
            attn = layer["o"](self.attn_out)
            add_rmsnorm(self.stream, attn, layer["norm2"], self.eps, self.normed)
            gate_up = layer["gate_up"](self.normed)
            silu_mul(gate_up, self.act)
            delta = layer["down"](self.act)
        add_rmsnorm(self.stream, delta, self.final_norm, self.eps, self.normed)
        self.logits = self.lm_head(self.normed)
        argmax_advance(self.logits, self.token, self.position)

    def step(self) -> None:
        """Consumes ``self.token`` at ``self.position``; leaves the greedy next token in ``self.token``."""
        if self.persistent:
            self._persistent_step()
            return
        with torch.inference_mode():
            if self._graph is None:
                keep = (self.token.clone(), self.position.clone(), self.k_cache.clone(), self.v_cache.clone())
                before = _native.core().w4a16_launch_count()
                self._enqueue_step()                      # warm-up outside capture: workspaces, lazy initialisation
                self.launches_per_step = _native.core().w4a16_launch_count() - before
                torch.cuda.synchronize()
                self.token.copy_(keep[0]); self.position.copy_(keep[1])
                self.k_cache.copy_(keep[2]); self.v_cache.copy_(keep[3])
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self._enqueue_step()
                self._graph = graph
                self.token.copy_(keep[0]); self.position.copy_(keep[1])
                self.k_cache.copy_(keep[2]); self.v_cache.copy_(keep[3])
            self._graph.replay()

    def reset(self) -> None:
        self.position.zero_()
        self.status.zero_()
        if self.persistent:
            self.step_status.zero_()

    # Prompts up to this many tokens are cheaper one decode step at a time than through the framework's
    # batched forward (about half a millisecond per token against a fixed ~12 ms).
    STEPPED_PREFILL_MAX = 24

    def prefill(self, prompt_ids: torch.Tensor, batched: bool | None = None) -> None:
        """Consume a 1-D prompt from position 0; leaves the first generated token in ``self.token``."""
        prompt = prompt_ids.reshape(-1).to(self.token.device)
        if prompt.numel() == 0 or prompt.numel() >= self.max_len:
            raise ValueError("the prompt must hold at least one token and fit the cache")
        self.reset()
        if batched is None:
            batched = prompt.numel() > self.STEPPED_PREFILL_MAX
        if not batched:
            for i in range(prompt.numel()):
                self.token.copy_(prompt[i:i + 1])
                self.step()
            return
        from transformers import StaticCache

        count = prompt.numel()
        with torch.inference_mode():
            cache = StaticCache(config=self.model.config, max_cache_len=self.max_len)
            out = self.model(input_ids=prompt.view(1, -1), past_key_values=cache,
                             cache_position=torch.arange(count, device=prompt.device), use_cache=True)
            for index, layer in enumerate(cache.layers):
                self.k_cache[index, :, :count].copy_(layer.keys[0, :, :count])
                self.v_cache[index, :, :count].copy_(layer.values[0, :, :count])
            self.token.copy_(out.logits[0, -1:].argmax(-1))
            self.position.fill_(count)
        from .cuda import check_device_status

        check_device_status()      # the batched forward ran the prefill kernels: none of their waits may have given up

    def generate(self, prompt_ids: torch.Tensor, new_tokens: int, batched_prefill: bool | None = None) -> torch.Tensor:
        """Greedy continuation of a 1-D prompt; returns the ``new_tokens`` generated ids."""
        prompt = prompt_ids.reshape(-1).to(self.token.device)
        if prompt.numel() + new_tokens > self.max_len:
            raise ValueError("prompt + new tokens exceed the cache length")
        out = torch.empty((new_tokens,), dtype=torch.long, device=self.token.device)
        self.prefill(prompt, batched_prefill)
        for i in range(new_tokens):
            out[i:i + 1].copy_(self.token)
            if i + 1 < new_tokens:
                self.step()
        if int(self.status.item()) != 0:
            raise RuntimeError("a decode step ran past the end of the KV cache")
        if self.persistent and int(self.step_status.item()) != 0:
            code = int(self.step_status.item())
            raise RuntimeError("a decode step ran past the end of the KV cache" if code == 1 else
                               f"the persistent decode step gave up waiting before operation {code - 0x100}")
        return out
