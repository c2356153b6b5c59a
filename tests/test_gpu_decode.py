"""-m gpu: the decode-step kernels and the runner against transformers' LLaMA code on the same weights."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

transformers = pytest.importorskip("transformers")


def _config(**overrides):
    base = dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=2, max_position_embeddings=128, rms_norm_eps=1e-5, tie_word_embeddings=False)
    base.update(overrides)
    return transformers.LlamaConfig(**base)


def test_add_rmsnorm_matches_the_framework_module():
    from transformers.models.llama.modeling_llama import LlamaRMSNorm

    from nibble_b200.decode import add_rmsnorm

    torch.manual_seed(0)
    for hidden in (256, 2048, 8192):
        norm = LlamaRMSNorm(hidden, eps=1e-5).half().cuda()
        norm.weight.data = (torch.randn(hidden) * 0.1 + 1).half().cuda()
        stream = torch.randn((1, hidden)).half().cuda()
        delta = torch.randn((1, hidden)).half().cuda()
        want_stream = stream + delta
        want = norm(want_stream)
        normed = torch.empty_like(stream)
        add_rmsnorm(stream, delta, norm.weight, 1e-5, normed)
        assert torch.equal(stream, want_stream)
        torch.testing.assert_close(normed, want, rtol=2e-3, atol=2e-3)
        # without a delta the stream is left as it is
        before = stream.clone()
        add_rmsnorm(stream, None, norm.weight, 1e-5, normed)
        assert torch.equal(stream, before)
        torch.testing.assert_close(normed, norm(before), rtol=2e-3, atol=2e-3)


def test_silu_mul_matches_torch():
    from nibble_b200.decode import silu_mul

    gate_up = (torch.randn((1, 2 * 5632), generator=torch.Generator().manual_seed(1)) * 3).half().cuda()
    out = torch.empty((1, 5632), dtype=torch.float16, device="cuda")
    silu_mul(gate_up, out)
    want = torch.nn.functional.silu(gate_up[:, :5632]) * gate_up[:, 5632:]
    torch.testing.assert_close(out, want, rtol=2e-3, atol=1e-3)


@pytest.mark.parametrize(("q_heads", "kv_heads", "head_dim"), [(4, 2, 64), (32, 4, 64), (8, 8, 128)])
def test_attention_decode_matches_rope_plus_sdpa(q_heads, kv_heads, head_dim):
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb

    from nibble_b200.decode import attention_decode

    g = torch.Generator().manual_seed(q_heads + head_dim)
    max_len, steps = 40, 37
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, head_dim, 2).float() / head_dim))).cuda()
    k_cache = torch.zeros((kv_heads, max_len, head_dim), dtype=torch.float16, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    ref_k = torch.zeros((1, kv_heads, max_len, head_dim), dtype=torch.float16, device="cuda")
    ref_v = torch.zeros_like(ref_k)
    position = torch.zeros((1,), dtype=torch.long, device="cuda")
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    out = torch.empty((1, q_heads * head_dim), dtype=torch.float16, device="cuda")
    for t in range(steps):
        qkv = torch.randn((1, (q_heads + 2 * kv_heads) * head_dim), generator=g).half().cuda()
        position.fill_(t)
        attention_decode(qkv, k_cache, v_cache, out, position, inv_freq, q_heads, kv_heads, head_dim, 1.0, status)
        # the framework's route on the same numbers
        q = qkv[:, : q_heads * head_dim].view(1, 1, q_heads, head_dim).transpose(1, 2)
        k = qkv[:, q_heads * head_dim:(q_heads + kv_heads) * head_dim].view(1, 1, kv_heads, head_dim).transpose(1, 2)
        v = qkv[:, (q_heads + kv_heads) * head_dim:].view(1, 1, kv_heads, head_dim).transpose(1, 2)
        freqs = position.float()[:, None] * inv_freq[None, :]
        emb = torch.cat((freqs, freqs), dim=-1)[None]
        q_r, k_r = apply_rotary_pos_emb(q, k, emb.cos().half(), emb.sin().half())
        ref_k[:, :, t] = k_r[:, :, 0]
        ref_v[:, :, t] = v[:, :, 0]
        want = torch.nn.functional.scaled_dot_product_attention(
            q_r, ref_k[:, :, : t + 1], ref_v[:, :, : t + 1], enable_gqa=True).transpose(1, 2).reshape(1, -1)
        torch.testing.assert_close(out, want, rtol=5e-3, atol=2e-3)
    # rotary products are rounded where the framework rounds them; cos/sin may differ in the last bit
    torch.testing.assert_close(k_cache[:, :steps], ref_k[0, :, :steps], rtol=2e-3, atol=2e-3)
    assert (k_cache[:, :steps] == ref_k[0, :, :steps]).float().mean().item() > 0.98
    assert torch.equal(v_cache[:, :steps], ref_v[0, :, :steps])
    assert status.item() == 0
    position.fill_(max_len)                                            # past the cache: reported, nothing written
    attention_decode(qkv, k_cache, v_cache, out, position, inv_freq, q_heads, kv_heads, head_dim, 1.0, status)
    assert status.item() == 1


def test_argmax_advance_picks_the_first_maximum():
    from nibble_b200.decode import argmax_advance

    g = torch.Generator().manual_seed(3)
    token = torch.zeros((1,), dtype=torch.long, device="cuda")
    position = torch.full((1,), 41, dtype=torch.long, device="cuda")
    for count in (1, 7, 512, 32000, 32003):
        logits = torch.randn((1, count), generator=g).half().cuda()
        argmax_advance(logits, token, position)
        assert token.item() == int(torch.argmax(logits.float()).item())
    assert position.item() == 46
    logits = torch.zeros((1, 32000), dtype=torch.float16, device="cuda")
    logits[0, 12345] = 3.0
    logits[0, 777] = 3.0                     # a tie: the lower index, as torch.argmax gives
    argmax_advance(logits, token, None)
    assert token.item() == 777 and position.item() == 46


def test_linear_with_fused_input_equals_the_separate_kernels():
    import ctypes

    from nibble_b200 import _native, quantize_and_pack_weights
    from nibble_b200.decode import add_rmsnorm, linear_with_input, silu_mul
    from nibble_b200.linear import QuantizedLinear

    g = torch.Generator().manual_seed(11)
    workspace = torch.zeros((8 << 20,), dtype=torch.uint8, device="cuda")
    for hidden, n in ((2048, 2560), (2048, 11264), (2048, 32000), (8192, 1024)):
        packed, scales = quantize_and_pack_weights((torch.randn((n, hidden), generator=g) * 0.02).cuda(), 128)
        layer = QuantizedLinear(packed, scales, 128)
        stream = torch.randn((1, hidden), generator=g).half().cuda()
        delta = torch.randn((1, hidden), generator=g).half().cuda()
        weight = (torch.randn((hidden,), generator=g) * 0.1 + 1).half().cuda()
        for second in (delta, None):
            want_stream, normed = stream.clone(), torch.empty_like(stream)
            add_rmsnorm(want_stream, second, weight, 1e-5, normed)
            want = torch.empty((1, n), dtype=torch.float16, device="cuda")
            linear_with_input(layer, normed, want, workspace, None)
            got, new_stream = torch.empty_like(want), torch.zeros_like(stream)
            transform = _native.InputTransform(_native.INPUT_ADD_RMSNORM, 0 if second is None else second.data_ptr(),
                                               weight.data_ptr(), new_stream.data_ptr(), 1e-5)
            linear_with_input(layer, stream, got, workspace, transform)
            assert torch.equal(new_stream, want_stream)
            torch.testing.assert_close(got, want, rtol=2e-3, atol=2e-3)   # the sum of squares is taken in another order
            again = torch.empty_like(got)
            linear_with_input(layer, stream, again, workspace, transform)  # the split-K scratch is reusable as it was left
            assert torch.equal(again, got)
    for inter, n in ((5632, 2048), (28672, 1024)):
        packed, scales = quantize_and_pack_weights((torch.randn((n, inter), generator=g) * 0.02).cuda(), 128)
        layer = QuantizedLinear(packed, scales, 128)
        for rows in (1, 3):
            gate_up = (torch.randn((rows, 2 * inter), generator=g) * 2).half().cuda()
            act = torch.empty((rows, inter), dtype=torch.float16, device="cuda")
            for r in range(rows):
                silu_mul(gate_up[r:r + 1], act[r:r + 1])
            want, got = (torch.empty((rows, n), dtype=torch.float16, device="cuda") for _ in range(2))
            linear_with_input(layer, act, want, workspace, None)
            linear_with_input(layer, gate_up, got, workspace, _native.InputTransform(_native.INPUT_SILU_MUL, 0, 0, 0, 0.0))
            assert torch.equal(got, want)                                 # same values staged, same kernel
    # refusals: RMSNorm input is for one row; the stream may not be updated in place
    lib = _native.core()
    bad = _native.InputTransform(_native.INPUT_ADD_RMSNORM, 0, weight.data_ptr(), stream.data_ptr(), 1e-5)
    out = torch.empty((1, n), dtype=torch.float16, device="cuda")
    args = lambda rows, t: (stream.data_ptr(), packed.data_ptr(), scales.data_ptr(), out.data_ptr(), rows, n, inter, 128,
                            None, 0, 0, ctypes.byref(t), None)
    assert lib.w4a16_linear_f16_input(*args(1, bad)) == -6
    ok = _native.InputTransform(_native.INPUT_ADD_RMSNORM, 0, weight.data_ptr(), 0, 1e-5)
    assert lib.w4a16_linear_f16_input(*args(2, ok)) == -2
    torch.cuda.synchronize()


def test_runner_logits_follow_the_framework_forward():
    from transformers import StaticCache

    from nibble_b200 import replace_linear_layers
    from nibble_b200.decode import LlamaDecodeRunner

    cfg = _config()
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = transformers.AutoModelForCausalLM.from_config(cfg, dtype=torch.float16)
    model.eval()
    assert replace_linear_layers(model, group_size=128) == 3 * 7 + 1
    tokens = torch.randint(0, cfg.vocab_size, (24,), generator=torch.Generator().manual_seed(2)).cuda()
    # framework, token by token, before the runner fuses the siblings (same packed weights either way)
    cache = StaticCache(config=cfg, max_cache_len=32)
    want = []
    with torch.inference_mode():
        for t in range(tokens.numel()):
            out = model(input_ids=tokens[t].view(1, 1), past_key_values=cache,
                        cache_position=torch.tensor([t], device="cuda"), use_cache=True)
            want.append(out.logits[0, -1].float().clone())
    for fuse_inputs, per_block, tail in ((False, 8, 3), (True, 5, 2)):
        runner = LlamaDecodeRunner(model, max_len=32, fuse_inputs=fuse_inputs)
        assert runner.launches_per_step == 0
        worst = 0.0
        for t in range(tokens.numel()):
            runner.token.copy_(tokens[t:t + 1])
            runner.step()
            got = runner.logits[0].float()
            scale = want[t].abs().max().item()
            worst = max(worst, (got - want[t]).abs().max().item() / scale)
            assert int(runner.position.item()) == t + 1
        assert runner.launches_per_step == per_block * 3 + tail     # our kernels per token
        assert worst < 2e-2, worst
        assert runner.status.item() == 0
        graph_cache = (runner.k_cache.clone(), runner.v_cache.clone())
    # the same step as ONE cooperative launch walking a list of operations: same logits, same caches
    runner = LlamaDecodeRunner(model, max_len=32, persistent=True)
    worst = 0.0
    for t in range(tokens.numel()):
        runner.token.copy_(tokens[t:t + 1])
        runner.step()
        got = runner.logits[0].float()
        scale = want[t].abs().max().item()
        worst = max(worst, (got - want[t]).abs().max().item() / scale)
        assert int(runner.position.item()) == t + 1
        assert int(runner.token.item()) == int(got.argmax().item())
    assert runner.launches_per_step == 1
    assert int(runner.step_status.item()) == 0
    assert worst < 2e-2, worst
    # the launch shapes differ from the graph runner's, so sums are taken in another order: close, not equal
    torch.testing.assert_close(runner.v_cache, graph_cache[1], rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(runner.k_cache, graph_cache[0], rtol=2e-2, atol=2e-2)
    assert torch.equal(runner.v_cache[0], graph_cache[1][0]) or (runner.v_cache[0] == graph_cache[1][0]).float().mean().item() > 0.9


def test_persistent_step_reports_a_full_cache_and_keeps_running():
    from nibble_b200 import replace_linear_layers
    from nibble_b200.decode import LlamaDecodeRunner

    cfg = _config(num_hidden_layers=2)
    torch.manual_seed(3)
    with torch.device("cuda"):
        model = transformers.AutoModelForCausalLM.from_config(cfg, dtype=torch.float16)
    model.eval()
    replace_linear_layers(model, group_size=128)
    runner = LlamaDecodeRunner(model, max_len=8, persistent=True)
    reference = LlamaDecodeRunner(model, max_len=8)
    prompt = torch.tensor([7, 1, 300])
    assert torch.equal(runner.generate(prompt, 5), reference.generate(prompt, 5))
    assert torch.equal(runner.generate(prompt, 5), reference.generate(prompt, 5))   # plans are reusable after reset
    for _ in range(3):
        runner.step()            # positions 7, then 8 and 9: past the cache
    torch.cuda.synchronize()
    assert int(runner.step_status.item()) == 1


def test_generate_is_repeatable_and_checks_the_cache_length():
    from nibble_b200 import replace_linear_layers
    from nibble_b200.decode import LlamaDecodeRunner

    cfg = _config(num_hidden_layers=2)
    torch.manual_seed(1)
    with torch.device("cuda"):
        model = transformers.AutoModelForCausalLM.from_config(cfg, dtype=torch.float16)
    model.eval()
    replace_linear_layers(model, group_size=128)
    runner = LlamaDecodeRunner(model, max_len=24)
    prompt = torch.tensor([5, 9, 100, 3])
    first = runner.generate(prompt, 12)
    second = runner.generate(prompt, 12)
    assert first.shape == (12,) and torch.equal(first, second)
    with pytest.raises(ValueError):
        runner.generate(prompt, 21)


def test_batched_prefill_through_the_model_lands_in_the_runners_cache():
    from nibble_b200 import replace_linear_layers
    from nibble_b200.decode import LlamaDecodeRunner

    cfg = _config(num_hidden_layers=2)
    torch.manual_seed(5)
    with torch.device("cuda"):
        model = transformers.AutoModelForCausalLM.from_config(cfg, dtype=torch.float16)
    model.eval()
    replace_linear_layers(model, group_size=128)
    runner = LlamaDecodeRunner(model, max_len=96)
    prompt = torch.randint(0, cfg.vocab_size, (70,), generator=torch.Generator().manual_seed(6))
    runner.prefill(prompt, batched=False)
    k_stepped, v_stepped = runner.k_cache[:, :, :70].clone(), runner.v_cache[:, :, :70].clone()
    runner.step()
    logits_stepped = runner.logits.float().clone()
    runner.prefill(prompt)                         # 70 tokens: the batched route by default
    assert int(runner.position.item()) == 70
    torch.testing.assert_close(runner.k_cache[:, :, :70], k_stepped, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(runner.v_cache[:, :, :70], v_stepped, rtol=3e-2, atol=3e-2)
    runner.step()
    scale = logits_stepped.abs().max().item()
    assert (runner.logits.float() - logits_stepped).abs().max().item() / scale < 3e-2
    out = runner.generate(prompt, 8)
    assert out.shape == (8,) and int(runner.position.item()) == 70 + 7
