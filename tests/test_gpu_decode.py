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
    runner = LlamaDecodeRunner(model, max_len=32)
    assert runner.launches_per_step == 0
    worst = 0.0
    for t in range(tokens.numel()):
        runner.token.copy_(tokens[t:t + 1])
        runner.step()
        got = runner.logits[0].float()
        scale = want[t].abs().max().item()
        worst = max(worst, (got - want[t]).abs().max().item() / scale)
        assert int(runner.position.item()) == t + 1
    assert runner.launches_per_step == 8 * 3 + 2          # our kernels per token: 8 per block, final norm, lm_head
    assert worst < 2e-2, worst
    assert runner.status.item() == 0


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
