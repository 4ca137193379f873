"""The numpy restatement of the Llama layer ops against the transformers modules themselves
(CPU, bf16), so the GPU tests can use the restatement as their oracle."""

import numpy as np
import pytest
import torch

from oracle import llama_ops
from oracle.quant_oracle import f32_to_bf16_bits


def _np(t):
    return t.detach().float().numpy()


@pytest.fixture(scope="module")
def hf():
    return pytest.importorskip("transformers.models.llama.modeling_llama")


def test_rmsnorm_matches_transformers(hf):
    torch.manual_seed(0)
    norm = hf.LlamaRMSNorm(256, eps=1e-5).to(torch.bfloat16)
    norm.weight.data = (torch.randn(256) * 0.1 + 1).bfloat16()
    x = (torch.randn(3, 256) * 2).bfloat16()
    got = llama_ops.rmsnorm(_np(x), _np(norm.weight), 1e-5)
    want = _np(norm(x))
    assert (f32_to_bf16_bits(got) == f32_to_bf16_bits(want)).mean() > 0.995
    assert np.allclose(got, want, rtol=2 ** -7)


def test_rope_matches_transformers(hf):
    from transformers import LlamaConfig

    cfg = LlamaConfig(hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                      intermediate_size=512, num_hidden_layers=1, vocab_size=64,
                      rope_parameters={"rope_type": "default", "rope_theta": 500000.0})
    rotary = hf.LlamaRotaryEmbedding(cfg)
    positions = torch.tensor([[0, 1, 5, 100, 2047]])
    x = torch.randn(1, 4, 5, 64).bfloat16()
    cos, sin = rotary(x, positions)
    got_cos, got_sin = llama_ops.rope_tables(_np(rotary.inv_freq), positions[0].numpy(),
                                             rotary.attention_scaling)
    assert np.array_equal(got_cos, _np(cos[0])) and np.array_equal(got_sin, _np(sin[0]))
    q, _ = hf.apply_rotary_pos_emb(x, x, cos, sin)
    got = llama_ops.apply_rope(_np(x[0]), got_cos[None], got_sin[None])
    assert np.array_equal(got, _np(q[0]))


def test_silu_mul_matches_transformers(hf):
    torch.manual_seed(1)
    gate, up = (torch.randn(4, 512) * 3).bfloat16(), torch.randn(4, 512).bfloat16()
    want = _np(torch.nn.functional.silu(gate) * up)
    got = llama_ops.silu_mul(_np(gate), _np(up))
    assert (f32_to_bf16_bits(got) == f32_to_bf16_bits(want)).mean() > 0.995
    assert np.allclose(got, want, rtol=2 ** -7, atol=1e-30)


def test_attention_decode_matches_transformers(hf):
    torch.manual_seed(2)
    q = torch.randn(1, 8, 1, 64).bfloat16()
    k = torch.randn(1, 2, 37, 64).bfloat16()
    v = torch.randn(1, 2, 37, 64).bfloat16()

    class M(torch.nn.Module):
        num_key_value_groups = 4
        training = False

    want, _ = hf.eager_attention_forward(M(), q, k, v, None, scaling=64 ** -0.5)
    got = llama_ops.attention_decode(_np(q[0, :, 0]), _np(k[0]), _np(v[0]), 64 ** -0.5)
    err = np.linalg.norm(got - _np(want[0, 0])) / np.linalg.norm(_np(want[0, 0]))
    assert err < 5e-3
