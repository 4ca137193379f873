"""numpy restatement of the Llama decoder-layer arithmetic that surrounds the quantized
linears. TEST INFRASTRUCTURE ONLY.

The reference does not implement these ops: it runs them through the third-party
`transformers` package (unpinned in the reference's pyproject; 5.5.0 in this image). The
functions follow transformers 5.5.0 `models/llama/modeling_llama.py` and mirror the
roundings a bfloat16 model performs there (each elementwise torch op on bf16 tensors
computes in fp32 and rounds its result to bf16).

Parity status: pinned against transformers itself by tests/test_oracle_llama_ops.py, which
runs the real modules on CPU and compares.
"""

import numpy as np

from oracle.quant_oracle import kv_fake_quantize, round_to_dtype


def _bf16(x):
    return round_to_dtype(np.asarray(x, dtype=np.float32), "bf16")


def rmsnorm(x, weight, eps):
    """LlamaRMSNorm.forward (modeling_llama.py:62-67) for bf16 x and bf16 weight, as fp32."""
    x = np.asarray(x, dtype=np.float32)
    variance = np.mean(x * x, axis=-1, keepdims=True, dtype=np.float32)
    normed = x * (np.float32(1.0) / np.sqrt(variance + np.float32(eps)))
    return _bf16(np.asarray(weight, dtype=np.float32) * _bf16(normed))


def rope_tables(inv_freq, positions, attention_scaling=1.0):
    """LlamaRotaryEmbedding.forward (modeling_llama.py:124-135): bf16 cos/sin [T, head_dim]."""
    freqs = np.asarray(positions, dtype=np.float32)[:, None] * np.asarray(inv_freq, dtype=np.float32)[None, :]
    emb = np.concatenate((freqs, freqs), axis=-1)
    return (_bf16(np.cos(emb) * np.float32(attention_scaling)),
            _bf16(np.sin(emb) * np.float32(attention_scaling)))


def apply_rope(x, cos, sin):
    """apply_rotary_pos_emb (modeling_llama.py:146-168) on [..., head_dim] bf16 values."""
    x = np.asarray(x, dtype=np.float32)
    half = x.shape[-1] // 2
    rotated = np.concatenate((-x[..., half:], x[..., :half]), axis=-1)
    return _bf16(_bf16(x * cos) + _bf16(rotated * sin))


def silu_mul(gate, up):
    """LlamaMLP.forward's act_fn(gate) * up (modeling_llama.py:182-184) in bf16."""
    gate = np.asarray(gate, dtype=np.float32)
    act = _bf16(gate / (np.float32(1.0) + np.exp(-gate)))
    return _bf16(act * np.asarray(up, dtype=np.float32))


def attention_decode(q, k, v, scaling):
    """One query token per head against a dense cache (eager_attention_forward,
    modeling_llama.py:199-222, without the mask): q [Hq, D], k/v [Hkv, T, D] -> [Hq, D].
    fp32 scores, fp32 softmax, probabilities rounded to bf16, output rounded to bf16."""
    q, k, v = (np.asarray(a, dtype=np.float32) for a in (q, k, v))
    rep = q.shape[0] // k.shape[0]
    k = np.repeat(k, rep, axis=0)
    v = np.repeat(v, rep, axis=0)
    scores = _bf16(_bf16(np.einsum("hd,htd->ht", q, k)) * np.float32(scaling))
    scores = scores - scores.max(axis=-1, keepdims=True)
    p = np.exp(scores)
    p = _bf16(p / p.sum(axis=-1, keepdims=True))
    return _bf16(np.einsum("ht,htd->hd", p, v))


def kv_store(states, num_bits=8):
    """What the quantized cache holds for new K or V [..., head_dim]: the reference's
    FakeQuantCache values (llmquant/quantizers/fake.py:46-55)."""
    return kv_fake_quantize(states, num_bits, 128, dtype="bf16")


def attention_decode_exact(q, k_codes, k_scales, v_codes, v_scales, scaling):
    """The rounding-free value of the same attention: float64 over the stored integers times
    their fp32 scales, q [Hq, D], codes [Hkv, T, D] int8, scales [Hkv, T, 1] -> [Hq, D].

    NOT the reference's arithmetic (that is `attention_decode`, which rounds scores,
    probabilities and the output to bf16 like transformers' eager path and reads bf16-rounded
    cache values): it is the quantity both of them approximate. The bf16 path is itself about
    1e-2 (relative L2) away from it at a few hundred tokens, so a kernel that accumulates in
    fp32 is held to a tight bound against this value and to the bf16 path's own noise against
    `attention_decode`."""
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k_codes, dtype=np.float64) * np.asarray(k_scales, dtype=np.float64)
    v = np.asarray(v_codes, dtype=np.float64) * np.asarray(v_scales, dtype=np.float64)
    rep = q.shape[0] // k.shape[0]
    k = np.repeat(k, rep, axis=0)
    v = np.repeat(v, rep, axis=0)
    scores = np.einsum("hd,htd->ht", q, k) * float(scaling)
    p = np.exp(scores - scores.max(axis=-1, keepdims=True))
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("ht,htd->hd", p, v)
