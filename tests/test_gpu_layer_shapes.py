"""One decoder layer of the Llama-3-8B shape and one of the Llama-3.2-1B shape through the fused
decode step (GEMV chain + attention block), at batch 1 and batch 8, against the numpy oracle
stage by stage: every stage takes the GPU's own input tensor and compares the GPU's output of
that stage with the oracle's (real-mode linear, transformers' norm / rotary / softmax / SiLU
arithmetic), so a tolerance is the tolerance of that stage alone.

The cached context (a few hundred tokens written by the prefill path, whose codes and scales
other tests hold bit-exact) is read back from the GPU cache as integers and dequantized by the
oracle."""

import numpy as np
import pytest
import torch

import oracle
from gpu_util import rel_l2
from llmquant_b200.core import QuantConfig, oneshot
from oracle import llama_ops

pytestmark = pytest.mark.gpu

SHAPES = {
    "8b": dict(hidden=4096, heads=32, kv_heads=8, head_dim=128, inter=14336),
    "1b": dict(hidden=2048, heads=32, kv_heads=8, head_dim=64, inter=8192),
}


def _np(t):
    return t.detach().float().cpu().numpy()


@pytest.mark.timeout(900)
@pytest.mark.parametrize("shape", ["8b", "1b"])
@pytest.mark.parametrize("B", [1, 8])
def test_decoder_layer_stage_by_stage(shape, B):
    from llmquant_b200.runtime.decoder import FusedLlamaDecoder
    from oracle.real_mode import tiny_llama

    kw = SHAPES[shape]
    hd, hq, hkv, hidden = kw["head_dim"], kw["heads"], kw["kv_heads"], kw["hidden"]
    T = 300
    model = tiny_llama(seed=5, layers=1, vocab=1024, **kw)
    layer = model.model.layers[0]
    weights = {n: getattr(layer.self_attn, n).weight.detach().float().numpy() for n in ("q_proj", "k_proj", "v_proj", "o_proj")}
    weights.update({n: getattr(layer.mlp, n).weight.detach().float().numpy() for n in ("gate_proj", "up_proj", "down_proj")})
    ln1 = layer.input_layernorm.weight.detach().float().numpy()
    ln2 = layer.post_attention_layernorm.weight.detach().float().numpy()
    embed = model.model.embed_tokens.weight.detach().float().numpy()
    inv_freq = model.model.rotary_emb.inv_freq.float().numpy()
    cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    model = oneshot(model.cuda(), cfg.to_modifier(mode="kernel"))
    dec = FusedLlamaDecoder(model, B, T + 8, kv_bits=8, use_graph=False)
    g = torch.Generator().manual_seed(B)
    prompt = torch.randint(0, 1024, (B, T), generator=g).cuda()
    dec.prefill(prompt)
    tok = torch.randint(0, 1024, (B,), generator=g)
    dec.tokens.copy_(tok)
    dec.step()
    torch.cuda.synchronize()
    cache = dec.cache.layers[0]

    def linear(x, name, bits, **scheme):
        q, scale = oracle.quantize_weight(weights[name], bits, 128, **scheme)
        return oracle.real_linear(x, q, scale, bits, 128, **scheme)

    # ---- q|k|v from the embedding row (RMSNorm fused into the GEMV); q/k/v share a scale per head
    x0 = embed[tok.numpy()]
    normed = llama_ops.rmsnorm(x0, ln1, 1e-5)
    want_qkv = np.concatenate([linear(normed, n, 8, out_group=hd) for n in ("q_proj", "k_proj", "v_proj")], -1)
    got_qkv = _np(dec.qkv)
    assert rel_l2(got_qkv, want_qkv) <= 2e-3

    # ---- attention block from the GPU's q|k|v row and the GPU's integer cache
    cos_np, sin_np = llama_ops.rope_tables(inv_freq, np.arange(T + 1))
    heads = got_qkv.reshape(B, hq + 2 * hkv, hd)
    q_rot = llama_ops.apply_rope(heads[:, :hq], cos_np[T], sin_np[T])
    k_new = llama_ops.kv_store(llama_ops.apply_rope(heads[:, hq:hq + hkv], cos_np[T], sin_np[T]))
    v_new = llama_ops.kv_store(heads[:, hq + hkv:])
    k_codes, v_codes = cache.k_codes[:, :, :T + 1].cpu().numpy(), cache.v_codes[:, :, :T + 1].cpu().numpy()
    k_scales, v_scales = cache.k_scales[:, :, :T + 1].cpu().numpy(), cache.v_scales[:, :, :T + 1].cpu().numpy()
    k_all = oracle.round_to_dtype(k_codes.astype(np.float32) * k_scales, "bf16")
    v_all = oracle.round_to_dtype(v_codes.astype(np.float32) * v_scales, "bf16")
    # the token appended by the step holds what the oracle stores for it
    assert np.array_equal(k_all[:, :, T], k_new) and np.array_equal(v_all[:, :, T], v_new)
    got_attn = _np(dec.attn).reshape(B, hq, hd)
    for b in range(B):
        # tight against the rounding-free value over the stored integers; against the bf16
        # path of transformers within that path's own rounding noise (about 1e-2 here)
        exact = llama_ops.attention_decode_exact(q_rot[b], k_codes[b], k_scales[b], v_codes[b], v_scales[b], hd ** -0.5)
        assert rel_l2(got_attn[b], exact) <= 5e-3, b
        want = llama_ops.attention_decode(q_rot[b], k_all[b], v_all[b], hd ** -0.5)
        assert rel_l2(got_attn[b], want) <= 1.5e-2, b

    # ---- o_proj + residual (per-head groups along K when the head is narrower than a group)
    o = linear(_np(dec.attn), "o_proj", 8, head_dim=hd)
    want_h1 = oracle.round_to_dtype(oracle.round_to_dtype(o, "bf16") + x0, "bf16")
    got_h1 = _np(dec.h[1])
    assert rel_l2(got_h1 - x0, want_h1 - x0) <= 4e-3  # the layer's own contribution, bf16-rounded twice
    assert rel_l2(got_h1, want_h1) <= 2e-3

    # ---- gate|up with the fused RMSNorm and SiLU * up
    normed2 = llama_ops.rmsnorm(got_h1, ln2, 1e-5)
    gate = oracle.round_to_dtype(linear(normed2, "gate_proj", 4), "bf16")
    up = oracle.round_to_dtype(linear(normed2, "up_proj", 4), "bf16")
    want_act = llama_ops.silu_mul(gate, up)
    got_act = _np(dec.act)
    assert rel_l2(got_act, want_act) <= 4e-3  # a product of two bf16-rounded linears

    # ---- down_proj + residual
    down = linear(got_act, "down_proj", 4)
    want_h2 = oracle.round_to_dtype(oracle.round_to_dtype(down, "bf16") + got_h1, "bf16")
    assert rel_l2(_np(dec.h[0]), want_h2) <= 2e-3
    dec.check_device_errors()
