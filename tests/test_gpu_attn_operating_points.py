"""The fused decode-attention block at the shapes and context lengths the decode benchmarks run
it at, against the numpy restatement of transformers' attention over the reference's
fake-quantized cache (oracle/llama_ops.py) -- directly, not against another kernel of this
library: Llama-3-8B heads (head_dim 128, 32 query / 8 KV heads) at a context of 4096+ tokens
with the slice counts the decoder uses, and Llama-3.2-1B heads (head_dim 64) past 512 tokens.

Two bounds per step: 1.5e-2 against that bf16 arithmetic (which rounds scores, probabilities and
outputs to bf16 and is itself about 1e-2 away from exact arithmetic at these lengths), and
5e-3 against the rounding-free float64 attention over the integers the cache holds."""

import numpy as np
import pytest
import torch

import oracle
from gpu_util import rel_l2
from llmquant_b200 import native
from oracle import llama_ops

pytestmark = pytest.mark.gpu


def _filled_cache(B, hkv, T, Tmax, hd, seed):
    """A cache holding T tokens: random keys / values quantized by the oracle (the codes and
    scales the write kernels are separately shown to produce), uploaded as they are."""
    rng = np.random.default_rng(seed)
    k = oracle.round_to_dtype(rng.standard_normal((B, hkv, T, hd)).astype(np.float32), "bf16")
    v = oracle.round_to_dtype(rng.standard_normal((B, hkv, T, hd)).astype(np.float32), "bf16")
    kc, ks = oracle.kv_quantize(k, 8)
    vc, vs = oracle.kv_quantize(v, 8)
    dev = {}
    for name, codes, scales in (("k", kc, ks), ("v", vc, vs)):
        c = torch.zeros(B, hkv, Tmax, hd, dtype=torch.int8, device="cuda")
        s = torch.zeros(B, hkv, Tmax, 1, dtype=torch.float32, device="cuda")
        c[:, :, :T] = torch.from_numpy(codes).cuda()
        s[:, :, :T] = torch.from_numpy(scales.reshape(B, hkv, T, 1)).cuda()
        dev[name] = (c, s)
    return dev, llama_ops.kv_store(k), llama_ops.kv_store(v)


@pytest.mark.parametrize("hd,hq,hkv,B,T,splits,impl", [
    (128, 32, 8, 1, 4096, 37, native.ATTN_AUTO),      # the 8B decode step as the decoder launches it
    (128, 32, 8, 1, 4096, 16, native.ATTN_CLUSTER),   # the same with one cluster per KV head
    (128, 32, 8, 1, 4096, 16, native.ATTN_SIMT),
    (128, 4, 1, 1, 4100, 64, native.ATTN_AUTO),       # one KV head per GPU (tensor parallel over 8)
    (128, 4, 1, 1, 4100, 16, native.ATTN_CLUSTER),
    (128, 32, 8, 2, 1030, 8, native.ATTN_CLUSTER),
    (128, 32, 8, 8, 1030, 5, native.ATTN_AUTO),       # batch 8
    (64, 32, 8, 1, 600, 37, native.ATTN_AUTO),        # the 1B decode step past 512 tokens
    (64, 32, 8, 1, 600, 16, native.ATTN_CLUSTER),
    (64, 32, 8, 1, 2040, 32, native.ATTN_AUTO),
])
def test_fused_attention_at_benchmark_contexts(hd, hq, hkv, B, T, splits, impl):
    steps, Tmax = 4, T + 16
    inv_freq = 1.0 / (500000.0 ** (np.arange(0, hd, 2, dtype=np.float32) / hd))
    cos_np, sin_np = llama_ops.rope_tables(inv_freq, np.arange(Tmax))
    cos = torch.from_numpy(cos_np).bfloat16().cuda()
    sin = torch.from_numpy(sin_np).bfloat16().cuda()
    dev, k_deq, v_deq = _filled_cache(B, hkv, T, Tmax, hd, seed=hd + T)
    (kc, ks), (vc, vs) = dev["k"], dev["v"]
    k_all = np.zeros((B, hkv, Tmax, hd), np.float32)
    v_all = np.zeros_like(k_all)
    k_all[:, :, :T], v_all[:, :, :T] = k_deq, v_deq
    lib = native.library()
    nbytes = lib.lq_attn_fused_scratch_bytes(B, hq, hkv, hd, splits)
    scratch = torch.zeros(-(-nbytes // 4), dtype=torch.float32, device="cuda")
    out = torch.zeros(B, hq, hd, dtype=torch.bfloat16, device="cuda")
    pos = torch.tensor([T], dtype=torch.long, device="cuda")
    g = torch.Generator().manual_seed(T)
    rows = torch.randn(steps, B, (hq + 2 * hkv) * hd, generator=g).bfloat16()
    stream = native.stream_ptr()
    raw_k = []
    for t in range(steps):
        row = rows[t].cuda()
        native.call("lq_attn_decode_fused", row.data_ptr(), cos.data_ptr(), sin.data_ptr(), kc.data_ptr(),
                    vc.data_ptr(), ks.data_ptr(), vs.data_ptr(), out.data_ptr(), scratch.data_ptr(),
                    B, hq, hkv, hd, Tmax, Tmax, pos.data_ptr(), 0, 8, hd ** -0.5, splits, impl, 0, stream)
        p = T + t
        heads = rows[t].float().numpy().reshape(B, hq + 2 * hkv, hd)
        q_rot = llama_ops.apply_rope(heads[:, :hq], cos_np[p], sin_np[p])
        raw_k.append(llama_ops.apply_rope(heads[:, hq:hq + hkv], cos_np[p], sin_np[p]))
        k_all[:, :, p] = llama_ops.kv_store(raw_k[-1])
        v_all[:, :, p] = llama_ops.kv_store(heads[:, hq + hkv:])
        got = out.float().cpu().numpy()
        codes = [a[:, :, :p + 1].cpu().numpy() for a in (kc, ks, vc, vs)]
        for b in range(B):
            # against transformers' bf16 arithmetic within that path's own rounding noise, and
            # tightly against the rounding-free value over the stored integers
            want = llama_ops.attention_decode(q_rot[b], k_all[b, :, :p + 1], v_all[b, :, :p + 1], hd ** -0.5)
            err = rel_l2(got[b], want)
            assert err <= 1.5e-2, (t, b, err)
            exact = llama_ops.attention_decode_exact(q_rot[b], codes[0][b], codes[1][b], codes[2][b], codes[3][b],
                                                     hd ** -0.5)
            err = rel_l2(got[b], exact)
            assert err <= 5e-3, (t, b, err)
        pos.add_(1)
    # the appended tokens hold exactly the codes and scales the oracle gives them
    want_codes, want_scales = oracle.kv_quantize(np.stack(raw_k, axis=2), 8)
    assert np.array_equal(kc[:, :, T:T + steps].cpu().numpy(), want_codes)
    assert np.array_equal(ks[:, :, T:T + steps, 0].cpu().numpy().view(np.uint32),
                          want_scales.reshape(B, hkv, steps).view(np.uint32))
    assert lib.lq_attn_device_error() == 0
