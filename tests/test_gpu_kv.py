"""GPU parity of the quantized KV cache kernels (through the C ABI and the Cache class)
against the reference's FakeQuantCache outputs (tests/golden/kv_cache.npz) and the numpy
oracle. Codes and scales are bit-exact; attention outputs within the stated tolerance."""

import numpy as np
import pytest
import torch

import oracle
from gpu_util import bf16_from_bits, bits_of, rel_l2, seeded
from llmquant_b200 import native
from oracle import llama_ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("hd", [64, 128])
def test_cache_update_matches_the_reference_cache(golden, bits, hd):
    from llmquant_b200.quantizers import KernelQuantCache, make_cache_factory

    blob = golden("kv_cache")
    tag = f"b{bits}_hd{hd}"
    cache = make_cache_factory(bits)()
    assert isinstance(cache, KernelQuantCache) and make_cache_factory(None) is None
    k, v = bf16_from_bits(blob[f"{tag}_k"]), bf16_from_bits(blob[f"{tag}_v"])
    # transformers hands the cache transposed views; keep that property
    k_view = k.transpose(1, 2).contiguous().transpose(1, 2)
    ck, cv = cache.update(k_view, v, 0)
    want_k, want_v = (oracle.bf16_bits_to_f32(blob[f"{tag}_c{n}"]) for n in "kv")
    assert np.array_equal(ck.float().cpu().numpy(), want_k)  # by value: -0.0 == 0.0
    assert np.array_equal(cv.float().cpu().numpy(), want_v)
    nz = want_k != 0
    assert np.array_equal(bits_of(ck)[nz], blob[f"{tag}_ck"][nz])
    # codes and scales themselves
    layer = cache.layers[0]
    codes, scales = oracle.kv_quantize(oracle.bf16_bits_to_f32(blob[f"{tag}_k"]), bits)
    t = k.shape[2]
    assert np.array_equal(layer.k_codes[:, :, :t].cpu().numpy(), codes)
    assert np.array_equal(layer.k_scales[:, :, :t].cpu().numpy().view(np.uint32), scales.view(np.uint32))
    # second update appends and leaves the stored tokens alone
    k2, v2 = bf16_from_bits(blob[f"{tag}_k2"]), bf16_from_bits(blob[f"{tag}_v2"])
    ck2, cv2 = cache.update(k2, v2, 0)
    assert np.array_equal(ck2.float().cpu().numpy(), oracle.bf16_bits_to_f32(blob[f"{tag}_ck2"]))
    assert np.array_equal(cv2.float().cpu().numpy(), oracle.bf16_bits_to_f32(blob[f"{tag}_cv2"]))
    assert cache.get_seq_length() == t + 2
    assert torch.equal(ck2[:, :, :t], ck)


def test_cache_grows_and_respects_a_fixed_capacity():
    from llmquant_b200.quantizers import KernelQuantCache

    cache = KernelQuantCache(8)
    chunks = [seeded((1, 2, n, 64), n).bfloat16().cuda() for n in (200, 100, 300)]
    for c in chunks:
        k, _ = cache.update(c, c, 0)
    full = torch.cat(chunks, 2)
    want = oracle.kv_fake_quantize(full.float().cpu().numpy(), 8)
    assert np.array_equal(k.float().cpu().numpy(), want)
    fixed = KernelQuantCache(8, max_cache_len=64)
    fixed.update(chunks[0][:, :, :60], chunks[0][:, :, :60], 0)
    with pytest.raises(RuntimeError, match="cannot take"):
        fixed.update(chunks[1][:, :, :10], chunks[1][:, :, :10], 0)


@pytest.mark.parametrize("hd,hq,hkv", [(64, 8, 2), (128, 8, 2), (128, 4, 4), (64, 8, 1)])
def test_rope_write_and_decode_attention(hd, hq, hkv):
    """Fused RoPE + KV write, then int8-KV decode attention, against the numpy restatement of
    transformers' ops over the reference's fake-quantized cache."""
    B, T, Tmax = 2, 333, 512
    g = torch.Generator().manual_seed(hd + hq)
    inv_freq = 1.0 / (500000.0 ** (np.arange(0, hd, 2, dtype=np.float32) / hd))
    cos_np, sin_np = llama_ops.rope_tables(inv_freq, np.arange(Tmax))
    cos = torch.from_numpy(cos_np).bfloat16().cuda()
    sin = torch.from_numpy(sin_np).bfloat16().cuda()
    kc = torch.zeros(B, hkv, Tmax, hd, dtype=torch.int8, device="cuda")
    vc = torch.zeros_like(kc)
    ks = torch.zeros(B, hkv, Tmax, 1, dtype=torch.float32, device="cuda")
    vs = torch.zeros_like(ks)
    pos = torch.zeros(1, dtype=torch.long, device="cuda")
    q_rot = torch.zeros(B, hq, hd, dtype=torch.bfloat16, device="cuda")
    qkv_all = (torch.randn(T, B, (hq + 2 * hkv) * hd, generator=g)).bfloat16()
    want_k = np.zeros((B, hkv, T, hd), np.float32)
    want_v = np.zeros((B, hkv, T, hd), np.float32)
    for t in range(T):
        row = qkv_all[t].cuda()
        native.call("lq_rope_kv_write", row.data_ptr(), cos.data_ptr(), sin.data_ptr(), q_rot.data_ptr(),
                    kc.data_ptr(), vc.data_ptr(), ks.data_ptr(), vs.data_ptr(), B, hq, hkv, hd, Tmax,
                    Tmax, pos.data_ptr(), 0, 8, 0, native.stream_ptr())
        pos.add_(1)
        heads = qkv_all[t].float().numpy().reshape(B, hq + 2 * hkv, hd)
        want_k[:, :, t] = llama_ops.apply_rope(heads[:, hq:hq + hkv], cos_np[t], sin_np[t])
        want_v[:, :, t] = heads[:, hq + hkv:]
    want_q = llama_ops.apply_rope(heads[:, :hq], cos_np[T - 1], sin_np[T - 1])
    assert np.array_equal(q_rot.float().cpu().numpy(), want_q)
    k_codes, k_scales = oracle.kv_quantize(want_k, 8)
    v_codes, v_scales = oracle.kv_quantize(want_v, 8)
    assert np.array_equal(kc[:, :, :T].cpu().numpy(), k_codes)
    assert np.array_equal(vc[:, :, :T].cpu().numpy(), v_codes)
    assert np.array_equal(ks[:, :, :T].cpu().numpy().view(np.uint32), k_scales.view(np.uint32))
    assert np.array_equal(vs[:, :, :T].cpu().numpy().view(np.uint32), v_scales.view(np.uint32))

    k_deq, v_deq = llama_ops.kv_store(want_k), llama_ops.kv_store(want_v)
    for splits in (1, 3, 16):
        nbytes = native.library().lq_attn_decode_scratch_bytes(B, hq, hd, splits)
        scratch = torch.zeros(nbytes // 4, dtype=torch.float32, device="cuda")
        out = torch.zeros(B, hq, hd, dtype=torch.bfloat16, device="cuda")
        # the cursor now points one past the last token: len = pos + 0
        native.call("lq_attn_decode_kv_i8", q_rot.data_ptr(), kc.data_ptr(), vc.data_ptr(), ks.data_ptr(),
                    vs.data_ptr(), out.data_ptr(), scratch.data_ptr(), B, hq, hkv, hd, Tmax,
                    pos.data_ptr(), 0, 0, hd ** -0.5, splits, 0, native.stream_ptr())
        for b in range(B):
            want = llama_ops.attention_decode(want_q[b], k_deq[b], v_deq[b], hd ** -0.5)
            assert rel_l2(out[b].float().cpu().numpy(), want) <= 1e-2, (splits, b)
    # host-side length gives the same result as the device cursor
    out2 = torch.zeros_like(out)
    native.call("lq_attn_decode_kv_i8", q_rot.data_ptr(), kc.data_ptr(), vc.data_ptr(), ks.data_ptr(),
                vs.data_ptr(), out2.data_ptr(), scratch.data_ptr(), B, hq, hkv, hd, Tmax, 0, T, 0,
                hd ** -0.5, 16, 0, native.stream_ptr())
    assert torch.equal(out, out2)


@pytest.mark.parametrize("hd,hq,hkv", [(64, 8, 2), (128, 8, 2), (128, 8, 8)])
@pytest.mark.parametrize("splits,impl", [(1, native.ATTN_AUTO), (7, native.ATTN_MMA), (7, native.ATTN_SIMT),
                                         (1, native.ATTN_SIMT), (8, native.ATTN_CLUSTER), (4, native.ATTN_CLUSTER)])
def test_fused_attention_block_matches_the_separate_kernels(hd, hq, hkv, splits, impl):
    """lq_attn_decode_fused = lq_rope_kv_write + lq_attn_decode_kv_i8 in one launch, with every
    kernel that can serve it (all-SIMT, tensor-core with the merge by the last CTA -- the
    library's own choice -- and the cluster kernel for 2 / 4 / 8 / 16 slices): the cache it leaves
    behind is bit-identical, its output agrees with the separate kernels (which
    test_rope_write_and_decode_attention holds against the oracle), and its tickets are back at
    zero so it can be replayed."""
    B, T, Tmax = 2, (150 if splits > 1 else 520), 600
    g = torch.Generator().manual_seed(7 * hd + hq + splits)
    inv_freq = 1.0 / (500000.0 ** (np.arange(0, hd, 2, dtype=np.float32) / hd))
    cos_np, sin_np = llama_ops.rope_tables(inv_freq, np.arange(Tmax))
    cos = torch.from_numpy(cos_np).bfloat16().cuda()
    sin = torch.from_numpy(sin_np).bfloat16().cuda()

    def fresh():
        kc = torch.zeros(B, hkv, Tmax, hd, dtype=torch.int8, device="cuda")
        ks = torch.zeros(B, hkv, Tmax, 1, dtype=torch.float32, device="cuda")
        return kc, torch.zeros_like(kc), ks, torch.zeros_like(ks)

    ref, fus = fresh(), fresh()
    pos = torch.zeros(1, dtype=torch.long, device="cuda")
    q_rot = torch.zeros(B, hq, hd, dtype=torch.bfloat16, device="cuda")
    out_ref = torch.zeros(B, hq, hd, dtype=torch.bfloat16, device="cuda")
    out_fus = torch.zeros_like(out_ref)
    lib = native.library()
    scratch_ref = torch.zeros(lib.lq_attn_decode_scratch_bytes(B, hq, hd, splits) // 4, device="cuda")
    nbytes = lib.lq_attn_fused_scratch_bytes(B, hq, hkv, hd, splits)
    scratch_fus = torch.zeros(-(-nbytes // 4), dtype=torch.float32, device="cuda")
    rows = torch.randn(T, B, (hq + 2 * hkv) * hd, generator=g).bfloat16().cuda()
    stream = native.stream_ptr()
    for t in range(T):
        row = rows[t]
        kc, vc, ks, vs = ref
        native.call("lq_rope_kv_write", row.data_ptr(), cos.data_ptr(), sin.data_ptr(), q_rot.data_ptr(),
                    kc.data_ptr(), vc.data_ptr(), ks.data_ptr(), vs.data_ptr(), B, hq, hkv, hd, Tmax,
                    Tmax, pos.data_ptr(), 0, 8, 0, stream)
        native.call("lq_attn_decode_kv_i8", q_rot.data_ptr(), kc.data_ptr(), vc.data_ptr(), ks.data_ptr(),
                    vs.data_ptr(), out_ref.data_ptr(), scratch_ref.data_ptr(), B, hq, hkv, hd, Tmax,
                    pos.data_ptr(), 0, 1, hd ** -0.5, splits, 0, stream)
        kc, vc, ks, vs = fus
        native.call("lq_attn_decode_fused", row.data_ptr(), cos.data_ptr(), sin.data_ptr(), kc.data_ptr(),
                    vc.data_ptr(), ks.data_ptr(), vs.data_ptr(), out_fus.data_ptr(), scratch_fus.data_ptr(),
                    B, hq, hkv, hd, Tmax, Tmax, pos.data_ptr(), 0, 8, hd ** -0.5, splits, impl, 0, stream)
        pos.add_(1)
        if t in (0, 1, 17, T - 1):
            err = rel_l2(out_fus.float().cpu().numpy(), out_ref.float().cpu().numpy())
            assert err <= 1e-2, (t, err)
    for a, b in zip(ref, fus):
        assert torch.equal(a, b)
    tickets = scratch_fus.view(torch.int32)[-(B * hkv):]
    assert int(tickets.abs().sum()) == 0
    assert lib.lq_attn_device_error() == 0


@pytest.mark.parametrize("kw", [dict(head_dim=64), dict(head_dim=128, hidden=512, inter=1024)])
def test_generate_reads_the_integer_cache_without_dequantizing_it(kw):
    """transformers' own `generate` on a model switched to the dequantize-on-read attention:
    after the prompt, no decode step dequantizes the cache (the reference's route materialises
    the whole bf16 cache at every step), and the logits agree with the dequantizing route."""
    from llmquant_b200.core import QuantConfig, oneshot
    from llmquant_b200.quantizers import kv_cache, make_cache_factory
    from oracle.real_mode import tiny_llama

    cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    model = oneshot(tiny_llama(seed=0, **kw).cuda(), cfg.to_modifier(mode="kernel"))
    assert model.config._attn_implementation == kv_cache.ATTENTION_NAME
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, 512, (1, 40), generator=g).cuda()
    fused, plain = make_cache_factory(8, model=model)(), make_cache_factory(8)()
    assert fused.fused_read and not plain.fused_read
    new = 10
    out = model.generate(ids, attention_mask=torch.ones_like(ids), max_new_tokens=new, do_sample=False,
                         pad_token_id=0, past_key_values=fused)
    assert out.shape == (1, 40 + new)
    layers = len(model.model.layers)
    assert [l.dequant_calls for l in fused.layers] == [1] * layers          # the prompt only
    assert [l.fused_reads for l in fused.layers] == [new - 1] * layers
    # teacher-forced over the generated tokens: fused reads against whole-cache dequantization
    a, b = make_cache_factory(8, model=model)(), make_cache_factory(8)()
    with torch.no_grad():
        model(out[:, :40], past_key_values=a, use_cache=True)
        model(out[:, :40], past_key_values=b, use_cache=True)
        for i in range(40, 40 + new - 1):
            la = model(out[:, i:i + 1], past_key_values=a, use_cache=True).logits[:, -1]
            lb = model(out[:, i:i + 1], past_key_values=b, use_cache=True).logits[:, -1]
            assert rel_l2(la.float().cpu().numpy(), lb.float().cpu().numpy()) <= 1e-2, i
    assert b.layers[0].dequant_calls == new and b.layers[0].fused_reads == 0
    # the first layer's keys depend on the embeddings only: both routes store the same integers
    # there (deeper layers see hidden states that differ by the two routes' rounding)
    assert torch.equal(a.layers[0].k_codes[:, :, : a.layers[0].length], b.layers[0].k_codes[:, :, : b.layers[0].length])
    assert a.layers[-1].length == b.layers[-1].length == 40 + new - 1
