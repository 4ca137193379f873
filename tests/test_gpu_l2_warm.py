"""Launches that pull later launches' weights into L2 (`lq_span`): the requests change no
result, and malformed spans are refused before anything is launched."""
import ctypes

import pytest
import torch

from gpu_util import seeded
from llmquant_b200.core import QuantConfig, oneshot

pytestmark = pytest.mark.gpu


def _module(n, k, bits, seed):
    from llmquant_b200.core import QuantizationArgs, QuantizationScheme
    from llmquant_b200.quantizers import KernelQuantLinear

    scheme = QuantizationScheme(
        weights=QuantizationArgs(num_bits=bits, strategy="group", group_size=128), input_activations=None)
    linear = torch.nn.Linear(k, n, bias=False)
    linear.weight.data = seeded((n, k), seed, 0.02, torch.bfloat16).float()
    return KernelQuantLinear.from_linear(linear.cuda(), scheme)


@pytest.mark.parametrize("bits,m", [(4, 1), (8, 2), (4, 4), (8, 8)])
def test_gemv_with_spans_gives_the_same_bits(bits, m):
    """Both GEMV kernels (the SIMT one at 1-2 rows, the tensor-core one above)."""
    module = _module(520, 2048, bits, 3)
    other = _module(1024, 2048, 4, 4)
    third = torch.zeros(3 << 20, dtype=torch.uint8, device="cuda")  # 3 MB: many pieces per CTA
    x = seeded((m, 2048), 5).bfloat16().cuda()
    gamma = (seeded((2048,), 6) * 0.1 + 1).bfloat16().cuda()
    plain = module.gemv(x, norm_weight=gamma)
    warmed = module.gemv(x, norm_weight=gamma, warm=[other.codes, third])
    torch.cuda.synchronize()
    assert torch.equal(plain, warmed)
    # a span whose size is not a multiple of the request size, and one of a few bytes
    odd = module.gemv(x, norm_weight=gamma, warm=[third[: (1 << 20) + 4080], third[16:40]])
    assert torch.equal(plain, odd)


def test_malformed_spans_are_refused():
    from llmquant_b200 import native

    module = _module(64, 256, 8, 7)
    x = seeded((1, 256), 8).bfloat16().cuda()
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="16-byte"):
        module.gemv(x, warm=[buf[8:]])
    with pytest.raises(ValueError, match="at most 2"):
        module.gemv(x, warm=[buf, buf, buf])
    # through the C ABI: a negative size, and more spans than a launch takes
    arr = (native.Span * 2)()
    arr[0].ptr, arr[0].bytes = buf.data_ptr(), -16
    status = native.library().lq_attn_decode_fused(
        *([buf.data_ptr()] * 9), 1, 4, 1, 64, 16, 16, buf.data_ptr(), 0, 8, ctypes.c_float(0.125), 1, 0,
        arr, 1, 0, native.stream_ptr())
    assert status != 0 and "negative size" in native.last_error()
    status = native.library().lq_attn_decode_fused(
        *([buf.data_ptr()] * 9), 1, 4, 1, 64, 16, 16, buf.data_ptr(), 0, 8, ctypes.c_float(0.125), 1, 0,
        arr, 3, 0, native.stream_ptr())
    assert status != 0 and "warm spans" in native.last_error()


@pytest.mark.parametrize("policy", ["attn", "chain", "next"])
def test_decoder_policies_decode_the_same_tokens(policy):
    """The fused decoder with every policy against the decoder without: same tokens, same
    logits bit for bit (graphed, 12 tokens; the attention launch carries the spans too)."""
    from llmquant_b200.runtime.decoder import FusedLlamaDecoder
    from oracle.real_mode import tiny_llama

    cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    model = oneshot(tiny_llama(seed=0, head_dim=128, hidden=512, inter=1024).cuda(), cfg.to_modifier(mode="kernel"))
    ids = torch.randint(0, model.config.vocab_size, (1, 24), generator=torch.Generator().manual_seed(2)).cuda()
    outs = []
    for pol in ("none", policy):
        dec = FusedLlamaDecoder(model, 1, 64, kv_bits=8, l2_warm=pol)
        dec.prefill(ids)
        dec.capture()
        logits = []
        for _ in range(12):
            dec.step()
            logits.append(dec.logits.clone())
        dec.check_device_errors()
        outs.append((dec.history[:, :40].clone(), torch.stack(logits)))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    with pytest.raises(ValueError, match="l2_warm"):
        FusedLlamaDecoder(model, 1, 64, kv_bits=8, l2_warm="everything")
