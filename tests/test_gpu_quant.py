"""GPU parity of the quantizer kernels, through the C ABI, against the golden vectors the
reference produced and against the numpy oracle on larger seeded inputs. Bit-exact."""

import numpy as np
import pytest
import torch

import oracle
from gpu_util import bf16_from_bits, bits_of, index_of, seeded, to_torch
from llmquant_b200.core import QuantizationArgs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fq():
    from llmquant_b200.cuda import fake_quantize_cuda
    return fake_quantize_cuda


def _args(bits, group):
    if group is None:
        return QuantizationArgs(num_bits=bits, strategy="channel")
    return QuantizationArgs(num_bits=bits, strategy="group", group_size=group)


def test_fake_quant_matches_golden_bit_exactly(golden, fq):
    blob = golden("fake_quant")
    for case in index_of(blob):
        key, dt = case["key"], case["dtype"]
        x = to_torch(blob[key + "_x"], dt)
        got, scale = fq(x, _args(case["bits"], case["group"]), return_scale=True)
        assert got.dtype == x.dtype and got.shape == x.shape
        assert np.array_equal(bits_of(got).view(np.uint8), blob[key + "_y"].view(np.uint8)), key
        assert np.array_equal(bits_of(scale).view(np.uint32).reshape(-1),
                              blob[key + "_s"].view(np.uint32).reshape(-1)), key


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("shape", [(2048, 2048), (512, 2048), (2048, 8192), (2, 7, 2048)])
def test_fake_quant_matches_oracle_at_layer_sizes(fq, bits, dtype, shape):
    tdt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    x = (seeded(shape, 0) * 3).to(tdt)
    got, scale = fq(x.cuda(), _args(bits, 128), return_scale=True)
    want = oracle.fake_quantize(x.float().numpy(), bits, 128, dtype=dtype)
    assert np.array_equal(got.float().cpu().numpy().view(np.uint32), want.view(np.uint32))
    want_scale = oracle.compute_scale(x.float().numpy(), bits, 128)[..., 0]
    assert np.array_equal(bits_of(scale).view(np.uint32), want_scale.view(np.uint32))


@pytest.mark.parametrize("group", [32, 128, 256, 2048, 20])
def test_fake_quant_other_group_sizes(fq, group):
    k = 2048 if group != 20 else 200
    x = seeded((64, k), 0).bfloat16()
    got = fq(x.cuda(), _args(4, group))
    want = oracle.fake_quantize(x.float().numpy(), 4, group, dtype="bf16")
    assert np.array_equal(got.float().cpu().numpy(), want)


def test_fake_quant_non_contiguous_padded_empty_and_errors(fq):
    args = _args(8, 128)
    x = seeded((128, 64), 0).bfloat16().cuda().t()
    assert not x.is_contiguous()
    want = oracle.fake_quantize(x.float().cpu().numpy(), 8, 128, dtype="bf16")
    assert np.array_equal(fq(x, args).float().cpu().numpy(), want)
    for shape in [(4, 100), (2, 3, 64), (8, 192)]:
        x = seeded(shape, 1).bfloat16()
        want = oracle.fake_quantize(x.float().numpy(), 8, 128, dtype="bf16")
        assert np.array_equal(fq(x.cuda(), args).float().cpu().numpy(), want), shape
    empty = fq(torch.empty(0, 128, device="cuda"), args)
    assert empty.shape == (0, 128)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        fq(torch.randn(4, 128), args)
    with pytest.raises(RuntimeError, match="float32, float16 or bfloat16"):
        fq(torch.randn(4, 128, device="cuda").double(), args)


def test_quantize_group_codes_are_bit_exact():
    """The code-emitting variant (activation / KV quantizer): int8 codes and fp32 scales."""
    from llmquant_b200 import native

    for bits in (4, 8):
        for shape in [(3, 5, 128), (64, 2048), (7, 64)]:
            x = seeded(shape, bits).bfloat16().cuda()
            gs = min(128, shape[-1])
            groups = x.numel() // gs
            codes = torch.empty(x.shape, dtype=torch.int8, device="cuda")
            scales = torch.empty(groups, dtype=torch.float32, device="cuda")
            native.call("lq_quantize_group_i8", x.data_ptr(), codes.data_ptr(), scales.data_ptr(),
                        groups, gs, bits, native.LQ_BF16, native.stream_ptr())
            xf = x.float().cpu().numpy()
            want_scale = oracle.compute_scale(xf, bits, gs)
            want_codes = oracle.ungroup(
                oracle.quantize(oracle.group_view(xf, gs), want_scale, bits), xf.shape, gs)
            assert np.array_equal(codes.cpu().numpy(), want_codes.astype(np.int8))
            assert np.array_equal(scales.cpu().numpy().view(np.uint32),
                                  want_scale.reshape(-1).view(np.uint32))


@pytest.mark.parametrize("name", ["plain8", "plain4", "oproj8", "oproj4", "qproj8", "tail4"])
def test_weight_quantizer_codes_scales_and_packed_bytes(golden, name):
    from llmquant_b200.packing import pack_weight, unpack_weight
    from llmquant_b200.quantizers import quantize_weight_canonical

    blob = golden("linear")
    spec = next(c for c in index_of(blob) if c["name"] == name)
    args = QuantizationArgs(num_bits=spec["bits"], strategy="group", group_size=128,
                            head_dim=spec.get("head_dim"), out_group=spec.get("out_group"))
    for dt in (torch.bfloat16, torch.float32):
        w = bf16_from_bits(blob[f"{name}_w"]).to(dt)
        canonical, wscale = quantize_weight_canonical(w, args)
        assert np.array_equal(canonical.cpu().numpy(), blob[f"{name}_canonical"])
        assert np.array_equal(bits_of(wscale).view(np.uint32), blob[f"{name}_wscale"].view(np.uint32))
    packed = pack_weight(canonical, spec["bits"])
    assert np.array_equal(packed.cpu().numpy(), blob[f"{name}_packed"])
    assert packed.cpu().numpy().dtype == blob[f"{name}_packed"].dtype
    assert torch.equal(unpack_weight(packed, spec["bits"]), canonical)


def test_config1_codes_scales_dequant_full_size(golden):
    """BASELINE config 1 at full size: hashes of codes, scales, dequantized weights, packed int4."""
    import hashlib
    import json

    from llmquant_b200 import native
    from llmquant_b200.packing import pack_weight
    from llmquant_b200.quantizers import quantize_weight_canonical

    blob = golden("config1")
    want = json.loads(bytes(blob["hashes"]).decode())

    def sha(t):
        return hashlib.sha256(np.ascontiguousarray(bits_of(t)).tobytes()).hexdigest()

    w = seeded((8192, 2048), 0, 0.02, torch.bfloat16)
    if sha(w) != want["w_sha"]:
        pytest.skip("torch's CPU generator produced different inputs than when the fixture was made")
    a8 = QuantizationArgs(num_bits=8, strategy="group", group_size=128)
    canonical, wscale = quantize_weight_canonical(w.cuda(), a8)
    assert sha(canonical.reshape(8192, 2048)) == want["q_sha"]
    assert sha(wscale) == want["scale_sha"]
    deq = torch.empty(8192, 2048, dtype=torch.float32, device="cuda")
    native.call("lq_dequant_weight", canonical.data_ptr(), wscale.data_ptr(), deq.data_ptr(),
                native.LQ_F32, 8192, 16, 128, 0, native.stream_ptr())
    assert sha(deq) == want["dequant_sha"]
    a4 = QuantizationArgs(num_bits=4, strategy="group", group_size=128)
    c4, s4 = quantize_weight_canonical(w.cuda(), a4)
    assert sha(c4.reshape(8192, 2048)) == want["q4_sha"] and sha(s4) == want["scale4_sha"]
    assert sha(pack_weight(c4, 4)) == want["packed4_sha"]
