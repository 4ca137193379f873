"""model.bin written from GPU-resident kernel modules is byte-identical to the file the
reference's save_packed_model wrote for the same weights (tests/golden/file_format.npz),
and loads back bit-exactly."""

import numpy as np
import pytest
import torch

from gpu_util import bf16_from_bits, bits_of
from llmquant_b200.core import QuantizationArgs, QuantizationScheme, preset_name_to_scheme

pytestmark = pytest.mark.gpu


class Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.proj = torch.nn.Linear(256, 32, bias=False)
        self.head = torch.nn.Linear(256, 16, bias=True)
        self.norm = torch.nn.LayerNorm(8)
        self.register_buffer("inv_freq", torch.arange(4, dtype=torch.float32) / 7, persistent=False)


def _tiny(blob):
    from llmquant_b200.quantizers import KernelQuantLinear

    model = Tiny().to(torch.bfloat16)
    model.proj.weight.data = bf16_from_bits(blob["tiny_proj_w"], "cpu")
    model.head.weight.data = bf16_from_bits(blob["tiny_head_w"], "cpu")
    model.head.bias.data = bf16_from_bits(blob["tiny_head_b"], "cpu")
    model.norm.weight.data = bf16_from_bits(blob["tiny_norm_w"], "cpu")
    model.norm.bias.data = bf16_from_bits(blob["tiny_norm_b"], "cpu")
    model = model.cuda()

    def w(bits):
        return QuantizationScheme(
            weights=QuantizationArgs(num_bits=bits, strategy="group", group_size=128),
            input_activations=None)

    model.proj = KernelQuantLinear.from_linear(model.proj, w(4))
    model.head = KernelQuantLinear.from_linear(model.head, w(8))
    return model


def test_saved_file_is_byte_identical_to_the_reference(golden, tmp_path):
    from llmquant_b200.packing import read_packed, save_packed_model
    from llmquant_b200.packing.model_io import build_quant_linear

    blob = golden("file_format")
    model = _tiny(blob)
    path = save_packed_model(model, tmp_path / "tiny.bin", "test/model", kv_cache_bits=8)
    assert path.read_bytes() == bytes(blob["tiny_file"])

    tensors, meta = read_packed(path)
    for name in ("proj", "head"):
        rebuilt = build_quant_linear(meta["layers"][name], tensors[f"{name}.qweight"],
                                     tensors[f"{name}.wscale"], tensors.get(f"{name}.bias"), "cuda")
        original = getattr(model, name)
        assert torch.equal(rebuilt.codes, original.codes)
        assert torch.equal(rebuilt.scale_tiles, original.scale_tiles)
        assert torch.equal(rebuilt.qweight, original.qweight)
        x = torch.randn(2, 256, device="cuda", dtype=torch.bfloat16)
        assert torch.equal(rebuilt(x), original(x))


@pytest.mark.parametrize("name", ["W4A16", "W8A16"])
def test_a_quantized_layer_round_trips_bit_exactly(tmp_path, name):
    from llmquant_b200.packing import read_packed, save_packed_model, unpack_weight
    from llmquant_b200.quantizers import KernelQuantLinear

    torch.manual_seed(0)
    linear = torch.nn.Linear(512, 128, bias=False).cuda().to(torch.bfloat16)
    module = KernelQuantLinear.from_linear(linear, preset_name_to_scheme(name))
    model = torch.nn.Module()
    model.proj = module
    path = save_packed_model(model, tmp_path / "layer.bin", "test/model")
    tensors, meta = read_packed(path)
    assert set(tensors) == {"proj.qweight", "proj.wscale"}
    bits = meta["layers"]["proj"]["weights"]["num_bits"]
    restored = unpack_weight(tensors["proj.qweight"], bits).reshape(
        meta["layers"]["proj"]["canonical_shape"])
    assert torch.equal(restored.cuda(), module.qweight)
    assert module.qweight.dtype == torch.int8 and module.qweight.shape[-1] == 128
    if bits == 4:
        assert module.qweight.min() >= -8 and module.qweight.max() <= 7
        assert module.codes.numel() * 2 == module.qweight.numel()  # true nibbles in HBM
