"""CPU-side checks: the C ABI loads and exports what the header declares; config, targeting
and the file format behave as the reference's do (tests/test_config.py, test_packing.py and
test_quantization.py of the reference are the model for these)."""

import json
import struct

import numpy as np
import pytest
import torch
import torch.nn as nn

from llmquant_b200 import native
from llmquant_b200.core import (
    QuantConfig,
    QuantizationArgs,
    QuantizationModifier,
    preset_name_to_scheme,
)
from llmquant_b200.packing import (
    describe_packed,
    pack_int4,
    pack_weight,
    packed_dtypes,
    read_header,
    read_packed,
    unpack_int4,
    unpack_weight,
    write_packed,
)
from llmquant_b200.packing.format import ALIGNMENT, MAGIC


def test_library_exports_every_declared_symbol():
    lib = native.library()
    declared = native.declared_symbols()
    assert "lq_wq_gemv_stream" in declared and "lq_fake_quant_group" in declared
    for name in declared:
        assert hasattr(lib, name), name
        assert name in native._SIGNATURES, f"{name} has no ctypes signature"
    assert lib.lq_version() >= 1


def test_argument_errors_come_back_as_messages():
    # no GPU work: both calls are rejected by validation before any launch
    with pytest.raises(RuntimeError, match="num_bits must be in"):
        native.call("lq_fake_quant_group", 0, 0, 0, 4, 128, 9, native.LQ_BF16, 0)
    with pytest.raises(RuntimeError, match="multiple of 4"):
        native.call("lq_wq_gemv", 0, 0, 0, 0, 1, 8, 2, 6, 0, native.LQ_BF16, 0)
    with pytest.raises(RuntimeError, match="float32, float16 or bfloat16"):
        native.call("lq_fake_quant_group", 8, 8, 0, 4, 128, 8, 7, 0)
    kd, span, npad = native.stream_layout_sizes(2048, 32, 128, 64, 8)
    assert (kd, span, npad) == (2048, 64, 2048)
    kd, span, npad = native.stream_layout_sizes(10, 16, 128, 0, 4)
    assert (kd, span, npad) == (2048, 128, 12)


def test_decode_gemm_size_arithmetic():
    """Sizes the decode GEMM asks its caller for (host arithmetic, no GPU): the tile-major
    weight is one block of codes + 128 fp32 scales per (128-row tile, 128-code group); the
    workspace is the activation planes (per group 2 * rows_padded plane rows of 128 bytes and
    the units, 128-byte padded) followed by 1..8 fp32 parts of the output."""
    lib = native.library()
    for n, kd in ((4096, 4096), (1000, 1152), (28672, 4096), (128256, 4096)):
        tiles, groups = -(-n // 128), kd // 128
        assert lib.lq_tile_weight_bytes(n, kd, 8) == tiles * groups * (128 * 128 + 512)
        assert lib.lq_tile_weight_bytes(n, kd, 4) == tiles * groups * (128 * 64 + 512)
        last = 0
        for rows in (1, 8, 9, 16, 17, 32, 33, 64):
            padded = next(p for p in (8, 16, 32, 64) if rows <= p)
            planes = groups * (2 * padded * 128 + -(-padded * 4 // 128) * 128)
            planes = -(-planes // 256) * 256
            total = lib.lq_decode_gemm_workspace_bytes(rows, n, kd)
            parts, rest = divmod(total - planes, rows * n * 4)
            assert rest == 0 and 1 <= parts <= 8, (n, kd, rows, total)
            assert total > last
            last = total
    assert lib.lq_decode_gemm_workspace_bytes(0, 4096, 4096) == 0
    assert lib.lq_decode_gemm_workspace_bytes(65, 4096, 4096) == 0


def test_scheme_rules():
    with pytest.raises(ValueError, match="requires a positive group_size"):
        QuantizationArgs(num_bits=4, strategy="group")
    with pytest.raises(ValueError, match="only valid for strategy"):
        QuantizationArgs(num_bits=4, strategy="channel", group_size=128)
    with pytest.raises(ValueError):
        preset_name_to_scheme("W3A8")
    w4a8 = preset_name_to_scheme("w4a8")
    assert w4a8.weights.num_bits == 4 and w4a8.input_activations.dynamic
    assert preset_name_to_scheme("W8A16").input_activations is None


def test_config_validation_and_modifier():
    for field in ("kv_cache", "head_weight", "activation"):
        with pytest.raises(ValueError, match="only"):
            QuantConfig(**{field: "int4"})
    with pytest.raises(ValueError, match="unknown dtype"):
        QuantConfig(attn_weight="int3")
    cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    assert cfg.kv_cache_bits == 8
    assert cfg.describe() == "attn-int8_mlp-int4_head-int8_act-bf16_kv-int8_g128"
    mod = cfg.to_modifier(mode="kernel")
    mod.head_dim = 64
    o = mod.scheme_for("model.layers.0.self_attn.o_proj")
    q = mod.scheme_for("model.layers.0.self_attn.q_proj")
    down = mod.scheme_for("model.layers.3.mlp.down_proj")
    assert o.weights.head_dim == 64 and o.weights.out_group is None
    assert q.weights.out_group == 64 and q.weights.head_dim is None
    assert down.weights.num_bits == 4 and mod.scheme_for("lm_head").weights.num_bits == 8
    assert mod.scheme_for("model.embed_tokens") is None
    assert QuantConfig().to_modifier().scheme_for("model.layers.0.mlp.up_proj") is None
    with pytest.raises(ValueError, match="unsupported mode"):
        QuantizationModifier(scheme="W4A16", mode="fake").apply(nn.Linear(4, 4))


def test_nibble_codec_on_host(golden):
    kat = golden("kat")
    assert int(pack_int4(torch.tensor([[-3, 5]], dtype=torch.int8))[0, 0]) == 0xD5
    values = torch.from_numpy(kat["all16_in"])
    assert np.array_equal(pack_int4(values).numpy(), kat["all16_packed"])
    assert torch.equal(unpack_int4(pack_int4(values)), values)
    assert pack_weight(values, 4).numel() * 2 == values.numel()
    assert torch.equal(unpack_weight(pack_weight(values, 8), 8), values)
    for bad in (9, -9):
        with pytest.raises(ValueError, match=r"must be in \[-8, 7\]"):
            pack_int4(torch.tensor([[bad, 0]], dtype=torch.int8))
    with pytest.raises(ValueError, match="must be even"):
        pack_int4(torch.zeros(1, 3, dtype=torch.int8))
    for bits in (2, 16):
        with pytest.raises(ValueError, match="unsupported num_bits"):
            pack_weight(torch.zeros(2, 2, dtype=torch.int8), bits)


def test_file_bytes_equal_the_reference_writer(golden, tmp_path):
    blob = golden("file_format")
    meta = json.loads(bytes(blob["meta"]).decode())
    tensors = {
        "packed": torch.from_numpy(blob["t_packed"]),
        "scale": torch.from_numpy(blob["t_scale"]),
        "norm": torch.from_numpy(blob["t_norm"]).view(torch.bfloat16),
        "codes": torch.from_numpy(blob["t_codes"]),
    }
    path = write_packed(tmp_path / "w.bin", tensors, meta)
    assert path.read_bytes() == bytes(blob["file_bytes"])
    restored, got_meta = read_packed(path)
    assert got_meta == meta
    for name, tensor in tensors.items():
        assert restored[name].dtype == tensor.dtype and torch.equal(restored[name], tensor), name
    for entry in read_header(path)["tensors"].values():
        assert entry["offset"] % ALIGNMENT == 0


def test_foreign_and_future_files_are_rejected(tmp_path):
    bad = tmp_path / "not-ours.bin"
    bad.write_bytes(b"SOMETHING" + b"\0" * 64)
    with pytest.raises(ValueError, match="not a llmquant weight file"):
        read_header(bad)
    header = json.dumps({"version": 999, "meta": {}, "tensors": {}}).encode()
    future = tmp_path / "future.bin"
    future.write_bytes(MAGIC + struct.pack("<Q", len(header)) + header)
    with pytest.raises(ValueError, match="unsupported file version"):
        read_header(future)


def test_reference_written_model_file_is_readable(golden, tmp_path):
    """A model.bin written by the reference's save_packed_model parses here."""
    blob = golden("file_format")
    path = tmp_path / "tiny.bin"
    path.write_bytes(bytes(blob["tiny_file"]))
    tensors, meta = read_packed(path)
    assert set(meta["layers"]) == {"proj", "head"}
    assert meta["layers"]["proj"]["canonical_shape"] == [32, 2, 128]
    assert tensors["proj.qweight"].dtype == torch.uint8 and tensors["proj.qweight"].shape == (32, 2, 64)
    assert tensors["head.qweight"].dtype == torch.int8
    assert meta["non_persistent_buffers"] == ["inv_freq"] and tensors["inv_freq"].dtype == torch.bfloat16
    assert packed_dtypes(path)["kv_cache"] == "int8"
    assert describe_packed(path)["quantized_layers"] == 2
    w = torch.from_numpy(blob["tiny_norm_w"]).view(torch.bfloat16)
    assert torch.equal(tensors["norm.weight"], w)


def test_kernel_module_refuses_cpu_tensors():
    from llmquant_b200.quantizers import KernelQuantLinear

    with pytest.raises(RuntimeError, match="no CPU fallback"):
        KernelQuantLinear.from_linear(nn.Linear(128, 8, bias=False), preset_name_to_scheme("W8A16"))
    with pytest.raises(ValueError, match="needs a weight scheme"):
        from llmquant_b200.core import QuantizationScheme
        KernelQuantLinear.from_linear(nn.Linear(128, 8), QuantizationScheme(None, None))
    if not torch.cuda.is_available():
        from llmquant_b200.cuda import load_extension
        with pytest.raises(RuntimeError, match="CUDA is not available"):
            load_extension()
