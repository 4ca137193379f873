"""The numpy oracle against the fixtures the reference itself produced (tests/golden/).

Equalities, not tolerances, for everything that is integer, byte or scale arithmetic; the
fp32 group matmul is compared to 1e-6 rel-L2 because BLAS libraries order fp32 sums
differently.
"""

import json

import numpy as np
import pytest

import oracle


def _index(blob):
    return json.loads(bytes(blob["index"]).decode())


def _as_f32(a, dtype):
    if dtype == "bf16":
        return oracle.bf16_bits_to_f32(a)
    return np.asarray(a, dtype=np.float32)


def test_known_answers(golden):
    kat = golden("kat")
    assert oracle.pack_int4(kat["nibble_in"])[0, 0] == 0xD5 == kat["nibble_out"][0, 0]
    assert np.array_equal(oracle.pack_int4(kat["all16_in"]), kat["all16_packed"])
    assert np.array_equal(oracle.unpack_int4(kat["all16_packed"]), kat["all16_in"])
    q = oracle.quantize(kat["ties_in"], np.float32(1.0), 8)
    assert q.tolist() == [0.0, 2.0, 2.0, -0.0] == kat["ties_out"].tolist()
    scale = oracle.compute_scale(kat["truediv_in"], 4, 128)
    assert scale.view(np.uint32).tolist() == kat["truediv_scale"].view(np.uint32).tolist()


def test_fake_quantize_bit_exact(golden):
    blob = golden("fake_quant")
    for case in _index(blob):
        key, dt = case["key"], case["dtype"]
        x = _as_f32(blob[key + "_x"], dt)
        want = _as_f32(blob[key + "_y"], dt)
        got = oracle.fake_quantize(x, case["bits"], case["group"], dtype=dt)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), key
        scale = oracle.compute_scale(x, case["bits"], case["group"])[..., 0]
        assert np.array_equal(scale.view(np.uint32), blob[key + "_s"].view(np.uint32)), key


@pytest.mark.parametrize("name", ["plain8", "plain4", "oproj8", "oproj4", "qproj8", "tail4"])
def test_weight_codes_scales_and_packed_bytes(golden, name):
    blob = golden("linear")
    spec = next(c for c in _index(blob) if c["name"] == name)
    w = oracle.bf16_bits_to_f32(blob[f"{name}_w"])
    kw = dict(head_dim=spec.get("head_dim"), out_group=spec.get("out_group"))
    q, scale = oracle.quantize_weight(w, spec["bits"], 128, **kw)
    assert np.array_equal(q, blob[f"{name}_q"])
    assert list(scale.shape) == blob[f"{name}_scale_raw_shape"].tolist()
    canonical, wscale = oracle.canonical_weight(w, spec["bits"], 128, **kw)
    assert np.array_equal(canonical, blob[f"{name}_canonical"])
    assert np.array_equal(wscale.view(np.uint32), blob[f"{name}_wscale"].view(np.uint32))
    packed = oracle.pack_weight(canonical, spec["bits"])
    assert packed.dtype == blob[f"{name}_packed"].dtype
    assert np.array_equal(packed, blob[f"{name}_packed"])
    assert np.array_equal(oracle.unpack_weight(packed, spec["bits"]), canonical)


@pytest.mark.parametrize("name", ["plain8", "plain4", "oproj8", "oproj4", "qproj8", "tail4"])
@pytest.mark.parametrize("M", [1, 4])
@pytest.mark.parametrize("act", [16, 8])
def test_real_linear_matches_reference(golden, name, M, act):
    blob = golden("linear")
    spec = next(c for c in _index(blob) if c["name"] == name)
    w = oracle.bf16_bits_to_f32(blob[f"{name}_w"])
    kw = dict(head_dim=spec.get("head_dim"), out_group=spec.get("out_group"))
    q, scale = oracle.quantize_weight(w, spec["bits"], 128, **kw)
    x = oracle.bf16_bits_to_f32(blob[f"{name}_x{M}"])
    got = oracle.real_linear(x, q, scale, spec["bits"], 128, act_bits=None if act == 16 else 8, **kw)
    want = blob[f"{name}_y{M}_a{act}_f32"]
    assert oracle.rel_l2(got, want) < 1e-6
    if act == 8:
        # integer x integer group sums are exact in fp32, so only the final scaling and the
        # cross-group additions could differ -- and they are done in the same order
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    got_bf16 = oracle.f32_to_bf16_bits(got)
    same = (got_bf16 == blob[f"{name}_y{M}_a{act}_bf16"]).mean()
    assert same > 0.98


def test_kv_cache_values(golden):
    blob = golden("kv_cache")
    for bits in (4, 8):
        for hd in (64, 128):
            tag = f"b{bits}_hd{hd}"
            for src, dst, dst2 in (("k", "ck", "ck2"), ("v", "cv", "cv2")):
                x = oracle.bf16_bits_to_f32(blob[f"{tag}_{src}"])
                got = oracle.f32_to_bf16_bits(oracle.kv_fake_quantize(x, bits))
                assert np.array_equal(got, blob[f"{tag}_{dst}"]), tag
                codes, scales = oracle.kv_quantize(x, bits)
                # integer storage cannot keep the sign of a zero, so the dequantized codes are
                # compared by value (-0.0 == 0.0), everything else bit for bit
                again = oracle.round_to_dtype(codes.astype(np.float32) * scales[..., :1], "bf16")
                stored = oracle.bf16_bits_to_f32(blob[f"{tag}_{dst}"])
                assert np.array_equal(again, stored), tag
                nonzero = stored != 0
                assert np.array_equal(oracle.f32_to_bf16_bits(again)[nonzero], blob[f"{tag}_{dst}"][nonzero])
                # the second update appends; what was stored is left alone
                x2 = oracle.bf16_bits_to_f32(blob[f"{tag}_{src}2"])
                got2 = oracle.f32_to_bf16_bits(oracle.kv_fake_quantize(x2, bits))
                full = blob[f"{tag}_{dst2}"]
                t = x.shape[2]
                assert np.array_equal(full[:, :, :t], blob[f"{tag}_{dst}"])
                assert np.array_equal(full[:, :, t:], got2)


def test_file_format_bytes(golden):
    blob = golden("file_format")
    meta = json.loads(bytes(blob["meta"]).decode())
    tensors = {
        "packed": ("uint8", blob["t_packed"]), "scale": ("float32", blob["t_scale"]),
        "norm": ("bfloat16", blob["t_norm"]), "codes": ("int8", blob["t_codes"]),
    }
    assert oracle.packed_file_bytes(tensors, meta) == bytes(blob["file_bytes"])
    parsed, parsed_meta = oracle.parse_packed_file(bytes(blob["file_bytes"]))
    assert parsed_meta == meta
    for name, (dtype, array) in tensors.items():
        assert parsed[name][0] == dtype and np.array_equal(parsed[name][1], array)
    with pytest.raises(ValueError, match="not a llmquant weight file"):
        oracle.parse_packed_file(b"SOMETHING" + b"\0" * 64)


def test_config1_full_size(golden):
    """BASELINE config 1: W[8192,2048] seed 0, int8 group 128, x[1,2048] seed 1."""
    import hashlib

    import torch

    blob = golden("config1")
    want = json.loads(bytes(blob["hashes"]).decode())

    def sha(a):
        return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()

    g = torch.Generator().manual_seed(0)
    w_bits = (torch.randn(8192, 2048, generator=g) * 0.02).bfloat16().view(torch.uint16).numpy()
    if sha(w_bits) != want["w_sha"]:
        pytest.skip("torch's CPU generator produced different inputs than when the fixture was made")
    w = oracle.bf16_bits_to_f32(w_bits)
    q, scale = oracle.quantize_weight(w, 8, 128)
    assert sha(q) == want["q_sha"]
    assert sha(scale.reshape(8192, 16)) == want["scale_sha"]
    assert (int(q.min()), int(q.max())) == (want["q_min"], want["q_max"])
    deq = (oracle.group_view(q.astype(np.float32), 128) * scale).reshape(8192, 2048)
    assert sha(deq) == want["dequant_sha"]
    x = oracle.bf16_bits_to_f32(blob["x"])
    y = oracle.real_linear(x, q, scale, 8, 128)
    assert oracle.rel_l2(y, blob["y_f32"]) < 1e-6
    q4, scale4 = oracle.quantize_weight(w, 4, 128)
    assert sha(q4) == want["q4_sha"] and sha(scale4.reshape(8192, 16)) == want["scale4_sha"]
    assert sha(oracle.pack_weight(oracle.group_view(q4, 128), 4)) == want["packed4_sha"]
    assert oracle.rel_l2(oracle.real_linear(x, q4, scale4, 4, 128), blob["y4_f32"]) < 1e-6
