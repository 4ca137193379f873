"""Generate tests/golden/*.npz by running the REFERENCE implementation on CPU.

Run once, where the reference checkout is available:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/llm-quant

The fixtures hold inputs and the reference's outputs, so the tests never need the reference
again. bfloat16 tensors are stored as uint16 bit patterns. Nothing here is imported by the
package or by the tests; it is the provenance of the fixtures.
"""

import hashlib
import json
import pathlib
import sys
import types

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent


def bits_of(t):
    """torch tensor -> numpy, bfloat16 as uint16 bit patterns."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy().copy()
    return t.numpy().copy()


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def seeded(shape, seed, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


def main(ref_root):
    sys.path.insert(0, ref_root)
    sys.dont_write_bytecode = True
    from llmquant.core.observers import compute_scale, group_view
    from llmquant.core.quant_ops import fake_quantize, quantize
    from llmquant.core.scheme import QuantizationArgs, QuantizationScheme
    from llmquant.packing import pack_int4, pack_weight, unpack_int4, write_packed
    from llmquant.quantizers.fake import FakeQuantCache
    from llmquant.quantizers.real import RealQuantLinear, quantize_weight

    def wargs(bits, **kw):
        return QuantizationArgs(num_bits=bits, strategy="group", group_size=128, **kw)

    # ------------------------------------------------------------------ known answers
    kat = {}
    kat["nibble_in"] = np.array([[-3, 5]], dtype=np.int8)
    kat["nibble_out"] = bits_of(pack_int4(torch.tensor([[-3, 5]], dtype=torch.int8)))
    allv = torch.arange(-8, 8, dtype=torch.int8).repeat(4, 1)
    kat["all16_in"] = bits_of(allv)
    kat["all16_packed"] = bits_of(pack_int4(allv))
    kat["all16_unpacked"] = bits_of(unpack_int4(pack_int4(allv)))
    a8 = QuantizationArgs(num_bits=8, strategy="group", group_size=128, dynamic=True)
    ties = torch.tensor([0.5, 1.5, 2.5, -0.5])
    kat["ties_in"] = bits_of(ties)
    kat["ties_out"] = bits_of(quantize(ties, torch.tensor(1.0), a8))
    x = torch.zeros(1, 128)
    x[0, 0] = 6.2982625961
    kat["truediv_in"] = bits_of(x)
    kat["truediv_scale"] = bits_of(compute_scale(x, wargs(4)))
    np.savez_compressed(HERE / "kat.npz", **kat)

    # ------------------------------------------------------------------ fake_quantize
    fq = {}
    index = []
    cases = [
        ("single", (16, 128), 128), ("act3d", (2, 7, 256), 128), ("padded100", (4, 100), 128),
        ("padded192", (8, 192), 128), ("g32", (8, 256), 32), ("g256", (8, 512), 256),
        ("channel", (8, 384), None),
    ]
    for bits in (4, 8):
        for dt_name, dt in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
            for name, shape, gs in cases:
                torch.manual_seed(0)
                xin = (torch.randn(*shape) * 3).to(dt)
                if gs is None:
                    args = QuantizationArgs(num_bits=bits, strategy="channel")
                else:
                    args = QuantizationArgs(num_bits=bits, strategy="group", group_size=gs)
                key = f"{name}_{dt_name}_b{bits}"
                fq[key + "_x"] = bits_of(xin) if dt != torch.float16 else xin.numpy()
                out = fake_quantize(xin, args)
                fq[key + "_y"] = bits_of(out) if dt != torch.float16 else out.numpy()
                fq[key + "_s"] = bits_of(compute_scale(xin, args).squeeze(-1))
                index.append({"key": key, "dtype": dt_name, "bits": bits, "group": gs})
    edge = {
        "zeros": torch.zeros(4, 128), "tiny": torch.full((4, 128), 1e-9),
        "huge": torch.full((4, 128), 3e38),
        "ties": torch.arange(512.0).reshape(4, 128) - 256 + 0.5,
    }
    for name, xin in edge.items():
        key = f"edge_{name}_f32_b8"
        fq[key + "_x"] = bits_of(xin)
        fq[key + "_y"] = bits_of(fake_quantize(xin, wargs(8)))
        fq[key + "_s"] = bits_of(compute_scale(xin, wargs(8)).squeeze(-1))
        index.append({"key": key, "dtype": "f32", "bits": 8, "group": 128})
    fq["index"] = np.frombuffer(json.dumps(index).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "fake_quant.npz", **fq)

    # ------------------------------------------------------------------ linear layouts
    lin = {}
    N, K, HD = 96, 512, 64
    layouts = {
        "plain8": dict(bits=8), "plain4": dict(bits=4),
        "oproj8": dict(bits=8, head_dim=HD), "oproj4": dict(bits=4, head_dim=HD),
        "qproj8": dict(bits=8, out_group=HD // 2),  # 96 rows -> 3 blocks of 32
        "tail4": dict(bits=4),  # K not a multiple of 128, see below
    }
    lindex = []
    for name, spec in layouts.items():
        k = 448 if name == "tail4" else K
        w = seeded((N, k), 10, 0.02, torch.bfloat16)
        bits = spec["bits"]
        args = wargs(bits, head_dim=spec.get("head_dim"), out_group=spec.get("out_group"))
        q, scale = quantize_weight(w, args)
        canonical = group_view(q, args.group_size, args.head_dim).contiguous()
        flat_scale = scale.reshape(-1, canonical.shape[1]).contiguous().float()
        lin[f"{name}_w"] = bits_of(w)
        lin[f"{name}_q"] = bits_of(q)
        lin[f"{name}_scale_raw_shape"] = np.array(scale.shape)
        lin[f"{name}_canonical"] = bits_of(canonical)
        lin[f"{name}_wscale"] = bits_of(flat_scale)
        lin[f"{name}_packed"] = bits_of(pack_weight(canonical, bits))
        for M in (1, 4):
            xin = seeded((M, k), 20 + M, 1.0, torch.bfloat16)
            lin[f"{name}_x{M}"] = bits_of(xin)
            for act_bits in (None, 8):
                act = a8 if act_bits else None
                if act is not None and args.head_dim:
                    act = QuantizationArgs(num_bits=8, strategy="group", group_size=128,
                                           dynamic=True, head_dim=args.head_dim)
                scheme = QuantizationScheme(weights=args, input_activations=act)
                layer = RealQuantLinear(q, scale, None, scheme)
                tag = f"{name}_y{M}_a{act_bits or 16}"
                lin[tag + "_bf16"] = bits_of(layer(xin))
                lin[tag + "_f32"] = bits_of(layer(xin.float()))
        lindex.append({"name": name, "k": k, **spec})
    lin["index"] = np.frombuffer(json.dumps(lindex).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "linear.npz", **lin)

    # ------------------------------------------------------------------ KV cache
    kv = {}
    for bits in (4, 8):
        for hd, shape in ((64, (1, 2, 5, 64)), (128, (2, 3, 4, 128))):
            torch.manual_seed(0)
            keys, values = torch.randn(*shape).bfloat16(), torch.randn(*shape).bfloat16()
            cache = FakeQuantCache(bits)
            ck, cv = cache.update(keys, values, 0)
            k2, v2 = torch.randn(*shape[:2], 2, hd).bfloat16(), torch.randn(*shape[:2], 2, hd).bfloat16()
            ck2, cv2 = cache.update(k2, v2, 0)
            tag = f"b{bits}_hd{hd}"
            for nm, t in (("k", keys), ("v", values), ("ck", ck), ("cv", cv), ("k2", k2),
                          ("v2", v2), ("ck2", ck2), ("cv2", cv2)):
                kv[f"{tag}_{nm}"] = bits_of(t)
    np.savez_compressed(HERE / "kv_cache.npz", **kv)

    # ------------------------------------------------------------------ file format
    tensors = {
        "packed": torch.arange(32, dtype=torch.uint8).reshape(4, 8),
        "scale": seeded((4, 2), 3),
        "norm": seeded((16,), 4).to(torch.bfloat16),
        "codes": (torch.arange(21, dtype=torch.int16) - 10).to(torch.int8),
    }
    meta = {"model_id": "test", "layers": {}, "kv_cache_bits": 8}
    path = write_packed(HERE / "_tmp_format.bin", tensors, meta)
    blob = path.read_bytes()
    path.unlink()
    ff = {"file_bytes": np.frombuffer(blob, dtype=np.uint8)}
    for name, t in tensors.items():
        ff["t_" + name] = bits_of(t)
    ff["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)

    # a whole (tiny) model file through the reference's save_packed_model. The reference's
    # KernelQuantLinear resolves its CUDA extension in __init__; there is no GPU here, so
    # the loader is replaced by an empty stand-in (no arithmetic goes through it).
    import llmquant.quantizers.kernel as ref_kernel
    ref_kernel.load_extension = lambda: types.SimpleNamespace(
        wq_gemv=None, wq_gemv_batched=None, wq_gemv_batched_max_rows=lambda: 8)
    from llmquant.packing.model_io import save_packed_model

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.proj = torch.nn.Linear(256, 32, bias=False)
            self.head = torch.nn.Linear(256, 16, bias=True)
            self.norm = torch.nn.LayerNorm(8)
            self.register_buffer("inv_freq", torch.arange(4, dtype=torch.float32) / 7, persistent=False)

    torch.manual_seed(5)
    tiny = Tiny().to(torch.bfloat16)
    ff["tiny_proj_w"] = bits_of(tiny.proj.weight)
    ff["tiny_head_w"] = bits_of(tiny.head.weight)
    ff["tiny_head_b"] = bits_of(tiny.head.bias)
    ff["tiny_norm_w"] = bits_of(tiny.norm.weight)
    ff["tiny_norm_b"] = bits_of(tiny.norm.bias)
    tiny.proj = ref_kernel.KernelQuantLinear.from_linear(
        tiny.proj, QuantizationScheme(weights=wargs(4), input_activations=None))
    tiny.head = ref_kernel.KernelQuantLinear.from_linear(
        tiny.head, QuantizationScheme(weights=wargs(8), input_activations=None))
    path = save_packed_model(tiny, HERE / "_tmp_model.bin", "test/model", kv_cache_bits=8)
    ff["tiny_file"] = np.frombuffer(path.read_bytes(), dtype=np.uint8)
    path.unlink()
    np.savez_compressed(HERE / "file_format.npz", **ff)

    # ------------------------------------------------------------------ config 1 (full size)
    # W[8192, 2048] bf16 ~N(0, 0.02) seed 0, int8 group 128; x[1, 2048] bf16 ~N(0,1) seed 1.
    w = seeded((8192, 2048), 0, 0.02, torch.bfloat16)
    xin = seeded((1, 2048), 1, 1.0, torch.bfloat16)
    args = wargs(8)
    q, scale = quantize_weight(w, args)
    layer = RealQuantLinear(q, scale, None, QuantizationScheme(weights=args, input_activations=None))
    y32 = layer(xin.float())
    deq = (group_view(q.float(), 128) * scale).reshape(8192, 2048)
    c1 = {
        "w_sha": sha(bits_of(w)), "x_sha": sha(bits_of(xin)), "q_sha": sha(bits_of(q)),
        "scale_sha": sha(bits_of(scale.reshape(8192, 16))), "dequant_sha": sha(bits_of(deq)),
        "q_min": int(q.min()), "q_max": int(q.max()),
    }
    args4 = wargs(4)
    q4, scale4 = quantize_weight(w, args4)
    c1["q4_sha"] = sha(bits_of(q4))
    c1["scale4_sha"] = sha(bits_of(scale4.reshape(8192, 16)))
    c1["packed4_sha"] = sha(bits_of(pack_weight(group_view(q4, 128).contiguous(), 4)))
    layer4 = RealQuantLinear(q4, scale4, None, QuantizationScheme(weights=args4, input_activations=None))
    np.savez_compressed(
        HERE / "config1.npz",
        hashes=np.frombuffer(json.dumps(c1).encode(), dtype=np.uint8),
        x=bits_of(xin), y_f32=bits_of(y32), y_bf16=bits_of(layer(xin)),
        y4_f32=bits_of(layer4(xin.float())),
        w_head=bits_of(w[:4]), q_head=bits_of(q[:4]), scale_head=bits_of(scale[:4].reshape(4, 16)),
    )
    print("fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python %s <path to an llm-quant checkout>" % sys.argv[0])
    main(sys.argv[1])
