"""numpy restatement of the reference's quantization arithmetic. TEST INFRASTRUCTURE ONLY.

Each function names the reference file:line it follows (paths inside pjh5672/llm-quant).
All floating point is IEEE binary32 with true division and round-half-to-even, which is
what numpy's float32 `/` and `np.rint` do; bfloat16 travels as uint16 bit patterns.

Parity status: pinned by tests/golden/ (generated from the reference itself).
"""

import json
import struct

import numpy as np

__all__ = [
    "SCALE_EPS", "bf16_bits_to_f32", "f32_to_bf16_bits", "f32_to_f16", "round_to_dtype",
    "pad_to_group", "group_view", "ungroup", "compute_scale", "quantize", "fake_quantize",
    "quantize_weight", "canonical_weight", "pack_int4", "unpack_int4", "pack_weight",
    "unpack_weight", "real_linear", "pad_activation", "kv_quantize", "kv_fake_quantize",
    "packed_file_bytes", "parse_packed_file", "rel_l2",
]

# core/observers.py:5
SCALE_EPS = np.float32(1e-8)


# --------------------------------------------------------------------------- dtypes
def bf16_bits_to_f32(bits):
    """uint16 bfloat16 patterns -> float32 (exact)."""
    bits = np.asarray(bits, dtype=np.uint16)
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x):
    """float32 -> bfloat16 bit patterns, round-to-nearest-even (torch's `.to(bfloat16)`)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    rounding = ((u >> 16) & 1) + np.uint32(0x7FFF)
    out = ((u + rounding) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def f32_to_f16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16)


def round_to_dtype(x, dtype):
    """Round a float32 array to `dtype` ("f32" | "f16" | "bf16") and come back to float32."""
    if dtype == "f32":
        return np.asarray(x, dtype=np.float32)
    if dtype == "f16":
        return f32_to_f16(x).astype(np.float32)
    if dtype == "bf16":
        return bf16_bits_to_f32(f32_to_bf16_bits(x))
    raise ValueError(dtype)


# --------------------------------------------------------------------------- grouping
def pad_to_group(x, group_size):
    """core/observers.py:8-20 -- zero-pad the last axis to a whole number of groups."""
    rem = x.shape[-1] % group_size
    if not rem:
        return x
    widths = [(0, 0)] * (x.ndim - 1) + [(0, group_size - rem)]
    return np.pad(x, widths)


def group_view(x, group_size, head_dim=None):
    """core/observers.py:23-43 -- [..., K] -> [..., G, group_size]; per head if head_dim."""
    if head_dim is None:
        p = pad_to_group(x, group_size)
        return p.reshape(*p.shape[:-1], p.shape[-1] // group_size, group_size)
    lead, k = x.shape[:-1], x.shape[-1]
    if k % head_dim:
        raise ValueError(f"last dim {k} is not a multiple of head_dim {head_dim}")
    per_head = pad_to_group(x.reshape(*lead, k // head_dim, head_dim), group_size)
    return per_head.reshape(*lead, -1, group_size)


def ungroup(y, shape, group_size, head_dim=None):
    """core/observers.py:46-53 -- undo group_view, dropping the padding."""
    lead, k = tuple(shape[:-1]), shape[-1]
    if head_dim is None:
        return y.reshape(*lead, -1)[..., :k]
    padded_head = -(-head_dim // group_size) * group_size
    per_head = y.reshape(*lead, k // head_dim, padded_head)
    return per_head[..., :head_dim].reshape(*lead, k)


def _out_block_view(x, out_group):
    """core/observers.py:56-68."""
    rem = x.shape[0] % out_group
    if rem:
        x = np.pad(x, [(0, out_group - rem)] + [(0, 0)] * (x.ndim - 1))
    return x.reshape(-1, out_group, *x.shape[1:])


# --------------------------------------------------------------------------- scale / codes
def compute_scale(x, num_bits, group_size=None, head_dim=None, out_group=None):
    """core/observers.py:74-98 -- symmetric abs-max scale, fp32, true division, eps floor.

    group_size None means one group spanning the last axis ("channel"/"token").
    Returns [..., G, 1] (or [N/out_group, 1, G, 1] with out_group).
    """
    qmax = np.float32(2 ** (num_bits - 1) - 1)
    xf = np.asarray(x, dtype=np.float32)
    if group_size is None:
        amax = np.abs(xf).max(axis=-1, keepdims=True)
    else:
        view = group_view(xf, group_size, head_dim)
        if out_group:
            amax = np.abs(_out_block_view(view, out_group)).max(axis=(1, -1), keepdims=True)
        else:
            amax = np.abs(view).max(axis=-1, keepdims=True)
    return np.maximum((amax / qmax).astype(np.float32), SCALE_EPS)


def quantize(x, scale, num_bits):
    """core/quant_ops.py:13-19 -- clamp(rint(x / scale), -qmax-1, qmax), integer-valued fp32."""
    qmax = 2 ** (num_bits - 1) - 1
    with np.errstate(over="ignore", invalid="ignore"):
        q = np.rint(np.asarray(x, dtype=np.float32) / np.asarray(scale, dtype=np.float32))
    return np.clip(q, -qmax - 1, qmax).astype(np.float32)


def fake_quantize(x, num_bits, group_size=None, head_dim=None, out_group=None, dtype="f32"):
    """core/quant_ops.py:26-37 -- quantize-dequantize; result rounded to `dtype`, as float32."""
    x = np.asarray(x, dtype=np.float32)
    scale = compute_scale(x, num_bits, group_size, head_dim, out_group)
    if group_size is None:
        return round_to_dtype(quantize(x, scale, num_bits) * scale, dtype)
    view = group_view(x, group_size, head_dim)
    if out_group:
        blocked = _out_block_view(view, out_group)
        out = (quantize(blocked, scale, num_bits) * scale).reshape(-1, *view.shape[1:])[: x.shape[0]]
    else:
        out = quantize(view, scale, num_bits) * scale
    return round_to_dtype(ungroup(out, x.shape, group_size, head_dim), dtype)


def quantize_weight(w, num_bits, group_size=128, head_dim=None, out_group=None):
    """quantizers/real.py:29-47 -- int8 codes in [out, in] plus the fp32 scales."""
    w = np.asarray(w, dtype=np.float32)
    scale = compute_scale(w, num_bits, group_size, head_dim, out_group)
    grouped = group_view(w, group_size, head_dim)
    if out_group:
        blocked = _out_block_view(grouped, out_group)
        q = quantize(blocked, scale, num_bits).reshape(-1, *grouped.shape[1:])[: w.shape[0]]
    else:
        q = quantize(grouped, scale, num_bits)
    q = ungroup(q, w.shape, group_size, head_dim)
    return q.astype(np.int8), scale


def canonical_weight(w, num_bits, group_size=128, head_dim=None, out_group=None):
    """quantizers/kernel.py:56-66 -- canonical [N, G, gs] int8 and [scale_rows, G] fp32."""
    q, scale = quantize_weight(w, num_bits, group_size, head_dim, out_group)
    canonical = np.ascontiguousarray(group_view(q, group_size, head_dim))
    flat_scale = np.ascontiguousarray(scale.reshape(-1, canonical.shape[1]).astype(np.float32))
    return canonical, flat_scale


# --------------------------------------------------------------------------- packing
def pack_int4(values):
    """packing/packing.py:20-32 -- (v+8) nibbles, even index low, odd index high."""
    values = np.asarray(values)
    if values.shape[-1] % 2:
        raise ValueError(f"last dim {values.shape[-1]} must be even to pack into nibbles")
    if values.size and (values.min() < -8 or values.max() > 7):
        raise ValueError(
            f"values must be in [-8, 7], got [{int(values.min())}, {int(values.max())}]"
        )
    biased = (values.astype(np.int16) + 8).astype(np.uint8)
    return np.ascontiguousarray(biased[..., 0::2] | (biased[..., 1::2] << 4))


def unpack_int4(packed):
    """packing/packing.py:35-40."""
    packed = np.asarray(packed, dtype=np.uint8)
    low = (packed & 0x0F).astype(np.int16) - 8
    high = ((packed >> 4) & 0x0F).astype(np.int16) - 8
    out = np.stack((low, high), axis=-1)
    return out.reshape(*packed.shape[:-1], -1).astype(np.int8)


def pack_weight(q, num_bits):
    """packing/packing.py:43-49."""
    if num_bits == 8:
        return np.ascontiguousarray(q)
    if num_bits == 4:
        return pack_int4(q)
    raise ValueError(f"unsupported num_bits {num_bits}, expected 4 or 8")


def unpack_weight(stored, num_bits):
    """packing/packing.py:52-57."""
    if num_bits == 8:
        return np.asarray(stored).astype(np.int8)
    if num_bits == 4:
        return unpack_int4(stored)
    raise ValueError(f"unsupported num_bits {num_bits}, expected 4 or 8")


# --------------------------------------------------------------------------- the linear
def pad_activation(flat, group_size, head_dim=None):
    """quantizers/kernel.py:17-25 -- pad x the way the weight's K axis was padded."""
    if head_dim:
        lead, k = flat.shape[:-1], flat.shape[-1]
        per_head = pad_to_group(flat.reshape(*lead, k // head_dim, head_dim), group_size)
        return per_head.reshape(*lead, -1)
    return pad_to_group(flat, group_size)


def real_linear(x, q, scale, num_bits, group_size=128, head_dim=None, out_group=None,
                act_bits=None, bias=None, out_dtype="f32"):
    """quantizers/real.py:76-103 -- RealQuantLinear.forward.

    x [M, K] float32 (already holding whatever dtype's values), q [N, K] int8 codes,
    scale as returned by quantize_weight. Per reduction group, in order: fp32 matmul of the
    integer-valued operands, times the weight scale (times the activation scale when
    act_bits is set: dynamic per-token per-group, same group size), accumulated in fp32.
    """
    x = np.asarray(x, dtype=np.float32)
    n_out = q.shape[0]
    wg = group_view(q.astype(np.float32), group_size, head_dim)  # [N, G, gs]
    if act_bits is None:
        xg = group_view(x, group_size, head_dim)
        act_scale = None
    else:
        act_scale = compute_scale(x, act_bits, group_size, head_dim)  # [M, G, 1]
        xg = quantize(group_view(x, group_size, head_dim), act_scale, act_bits)
    out = np.zeros((x.shape[0], n_out), dtype=np.float32)
    for g in range(wg.shape[1]):
        partial = (xg[:, g] @ wg[:, g].T).astype(np.float32)
        if out_group:
            ws = np.repeat(scale[:, 0, g, 0], out_group)[:n_out]
        else:
            ws = scale[:, g, 0]
        partial = partial * ws
        if act_scale is not None:
            partial = partial * act_scale[:, g]
        out += partial
    if bias is not None:
        out = out + np.asarray(bias, dtype=np.float32)
    return round_to_dtype(out, out_dtype)


# --------------------------------------------------------------------------- KV cache
def kv_quantize(states, num_bits=8, group_size=128):
    """quantizers/fake.py:46-55 -- what FakeQuantCache.update does to new K or V.

    states [..., head_dim] float32. The group is 128 over head_dim (a shorter head is one
    zero-padded group, i.e. one scale per token per head). Returns (codes int8
    [..., head_dim], scales fp32 [..., ceil(head_dim/group)]).
    """
    states = np.asarray(states, dtype=np.float32)
    scale = compute_scale(states, num_bits, group_size)
    q = quantize(group_view(states, group_size), scale, num_bits)
    codes = ungroup(q, states.shape, group_size).astype(np.int8)
    return codes, scale[..., 0]


def kv_fake_quantize(states, num_bits=8, group_size=128, dtype="bf16"):
    """The value the reference cache stores: dtype(q * scale) (core/quant_ops.py:36-37)."""
    return fake_quantize(states, num_bits, group_size, dtype=dtype)


# --------------------------------------------------------------------------- file format
_NP_OF = {"uint8": np.uint8, "int8": np.int8, "float32": np.float32, "bfloat16": np.uint16}


def packed_file_bytes(tensors, meta):
    """packing/format.py:65-93 -- the bytes write_packed produces.

    `tensors` maps name -> (dtype_name, ndarray); bfloat16 arrays are uint16 bit patterns.
    Blobs are 64-byte aligned relative to the start of the data section.
    """
    entries, blobs, offset = {}, [], 0
    for name, (dtype_name, array) in tensors.items():
        payload = np.ascontiguousarray(array, dtype=_NP_OF[dtype_name]).tobytes()
        padding = -offset % 64
        if padding:
            blobs.append(b"\0" * padding)
            offset += padding
        entries[name] = {"dtype": dtype_name, "shape": list(array.shape), "offset": offset,
                         "nbytes": len(payload)}
        blobs.append(payload)
        offset += len(payload)
    header = json.dumps({"version": 1, "meta": meta, "tensors": entries}).encode("utf-8")
    return b"LLMQUANT" + struct.pack("<Q", len(header)) + header + b"".join(blobs)


def parse_packed_file(blob):
    """packing/format.py:96-118 -- (tensors, meta) from file bytes."""
    if blob[:8] != b"LLMQUANT":
        raise ValueError("not a llmquant weight file")
    (length,) = struct.unpack("<Q", blob[8:16])
    header = json.loads(blob[16:16 + length].decode("utf-8"))
    if header["version"] != 1:
        raise ValueError(f"unsupported file version {header['version']}, expected 1")
    data = memoryview(blob)[16 + length:]
    tensors = {}
    for name, e in header["tensors"].items():
        raw = data[e["offset"]: e["offset"] + e["nbytes"]]
        tensors[name] = (e["dtype"], np.frombuffer(raw, dtype=_NP_OF[e["dtype"]]).reshape(e["shape"]).copy())
    return tensors, header["meta"]


def rel_l2(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    denom = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / (denom if denom else 1.0))
