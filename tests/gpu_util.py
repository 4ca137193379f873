"""Helpers shared by the GPU parity tests (they run on the B200 box, never on CPU)."""

import json

import numpy as np
import torch


def index_of(blob):
    return json.loads(bytes(blob["index"]).decode())


def bf16_from_bits(bits, device="cuda"):
    return torch.from_numpy(np.ascontiguousarray(bits)).view(torch.bfloat16).to(device)


def to_torch(array, dtype_name, device="cuda"):
    if dtype_name == "bf16":
        return bf16_from_bits(array, device)
    return torch.from_numpy(np.ascontiguousarray(array)).to(device)


def bits_of(t):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy()
    return t.numpy()


def rel_l2(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def seeded(shape, seed, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)
