"""Nibble codec of the model.bin payload (llmquant/packing/packing.py:16-57).

int8 is stored as is. int4 goes two to a byte: value + 8 (0..15), even index in the low
nibble, odd index in the high one, so (-3, 5) -> 0xD5. CUDA tensors are packed by the
library's kernels; host tensors (file I/O) by the same bit operations in numpy.
"""

import numpy as np
import torch

from llmquant_b200 import native

INT4_BIAS = 8
INT4_MIN, INT4_MAX = -8, 7


def _check_range(values: torch.Tensor):
    if values.shape[-1] % 2:
        raise ValueError(f"last dim {values.shape[-1]} must be even to pack into nibbles")
    if values.numel():
        lo, hi = int(values.min()), int(values.max())
        if lo < INT4_MIN or hi > INT4_MAX:
            raise ValueError(f"values must be in [{INT4_MIN}, {INT4_MAX}], got [{lo}, {hi}]")


def pack_int4(values: torch.Tensor) -> torch.Tensor:
    """[..., n] int8 in -8..7 -> [..., n // 2] uint8."""
    _check_range(values)
    shape = (*values.shape[:-1], values.shape[-1] // 2)
    if values.is_cuda:
        src = values.to(torch.int8).contiguous()
        out = torch.empty(shape, dtype=torch.uint8, device=values.device)
        with torch.cuda.device(values.device):
            native.call("lq_pack_int4", src.data_ptr(), out.data_ptr(), src.numel(),
                        native.stream_ptr(values.device))
        return out
    biased = (values.numpy().astype(np.int16) + INT4_BIAS).astype(np.uint8)
    return torch.from_numpy(np.ascontiguousarray(biased[..., 0::2] | (biased[..., 1::2] << 4)))


def unpack_int4(packed: torch.Tensor) -> torch.Tensor:
    """[..., n // 2] uint8 -> [..., n] int8."""
    shape = (*packed.shape[:-1], packed.shape[-1] * 2)
    if packed.is_cuda:
        src = packed.to(torch.uint8).contiguous()
        out = torch.empty(shape, dtype=torch.int8, device=packed.device)
        with torch.cuda.device(packed.device):
            native.call("lq_unpack_int4", src.data_ptr(), out.data_ptr(), out.numel(),
                        native.stream_ptr(packed.device))
        return out
    raw = packed.numpy().astype(np.uint8)
    pair = np.stack(((raw & 0x0F).astype(np.int16) - INT4_BIAS,
                     (raw >> 4).astype(np.int16) - INT4_BIAS), axis=-1)
    return torch.from_numpy(pair.reshape(shape).astype(np.int8))


def pack_weight(qweight: torch.Tensor, num_bits: int) -> torch.Tensor:
    if num_bits == 8:
        return qweight.contiguous()
    if num_bits == 4:
        return pack_int4(qweight)
    raise ValueError(f"unsupported num_bits {num_bits}, expected 4 or 8")


def unpack_weight(stored: torch.Tensor, num_bits: int) -> torch.Tensor:
    if num_bits == 8:
        return stored.to(torch.int8)
    if num_bits == 4:
        return unpack_int4(stored)
    raise ValueError(f"unsupported num_bits {num_bits}, expected 4 or 8")
