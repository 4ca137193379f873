"""An integer KV cache behind transformers' `Cache` interface.

The reference's `FakeQuantCache` (llmquant/quantizers/fake.py:39-62) rounds new keys and
values to the int grid and keeps the dequantized bf16 tensors. Here the int8 codes and the
fp32 per-token-per-head scales are what is stored; `update()` quantizes the new tokens with
`lq_kv_write` and returns `codes * scale` in the model dtype, i.e. the very values the
reference would have stored (an integer cannot keep the sign of a zero, nothing else
differs). Tokens already in the cache are never re-quantized. The fused decoder
(`llmquant_b200.runtime.decoder`) reads the same storage directly with the decode-attention
kernel instead of going through the dequantized copy.
"""

import ctypes
import functools

import torch
from transformers.cache_utils import Cache, CacheLayerMixin

from llmquant_b200 import native

KV_GROUP = 128


class QuantizedKVLayer(CacheLayerMixin):
    """One layer: codes [B, H, capacity, D] int8 and scales [B, H, capacity, ceil(D/128)] fp32."""

    is_sliding = False
    is_compileable = False

    def __init__(self, num_bits: int = 8, max_cache_len=None):
        super().__init__()
        self.num_bits = num_bits
        self.max_cache_len = max_cache_len
        self.length = 0
        self.capacity = 0
        self.k_codes = self.v_codes = self.k_scales = self.v_scales = None

    def lazy_initialization(self, key_states, value_states):
        if not key_states.is_cuda:
            raise RuntimeError("the quantized KV cache needs CUDA tensors: there is no CPU fallback")
        native.library()
        self.dtype, self.device = key_states.dtype, key_states.device
        self.batch, self.heads, _, self.head_dim = key_states.shape
        self.groups = -(-self.head_dim // KV_GROUP)
        self._allocate(self.max_cache_len or 256)
        self.is_initialized = True

    def _allocate(self, capacity):
        shape = (self.batch, self.heads, capacity)
        new = [torch.zeros(*shape, self.head_dim, dtype=torch.int8, device=self.device) for _ in range(2)]
        new += [torch.zeros(*shape, self.groups, dtype=torch.float32, device=self.device) for _ in range(2)]
        if self.length:
            for dst, src in zip(new, (self.k_codes, self.v_codes, self.k_scales, self.v_scales)):
                dst[:, :, : self.length] = src[:, :, : self.length]
        self.k_codes, self.v_codes, self.k_scales, self.v_scales = new
        self.capacity = capacity

    def _strides(self, t):
        if t.stride(-1) != 1:
            t = t.contiguous()
        return t, (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))

    def append(self, key_states, value_states):
        """Quantize and store new tokens; returns nothing (the fused decoder's entry)."""
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        new = key_states.shape[-2]
        need = self.length + new
        if need > self.capacity:
            if self.max_cache_len is not None:
                raise RuntimeError(
                    f"KV cache of {self.max_cache_len} tokens cannot take {need}")
            self._allocate(max(need, 2 * self.capacity))
        k, ks = self._strides(key_states)
        v, vs = self._strides(value_states)
        with torch.cuda.device(self.device):
            native.call("lq_kv_write", k.data_ptr(), v.data_ptr(), ks, vs,
                        native.DTYPE_ID[k.dtype], self.k_codes.data_ptr(), self.v_codes.data_ptr(),
                        self.k_scales.data_ptr(), self.v_scales.data_ptr(), self.batch, self.heads,
                        new, self.head_dim, self.capacity, 0, self.length, self.num_bits,
                        native.stream_ptr(self.device))
        self.length = need

    def dequantized(self, length=None):
        """(K, V) in the model dtype, [B, H, length, D]."""
        length = self.length if length is None else length
        outs = []
        for codes, scales in ((self.k_codes, self.k_scales), (self.v_codes, self.v_scales)):
            out = torch.empty(self.batch, self.heads, length, self.head_dim, dtype=self.dtype,
                              device=self.device)
            with torch.cuda.device(self.device):
                native.call("lq_kv_dequant", codes.data_ptr(), scales.data_ptr(), out.data_ptr(),
                            native.DTYPE_ID[self.dtype], self.batch, self.heads, length,
                            self.head_dim, self.capacity, native.stream_ptr(self.device))
            outs.append(out)
        return tuple(outs)

    def update(self, key_states, value_states, *args, **kwargs):
        self.append(key_states, value_states)
        return self.dequantized()

    def get_mask_sizes(self, query_length: int):
        return self.get_seq_length() + query_length, 0

    def get_seq_length(self) -> int:
        return self.length

    def get_max_cache_shape(self) -> int:
        return self.max_cache_len if self.max_cache_len is not None else -1

    def reset(self):
        self.length = 0

    def crop(self, max_length: int):
        if max_length < 0:
            max_length = self.length - abs(max_length)
        self.length = min(self.length, max(max_length, 0))

    def offload(self):
        pass

    def prefetch(self):
        pass

    def reorder_cache(self, beam_idx):
        if self.length:
            idx = beam_idx.to(self.device)
            for name in ("k_codes", "v_codes", "k_scales", "v_scales"):
                setattr(self, name, getattr(self, name).index_select(0, idx))


class KernelQuantCache(Cache):
    """`Cache` whose layers store int codes. `KernelQuantCache(8)` is what
    `make_cache_factory(8)()` returns; `max_cache_len` fixes the capacity up front (needed
    when a captured graph is going to write into it)."""

    def __init__(self, num_bits: int = 8, max_cache_len=None):
        super().__init__(layer_class_to_replicate=functools.partial(
            QuantizedKVLayer, num_bits, max_cache_len))
        self.num_bits = num_bits
        self.capacity_limit = max_cache_len

    def crop(self, max_length: int):
        for layer in self.layers:
            layer.crop(max_length)


def make_cache_factory(num_bits, max_cache_len=None):
    """Zero-arg factory for `generate(past_key_values=...)`, or None to keep the bf16 cache
    (same contract as llmquant/quantizers/fake.py:58-62)."""
    if num_bits is None:
        return None
    return lambda: KernelQuantCache(num_bits, max_cache_len)
