"""An integer KV cache behind transformers' `Cache` interface.

The reference's `FakeQuantCache` (llmquant/quantizers/fake.py:39-62) rounds new keys and
values to the int grid and keeps the dequantized bf16 tensors. Here the int8 codes and the
fp32 per-token-per-head scales are what is stored; `update()` quantizes the new tokens with
`lq_kv_write` and returns `codes * scale` in the model dtype, i.e. the very values the
reference would have stored (an integer cannot keep the sign of a zero, nothing else
differs). Tokens already in the cache are never re-quantized. The fused decoder
(`llmquant_b200.runtime.decoder`) reads the same storage directly with the decode-attention
kernel instead of going through the dequantized copy.

So can transformers' own `generate`: `enable_fused_kv_attention(model)` registers an attention
function with transformers' `AttentionInterface` and selects it for the model; a cache made by
`make_cache_factory(bits, model=model)` then hands that function its integer storage instead
of a dequantized copy, and a decode step (one query token) runs the dequantize-on-read
attention kernel over the codes. Prefill, padded batches and shapes the kernel is not built
for dequantize once and take transformers' SDPA path, as before.
"""

import ctypes
import functools

import torch
from transformers.cache_utils import Cache, CacheLayerMixin

from llmquant_b200 import native

KV_GROUP = 128
ATTENTION_NAME = "llmquant_b200_int_kv"


def int_kv_attention(module, query, key, value, attention_mask, dropout=0.0, scaling=None, **kwargs):
    """Attention function for transformers' `AttentionInterface`. `key` / `value` are what
    `Cache.update` returned: int8 code views tagged with their cache layer when the cache was
    made for fused reading, ordinary tensors otherwise."""
    from transformers.integrations.sdpa_attention import sdpa_attention_forward

    layer = getattr(key, "lq_layer", None)
    if layer is None:
        return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout,
                                      scaling=scaling, **kwargs)
    batch, heads, q_len, head_dim = query.shape
    groups = heads // layer.heads if heads % layer.heads == 0 else 0
    fused = (q_len == 1 and query.dtype == torch.bfloat16 and head_dim in (64, 128) and groups in (1, 2, 4, 8)
             and (attention_mask is None or batch == 1) and layer.num_bits <= 8 and not dropout)
    if fused:
        scale = head_dim ** -0.5 if scaling is None else scaling
        out = layer.attend(query.reshape(batch, heads, head_dim), scale)
        return out.view(batch, 1, heads, head_dim), None
    k, v = layer.dequantized()
    return sdpa_attention_forward(module, query, k, v, attention_mask, dropout=dropout, scaling=scaling, **kwargs)


def enable_fused_kv_attention(model):
    """Select the dequantize-on-read attention for `model` (any transformers model whose
    attention goes through `AttentionInterface`). Safe with every cache: only a cache made
    with `make_cache_factory(bits, model=model)` is read as integers."""
    from transformers import AttentionInterface, AttentionMaskInterface
    from transformers.masking_utils import sdpa_mask
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    if ATTENTION_NAME not in ALL_ATTENTION_FUNCTIONS.valid_keys():
        AttentionInterface.register(ATTENTION_NAME, int_kv_attention)
        AttentionMaskInterface.register(ATTENTION_NAME, sdpa_mask)
    model.set_attn_implementation(ATTENTION_NAME)
    return model


class QuantizedKVLayer(CacheLayerMixin):
    """One layer: codes [B, H, capacity, D] int8 and scales [B, H, capacity, ceil(D/128)] fp32."""

    is_sliding = False
    is_compileable = False

    def __init__(self, num_bits: int = 8, max_cache_len=None, fused_read: bool = False):
        super().__init__()
        self.num_bits = num_bits
        self.max_cache_len = max_cache_len
        self.fused_read = fused_read
        self.dequant_calls = self.fused_reads = 0  # how the cache has been read so far
        self._scratch = None
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
        self.dequant_calls += 1
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
        if not self.fused_read:
            return self.dequantized()
        # the integer storage itself, tagged so that int_kv_attention knows what it was given
        k, v = self.k_codes[:, :, : self.length], self.v_codes[:, :, : self.length]
        k.lq_layer = v.lq_layer = self
        return k, v

    def attend(self, q, scaling):
        """softmax(q k^T * scaling) v for one query token per sequence over the stored codes:
        q [B, Hq, D] bf16 -> [B, Hq, D] bf16 (`lq_attn_decode_kv_i8`)."""
        batch, heads, head_dim = q.shape
        splits = max(1, min(-(-2 * 148 // (batch * self.heads)), self.length // 64 or 1))
        lib = native.library()
        need = lib.lq_attn_decode_scratch_bytes(batch, heads, head_dim, splits) // 4
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, dtype=torch.float32, device=self.device)
        q = q.contiguous()
        out = torch.empty_like(q)
        with torch.cuda.device(self.device):
            native.call("lq_attn_decode_kv_i8", q.data_ptr(), self.k_codes.data_ptr(), self.v_codes.data_ptr(),
                        self.k_scales.data_ptr(), self.v_scales.data_ptr(), out.data_ptr(),
                        self._scratch.data_ptr(), batch, heads, self.heads, head_dim, self.capacity, 0,
                        self.length, 0, float(scaling), splits, 0, native.stream_ptr(self.device))
        self.fused_reads += 1
        return out

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

    def __init__(self, num_bits: int = 8, max_cache_len=None, fused_read: bool = False):
        super().__init__(layer_class_to_replicate=functools.partial(
            QuantizedKVLayer, num_bits, max_cache_len, fused_read))
        self.num_bits = num_bits
        self.capacity_limit = max_cache_len
        self.fused_read = fused_read

    def crop(self, max_length: int):
        for layer in self.layers:
            layer.crop(max_length)


def make_cache_factory(num_bits, max_cache_len=None, model=None):
    """Zero-arg factory for `generate(past_key_values=...)`, or None to keep the bf16 cache
    (same contract as llmquant/quantizers/fake.py:58-62). With `model` given and switched to
    the dequantize-on-read attention (`enable_fused_kv_attention`), the caches it makes are
    read as integers by that model's decode steps instead of being dequantized whole."""
    if num_bits is None:
        return None
    fused = model is not None and getattr(getattr(model, "config", None), "_attn_implementation", None) == ATTENTION_NAME
    return lambda: KernelQuantCache(num_bits, max_cache_len, fused_read=fused)
