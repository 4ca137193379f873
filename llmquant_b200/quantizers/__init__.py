"""The deployed ("kernel") implementation of a quantized layer and of the quantized KV cache."""

from llmquant_b200.quantizers.kernel import (
    DECODE_MAX_ROWS,
    KERNEL_MAX_ROWS,
    KernelQuantLinear,
    pad_activation,
    quantize_weight_canonical,
)

from llmquant_b200.quantizers.experts import KernelQuantExperts, quantize_expert_stack
from llmquant_b200.quantizers.kv_cache import (
    KernelQuantCache,
    QuantizedKVLayer,
    enable_fused_kv_attention,
    make_cache_factory,
)

AVAILABLE_MODES = frozenset({"kernel"})


def quant_linear_for(mode: str):
    """The module class a mode swaps each Linear for (llmquant/quantizers/dispatch.py:12-34)."""
    if mode == "kernel":
        return KernelQuantLinear
    raise ValueError(f"unsupported mode {mode!r}, expected one of {sorted(AVAILABLE_MODES)}")


__all__ = [
    "AVAILABLE_MODES", "DECODE_MAX_ROWS", "KERNEL_MAX_ROWS", "KernelQuantCache", "KernelQuantExperts",
    "KernelQuantLinear", "quantize_expert_stack",
    "QuantizedKVLayer", "enable_fused_kv_attention", "make_cache_factory",
    "pad_activation", "quant_linear_for", "quantize_weight_canonical",
]
