"""Which Linear gets which scheme, and the in-place swap.

Same targeting rules as the reference (llmquant/core/modifier.py:8-199): Llama module names,
`lm_head` handled by its own scheme, `self_attn.o_proj` grouped inside each head of its
reduction axis, `self_attn.{q,k,v,qkv}_proj` given one scale per output head when
`qkv_out_scale_per_head` is set. Only mode "kernel" exists here: the swapped-in module is
`KernelQuantLinear`, whose arithmetic runs in the CUDA library.
"""

import re
from dataclasses import dataclass, replace
from typing import Optional, Tuple, Union

import torch.nn as nn

from llmquant_b200.core.scheme import QuantizationScheme, preset_name_to_scheme

ATTN_RE = re.compile(r".*\.self_attn\..*_proj$")
MLP_RE = re.compile(r".*\.mlp\..*_proj$")
O_PROJ_RE = re.compile(r".*\.self_attn\.o_proj$")
QKV_RE = re.compile(r".*\.self_attn\.(q|k|v|qkv)_proj$")

# stacked Mixture-of-Experts weights: one Parameter per projection holding every expert
# (llmquant/core/modifier.py:24-38 of the reference); the router is left alone
MOE_EXPERT_RE = re.compile(r".*\.experts\.(gate_up_proj|down_proj|w1|w2|w3)$")

SchemeLike = Union[str, QuantizationScheme, None]
AVAILABLE_MODES = frozenset({"kernel"})


def _resolve(scheme: SchemeLike) -> Optional[QuantizationScheme]:
    if scheme is None or isinstance(scheme, QuantizationScheme):
        return scheme
    return preset_name_to_scheme(scheme)


def _listed(name: str, patterns) -> bool:
    for pattern in patterns:
        if pattern.startswith("re:"):
            if re.match(pattern[3:], name):
                return True
        elif name == pattern:
            return True
    return False


def stacked_expert_blocks(model):
    """(name, module) of every module that directly owns stacked expert weights, found by
    structure rather than class name (llmquant/core/modifier.py:66-90 of the reference). A
    block that lacks what the quantized expert module mirrors is refused, not half-converted."""
    owners = []
    for name, param in model.named_parameters():
        if param.ndim >= 2 and MOE_EXPERT_RE.match(name):
            parent = name.rpartition(".")[0]
            if parent not in owners:
                owners.append(parent)
    blocks = []
    for name in owners:
        module = model.get_submodule(name)
        missing = [a for a in ("gate_up_proj", "down_proj", "act_fn") if not hasattr(module, a)]
        if missing:
            raise NotImplementedError(
                f"{name} ({type(module).__name__}) holds stacked expert weights but is missing "
                f"{missing}. The quantized expert module mirrors the Mixtral/OLMoE block; this "
                f"architecture needs its own.")
        blocks.append((name, module))
    return blocks


@dataclass
class QuantizationModifier:
    scheme: SchemeLike = None
    targets: Tuple[str, ...] = ("Linear",)
    ignore: Tuple[str, ...] = ("lm_head",)
    lm_head_scheme: SchemeLike = None
    mode: str = "kernel"
    attn_scheme: SchemeLike = None
    mlp_scheme: SchemeLike = None
    kv_cache_bits: Optional[int] = None
    head_dim: Optional[int] = None
    qkv_out_scale_per_head: bool = True

    def resolve(self, model) -> "QuantizationModifier":
        """Take head_dim from the model's config unless it was given."""
        config = getattr(model, "config", None)
        if config is not None and self.head_dim is None:
            head_dim = getattr(config, "head_dim", None)
            if head_dim is None and getattr(config, "num_attention_heads", None):
                head_dim = config.hidden_size // config.num_attention_heads
            self.head_dim = head_dim
        return self

    def scheme_for(self, name: str) -> Optional[QuantizationScheme]:
        if name == "lm_head":
            return _resolve(self.lm_head_scheme)
        if _listed(name, self.ignore):
            return None
        if self.attn_scheme is not None and ATTN_RE.match(name):
            scheme = _resolve(self.attn_scheme)
            if self.head_dim and O_PROJ_RE.match(name):
                act = scheme.input_activations
                return QuantizationScheme(
                    weights=replace(scheme.weights, head_dim=self.head_dim) if scheme.weights else None,
                    input_activations=replace(act, head_dim=self.head_dim) if act else None)
            if self.head_dim and self.qkv_out_scale_per_head and QKV_RE.match(name) and scheme.weights:
                return QuantizationScheme(
                    weights=replace(scheme.weights, out_group=self.head_dim),
                    input_activations=scheme.input_activations)
            return scheme
        if self.mlp_scheme is not None and MLP_RE.match(name):
            return _resolve(self.mlp_scheme)
        return _resolve(self.scheme)

    def apply(self, model: nn.Module) -> nn.Module:
        if self.mode not in AVAILABLE_MODES:
            raise ValueError(
                f"unsupported mode {self.mode!r}: this library only carries the deployed "
                f"'kernel' path (the reference's 'fake' and 'real' modes are its own CPU/torch paths)")
        from llmquant_b200.quantizers import KernelQuantExperts, KernelQuantLinear

        self.resolve(model)
        swaps = []
        expert_blocks = set()
        if self.mlp_scheme is not None:
            # stacked experts are the MLP of a Mixture-of-Experts block: they take the mlp scheme
            # and are swapped as one module (llmquant/core/modifier.py:176-185 of the reference)
            for name, module in stacked_expert_blocks(model):
                expert_blocks.add(name)
                swaps.append((name, KernelQuantExperts.from_experts(module, _resolve(self.mlp_scheme))))
        for name, module in model.named_modules():
            if name in expert_blocks or type(module).__name__ not in self.targets:
                continue
            scheme = self.scheme_for(name)
            if scheme is not None:
                swaps.append((name, KernelQuantLinear.from_linear(module, scheme)))
        for name, module in swaps:
            parent_name, _, child = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            setattr(parent, child, module)
        if self.kv_cache_bits and hasattr(model, "set_attn_implementation"):
            # a recipe with an integer KV cache also selects the attention that reads one as
            # integers (it behaves like transformers' SDPA for every other cache)
            from llmquant_b200.quantizers.kv_cache import enable_fused_kv_attention

            enable_fused_kv_attention(model)
        return model
