"""Quantization descriptors, field-compatible with the reference (llmquant/core/scheme.py:6-63):
the same names travel through `model.bin` metadata, so they are part of the file format."""

from dataclasses import dataclass
from typing import Optional

GROUP_SIZE = 128  # codes per scale along the reduction axis


@dataclass(frozen=True)
class QuantizationArgs:
    """How one tensor is quantized.

    strategy "group" puts one scale on every `group_size` elements of the last axis;
    "channel" (weights) and "token" (activations) use one scale for the whole axis.
    `head_dim` makes the groups restart at every head of the reduction axis (o_proj);
    `out_group` makes that many consecutive output rows share a scale (q/k/v per head).
    """

    num_bits: int
    strategy: str
    symmetric: bool = True
    dynamic: bool = False
    group_size: Optional[int] = None
    head_dim: Optional[int] = None
    out_group: Optional[int] = None

    def __post_init__(self):
        grouped = self.strategy == "group"
        if grouped and not (self.group_size and self.group_size > 0):
            raise ValueError("strategy='group' requires a positive group_size")
        if not grouped and self.group_size is not None:
            raise ValueError(
                f"group_size is only valid for strategy='group', got {self.strategy!r}")

    @property
    def qmax(self) -> int:
        return (1 << (self.num_bits - 1)) - 1


@dataclass(frozen=True)
class QuantizationScheme:
    weights: Optional[QuantizationArgs]
    input_activations: Optional[QuantizationArgs]


def weight_args(bits: int, group_size: int = GROUP_SIZE) -> QuantizationArgs:
    return QuantizationArgs(num_bits=bits, strategy="group", group_size=group_size)


def activation_args(bits: int, group_size: int = GROUP_SIZE) -> QuantizationArgs:
    """Dynamic, per token and per group: aligned with the weight groups, causal per token."""
    return QuantizationArgs(num_bits=bits, strategy="group", group_size=group_size, dynamic=True)


PRESET_SCHEMES = {
    f"W{w}A{a}": QuantizationScheme(
        weights=weight_args(w), input_activations=activation_args(a) if a == 8 else None)
    for w in (4, 8) for a in (8, 16)
}


def preset_name_to_scheme(name: str) -> QuantizationScheme:
    scheme = PRESET_SCHEMES.get(str(name).upper())
    if scheme is None:
        raise ValueError(f"unknown scheme {name!r}, expected one of {list(PRESET_SCHEMES)}")
    return scheme
