from llmquant_b200.core.config import BF16, DTYPE_BITS, ModelArgs, QuantConfig
from llmquant_b200.core.modifier import QuantizationModifier
from llmquant_b200.core.scheme import (
    GROUP_SIZE,
    PRESET_SCHEMES,
    QuantizationArgs,
    QuantizationScheme,
    preset_name_to_scheme,
)


def oneshot(model, recipe: QuantizationModifier):
    """Apply `recipe` to a loaded model in place (llmquant/core/oneshot.py:6-12)."""
    if isinstance(model, str):
        raise ValueError(
            "oneshot() takes a loaded model here; load it with transformers and pass the module")
    recipe.apply(model)
    return model


__all__ = [
    "BF16", "DTYPE_BITS", "GROUP_SIZE", "PRESET_SCHEMES", "ModelArgs", "QuantConfig",
    "QuantizationArgs", "QuantizationModifier", "QuantizationScheme", "oneshot",
    "preset_name_to_scheme",
]
