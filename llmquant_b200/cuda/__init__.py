"""The operator boundary: the same callables the reference's `llmquant.cuda` exposes,
served by the prebuilt sm_100a library instead of a JIT-compiled torch extension."""

from llmquant_b200.cuda.build import load_extension
from llmquant_b200.cuda.ops import fake_quantize_cuda

__all__ = ["fake_quantize_cuda", "load_extension"]
