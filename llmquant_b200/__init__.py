"""B200-native quantized-linear / quantized-KV path with the llm-quant user surface.

  csrc/        hand-written sm_100a kernels behind the C ABI of include/llmquant_b200.h
  native       ctypes binding of that library (no JIT, no CPU fallback)
  cuda         load_extension() / fake_quantize_cuda -- the reference's operator boundary
  core         QuantizationArgs / QuantConfig / QuantizationModifier / oneshot
  quantizers   KernelQuantLinear and the int8 KV cache
  packing      the single-file model.bin format
  runtime      graphed decode and the tensor-parallel decoder
"""

__version__ = "0.1.0"
