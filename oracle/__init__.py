"""CPU oracle for the quantized-linear / quantized-KV path. TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory. It restates, in numpy, the
arithmetic the reference defines for this path so that the CUDA kernels can be checked
against it; the only callers are the test suite, the smoke check and the CPU-baseline leg
of the benchmark.

Parity status: PINNED. Every function here is compared with the reference's own
implementation (imported and run on CPU when the fixtures were generated) through the
golden vectors under tests/golden/, and with the known-answer vectors the reference's
tests hold (nibble 0xD5, round-half-even, true division).
"""

from oracle.quant_oracle import *  # noqa: F401,F403
