// Instantiation unit: streaming GEMV, 8-bit codes, arithmetic variant 1.
#include "gemv_stream.cuh"

namespace lq {
namespace gemv {
int run_b8v1(GemvParams p, const lq_gemv_args& a, int spw, int threads, cudaStream_t s) {
  return launch_passes<8, 1>(p, a, spw, threads, s);
}
}  // namespace gemv
}  // namespace lq
