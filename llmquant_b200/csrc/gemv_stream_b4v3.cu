// Instantiation unit: streaming GEMV, 4-bit codes, arithmetic variant 3.
#include "gemv_stream.cuh"

namespace lq {
namespace gemv {
int run_b4v3(GemvParams p, const lq_gemv_args& a, int spw, int threads, cudaStream_t s) {
  return launch_passes<4, 3>(p, a, spw, threads, s);
}
}  // namespace gemv
}  // namespace lq
