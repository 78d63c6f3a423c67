// Host side of the integer decode-shape kernel: picks the token and row blocking.
#include "int8_skinny_launch.h"

#include "int8_skinny.cuh"

namespace b200dq {

namespace {

template <int NT, int MT>
cudaError_t launch(int wf, const GemmParams& p, cudaStream_t stream) {
  const int grid = (p.N + 16 * MT - 1) / (16 * MT);
  // few tokens: latency is everything, so K is cut over 16 warps; more tokens need the registers
  const int threads = NT <= 2 ? 512 : 256;
  if (wf == WF_I2_I8) int8_skinny_gemm_kernel<NT, MT, WF_I2_I8><<<grid, threads, 0, stream>>>(p);
  else if (wf == WF_I4_I8) int8_skinny_gemm_kernel<NT, MT, WF_I4_I8><<<grid, threads, 0, stream>>>(p);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_int8_skinny_gemm(int wf, const GemmParams& p, cudaStream_t stream) {
  if (p.M <= 8) return launch<1, 1>(wf, p, stream);
  if (p.M <= 16) return launch<2, 1>(wf, p, stream);
  if (p.M <= kInt8SkinnyMaxTokens) return launch<4, 2>(wf, p, stream);
  return cudaErrorInvalidValue;
}

}  // namespace b200dq
