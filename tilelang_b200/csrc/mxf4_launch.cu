// Host side of the native MXFP4 path: shared-memory attribute once per device, persistent grid.
#include "mxf4_launch.h"

#include "mxf4_gemm.cuh"

namespace b200dq {

cudaError_t launch_mxf4_gemm(const CUtensorMap& tmap_a, const CUtensorMap& tmap_w, const Mxf4Params& p, int sm_count,
                             cudaStream_t stream) {
  static bool attr_set[32] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 32) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    e = cudaFuncSetAttribute(mxf4_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMxf4SmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  const long long tiles = static_cast<long long>(p.m_tiles) * p.n_tiles;
  const int grid = static_cast<int>(tiles < sm_count ? tiles : sm_count);
  mxf4_gemm_kernel<<<grid, kMxf4Threads, kMxf4SmemBytes, stream>>>(tmap_a, tmap_w, p);
  return cudaGetLastError();
}

}  // namespace b200dq
