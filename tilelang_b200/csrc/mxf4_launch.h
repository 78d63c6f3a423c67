// Launcher of the native MXFP4 kernel (mxf4_gemm.cuh), in a translation unit of its own.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace b200dq {

struct DeviceStatus;

struct Mxf4Params {
  const uint32_t* sfa;   // activation scales, 128 x 4 blocked words: [ceil(M/128)][K/128][32][4]
  const uint32_t* sfw;   // weight scales, the same layout over N
  void* c;               // output (M, N) row-major
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;   // 128-token tiles, 128-row tiles, k-blocks of 256
  int out_type;          // OUT_BF16, OUT_F16 or OUT_F32
  DeviceStatus* status;
};

// Bytes per code row of the tensor maps' box and rows per box: the caller encodes two 2-D
// uint8 tensor maps over the (rows, K/2) code tensors with box {128, 128} and the 128-byte swizzle.
constexpr int kMxf4BoxBytes = 128;
constexpr int kMxf4BoxRows = 128;

cudaError_t launch_mxf4_gemm(const CUtensorMap& tmap_a, const CUtensorMap& tmap_w, const Mxf4Params& p, int sm_count,
                             cudaStream_t stream);

}  // namespace b200dq
