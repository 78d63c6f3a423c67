// Shared by the umma_inst_*.cu translation units: sets the shared-memory attribute of one
// kernel instance once per device, launches it and the stream-K fix-up pass.
#pragma once
#include "umma_gemm.cuh"
#include "umma_launch.h"

namespace b200dq {

constexpr int kMaxDevicesUmma = 32;

#define UMMA_OK(expr)                      \
  do {                                     \
    cudaError_t _e = (expr);               \
    if (_e != cudaSuccess) return _e;      \
  } while (0)

template <int TN, int WF, int ACT>
cudaError_t launch_umma_instance(const CUtensorMap& tmap, const GemmParams& p, int grid, cudaStream_t stream) {
  using Ring = RingConfig<TN, WF>;
  auto kernel = umma_dequant_gemm_kernel<TN, WF, ACT>;
  static bool attr_set[kMaxDevicesUmma] = {};
  int dev = 0;
  UMMA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevicesUmma) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    UMMA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Ring::kSmemBytes));
    attr_set[dev] = true;
  }
  kernel<<<grid, kThreads, Ring::kSmemBytes, stream>>>(tmap, p);
  UMMA_OK(cudaGetLastError());
  // stream-K second pass: one block column per cut between neighbouring CTAs
  if (((p.dyn_grid > 0 && !p.dyn_whole) || (p.dyn_grid == 0 && p.span % p.st_units != 0)) && grid > 1) {
    constexpr bool kInt = (ACT == ACT_I8);
    const dim3 fgrid(grid - 1, TN / fixup_tokens_per_block(TN));
    switch (p.out_type) {
      case OUT_F16: streamk_fixup_kernel<__half, TN, kInt><<<fgrid, kTileRows, 0, stream>>>(p); break;
      case OUT_BF16: streamk_fixup_kernel<__nv_bfloat16, TN, kInt><<<fgrid, kTileRows, 0, stream>>>(p); break;
      case OUT_F32: streamk_fixup_kernel<float, TN, kInt><<<fgrid, kTileRows, 0, stream>>>(p); break;
      default: streamk_fixup_kernel<int, TN, kInt><<<fgrid, kTileRows, 0, stream>>>(p); break;
    }
    UMMA_OK(cudaGetLastError());
  }
  return cudaSuccess;
}

template <int WF, int ACT>
cudaError_t launch_umma_format(int tn, const CUtensorMap& tmap, const GemmParams& p, int grid, cudaStream_t stream) {
  switch (tn) {
    case 16: return launch_umma_instance<16, WF, ACT>(tmap, p, grid, stream);
    case 32: return launch_umma_instance<32, WF, ACT>(tmap, p, grid, stream);
    case 64: return launch_umma_instance<64, WF, ACT>(tmap, p, grid, stream);
    case 128: return launch_umma_instance<128, WF, ACT>(tmap, p, grid, stream);
    case 256: return launch_umma_instance<256, WF, ACT>(tmap, p, grid, stream);
    default: return cudaErrorInvalidValue;
  }
}

// one entry per translation unit
cudaError_t launch_umma_u4sz_f16(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_u4sz_bf16(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_u2sz_f16(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_u2sz_bf16(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_lut4_f16(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_lut4_bf16(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_u4raw_f16(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_u4raw_bf16(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_s4raw_f16(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_s4raw_bf16(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_fp4_bf16(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_fp4_f16(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_i2_i8(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);
cudaError_t launch_umma_i4_i8(int, const CUtensorMap&, const GemmParams&, int, cudaStream_t);

#define B200DQ_UMMA_INSTANCE(name, WF, ACT)                                                              \
  cudaError_t name(int tn, const CUtensorMap& tmap, const GemmParams& p, int grid, cudaStream_t stream) { \
    return launch_umma_format<WF, ACT>(tn, tmap, p, grid, stream);                                       \
  }

}  // namespace b200dq
