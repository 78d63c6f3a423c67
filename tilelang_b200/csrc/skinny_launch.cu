// Host side of the small-M path: picks the kernel instance, sets its shared-memory
// attribute once per device and launches it followed by the stream-K fix-up pass.
#include "skinny_launch.h"

#include "skinny_gemm.cuh"

namespace b200dq {

namespace {

constexpr int kMaxDevicesSkinny = 32;

#define SKINNY_OK(expr)                    \
  do {                                     \
    cudaError_t _e = (expr);               \
    if (_e != cudaSuccess) return _e;      \
  } while (0)

template <int NT, int WF, int ACT>
cudaError_t launch_one(const CUtensorMap& tmap_a, const GemmParams& p, int grid, cudaStream_t stream) {
  using Ring = SkinnyRing<NT, WF>;
  static bool attr_set[kMaxDevicesSkinny] = {};
  constexpr int smem = Ring::kSmemBytes;
  static_assert(smem <= 232448, "over the 227 KiB shared-memory limit");
  auto kernel = skinny_dequant_gemm_kernel<NT, WF, ACT>;
  int dev = 0;
  SKINNY_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevicesSkinny) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    SKINNY_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set[dev] = true;
  }
  kernel<<<grid, kSkinnyThreads, smem, stream>>>(tmap_a, p);
  return cudaGetLastError();
}

template <int WF, int ACT>
cudaError_t launch_format(const CUtensorMap& tmap_a, const GemmParams& p, int grid, cudaStream_t stream) {
  if (p.M <= 8) SKINNY_OK((launch_one<1, WF, ACT>(tmap_a, p, grid, stream)));
  else SKINNY_OK((launch_one<2, WF, ACT>(tmap_a, p, grid, stream)));
  return cudaSuccess;
}

}  // namespace

cudaError_t launch_skinny_gemm(int wf, int act, const CUtensorMap& tmap_a, const GemmParams& p, int grid,
                               cudaStream_t stream) {
  if (p.K % 128 != 0) return cudaErrorInvalidValue;
  if (wf == WF_FP4_E8M0 && act == ACT_BF16) return launch_format<WF_FP4_E8M0, ACT_BF16>(tmap_a, p, grid, stream);
  if (wf == WF_FP4_E8M0 && act == ACT_F16) return launch_format<WF_FP4_E8M0, ACT_F16>(tmap_a, p, grid, stream);
  if (wf == WF_U4_SZ && act == ACT_F16) return launch_format<WF_U4_SZ, ACT_F16>(tmap_a, p, grid, stream);
  if (wf == WF_U4_SZ && act == ACT_BF16) return launch_format<WF_U4_SZ, ACT_BF16>(tmap_a, p, grid, stream);
  if (wf == WF_U4_RAW && act == ACT_F16) return launch_format<WF_U4_RAW, ACT_F16>(tmap_a, p, grid, stream);
  if (wf == WF_U4_RAW && act == ACT_BF16) return launch_format<WF_U4_RAW, ACT_BF16>(tmap_a, p, grid, stream);
  if (wf == WF_S4_RAW && act == ACT_F16) return launch_format<WF_S4_RAW, ACT_F16>(tmap_a, p, grid, stream);
  if (wf == WF_S4_RAW && act == ACT_BF16) return launch_format<WF_S4_RAW, ACT_BF16>(tmap_a, p, grid, stream);
  return cudaErrorInvalidValue;
}

}  // namespace b200dq
