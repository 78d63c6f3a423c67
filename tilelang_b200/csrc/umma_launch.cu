// Routes a (weight format, activation type) pair to the translation unit that holds its
// tcgen05 kernel instances.
#include "umma_launch_impl.cuh"

namespace b200dq {

cudaError_t launch_umma_gemm(int wf, int act, int tn, const CUtensorMap& tmap, const GemmParams& p, int grid,
                             cudaStream_t stream) {
  if (wf == WF_U4_SZ && act == ACT_F16) return launch_umma_u4sz_f16(tn, tmap, p, grid, stream);
  if (wf == WF_U4_SZ && act == ACT_BF16) return launch_umma_u4sz_bf16(tn, tmap, p, grid, stream);
  if (wf == WF_U2_SZ && act == ACT_F16) return launch_umma_u2sz_f16(tn, tmap, p, grid, stream);
  if (wf == WF_U2_SZ && act == ACT_BF16) return launch_umma_u2sz_bf16(tn, tmap, p, grid, stream);
  if (wf == WF_LUT4_S && act == ACT_F16) return launch_umma_lut4_f16(tn, tmap, p, grid, stream);
  if (wf == WF_LUT4_S && act == ACT_BF16) return launch_umma_lut4_bf16(tn, tmap, p, grid, stream);
  if (wf == WF_U4_RAW && act == ACT_F16) return launch_umma_u4raw_f16(tn, tmap, p, grid, stream);
  if (wf == WF_U4_RAW && act == ACT_BF16) return launch_umma_u4raw_bf16(tn, tmap, p, grid, stream);
  if (wf == WF_S4_RAW && act == ACT_F16) return launch_umma_s4raw_f16(tn, tmap, p, grid, stream);
  if (wf == WF_S4_RAW && act == ACT_BF16) return launch_umma_s4raw_bf16(tn, tmap, p, grid, stream);
  if (wf == WF_FP4_E8M0 && act == ACT_BF16) return launch_umma_fp4_bf16(tn, tmap, p, grid, stream);
  if (wf == WF_FP4_E8M0 && act == ACT_F16) return launch_umma_fp4_f16(tn, tmap, p, grid, stream);
  if (wf == WF_I2_I8 && act == ACT_I8) return launch_umma_i2_i8(tn, tmap, p, grid, stream);
  if (wf == WF_I4_I8 && act == ACT_I8) return launch_umma_i4_i8(tn, tmap, p, grid, stream);
  return cudaErrorInvalidValue;
}

}  // namespace b200dq
