// tcgen05 kernel instances for WF_FP4_E8M0 weights on ACT_F16 activations (all token tiles).
#include "umma_launch_impl.cuh"

namespace b200dq {
B200DQ_UMMA_INSTANCE(launch_umma_fp4_f16, WF_FP4_E8M0, ACT_F16)
}  // namespace b200dq
