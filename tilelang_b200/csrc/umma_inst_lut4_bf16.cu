// tcgen05 kernel instances for WF_LUT4_S weights on ACT_BF16 activations (all token tiles).
#include "umma_launch_impl.cuh"

namespace b200dq {
B200DQ_UMMA_INSTANCE(launch_umma_lut4_bf16, WF_LUT4_S, ACT_BF16)
}  // namespace b200dq
