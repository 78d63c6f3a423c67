// tcgen05 kernel instances for WF_U4_RAW weights on ACT_BF16 activations (all token tiles).
#include "umma_launch_impl.cuh"

namespace b200dq {
B200DQ_UMMA_INSTANCE(launch_umma_u4raw_bf16, WF_U4_RAW, ACT_BF16)
}  // namespace b200dq
