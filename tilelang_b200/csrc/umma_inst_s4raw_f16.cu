// tcgen05 kernel instances for WF_S4_RAW weights on ACT_F16 activations (all token tiles).
#include "umma_launch_impl.cuh"

namespace b200dq {
B200DQ_UMMA_INSTANCE(launch_umma_s4raw_f16, WF_S4_RAW, ACT_F16)
}  // namespace b200dq
