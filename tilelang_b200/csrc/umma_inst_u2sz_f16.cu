// tcgen05 kernel instances for WF_U2_SZ weights on ACT_F16 activations (all token tiles).
#include "umma_launch_impl.cuh"

namespace b200dq {
B200DQ_UMMA_INSTANCE(launch_umma_u2sz_f16, WF_U2_SZ, ACT_F16)
}  // namespace b200dq
