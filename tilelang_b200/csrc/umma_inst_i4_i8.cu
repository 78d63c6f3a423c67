// tcgen05 kernel instances for WF_I4_I8 weights on ACT_I8 activations (all token tiles).
#include "umma_launch_impl.cuh"

namespace b200dq {
B200DQ_UMMA_INSTANCE(launch_umma_i4_i8, WF_I4_I8, ACT_I8)
}  // namespace b200dq
