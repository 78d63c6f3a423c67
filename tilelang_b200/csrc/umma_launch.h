// Launcher of the tcgen05 kernels (umma_gemm.cuh). Every (weight format, activation type)
// pair is instantiated in a translation unit of its own (umma_inst_*.cu) so the pairs
// compile in parallel and a change elsewhere does not rebuild them.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace b200dq {

struct GemmParams;

// Launches umma_dequant_gemm_kernel<token_tile, weight_format, act_type> on the schedule in
// `p`, then the stream-K fix-up pass when tiles were split between CTAs. Returns
// cudaErrorInvalidValue for a combination that has no kernel.
cudaError_t launch_umma_gemm(int weight_format, int act_type, int token_tile, const CUtensorMap& tmap_a,
                             const GemmParams& p, int grid, cudaStream_t stream);

}  // namespace b200dq
