// Launcher of the small-M kernels (skinny_gemm.cuh), compiled in a translation unit of its
// own (skinny_launch.cu) so that a change to those kernels does not rebuild the tcgen05 ones.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace b200dq {

struct GemmParams;

constexpr int kSkinnyTokens = 16;   // most tokens the small-M kernels take (their schedule's token tile)

// Tokens per activation box of the kernel instance that serves M tokens (8 or 16): the
// caller encodes the 4-D activation tensor map {64 k, k-block parity, token, stage} with
// box {64, 2, this, 1} and the 128-byte swizzle.
inline int skinny_box_tokens(int M) { return M <= 8 ? 8 : 16; }

// Launches skinny_dequant_gemm_kernel for the given weight format / activation type on the
// token-tile-16 stream-K schedule in `p`, then the fix-up pass when tiles were split between
// CTAs. K must be a multiple of 128. Returns cudaErrorInvalidValue for a combination the
// kernels do not cover.
cudaError_t launch_skinny_gemm(int weight_format, int act_type, const CUtensorMap& tmap_a, const GemmParams& p,
                               int grid, cudaStream_t stream);

}  // namespace b200dq
