// Launcher of the integer decode-shape kernel (int8_skinny.cuh).
#pragma once
#include <cuda_runtime.h>

namespace b200dq {

struct GemmParams;

// WF_I2_I8 / WF_I4_I8 on int8 activations, at most 32 tokens, K a multiple of 16, dense.
// Uses p.wp, a, c, bias, row_scale, tensor_scale, code_bias, M, N, K, st_total, stage_bytes, ldc,
// flags, out_type. Needs no scratch and no tensor map.
cudaError_t launch_int8_skinny_gemm(int weight_format, const GemmParams& p, cudaStream_t stream);

}  // namespace b200dq
