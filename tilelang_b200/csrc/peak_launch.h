// Launcher of the tensor-pipe calibration kernels (peak_kernels.cu).
#pragma once
#include <cuda_runtime.h>

namespace b200dq {

struct DeviceStatus;

// kind: 0 bf16 (kind::f16), 1 int8 (kind::i8), 2 MXFP4 (kind::mxf4.block_scale). One CTA per SM
// issues `mmas` instructions of 128 x 256 x 32 bytes of K; `*ops` receives the arithmetic
// operations of the whole launch (2 per multiply-add).
cudaError_t launch_tensor_peak(int kind, int mmas, int sm_count, DeviceStatus* st, double* ops, cudaStream_t stream);

}  // namespace b200dq
