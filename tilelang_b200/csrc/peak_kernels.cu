// Tensor-pipe calibration: how fast this GPU runs back-to-back tcgen05.mma of one kind when
// nothing else is in the way. One CTA per SM; one thread issues `mmas` instructions of shape
// 128 x 256 x (32 bytes of K) on operands that sit in shared memory, into one TMEM accumulator,
// then commits and waits. The caller times the launch with events; ops per launch come back
// from the entry point. This is the denominator for the integer and fp4 kernels, the way a
// library bf16 GEMM is the denominator for the bf16 ones (kind 0 measures bf16 the same way,
// as a cross-check of the method). The reference's survey of its own benchmarks quotes int8
// and fp4 results against nominal peaks only.
#include "peak_launch.h"

#include "ptx.cuh"

namespace b200dq {

constexpr int kPeakN = 256;
constexpr int kPeakSmem = 1024 + 128 * 128 + kPeakN * 128 + 64;

template <int KIND>
__global__ void __launch_bounds__(128, 1) tensor_peak_kernel(int mmas, DeviceStatus* st) {
  extern __shared__ uint8_t peak_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(peak_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_tile = smem;
  uint8_t* b_tile = smem + 128 * 128;
  uint64_t* bar = reinterpret_cast<uint64_t*>(b_tile + kPeakN * 128);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5;

  // operand bytes: high bits clear, so every 16-bit pattern is a small finite bf16 and every byte a small int8
  for (int i = threadIdx.x; i < (128 + kPeakN) * 128 / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem)[i] = (0x9e3779b9u * static_cast<uint32_t>(i + 1)) & 0x3f1f3f1fu;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  fence_proxy_async_smem();
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (KIND == 2) {
    // scale factors 2^0 for both operands in columns [256, 272) of every lane
    uint32_t ones[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) ones[i] = 0x7f7f7f7fu;
    tmem_st_32x32b_x16(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + 256, ones);
    tc_wait_st();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  if (threadIdx.x == 0) {
    const uint64_t a_desc = make_smem_desc_sw128(smem_u32(a_tile));
    const uint64_t b_desc = make_smem_desc_sw128(smem_u32(b_tile));
    constexpr uint32_t idesc = KIND == 0   ? make_idesc(1, 1, 1, 128, kPeakN)
                               : KIND == 1 ? make_idesc(2, 1, 1, 128, kPeakN)
                                           : make_idesc_mxf4(128, kPeakN, 0, 0);
    for (int i = 0; i < mmas; ++i) {
      const int m = i & 3;
      if (KIND == 0) {
        umma_ss_f16(tmem_base, a_desc + 2 * m, b_desc + 2 * m, idesc, i != 0);
      } else if (KIND == 1) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_base),
            "l"(a_desc + 2 * m), "l"(b_desc + 2 * m), "r"(idesc), "r"(static_cast<uint32_t>(i != 0))
            : "memory");
      } else {
        umma_mxf4_ss(tmem_base, a_desc + 2 * m, b_desc + 2 * m, idesc, tmem_base + 256, tmem_base + 260, i != 0);
      }
    }
    tc_commit(bar);
    mbar_wait(bar, 0, abort_flag, st, 31);
    tc_fence_after_sync();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

cudaError_t launch_tensor_peak(int kind, int mmas, int sm_count, DeviceStatus* st, double* ops, cudaStream_t stream) {
  static bool attr_set[32][3] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 32 || kind < 0 || kind > 2) return cudaErrorInvalidValue;
  void (*kernel)(int, DeviceStatus*) =
      kind == 0 ? tensor_peak_kernel<0> : kind == 1 ? tensor_peak_kernel<1> : tensor_peak_kernel<2>;
  if (!attr_set[dev][kind]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem);
    if (e != cudaSuccess) return e;
    attr_set[dev][kind] = true;
  }
  kernel<<<sm_count, 128, kPeakSmem, stream>>>(mmas, st);
  const int k_per_mma = kind == 0 ? 16 : kind == 1 ? 32 : 64;
  if (ops != nullptr) *ops = 2.0 * 128 * kPeakN * k_per_mma * static_cast<double>(mmas) * sm_count;
  return cudaGetLastError();
}

}  // namespace b200dq
