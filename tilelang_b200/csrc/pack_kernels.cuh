// Offline layout transform (device side): natural little-endian packed codes
// (N, K*bits/8) -> the tiled, pre-interleaved image the GEMM streams.
//
// Packed image: [n_tile][k_block][chunk][row 0..127][16 bytes]. One
// (n_tile, k_block) stage is contiguous (4 KiB, or 8 KiB for 4-bit codes feeding
// int8), so the kernel fetches it with a single bulk copy, and the dequant
// thread of row r reads chunk c at byte c*2048 + r*16 — consecutive rows hit
// consecutive 16-byte slots, which is bank-conflict free.
//
// Inside a 32-bit word the codes are permuted for the shift-and-mask decoders
// (decode.cuh). For integer codes this is the permutation of the reference's
// interleave_weight (examples/dequantize_gemm/quantize/utils.py:71-125, the
// cases without the extra 1-/2-bit byte shuffles); the e2m1 permutation is this
// library's own (the reference's twiddled layout, quantize/mxfp.py:6-49 and
// dequantize_utils.py:4-54, solves the same problem with different positions).
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200dq {

// codes of `bits` bits, element e -> bit (e % G) * S + (e / G) * bits, G = 32 / S
__host__ __device__ inline uint32_t interleave_word(uint32_t w, int bits, int stride_bits) {
  const int per_word = 32 / bits;
  const int groups = 32 / stride_bits;
  const uint32_t mask = (1u << bits) - 1u;
  uint32_t out = 0;
  for (int e = 0; e < per_word; ++e) {
    const uint32_t code = (w >> (bits * e)) & mask;
    out |= code << ((e % groups) * stride_bits + (e / groups) * bits);
  }
  return out;
}

// e2m1 codes (s e1 e0 m = bits 3 2 1 0). Element e = 2*i + h goes to half h,
// code slot i; slot positions inside the 16-bit half are listed in decode.cuh.
__host__ __device__ inline uint32_t twiddle_fp4_word(uint32_t w) {
  uint32_t out = 0;
  for (int e = 0; e < 8; ++e) {
    const uint32_t code = (w >> (4 * e)) & 0xf;
    const uint32_t s = (code >> 3) & 1, e1 = (code >> 2) & 1, e0 = (code >> 1) & 1, m = code & 1;
    const int i = e >> 1, h = e & 1;
    uint32_t half = 0;
    if (i == 0) half = (s << 15) | (e1 << 8) | (e0 << 7) | (m << 6);
    else if (i == 1) half = (s << 12) | (e1 << 5) | (e0 << 4) | (m << 3);
    else if (i == 2) half = (s << 9) | (e1 << 2) | (e0 << 1) | m;
    else half = (s << 14) | (e1 << 13) | (e0 << 11) | (m << 10);
    out |= half << (16 * h);
  }
  return out;
}

// mode: 0 = integer codes -> 16-bit target, 1 = integer codes -> 8-bit target, 2 = e2m1 -> bf16
__global__ void pack_weights_kernel(const uint32_t* __restrict__ q, uint32_t* __restrict__ wp, int N, int K,
                                    int bits, int mode, int n_tiles, int kb_total, int chunks,
                                    int elems_per_kblock) {
  // one thread per output word
  const long long total = static_cast<long long>(n_tiles) * kb_total * chunks * 128 * 4;
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  const int j = static_cast<int>(idx & 3);                 // word in the 16-byte slot
  const int r = static_cast<int>((idx >> 2) & 127);        // row in tile
  long long rest = idx >> 9;
  const int c = static_cast<int>(rest % chunks); rest /= chunks;
  const int kb = static_cast<int>(rest % kb_total);
  const int nt = static_cast<int>(rest / kb_total);
  const int n = nt * 128 + r;
  const int elems_per_word = 32 / bits;
  const int k0 = kb * elems_per_kblock + (c * 4 + j) * elems_per_word;
  uint32_t w = 0;
  if (n < N && k0 < K) {
    const long long word_idx = (static_cast<long long>(n) * K + k0) / elems_per_word;
    w = q[word_idx];
  }
  uint32_t out;
  if (mode == 0) out = interleave_word(w, bits, 16);
  else if (mode == 1) out = interleave_word(w, bits, 8);
  else out = twiddle_fp4_word(w);
  wp[idx] = out;
}

template <bool kBf16>
__global__ void pack_scales_u4_kernel(const uint16_t* __restrict__ scales, const uint16_t* __restrict__ zeros,
                                      uint32_t* __restrict__ sz, int N, int groups, int n_pad) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int g = blockIdx.y;
  if (n >= n_pad) return;
  uint32_t out = 0;
  if (n < N) {
    const uint16_t s_raw = scales[static_cast<size_t>(n) * groups + g];
    float s, z = 8.f;
    if constexpr (kBf16) {
      s = __bfloat162float(__ushort_as_bfloat16(s_raw));
      if (zeros) z = __bfloat162float(__ushort_as_bfloat16(zeros[static_cast<size_t>(n) * groups + g]));
      const float c = (8.f - z) * s;
      out = s_raw | (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(c))) << 16);
    } else {
      s = __half2float(__ushort_as_half(s_raw));
      if (zeros) z = __half2float(__ushort_as_half(zeros[static_cast<size_t>(n) * groups + g]));
      const float c = (8.f - z) * s;
      out = s_raw | (static_cast<uint32_t>(__half_as_ushort(__float2half_rn(c))) << 16);
    }
  }
  sz[static_cast<size_t>(g) * n_pad + n] = out;
}

__global__ void pack_scales_e8m0_kernel(const uint8_t* __restrict__ exps, uint16_t* __restrict__ sz, int N,
                                        int blocks32, int n_pad) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int kb = blockIdx.y;
  if (n >= n_pad) return;
  uint16_t out = 0;
  if (n < N) {
    const uint8_t e0 = exps[static_cast<size_t>(n) * blocks32 + 2 * kb];
    const uint8_t e1 = exps[static_cast<size_t>(n) * blocks32 + 2 * kb + 1];
    out = static_cast<uint16_t>(e0) | (static_cast<uint16_t>(e1) << 8);
  }
  sz[static_cast<size_t>(kb) * n_pad + n] = out;
}

}  // namespace b200dq
