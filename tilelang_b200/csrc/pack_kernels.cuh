// Offline layout transform (device side): natural little-endian packed codes
// (N, K*bits/8) -> the tiled, pre-interleaved image the GEMM streams.
//
// Packed image: [n_tile][stage][ codes of 2 k-blocks | scale words ], where the
// codes of a stage are [chunk][position 0..127][16 bytes] and the scale words are
// [word][row 0..127][4 bytes]. One (n_tile, stage) record is contiguous, so the
// kernel fetches it with a single bulk copy. Chunk c (counted over the whole stage) of
// row r sits at position r ^ (2c & 6) of its 2 KiB slab. Both readers are then free
// of shared-memory bank conflicts: the tcgen05 dequant thread of row r reads chunk c
// at byte c*2048 + (r ^ (2c & 6))*16 (consecutive rows, one chunk: a permutation of 8
// consecutive 16-byte slots), and a lane quad of the small-M kernel reads chunks 0..3
// of rows r and r+1 (eight different slots modulo 8). The scale words of the k-blocks
// travel in the same record, so the dequant warps never touch global memory. K is
// padded to a whole stage with zero codes and zero scales.
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

#include "decode.cuh"

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

struct PackParams {
  const uint32_t* q;        // natural codes, (N, K*bits/8) bytes viewed as words
  const uint16_t* scales;   // U4_SZ: (N, groups) in the activation dtype
  const uint16_t* zeros;    // U4_SZ: (N, groups) or nullptr (zero-point 8)
  const uint8_t* exps;      // FP4_E8M0: (N, K/32) exponent bytes
  uint32_t* wp;             // packed image
  int N, K, bits;
  int mode;                 // 0 integer codes -> 16-bit, 1 integer codes -> 8-bit, 2 e2m1 -> bf16, 3 natural order
  int sz_kind;              // 0 none, 1 u4 scale/zero words, 2 e8m0 byte quads, 3 plain scale in the low half
  int bf16;                 // activation dtype of the scale words
  int n_tiles, st_total;
  int code_words_per_kb;    // 1024 or 2048
  int stage_words;          // 2 * code_words_per_kb + 128 * nsz
  int elems_per_kblock;     // 64 or 128
  int group_size;           // U4_SZ
  int groups;               // K / group_size (U4_SZ)
  int nsz;                  // scale words per row and stage (0, 1 or 2)
};

// One thread per 32-bit word of the packed image:
//   [n_tile][stage][ codes: [k-block 2][chunk][row 128][4 words] | scale words: [nsz][row 128] ]
__global__ void pack_image_kernel(const PackParams p) {
  const long long total = static_cast<long long>(p.n_tiles) * p.st_total * p.stage_words;
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  const int wi = static_cast<int>(idx % p.stage_words);
  const long long rest = idx / p.stage_words;
  const int stg = static_cast<int>(rest % p.st_total);
  const int nt = static_cast<int>(rest / p.st_total);
  uint32_t out = 0;
  if (wi < 2 * p.code_words_per_kb) {
    const int h = wi / p.code_words_per_kb;
    const int r = wi % p.code_words_per_kb;
    const int j = r & 3;
    const int c = r >> 9;
    const int chunk_in_stage = h * (p.code_words_per_kb >> 9) + c;
    const int row = ((r >> 2) & 127) ^ chunk_swizzle(chunk_in_stage);   // the row stored at this position
    const int n = nt * 128 + row;
    const int elems_per_word = 32 / p.bits;
    const int k0 = (stg * 2 + h) * p.elems_per_kblock + (c * 4 + j) * elems_per_word;
    uint32_t w = 0;
    if (n < p.N && k0 < p.K) w = p.q[(static_cast<long long>(n) * p.K + k0) / elems_per_word];
    if (p.mode == 0) out = interleave_word(w, p.bits, 16);
    else if (p.mode == 1) out = interleave_word(w, p.bits, 8);
    else if (p.mode == 2) out = twiddle_fp4_word(w);
    else out = w;
  } else {
    const int r = wi - 2 * p.code_words_per_kb;
    const int si = r >> 7;
    const int row = r & 127;
    const int n = nt * 128 + row;
    if (n < p.N) {
      if (p.sz_kind == 1 || p.sz_kind == 3) {
        const int k_start = (stg * 2 + (p.nsz == 2 ? si : 0)) * 64;
        if (k_start < p.K) {
          const int g = min(k_start / p.group_size, p.groups - 1);
          const uint16_t s_raw = p.scales[static_cast<size_t>(n) * p.groups + g];
          uint16_t lo, hi;
          if (p.sz_kind == 3) {
            lo = s_raw;
            hi = 0;
          } else if (p.bf16) {
            const float s = __bfloat162float(__ushort_as_bfloat16(s_raw));
            const float z = p.zeros ? __bfloat162float(__ushort_as_bfloat16(p.zeros[static_cast<size_t>(n) * p.groups + g])) : 8.f;
            lo = __bfloat16_as_ushort(__float2bfloat16_rn(s * 64.f));
            hi = __bfloat16_as_ushort(__float2bfloat16_rn(-z * 0.015625f));
          } else {
            const float s = __half2float(__ushort_as_half(s_raw));
            const float z = p.zeros ? __half2float(__ushort_as_half(p.zeros[static_cast<size_t>(n) * p.groups + g])) : 8.f;
            lo = __half_as_ushort(__float2half_rn(s * 512.f));
            hi = __half_as_ushort(__float2half_rn(-z * 0.001953125f));
          }
          out = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
        }
      } else if (p.sz_kind == 2) {
        const int blocks32 = p.K / 32;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int kb32 = stg * 4 + b;
          if (kb32 < blocks32) out |= static_cast<uint32_t>(p.exps[static_cast<size_t>(n) * blocks32 + kb32]) << (8 * b);
        }
      }
    }
  }
  p.wp[idx] = out;
}

}  // namespace b200dq
