// Register dequantisation of packed low-bit weights, one 16-byte chunk at a
// time. Each routine turns 4 packed 32-bit words into 16 registers that are
// stored to consecutive TMEM columns (or used directly by the SIMT GEMV):
//   * 16-bit targets: register r holds K elements (2r, 2r+1), even k in the low half;
//   * 8-bit targets:  register r holds K elements (4r .. 4r+3), lowest k in byte 0.
//
// The bit tricks restate what the reference emits from
// examples/dequantize_gemm/quantize/lop3.py (decode_i4u_to_f16 :6-39, the
// scale/zeros variants :41-176, decode_i2s_to_i8s / decode_i4s_to_i8s :893-1047)
// and quantize/mxfp.py:6-49 (fp4 -> bf16 by mask/shift then * 2^126). The
// reference has fp16 LOP3 decoders only. Here the scaled uint4 decoders read the
// masked code as a 16-bit subnormal (see decode_u4_chunk); the unscaled ones use the
// magic-exponent trick (0x6400 | q = 1024 + q in fp16, 0x4300 | q = 128 + q in bf16,
// which has 7 mantissa bits, so 128 + q is exact).
//
// Offline layouts expected in each 32-bit word (produced by pack_weight):
//   u4 -> 16 bit : element e at bit (e % 2) * 16 + (e / 2) * 4        (8 per word)
//   u2 -> 16 bit : element e at bit (e % 2) * 16 + (e / 2) * 2        (16 per word)
//   u2/u4 -> 8 bit: element e at bit (e % 4) * 8 + (e / 4) * nbits    (16 or 8 per word)
//   e2m1 -> bf16 : see decode_fp4_chunk
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200dq {

// Position of row r inside the 2 KiB slab that holds chunk c (counted over the whole stage)
// of a packed stage: r ^ chunk_swizzle(c). See pack_kernels.cuh for why.
__host__ __device__ constexpr int chunk_swizzle(int chunk_in_stage) { return (2 * chunk_in_stage) & 6; }

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t magic) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(magic));
  return r;
}

__device__ __forceinline__ uint32_t bf162_as_u32(__nv_bfloat162 v) {
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ __nv_bfloat162 u32_as_bf162(uint32_t v) {
  return *reinterpret_cast<__nv_bfloat162*>(&v);
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

// uint4 with per-group scale s and zero-point z, weight = (q - z) * s.
// The 4-bit code is masked in place: as a 16-bit float pattern it is the
// subnormal q * 2^-133 (bf16) or q * 2^-24 (fp16). One fma by P = 2^127 (2^15)
// with addend -z * 2^-6 (-z * 2^-9) gives (q - z) * 2^-6 (2^-9) -- exact whenever
// q - z fits the mantissa (always for integer z) -- and one multiply by
// s * 2^6 (s * 2^9) lands on the same value the reference's ref_program computes in
// fp32 and rounds once: RN((q - z) * s). sz word: low 16 bits = s * 2^6 (2^9),
// high 16 bits = -z * 2^-6 (2^-9), both prepared offline in the activation dtype.
// Codes 1 and 3 of each 16-bit half stay one nibble up (mask 0x00f0): the pattern is then
// 16 q in the same units (a bf16 with q >= 8 has exponent field 1, which continues the
// subnormal scale, so it still reads q * 2^-129 exactly) and the fma's factor is 2^123 (2^11)
// instead -- one shift and four masks per eight codes.
// One 32-bit word (8 codes) -> 4 registers; s2 / nz2 are the scale word's halves, each
// duplicated into both 16-bit lanes.
template <bool kBf16>
__device__ __forceinline__ void decode_u4_word(uint32_t w, uint32_t s2, uint32_t nz2, uint32_t* out) {
  const uint32_t wh = w >> 8;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t src = (i & 2) ? wh : w;
    const uint32_t x = src & ((i & 1) ? 0x00f000f0u : 0x000f000fu);
    if constexpr (kBf16) {
      const uint32_t pw2 = (i & 1) ? 0x7d007d00u : 0x7f007f00u;   // 2^123 : 2^127
      const __nv_bfloat162 t = __hfma2(u32_as_bf162(x), u32_as_bf162(pw2), u32_as_bf162(nz2));
      out[i] = bf162_as_u32(__hmul2(t, u32_as_bf162(s2)));
    } else {
      const uint32_t pw2 = (i & 1) ? 0x68006800u : 0x78007800u;   // 2^11 : 2^15
      const __half2 t = __hfma2(u32_as_h2(x), u32_as_h2(pw2), u32_as_h2(nz2));
      out[i] = h2_as_u32(__hmul2(t, u32_as_h2(s2)));
    }
  }
}

template <bool kBf16>
__device__ __forceinline__ void decode_u4_chunk(const uint4& packed, uint32_t sz, uint32_t (&out)[16]) {
  const uint32_t s2 = __byte_perm(sz, 0, 0x1010);
  const uint32_t nz2 = __byte_perm(sz, 0, 0x3232);
  decode_u4_word<kBf16>(packed.x, s2, nz2, &out[0]);
  decode_u4_word<kBf16>(packed.y, s2, nz2, &out[4]);
  decode_u4_word<kBf16>(packed.z, s2, nz2, &out[8]);
  decode_u4_word<kBf16>(packed.w, s2, nz2, &out[12]);
}

// 2-bit codes with per-group scale and zero-point, weight = (q - z) * s: the same subnormal
// trick as decode_u4_word. A word holds 16 codes, element e at bit (e % 2) * 16 + (e / 2) * 2;
// the pair (2i, 2i + 1) is masked in place at bits [2 (i % 4), +2) of the word or of the word
// shifted down by 8 (a 16-bit pattern is linear in its low 8 bits for bf16 -- 7 mantissa bits and
// the lowest exponent bit -- so the field may sit at bits 0, 2, 4 or 6), and the fma's
// power-of-two factor takes out the field's position: 2^(127 - 2 (i % 4)) in bf16,
// 2^(15 - 2 (i % 4)) in fp16. Restates what the reference's decode_i2u_to_f16 / decode_i2s_to_f16
// and their scale / zeros variants compute (quantize/lop3.py:424-677); z = 2 is its signed form.
template <bool kBf16>
__device__ __forceinline__ void decode_u2_word(uint32_t w, uint32_t s2, uint32_t nz2, uint32_t* out) {
  const uint32_t wh = w >> 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t src = (i & 4) ? wh : w;
    const int pos = i & 3;
    const uint32_t x = src & (0x00030003u << (2 * pos));
    if constexpr (kBf16) {
      const uint32_t pw2 = 0x7f007f00u - 0x01000100u * pos;       // 2^(127 - 2 pos) in both halves
      const __nv_bfloat162 t = __hfma2(u32_as_bf162(x), u32_as_bf162(pw2), u32_as_bf162(nz2));
      out[i] = bf162_as_u32(__hmul2(t, u32_as_bf162(s2)));
    } else {
      const uint32_t pw2 = 0x78007800u - 0x08000800u * pos;       // 2^(15 - 2 pos)
      const __half2 t = __hfma2(u32_as_h2(x), u32_as_h2(pw2), u32_as_h2(nz2));
      out[i] = h2_as_u32(__hmul2(t, u32_as_h2(s2)));
    }
  }
}

// One 16-byte chunk = 64 codes of one row = a whole k-block: 32 registers.
template <bool kBf16>
__device__ __forceinline__ void decode_u2_chunk(const uint4& packed, uint32_t sz, uint32_t (&out)[32]) {
  const uint32_t s2 = __byte_perm(sz, 0, 0x1010);
  const uint32_t nz2 = __byte_perm(sz, 0, 0x3232);
  decode_u2_word<kBf16>(packed.x, s2, nz2, &out[0]);
  decode_u2_word<kBf16>(packed.y, s2, nz2, &out[8]);
  decode_u2_word<kBf16>(packed.z, s2, nz2, &out[16]);
  decode_u2_word<kBf16>(packed.w, s2, nz2, &out[24]);
}

// 4-bit index into a 16-entry table of 16-bit floats, times a per-group scale (NF4 and other
// codebooks; the reference names NF4 among its benchmarked formats but ships no decoder).
// Codes are in natural nibble order (element e at bit 4 e). The table lives in eight registers,
// low bytes and high bytes apart; four codes are looked up at once with byte permutes: the low
// three bits of each nibble select among entries 0-7 and among entries 8-15, bit 3 (turned into
// a byte mask by the permute's sign replication) picks between the two, and two more permutes
// interleave low and high bytes into two registers of two elements each.
template <bool kBf16>
__device__ __forceinline__ void decode_lut4_word(uint32_t w, uint32_t s2, const uint32_t (&lo)[4],
                                                 const uint32_t (&hi)[4], uint32_t* out) {
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const uint32_t x = k ? (w >> 16) : w;
    const uint32_t sel = x & 0x7777u;
    uint32_t m;                                            // byte j = 0xff if bit 3 of nibble j is set
    asm("prmt.b32 %0, %1, %2, 0xD9C8;" : "=r"(m) : "r"(x << 4), "r"(x));   // selector bit 3: replicate the byte's sign
    const uint32_t l = (__byte_perm(lo[0], lo[1], sel) & ~m) | (__byte_perm(lo[2], lo[3], sel) & m);
    const uint32_t h = (__byte_perm(hi[0], hi[1], sel) & ~m) | (__byte_perm(hi[2], hi[3], sel) & m);
    const uint32_t v0 = __byte_perm(l, h, 0x5140), v1 = __byte_perm(l, h, 0x7362);
    if constexpr (kBf16) {
      out[2 * k] = bf162_as_u32(__hmul2(u32_as_bf162(v0), u32_as_bf162(s2)));
      out[2 * k + 1] = bf162_as_u32(__hmul2(u32_as_bf162(v1), u32_as_bf162(s2)));
    } else {
      out[2 * k] = h2_as_u32(__hmul2(u32_as_h2(v0), u32_as_h2(s2)));
      out[2 * k + 1] = h2_as_u32(__hmul2(u32_as_h2(v1), u32_as_h2(s2)));
    }
  }
}

template <bool kBf16>
__device__ __forceinline__ void decode_lut4_chunk(const uint4& packed, uint32_t sz, const uint32_t (&lo)[4],
                                                  const uint32_t (&hi)[4], uint32_t (&out)[16]) {
  const uint32_t s2 = __byte_perm(sz, 0, 0x1010);
  decode_lut4_word<kBf16>(packed.x, s2, lo, hi, &out[0]);
  decode_lut4_word<kBf16>(packed.y, s2, lo, hi, &out[4]);
  decode_lut4_word<kBf16>(packed.z, s2, lo, hi, &out[8]);
  decode_lut4_word<kBf16>(packed.w, s2, lo, hi, &out[12]);
}

// No scale at all: weight = q (unsigned) or q - 8 (signed storage), as in the
// reference's fine-grained example (example_dequant_gemm_fine_grained.py:11-13).
template <bool kBf16, bool kSigned>
__device__ __forceinline__ void decode_u4_word_noscale(uint32_t w, uint32_t* out) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t t = w >> (4 * i);
    if constexpr (kBf16) {
      const uint32_t x = lop3_and_or(t, 0x000f000fu, 0x43004300u);
      out[i] = bf162_as_u32(__hsub2(u32_as_bf162(x), u32_as_bf162(kSigned ? 0x43084308u : 0x43004300u)));
    } else {
      const uint32_t x = lop3_and_or(t, 0x000f000fu, 0x64006400u);
      out[i] = h2_as_u32(__hsub2(u32_as_h2(x), u32_as_h2(kSigned ? 0x64086408u : 0x64006400u)));
    }
  }
}

template <bool kBf16, bool kSigned>
__device__ __forceinline__ void decode_u4_chunk_noscale(const uint4& packed, uint32_t (&out)[16]) {
  decode_u4_word_noscale<kBf16, kSigned>(packed.x, &out[0]);
  decode_u4_word_noscale<kBf16, kSigned>(packed.y, &out[4]);
  decode_u4_word_noscale<kBf16, kSigned>(packed.z, &out[8]);
  decode_u4_word_noscale<kBf16, kSigned>(packed.w, &out[12]);
}

// 2-bit codes -> int8. 16 codes per word, word j of the chunk covers K
// elements 16j .. 16j+15. `bias` is subtracted bytewise (0x02020202 for the
// ternary code q = w + 2, 0 for unsigned codes).
__device__ __forceinline__ void decode_i2_chunk(const uint4& packed, uint32_t bias, uint32_t (&out)[16]) {
  const uint32_t w[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t x = (w[j] >> (2 * i)) & 0x03030303u;
      out[4 * j + i] = __vsub4(x, bias);
    }
  }
}

// 4-bit codes -> int8. 8 codes per word; a 16-byte chunk yields only 8
// registers (32 K elements), so the caller decodes two chunks per 64 elements.
__device__ __forceinline__ void decode_i4_chunk(const uint4& packed, uint32_t bias, uint32_t (&out)[8]) {
  const uint32_t w[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint32_t x = (w[j] >> (4 * i)) & 0x0f0f0f0fu;
      out[2 * j + i] = __vsub4(x, bias);
    }
  }
}

// e2m1 -> bf16 (or fp16) with a power-of-two block scale.
// Offline bit layout per 16-bit half (4 codes; code = s e1 e0 m): the first
// three codes sit where one shift and one mask move them to bf16 bit positions
// (sign -> 15, e1 e0 m -> 8..6):
//   code 0: s@15  e1 e0 m @ 8 7 6      (mask 0x81c0, no shift)
//   code 1: s@12  e1 e0 m @ 5 4 3      (shift left 3)
//   code 2: s@9   e1 e0 m @ 2 1 0      (shift left 6)
//   code 3: s@14  e1@13   e0 m @ 11 10 (three pieces)
// and the two halves of a word carry K elements (8j+2i, 8j+2i+1) for code i.
// The masked pattern is a bf16 whose exponent field is only e (0..3); times
// 2^126 it becomes the e2m1 value {0, .5, 1, 1.5, 2, 3, 4, 6} exactly (e = 0 is
// a bf16 subnormal, which the multiply normalises). `mul_lo`/`mul_hi` are the
// two factors whose product is 2^126 * 2^(block exponent).
//
// `exp_add` = 0x00800080 selects the reference's other fp4 rule, value = 2^(e-1) * (1 + m/2)
// for every code (no zero, no subnormal: _tir_u8_to_f4_to_f16,
// examples/dequantize_gemm/example_dequant_gemm_fp4_hopper.py:10-29, and torch_convert,
// dequantize_utils.py:57-84): one more in the exponent field makes every pattern a normal
// number, and the caller halves the factor.
//
// fp16 target: the three bits e1 e0 m move up to fp16's positions 11..9 (exponent field e of
// five bits, mantissa top bit m); times 2^14 the same values come out (e = 0 is an fp16
// subnormal). fp16 has no room for a block exponent, so only one fixed factor is applied.
template <bool kBf16>
__device__ __forceinline__ void decode_fp4_word(uint32_t w, uint32_t m1, uint32_t m2, uint32_t exp_add, uint32_t* out) {
  const uint32_t kMask = 0x81c081c0u;
  uint32_t v[4];
  v[0] = w & kMask;
  v[1] = (w << 3) & kMask;
  v[2] = (w << 6) & kMask;
  uint32_t t = (w << 1) & 0x80008000u;
  t = lop3_and_or(w >> 5, 0x01000100u, t);
  t = lop3_and_or(w >> 4, 0x00c000c0u, t);
  v[3] = t;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (kBf16) {
      __nv_bfloat162 x = __hmul2(u32_as_bf162(v[i] + exp_add), u32_as_bf162(m1));
      out[i] = bf162_as_u32(__hmul2(x, u32_as_bf162(m2)));
    } else {
      const uint32_t h = lop3_and_or(v[i] << 3, 0x0e000e00u, v[i] & 0x80008000u) + exp_add;
      out[i] = h2_as_u32(__hmul2(u32_as_h2(h), u32_as_h2(m1)));
    }
  }
}

// e8m0 byte e -> the pair of bf16 factors (m1, m2) with m1 * m2 = 2^126 * 2^(e - bias_e).
// exp_total = 126 + e - bias_e is split so both factors are normal bf16 numbers.
__device__ __forceinline__ void fp4_scale_factors(int exp_total, uint32_t& m1, uint32_t& m2) {
  // m1 = 2^a, m2 = 2^b, a + b = exp_total, a = clamp(exp_total, -126, 127) / 2 rounded toward +inf
  int a = (exp_total + 1) >> 1;
  int b = exp_total - a;
  a = max(-126, min(127, a));
  b = max(-126, min(127, b));
  const uint32_t ha = static_cast<uint32_t>(a + 127) << 7;
  const uint32_t hb = static_cast<uint32_t>(b + 127) << 7;
  m1 = ha | (ha << 16);
  m2 = hb | (hb << 16);
}

// `exp_total`: power of two that takes the masked pattern to the weight (126 + block exponent
// for true e2m1 in bf16, one less for the reference's simple rule); `simple`: that rule. The
// fp16 form ignores the block exponent: 2^14 (true e2m1) or 2^13 (simple).
template <bool kBf16>
__device__ __forceinline__ void decode_fp4_chunk(const uint4& packed, int exp_total, bool simple, uint32_t (&out)[16]) {
  uint32_t m1, m2 = 0;
  uint32_t exp_add;
  if constexpr (kBf16) {
    fp4_scale_factors(exp_total - (simple ? 1 : 0), m1, m2);
    exp_add = simple ? 0x00800080u : 0u;
  } else {
    m1 = simple ? 0x70007000u : 0x74007400u;     // 2^13 : 2^14
    exp_add = simple ? 0x04000400u : 0u;
  }
  decode_fp4_word<kBf16>(packed.x, m1, m2, exp_add, &out[0]);
  decode_fp4_word<kBf16>(packed.y, m1, m2, exp_add, &out[4]);
  decode_fp4_word<kBf16>(packed.z, m1, m2, exp_add, &out[8]);
  decode_fp4_word<kBf16>(packed.w, m1, m2, exp_add, &out[12]);
}

}  // namespace b200dq
