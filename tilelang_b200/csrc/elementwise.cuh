// Small HBM-bound kernels that sit directly in front of / between the GEMMs.
//
//  * absmax_quant_int8: per-token absmax int8 quantisation of the activations,
//    the reference's BitLinear.activation_quant
//    (examples/bitnet-1.58b/utils_quant.py:156-163): s = 127 / max|x| (max clamped
//    at 1e-5; evaluated as reciprocal-then-multiply, as torch does for a scalar numerator), q = round(x * s) clamped to [-128, 127], round half to even as
//    torch.round does.
//  * silu_mul: act = silu(h[:, :H]) * h[:, H:] between the two expert GEMMs of a
//    mixture-of-experts MLP (examples/fusedmoe/example_fusedmoe_torch.py:8-23),
//    computed in fp32 and rounded once to the activation dtype.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200dq {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// one CTA per row; K % 8 == 0; 16-byte loads
template <typename T>
__global__ void __launch_bounds__(256) absmax_quant_int8_kernel(const T* __restrict__ x, int8_t* __restrict__ q,
                                                                float* __restrict__ scale, int K) {
  const int row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * K);
  const int nvec = K / 8;
  float amax = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 v = xr[i];
    const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(to_f32<T>(e[j])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  __shared__ float warp_max[8];
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = warp_max[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, warp_max[w]);
  // torch evaluates `127 / t` for a Python scalar numerator as t.reciprocal() * 127
  // (two roundings); the reference's scale is that value, so the same two steps here
  const float s = __frcp_rn(fmaxf(amax, 1e-5f)) * 127.0f;
  if (threadIdx.x == 0) scale[row] = s;
  uint2* qr = reinterpret_cast<uint2*>(q + static_cast<size_t>(row) * K);
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 v = xr[i];     // second read of the row comes from L2
    const T* e = reinterpret_cast<const T*>(&v);
    uint32_t packed[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float r = rintf(to_f32<T>(e[j]) * s);
      r = fminf(fmaxf(r, -128.f), 127.f);
      packed[j >> 2] |= (static_cast<uint32_t>(static_cast<int>(r)) & 0xffu) << (8 * (j & 3));
    }
    qr[i] = make_uint2(packed[0], packed[1]);
  }
}

// h: (rows, 2H); out: (rows, H); H % 8 == 0
template <typename T>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* __restrict__ h, T* __restrict__ out, long long rows,
                                                       int H) {
  const int vec_per_row = H / 8;
  const long long total = rows * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / vec_per_row;
    const int c = static_cast<int>(idx - r * vec_per_row);
    const uint4 g = reinterpret_cast<const uint4*>(h + r * 2 * H)[c];
    const uint4 u = reinterpret_cast<const uint4*>(h + r * 2 * H + H)[c];
    const T* ge = reinterpret_cast<const T*>(&g);
    const T* ue = reinterpret_cast<const T*>(&u);
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gv = to_f32<T>(ge[j]);
      const float sv = gv / (1.0f + expf(-gv));
      oe[j] = from_f32<T>(sv * to_f32<T>(ue[j]));
    }
    reinterpret_cast<uint4*>(out + r * H)[c] = o;
  }
}

// Score-weighted combine of a mixture-of-experts layer: out[t] = sum_s w[t, s] * y[row_of[t, s]]
// over the token's top_k expert rows, accumulated in fp32 in slot order (deterministic,
// unlike an atomic scatter-add) and rounded once (the reference's combine,
// examples/fusedmoe/example_fusedmoe_torch.py:83-91, is a scatter_reduce sum).
template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const T* __restrict__ y, const long long* __restrict__ row_of,
                                                          const float* __restrict__ w, T* __restrict__ out,
                                                          long long tokens, int top_k, int H) {
  const int vec_per_row = H / 8;
  const long long total = tokens * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / vec_per_row;
    const int c = static_cast<int>(idx - t * vec_per_row);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < top_k; ++s) {
      const long long r = row_of[t * top_k + s];
      const float ws = w[t * top_k + s];
      const uint4 v = reinterpret_cast<const uint4*>(y + r * H)[c];
      const T* ve = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(ws, to_f32<T>(ve[j]), acc[j]);
    }
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) oe[j] = from_f32<T>(acc[j]);
    reinterpret_cast<uint4*>(out + t * H)[c] = o;
  }
}

// Signed int4 pairs (low nibble = even index) -> int8, 8 packed bytes per thread.
// Feeds the int8 tensor-core path for the reference's int4 x int4 GEMM
// (examples/gemm_int4/example_tilelang_gemm_int4.py:17-38, pack rule :59-67); tcgen05
// has no 4-bit integer kind.
__global__ void __launch_bounds__(256) unpack_int4_to_int8_kernel(const uint2* __restrict__ packed,
                                                                  uint4* __restrict__ out, long long nvec) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint2 v = packed[i];
    const uint32_t w[2] = {v.x, v.y};
    uint32_t o[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      // bytes b0..b3 of w[h] hold elements (2b, 2b+1); sign-extend each nibble
      const uint32_t lo = w[h] & 0x0f0f0f0fu, hi = (w[h] >> 4) & 0x0f0f0f0fu;
      const uint32_t slo = __vsub4(lo ^ 0x08080808u, 0x08080808u);   // (x ^ 8) - 8
      const uint32_t shi = __vsub4(hi ^ 0x08080808u, 0x08080808u);
      o[2 * h] = __byte_perm(slo, shi, 0x5140);       // e0 e1 e2 e3
      o[2 * h + 1] = __byte_perm(slo, shi, 0x7362);   // e4 e5 e6 e7
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// bf16 / fp16 activations -> MXFP4: per row and 32 consecutive K elements one power-of-two
// scale 2^ceil(log2(amax / 6)) (amax clamped below at 6 * 2^-126), codes = e2m1 of x / scale
// by the hardware's round-to-nearest-even conversion, two per byte with the even k in the low
// nibble, scale as an e8m0 byte. The reference's quantiser
// (examples/deepseek_v4/act_quant.py:112-164) does the same with a cast to float4_e2m1fn.
// One thread takes 8 elements (one 16-byte load, one 4-byte store); the four threads of a
// block of 32 agree on the maximum with two shuffles. Pure streaming: 2 bytes in, 0.53 out.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float hi, float lo) {
  uint32_t r;
  asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// `sf_blocked`: write the scale bytes in the 128 x 4 blocked word layout the block-scaled MMA's
// scale-factor copy reads -- byte j of word [row block m / 128][k word kb / 4][m % 32][(m % 128) / 32]
// for block kb = 4 * word + j -- instead of row-major (M, K / 32).
template <typename T>
__global__ void __launch_bounds__(256) quant_mxfp4_kernel(const T* __restrict__ x, uint32_t* __restrict__ codes,
                                                          uint8_t* __restrict__ scale_bytes, long long n_vec,
                                                          int K, int sf_blocked) {
  // n_vec = M * K / 8 is a multiple of 4 (K % 32 == 0), so the four lanes of a block are
  // in range together and the shuffles below see whole blocks
  const long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const bool in_range = v < n_vec;
  float f[8];
  if (in_range) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[v];
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = static_cast<float>(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = 0.f;
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, 6.0f * 1.17549435e-38f);                     // 6 * 2^-126
  // smallest power of two >= amax / 6, from the exponent field
  const uint32_t bits = __float_as_uint(amax / 6.0f);
  uint32_t e8 = ((bits >> 23) & 0xffu) + ((bits & 0x7fffffu) != 0u ? 1u : 0u);
  e8 = min(max(e8, 1u), 254u);
  const float inv = __uint_as_float((254u - e8) << 23);           // 2^-(e8 - 127), exact
  if (!in_range) return;
  uint32_t word = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) word |= cvt_e2m1x2(f[2 * i + 1] * inv, f[2 * i] * inv) << (8 * i);
  codes[v] = word;
  if ((threadIdx.x & 3) == 0) {
    long long at = v >> 2;                                         // row-major: m * (K / 32) + kb
    if (sf_blocked) {
      const int blocks_per_row = K >> 5;
      const long long m = at / blocks_per_row;
      const int kb = static_cast<int>(at - m * blocks_per_row);
      const int r = static_cast<int>(m & 127);
      const long long word = (m >> 7) * (static_cast<long long>(K >> 7) * 128) + ((kb >> 2) * 32 + (r & 31)) * 4 + (r >> 5);
      at = word * 4 + (kb & 3);
    }
    scale_bytes[at] = static_cast<uint8_t>(e8);
  }
}

// Row and tile prefixes of a grouped GEMM from per-group row counts that live on the device
// (a router's bincount): row_prefix[g] = rows before group g, tile_prefix[g] = tiles before it,
// a group of c rows having ceil(c / token_tile) * n_tiles tiles. One warp, a shuffle scan per 32 groups.
__global__ void grouped_prefix_kernel(const void* counts, int is_int64, int num_groups, int n_tiles, int token_tile,
                                      int32_t* __restrict__ row_prefix, int32_t* __restrict__ tile_prefix) {
  const int lane = threadIdx.x;
  int rows_before = 0, tiles_before = 0;
  for (int base = 0; base < num_groups; base += 32) {
    const int g = base + lane;
    int c = 0;
    if (g < num_groups)
      c = is_int64 ? static_cast<int>(static_cast<const long long*>(counts)[g]) : static_cast<const int*>(counts)[g];
    int r = c, t = ((c + token_tile - 1) / token_tile) * n_tiles;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int ru = __shfl_up_sync(0xffffffffu, r, d), tu = __shfl_up_sync(0xffffffffu, t, d);
      if (lane >= d) { r += ru; t += tu; }
    }
    if (g < num_groups) {
      row_prefix[g + 1] = rows_before + r;
      tile_prefix[g + 1] = tiles_before + t;
    }
    rows_before += __shfl_sync(0xffffffffu, r, 31);
    tiles_before += __shfl_sync(0xffffffffu, t, 31);
  }
  if (lane == 0) { row_prefix[0] = 0; tile_prefix[0] = 0; }
}

}  // namespace b200dq
