// Memory-bound path for at most 16 tokens (decode shapes): C[m, n] = sum_k A[m, k] * W[n, k]
// with W dequantised in registers from the same packed image the tcgen05 kernel streams.
//
// With so few tokens the tcgen05 pipeline (TMA -> registers -> TMEM -> MMA, a chain of
// barrier hand-offs per k-block) is latency-bound far below HBM speed. Here every warp is
// independent: it reads packed codes straight from global memory with 128-bit loads (a
// bulk L2 prefetch runs a few stages ahead), decodes them with the same register
// routines, and multiplies with warp-level mma.sync.m16n8k16 -- weights are the 16-row
// operand, tokens the 8-column one -- so the only waits are the hardware scoreboard's.
// The reference's counterpart is its split-K SIMT GEMV (examples/dequantize_gemm/
// example_dequant_gemv_fp16xint4.py:21-136, examples/gemv/example_gemv.py:58-96).
// Measured alternatives that lost on B200: a plain SIMT variant on the mixed-precision
// scalar FMA (fma.rn.f32.bf16) for 1-2 tokens, and a lane-private cp.async ring in
// shared memory in place of the direct loads. mma.sync.m16n8k16 (bf16) sustains one
// instruction per 8 cycles per SM sub-partition here (dependent-issue latency 21 cycles), so
// the legacy tensor path is not the limit (1.5 k to 3.1 k instructions per sub-partition on
// the 28672 x 8192 benchmark weight). 4-bit integer weights (with or without scales) and
// e2m1 weights with e8m0 block scales take this path.
//
// Work split: the same stream-K schedule, segments and scratch format as the tcgen05
// kernel (token tile 16), so the same fix-up pass finishes tiles cut between CTAs. Inside
// a CTA, warp w takes weight rows [64 * (w & 1), +64) of the 128-row tile and the stages
// st_begin + (w >> 1), + 8, ...; the 8 partial sums of every output are added in a fixed
// order through shared memory when the segment ends (deterministic).
//
// Fragment mapping. The instruction fixes which lane holds which (row, k) slot: lanes
// 4j..4j+3 hold rows j and j+8, lane l the k slots {2q, 2q+1, 2q+8, 2q+9}, q = l % 4. A
// dot product does not care which real k sits in which slot as long as both operands
// agree, so lane (j, q) loads the 16-byte chunk q of rows j and j+8 (32 consecutive k
// each) and MMA i of 8 uses the lane's real k = 32q + 4i .. 4i+3 for its four slots; the
// activation fragment is then 8 contiguous bytes of the token row.
#pragma once
#include "skinny_launch.h"
#include "umma_gemm.cuh"

namespace b200dq {

constexpr int kSkinnyThreads = 512;
constexpr int kSkinnyRedStride = kTileRows + 4;      // padded row pitch of the reduction buffer (floats)
constexpr int kSkinnyPhases = kSkinnyThreads / 64;   // mma.sync kernel: 2 row halves x 8 phases
constexpr int kSkinnySmemBytes = kSkinnyPhases * kSkinnyTokens * kSkinnyRedStride * 4;
#ifndef B200DQ_SKINNY_PREFETCH
#define B200DQ_SKINNY_PREFETCH 2                     // stages (per warp) requested into L2 ahead of use
#endif

__device__ __forceinline__ uint4 ldg_stream_v4(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}

__device__ __forceinline__ void prefetch_l2_bulk(const void* ptr, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(ptr), "r"(bytes) : "memory");
}

template <bool kBf16>
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  if constexpr (kBf16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

// `sz` is the row's scale word of the stage; `q` the lane's chunk (uint4: one {scale, zero}
// pair per group; e2m1: one e8m0 byte per chunk of 32 codes).
template <int WF, bool kBf16>
__device__ __forceinline__ void skinny_decode(const GemmParams& p, const uint4& codes, uint32_t sz, int q,
                                              uint32_t (&out)[16]) {
  if constexpr (WF == WF_U4_SZ) decode_u4_chunk<kBf16>(codes, sz, out);
  else if constexpr (WF == WF_U4_RAW) decode_u4_chunk_noscale<kBf16, false>(codes, out);
  else if constexpr (WF == WF_S4_RAW) decode_u4_chunk_noscale<kBf16, true>(codes, out);
  else decode_fp4_chunk(codes, 126 + static_cast<int>((sz >> (8 * q)) & 0xffu) - p.fp4_exp_bias, out);
}

// One summed output of a segment: a raw partial into the CTA's scratch slot, or the
// finished value into C.
__device__ __forceinline__ void skinny_store(const GemmParams& p, const Segment& w, int tok, int row, float v) {
  const uint32_t bits = __float_as_uint(v);
  if (w.slot >= 0) {
    p.partial[(static_cast<size_t>(w.slot) * kSkinnyTokens + tok) * kTileRows + row] = bits;
    return;
  }
  const int m = w.row0 + tok;
  const int n = w.n_tile * kTileRows + row;
  if (m >= w.row_end || n >= p.N) return;
  const bool trans = (p.flags & GF_TRANS_C) != 0;
  const size_t idx = trans ? static_cast<size_t>(n) * p.ldc + m : static_cast<size_t>(m) * p.ldc + n;
  switch (p.out_type) {
    case OUT_F16: reinterpret_cast<__half*>(p.c)[idx] = finish_value<__half, false>(p, bits, m, n); break;
    case OUT_BF16: reinterpret_cast<__nv_bfloat16*>(p.c)[idx] = finish_value<__nv_bfloat16, false>(p, bits, m, n); break;
    default: reinterpret_cast<float*>(p.c)[idx] = finish_value<float, false>(p, bits, m, n); break;
  }
}

// ---------------------------------------------------------------------------------------
// mma.sync kernel. NT: 8-token column blocks (1 for M <= 8, else 2).
// Warp w: rows [64 * (w & 1), +64) of the tile, phase w >> 1.
// ---------------------------------------------------------------------------------------
template <int NT, int WF, int ACT>
__global__ void __launch_bounds__(kSkinnyThreads, 1) skinny_dequant_gemm_kernel(const GemmParams p) {
  static_assert(WF == WF_U4_SZ || WF == WF_U4_RAW || WF == WF_S4_RAW || WF == WF_FP4_E8M0,
                "4-bit weights on 16-bit activations");
  static_assert(WF != WF_FP4_E8M0 || ACT == ACT_BF16, "e2m1 weights decode to bf16");
  constexpr bool kBf16 = (ACT == ACT_BF16);
  constexpr int PH = kSkinnyPhases;
  constexpr int PD = B200DQ_SKINNY_PREFETCH;
  constexpr int kCodeBytes = 2 * codes_per_kblock_bytes(WF);   // 8192: four 2 KiB chunk slabs
  extern __shared__ float red[];                               // [phase][token][row (padded)]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int half = warp & 1;
  const int phase = warp >> 1;
  const int j = lane >> 2;
  const int q = lane & 3;
  const uint16_t* A = reinterpret_cast<const uint16_t*>(p.a);

  SegmentWalk walk(p);
  Segment w;
  while (walk.next(p, w)) {
    float acc[4][NT][4];
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[mt][nt][c] = 0.f;

    const uint8_t* tile_base = p.wp + w.wp_off + static_cast<size_t>(w.n_tile) * p.st_total * p.stage_bytes;
    const bool prefetcher = (PD > 0) && half == 0 && lane == 0;
    if (prefetcher) {
#pragma unroll
      for (int d = 0; d < PD; ++d) {
        const int s = w.st_begin + phase + PH * d;
        if (s < w.st_end) prefetch_l2_bulk(tile_base + static_cast<size_t>(s) * p.stage_bytes, p.stage_bytes);
      }
    }
    // the lane's token rows (one per 8-token block)
    const uint16_t* arow[NT];
    bool tok_ok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int t = w.row0 + nt * 8 + j;
      tok_ok[nt] = t < w.row_end;
      arow[nt] = A + static_cast<size_t>(tok_ok[nt] ? t : 0) * p.K;
    }
    const int row_lo = half * 64 + j;

    for (int st = w.st_begin + phase; st < w.st_end; st += PH) {
      const uint8_t* stage = tile_base + static_cast<size_t>(st) * p.stage_bytes;
      if (prefetcher) {
        const int s = st + PH * PD;
        if (s < w.st_end) prefetch_l2_bulk(tile_base + static_cast<size_t>(s) * p.stage_bytes, p.stage_bytes);
      }
      // ---- all loads of the stage first: 8 code chunks, their scale words, the activations
      uint4 codes[4][2];
      uint32_t szw[4][2];
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = row_lo + mt * 16 + h * 8;
          codes[mt][h] = ldg_stream_v4(stage + q * 2048 + r * 16);
          if constexpr (WF == WF_U4_SZ) {
            const int si = p.sz_per_kb ? (q >> 1) : 0;
            szw[mt][h] = __ldg(reinterpret_cast<const uint32_t*>(stage + kCodeBytes + si * 512) + r);
          } else if constexpr (WF == WF_FP4_E8M0) {
            szw[mt][h] = __ldg(reinterpret_cast<const uint32_t*>(stage + kCodeBytes) + r);
          } else {
            szw[mt][h] = 0;
          }
        }
      }
      const int k0 = st * 128 + q * 32;
      uint4 av[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        if (tok_ok[nt] && k0 < p.K) {
          const uint4* src = reinterpret_cast<const uint4*>(arow[nt] + k0);
#pragma unroll
          for (int v = 0; v < 4; ++v) av[nt][v] = __ldg(src + v);
        } else {
#pragma unroll
          for (int v = 0; v < 4; ++v) av[nt][v] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      // ---- decode and multiply, one 16-row block at a time
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        uint32_t wa[16], wb[16];
        skinny_decode<WF, kBf16>(p, codes[mt][0], szw[mt][0], q, wa);
        skinny_decode<WF, kBf16>(p, codes[mt][1], szw[mt][1], q, wb);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t* b = reinterpret_cast<const uint32_t*>(&av[nt][0]);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            mma_m16n8k16<kBf16>(acc[mt][nt], wa[2 * i], wb[2 * i], wa[2 * i + 1], wb[2 * i + 1], b[2 * i], b[2 * i + 1]);
        }
      }
    }

    // ---- add the phases' partial sums in a fixed order
    __syncthreads();   // the previous segment's readers are done with the buffer
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int row = half * 64 + mt * 16 + j + (c >> 1) * 8;
          const int tok = nt * 8 + 2 * q + (c & 1);
          red[(phase * kSkinnyTokens + tok) * kSkinnyRedStride + row] = acc[mt][nt][c];
        }
    __syncthreads();
    const int n_tok = NT * 8;
    for (int o = threadIdx.x; o < n_tok * kTileRows; o += kSkinnyThreads) {
      const int tok = o >> 7;
      const int row = o & (kTileRows - 1);
      float v = 0.f;
#pragma unroll
      for (int ph = 0; ph < PH; ++ph) v += red[(ph * kSkinnyTokens + tok) * kSkinnyRedStride + row];
      skinny_store(p, w, tok, row, v);
    }
  }
}

}  // namespace b200dq
