// Decode shapes of the integer formats: C[m, n] = sum_k A_int8[m, k] * (code[n, k] - bias) for
// at most 64 tokens, with 2- or 4-bit codes read straight from the packed image in global
// memory (no shared-memory ring, no scratch, one launch). The reference's counterpart is its
// dp4a GEMV (examples/bitnet-1.58b/kernel_benchmark/tilelang_bitnet_158_int8xint2_decode.py:
// 66-175); the weights it serves are a few megabytes, so what counts is latency: the work
// is cut into many small CTAs that each issue all their loads at once.
//
// A CTA owns 16 * MT weight rows; its 8 or 16 warps split K by stage (256 k) and add their
// int32 sums with shared-memory atomics -- integer addition, so the result does not depend on
// the order. A warp multiplies with mma.sync.m16n8k32 (u8 codes x s8 activations): weights are
// the 16-row operand, 8 tokens the column operand. The bias of the codes is taken out at the
// end, sum_k a (q - b) = sum_k a q - b sum_k a, with sum_k a accumulated by dp4a from the
// activation fragments the lanes hold anyway.
//
// Fragment mapping (the k slots of a fragment are permuted the same way in both operands, so a
// lane can use contiguous bytes): lane (j, q) = (lane / 4, lane % 4) owns the 64 k of the stage
// starting at 64 q for weight rows j and j + 8 and for token j; MMA i of 8 multiplies its
// k = 8 i .. 8 i + 7. In the image a 32-bit word holds element e at byte e % 4, field e / 4, so
// one shift and one mask give four codes of consecutive k as four bytes.
#pragma once
#include "umma_gemm.cuh"

namespace b200dq {

constexpr int kInt8SkinnyMaxThreads = 512;   // 8 or 16 warps split K (the launcher picks)
constexpr int kInt8SkinnyMaxTokens = 32;

__device__ __forceinline__ void mma_m16n8k32_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_nc_16(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}

// NT: 8-token blocks (1, 2 or 4); MT: 16-row blocks per CTA (1 or 2); WF_I2_I8 or WF_I4_I8.
template <int NT, int MT, int WF>
__global__ void __launch_bounds__(NT <= 2 ? kInt8SkinnyMaxThreads : kInt8SkinnyMaxThreads / 2) int8_skinny_gemm_kernel(const GemmParams p) {
  static_assert(WF == WF_I2_I8 || WF == WF_I4_I8, "integer codes on int8 activations");
  constexpr int kRows = 16 * MT;
  constexpr int kTok = 8 * NT;
  constexpr int kChunks = WF == WF_I2_I8 ? 1 : 2;    // 16-byte chunks that hold a lane's 64 k of one row
  __shared__ int red[kTok][kRows + 1];
  __shared__ int asum[kTok];

  const int warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int j = lane >> 2;
  const int q = lane & 3;
  for (int i = threadIdx.x; i < kTok * (kRows + 1); i += blockDim.x) (&red[0][0])[i] = 0;
  if (threadIdx.x < kTok) asum[threadIdx.x] = 0;
  __syncthreads();

  const int row0 = blockIdx.x * kRows;                  // first weight row of the CTA
  const int n_tile = row0 / kTileRows;
  const int row_in_tile = row0 % kTileRows;
  const uint8_t* tile = p.wp + static_cast<size_t>(n_tile) * p.st_total * p.stage_bytes;
  const int8_t* a = static_cast<const int8_t*>(p.a);

  int acc[MT][NT][4];
  int ones[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    ones[nt] = 0;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[mt][nt][c] = 0;
  }

  // codes of rows j and j + 8 of every 16-row block: chunk c of row r at c * 2048 + (r ^ swizzle(c)) * 16;
  // the next stage's codes are requested before this stage's are used
  uint32_t c_off[MT][2][kChunks];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int cc = 0; cc < kChunks; ++cc) {
        const int chunk = q * kChunks + cc;
        const int r = row_in_tile + mt * 16 + h * 8 + j;
        c_off[mt][h][cc] = static_cast<uint32_t>(chunk * 2048 + ((r ^ chunk_swizzle(chunk)) << 4));
      }
  uint4 next[MT][2][kChunks];
  if (warp < p.st_total) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int cc = 0; cc < kChunks; ++cc)
          next[mt][h][cc] = ldg_nc_16(tile + static_cast<size_t>(warp) * p.stage_bytes + c_off[mt][h][cc]);
  }
  for (int s = warp; s < p.st_total; s += warps) {
    uint4 codes[MT][2][kChunks];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int cc = 0; cc < kChunks; ++cc) {
          codes[mt][h][cc] = next[mt][h][cc];
          if (s + warps < p.st_total)
            next[mt][h][cc] = ldg_nc_16(tile + static_cast<size_t>(s + warps) * p.stage_bytes + c_off[mt][h][cc]);
        }
    const int k0 = s * 256 + q * 64;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      // weights of MMAs 4 half .. 4 half + 3
      uint32_t wa[MT][4][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t lo, hi;
            if constexpr (WF == WF_I2_I8) {
              const uint4& cw = codes[mt][h][0];
              const int wd = half * 2 + (i >> 1);
              const uint32_t w = wd == 0 ? cw.x : wd == 1 ? cw.y : wd == 2 ? cw.z : cw.w;
              lo = (w >> ((i & 1) * 4)) & 0x03030303u;
              hi = (w >> ((i & 1) * 4 + 2)) & 0x03030303u;
            } else {
              const uint4& cw = codes[mt][h][half];
              const uint32_t w = i == 0 ? cw.x : i == 1 ? cw.y : i == 2 ? cw.z : cw.w;
              lo = w & 0x0f0f0f0fu;
              hi = (w >> 4) & 0x0f0f0f0fu;
            }
            wa[mt][i][h] = lo;          // a0 (row j) / a1 (row j + 8): k 8 i .. 8 i + 3
            wa[mt][i][2 + h] = hi;      // a2 / a3: k 8 i + 4 .. 8 i + 7
          }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int tok = nt * 8 + j;
        uint4 b[2];
#pragma unroll
        for (int v = 0; v < 2; ++v) {
          const int k = k0 + half * 32 + v * 16;
          b[v] = (tok < p.M && k < p.K) ? *reinterpret_cast<const uint4*>(a + static_cast<size_t>(tok) * p.K + k)
                                        : make_uint4(0, 0, 0, 0);
        }
        const uint32_t bw[8] = {b[0].x, b[0].y, b[0].z, b[0].w, b[1].x, b[1].y, b[1].z, b[1].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ones[nt] = __dp4a(static_cast<int>(bw[2 * i]), 0x01010101, ones[nt]);
          ones[nt] = __dp4a(static_cast<int>(bw[2 * i + 1]), 0x01010101, ones[nt]);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            mma_m16n8k32_u8s8(acc[mt][nt], wa[mt][i][0], wa[mt][i][1], wa[mt][i][2], wa[mt][i][3], bw[2 * i], bw[2 * i + 1]);
        }
      }
    }
  }

  // ---- add the warps' sums (integers: any order gives the same bits)
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    atomicAdd(&asum[nt * 8 + j], ones[nt]);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        atomicAdd(&red[nt * 8 + 2 * q + (c & 1)][mt * 16 + j + (c >> 1) * 8], acc[mt][nt][c]);
  }
  __syncthreads();
  const int bias = static_cast<int>(p.code_bias & 0xffu);
  const bool trans = (p.flags & GF_TRANS_C) != 0;
  for (int o = threadIdx.x; o < kTok * kRows; o += blockDim.x) {
    const int m = o / kRows;
    const int n = row0 + o % kRows;
    if (m >= p.M || n >= p.N) continue;
    const uint32_t raw = static_cast<uint32_t>(red[m][o % kRows] - bias * asum[m]);
    const size_t idx = trans ? static_cast<size_t>(n) * p.ldc + m : static_cast<size_t>(m) * p.ldc + n;
    switch (p.out_type) {
      case OUT_I32: store_everywhere(p, idx, finish_value<int, true>(p, raw, m, n)); break;
      case OUT_F16: store_everywhere(p, idx, finish_value<__half, true>(p, raw, m, n)); break;
      case OUT_BF16: store_everywhere(p, idx, finish_value<__nv_bfloat16, true>(p, raw, m, n)); break;
      default: store_everywhere(p, idx, finish_value<float, true>(p, raw, m, n)); break;
    }
  }
}

}  // namespace b200dq
