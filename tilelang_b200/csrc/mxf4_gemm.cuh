// Native MXFP4 GEMM: C[M, N] = A[M, K] * W[N, K]^T with BOTH operands e2m1 codes carrying one
// e8m0 scale per 32 K elements, multiplied by tcgen05.mma kind::mxf4.block_scale (packed
// 4-bit operands straight from shared memory, the scale factors from tensor memory, fp32
// accumulation). Nothing is dequantised in registers: this is the path for activations that
// have been re-quantised to MXFP4 (b200dq_quant_mxfp4), at twice the bf16 tensor rate and a
// quarter of the operand bytes.
//
// The reference's building blocks for it are src/tl_templates/cuda/tcgen_05.h:123-178
// (tcgen05.cp of scale factors, the scale-factor shared-memory descriptor),
// src/op/tcgen5_meta.h:273-335 (block-scaled instruction descriptor; kind::mxf4 itself is not
// wired up there) and examples/deepseek_v4/fp8_fp4_gemm_1d1d_sm100.py:18-185 (the block-scaled
// mainloop, which keeps its scales group-major and transposes them in shared memory; here both
// scale tensors are stored in the 128 x 4 blocked layout, so a 512-byte piece is already the
// 32 x 16 B source tcgen05.cp.32x128b.warpx4 wants).
//
// Tile: 128 tokens (the MMA's M, one TMEM lane each) x 128 weight rows (N, fp32 columns),
// k-block = 256 K = one 128-byte swizzle atom per row = four MMAs of K = 64.
//   warp 0      : producer -- per k-block two tiled TMA loads (A codes, W codes: plain
//                 row-major (rows, K/2) byte tensors, no private image) and two bulk copies of
//                 1 KiB of scale words each
//   warp 1      : one thread copies the stage's scale factors to TMEM (4 x tcgen05.cp) and
//                 issues its four MMAs; tcgen05.commit frees the stage
//   warps 2-5   : epilogue, TMEM -> registers -> 16-byte global stores (a thread owns one
//                 output row, so its 128 values are contiguous); two accumulators, so the
//                 drain of one tile runs under the MMAs of the next
// Tiles are whole (no split-K): CTA b takes tiles b, b + grid, ... with the weight tile
// fastest. Every wait is bounded (ptx.cuh).
#pragma once
#include "mxf4_launch.h"
#include "umma_gemm.cuh"   // OutType, the SW128 descriptor helper, packed-float bit casts

namespace b200dq {

constexpr int kMxf4Threads = 192;
constexpr int kMxf4Stages = 6;
constexpr int kMxf4TileBytes = 128 * 128;          // 128 rows x 128 B of codes (256 K)
constexpr int kMxf4SfBytes = 1024;                 // scale words of 128 rows x 256 K: two 512 B pieces
constexpr int kMxf4StageBytes = 2 * kMxf4TileBytes + 2 * kMxf4SfBytes;
constexpr int kMxf4SmemBytes = 1024 + kMxf4Stages * kMxf4StageBytes + 1024;
constexpr int kMxf4AccCols = 128;                  // one accumulator: 128 fp32 columns
constexpr int kMxf4SfCol0 = 2 * kMxf4AccCols;      // scale factors behind the two accumulators

struct Mxf4Ctl {
  uint64_t full[kMxf4Stages];
  uint64_t empty[kMxf4Stages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(kMxf4Threads, 1)
mxf4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                 const Mxf4Params p) {
  extern __shared__ uint8_t mxf4_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(mxf4_smem_raw) + 1023) & ~uintptr_t(1023));
  Mxf4Ctl* ctl = reinterpret_cast<Mxf4Ctl*>(smem + kMxf4Stages * kMxf4StageBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &ctl->abort_flag;
  DeviceStatus* st = p.status;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMxf4Stages; ++i) { mbar_init(&ctl->full[i], 1); mbar_init(&ctl->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&ctl->acc_full[i], 1); mbar_init(&ctl->acc_empty[i], 4); }
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_w);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  const long long tiles = static_cast<long long>(p.m_tiles) * p.n_tiles;
  const int sf_words_per_rowblock = (p.K / 128) * 128;     // [K/128][32][4] words per 128 rows

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (long long t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        const int n_tile = static_cast<int>(t % p.n_tiles), m_tile = static_cast<int>(t / p.n_tiles);
        const uint32_t* sfa = p.sfa + static_cast<size_t>(m_tile) * sf_words_per_rowblock;
        const uint32_t* sfw = p.sfw + static_cast<size_t>(n_tile) * sf_words_per_rowblock;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          ok = mbar_wait(&ctl->empty[s], phase ^ 1u, abort_flag, st, 21);
          if (!ok) break;
          uint8_t* stage = smem + s * kMxf4StageBytes;
          mbar_arrive_expect_tx(&ctl->full[s], kMxf4StageBytes);
          tma_load_2d(stage, &tmap_a, kb * 128, m_tile * 128, &ctl->full[s]);
          tma_load_2d(stage + kMxf4TileBytes, &tmap_w, kb * 128, n_tile * 128, &ctl->full[s]);
          tma_bulk_g2s(stage + 2 * kMxf4TileBytes, sfa + static_cast<size_t>(kb) * 256, kMxf4SfBytes, &ctl->full[s]);
          tma_bulk_g2s(stage + 2 * kMxf4TileBytes + kMxf4SfBytes, sfw + static_cast<size_t>(kb) * 256, kMxf4SfBytes,
                       &ctl->full[s]);
          if (++s == kMxf4Stages) { s = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- scale-factor copies and MMAs ----------------
    if (lane == 0) {
      uint32_t s = 0, phase = 0, tc = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < tiles; t += gridDim.x, ++tc) {
        const uint32_t buf = tc & 1u;
        ok &= mbar_wait(&ctl->acc_empty[buf], ((tc >> 1) & 1u) ^ 1u, abort_flag, st, 22);
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + buf * kMxf4AccCols;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          ok &= mbar_wait(&ctl->full[s], phase, abort_flag, st, 23);
          tc_fence_after_sync();
          if (ok) {
            const uint32_t stage = smem_u32(smem + s * kMxf4StageBytes);
            const uint32_t sf_cols = tmem_base + kMxf4SfCol0 + s * 16;       // A: 8 columns, W: 8 columns
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              tmem_cp_32x128b_warpx4(sf_cols + c * 4, make_sf_desc(stage + 2 * kMxf4TileBytes + c * 512));
              tmem_cp_32x128b_warpx4(sf_cols + 8 + c * 4, make_sf_desc(stage + 2 * kMxf4TileBytes + kMxf4SfBytes + c * 512));
            }
            const uint64_t a_desc = make_smem_desc_sw128(stage);
            const uint64_t b_desc = make_smem_desc_sw128(stage + kMxf4TileBytes);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              // MMA j covers K [64 j, 64 j + 64) of the k-block: scale bytes 2j, 2j + 1 of the row,
              // i.e. word j / 2, byte pair (j % 2)
              const uint32_t sf_id = static_cast<uint32_t>(j & 1) * 2u;
              const uint32_t idesc = make_idesc_mxf4(128, 128, sf_id, sf_id);
              umma_mxf4_ss(acc, a_desc + 2 * j, b_desc + 2 * j, idesc, sf_cols + (j >> 1) * 4,
                           sf_cols + 8 + (j >> 1) * 4, (kb | j) != 0 ? 1u : 0u);
            }
          }
          tc_commit(&ctl->empty[s]);
          if (++s == kMxf4Stages) { s = 0; phase ^= 1u; }
        }
        tc_commit(&ctl->acc_full[buf]);
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 take TMEM lane quarters (warp % 4) ----------------
    const int quarter = warp & 3;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t tc = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < tiles; t += gridDim.x, ++tc) {
      const int n_tile = static_cast<int>(t % p.n_tiles), m_tile = static_cast<int>(t / p.n_tiles);
      const uint32_t buf = tc & 1u;
      ok &= mbar_wait(&ctl->acc_full[buf], (tc >> 1) & 1u, abort_flag, st, 24);
      tc_fence_after_sync();
      const int m = m_tile * 128 + quarter * 32 + lane;
      const int n0 = n_tile * 128;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + buf * kMxf4AccCols + c * 32, v);
        tc_wait_ld();
        if (c == 3) {
          // the accumulator goes back to the MMA thread as soon as its last columns are in registers
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
        }
        if (m < p.M && ok) {
          const int n = n0 + c * 32;
          if (p.out_type == OUT_F32) {
            float* dst = reinterpret_cast<float*>(p.c) + static_cast<size_t>(m) * p.N + n;
            if (n + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (n + i < p.N) dst[i] = __uint_as_float(v[i]);
            }
          } else {
            uint32_t h[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float lo = __uint_as_float(v[2 * i]), hi = __uint_as_float(v[2 * i + 1]);
              if (p.out_type == OUT_BF16) h[i] = bf162_as_u32(__floats2bfloat162_rn(lo, hi));
              else h[i] = h2_as_u32(__floats2half2_rn(lo, hi));
            }
            uint16_t* dst = reinterpret_cast<uint16_t*>(p.c) + static_cast<size_t>(m) * p.N + n;
            if (n + 32 <= p.N && (p.N & 7) == 0) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (n + i < p.N) dst[i] = static_cast<uint16_t>(h[i >> 1] >> (16 * (i & 1)));
            }
          }
        }
      }
    }
  }

  // ---------------- teardown ----------------
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace b200dq
