// Memory-bound path for at most 16 tokens (decode shapes): C[m, n] = sum_k A[m, k] * W[n, k]
// with W dequantised in registers from the same packed image the tcgen05 kernel streams.
//
// With so few tokens the tcgen05 pipeline (TMA -> registers -> TMEM -> MMA, a chain of
// barrier hand-offs per k-block) is latency-bound far below HBM speed. Here a producer warp
// streams packed stages into a shared-memory ring, one bulk copy (cp.async.bulk) each, and
// 16 independent warps read their code chunks from the ring with 128-bit shared loads,
// decode them with the same register routines and multiply with warp-level
// mma.sync.m16n8k16 -- weights are the 16-row operand, tokens the 8-column one. Weights of
// 4-bit integers (with or without scales) and e2m1 with e8m0 block scales take this path.
// The reference's counterpart is its split-K SIMT GEMV (examples/dequantize_gemm/
// example_dequant_gemv_fp16xint4.py:21-136, examples/gemv/example_gemv.py:58-96).
// Measured on B200: mma.sync.m16n8k16 (bf16) sustains one instruction per 8 cycles per SM
// sub-partition with a dependent-issue latency of 21 cycles, so the legacy tensor path is
// not the limit here (1.5 k to 3.1 k instructions per sub-partition on the 28672 x 8192
// benchmark weight). Alternatives that lost: a plain SIMT variant on the mixed-precision
// scalar FMA (fma.rn.f32.bf16) for 1-2 tokens; a lane-private cp.async ring; direct 128-bit
// global loads with a bulk L2 prefetch (46 us against 42 us for the ring at one token); the
// ring refilled by the multiply warps themselves with 128 registers per thread and the next
// stage's activations held in registers (same 42 us); applying the group scale to partial
// sums instead of to every weight (fewer instructions, no faster).
//
// Work split: the same stream-K schedule, segments and scratch format as the tcgen05
// kernel (token tile 16), so the same fix-up pass finishes tiles cut between CTAs. Inside
// a CTA, warp w takes weight rows [64 * (w & 1), +64) of the 128-row tile and the stages
// whose CTA-wide index is w >> 1 modulo 8; the 8 partial sums of every output are added in
// a fixed order through shared memory when the segment ends (deterministic).
//
// Fragment mapping. The instruction fixes which lane holds which (row, k) slot: lanes
// 4j..4j+3 hold rows j and j+8, lane l the k slots {2q, 2q+1, 2q+8, 2q+9}, q = l % 4. A
// dot product does not care which real k sits in which slot as long as both operands
// agree, so lane (j, q) reads the 16-byte chunk q of rows j and j+8 (32 consecutive k
// each) and MMA i of 8 uses the lane's real k = 32q + 4i .. 4i+3 for its four slots; the
// activation fragment is then 8 contiguous bytes of the token row.
#pragma once
#include "skinny_launch.h"
#include "umma_gemm.cuh"

namespace b200dq {

constexpr int kSkinnyConsumers = 512;                // 16 multiply warps
constexpr int kSkinnyThreads = kSkinnyConsumers + 32;  // + one producer warp
constexpr int kSkinnyRedStride = kTileRows + 4;      // padded row pitch of the reduction buffer (floats)
constexpr int kSkinnyPhases = kSkinnyConsumers / 64; // 2 row halves x 8 phases
// Shared-memory ring of packed stages. Its depth is a multiple of the phase count and a
// stage's phase is its CTA-wide index modulo the phase count, so a ring slot is always
// consumed by the same two warps and they see every phase of its barriers (a 1-bit parity
// wait cannot tell "one phase behind" from "done").
constexpr int kSkinnyRing = 2 * kSkinnyPhases;
constexpr int kSkinnyStagePitch = 2 * 4096 + 1024;   // largest packed stage (uint4, group 64)
constexpr int kSkinnyCtlBytes = 512;
constexpr int kSkinnyRedBytes = kSkinnyPhases * kSkinnyTokens * kSkinnyRedStride * 4;
constexpr int kSkinnySmemBytes = kSkinnyCtlBytes + kSkinnyRing * kSkinnyStagePitch + kSkinnyRedBytes;
static_assert(kSkinnySmemBytes <= 232448, "over the 227 KiB shared-memory limit");

struct SkinnyCtl {
  uint64_t full[kSkinnyRing];    // stage landed (bulk copy's byte count)
  uint64_t empty[kSkinnyRing];   // both row halves are done with the stage
  int abort_flag;
};
static_assert(sizeof(SkinnyCtl) <= kSkinnyCtlBytes, "control block must fit its slot");

// the 512 multiply threads only (the producer warp never joins)
__device__ __forceinline__ void skinny_consumer_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

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
// Warps 0-15 multiply: warp w takes rows [64 * (w & 1), +64) of the tile and the stages
// whose CTA-wide index is w >> 1 modulo 8. Warp 16 is the producer: one bulk copy per
// packed stage into the ring, running ahead across segment boundaries.
// ---------------------------------------------------------------------------------------
template <int NT, int WF, int ACT>
__global__ void __launch_bounds__(kSkinnyThreads, 1) skinny_dequant_gemm_kernel(const GemmParams p) {
  static_assert(WF == WF_U4_SZ || WF == WF_U4_RAW || WF == WF_S4_RAW || WF == WF_FP4_E8M0,
                "4-bit weights on 16-bit activations");
  static_assert(WF != WF_FP4_E8M0 || ACT == ACT_BF16, "e2m1 weights decode to bf16");
  constexpr bool kBf16 = (ACT == ACT_BF16);
  constexpr int PH = kSkinnyPhases;
  constexpr int RING = kSkinnyRing;
  constexpr int kCodeBytes = 2 * codes_per_kblock_bytes(WF);   // 8192: four 2 KiB chunk slabs
  extern __shared__ __align__(128) uint8_t skinny_smem[];
  SkinnyCtl* ctl = reinterpret_cast<SkinnyCtl*>(skinny_smem);
  uint8_t* ring = skinny_smem + kSkinnyCtlBytes;
  float* red = reinterpret_cast<float*>(ring + RING * kSkinnyStagePitch);   // [phase][token][row (padded)]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &ctl->abort_flag;
  DeviceStatus* st_word = p.status;

  if (threadIdx.x == 0) {
    for (int i = 0; i < RING; ++i) { mbar_init(&ctl->full[i], 1); mbar_init(&ctl->empty[i], 2); }
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kSkinnyConsumers / 32) {
    // ---------------- producer ----------------
    if (lane == 0) {
      uint32_t cnt = 0;   // stages issued by this CTA
      bool ok = true;
      SegmentWalk walk(p);
      Segment w;
      while (ok && walk.next(p, w)) {
        const uint8_t* tile_base = p.wp + w.wp_off + static_cast<size_t>(w.n_tile) * p.st_total * p.stage_bytes;
        for (int st = w.st_begin; st < w.st_end; ++st, ++cnt) {
          const uint32_t slot = cnt % RING;
          ok = mbar_wait(&ctl->empty[slot], ((cnt / RING) & 1u) ^ 1u, abort_flag, st_word, 11);
          if (!ok) break;
          mbar_arrive_expect_tx(&ctl->full[slot], static_cast<uint32_t>(p.stage_bytes));
          tma_bulk_g2s(ring + slot * kSkinnyStagePitch, tile_base + static_cast<size_t>(st) * p.stage_bytes,
                       static_cast<uint32_t>(p.stage_bytes), &ctl->full[slot]);
        }
      }
    }
  } else {
    // ---------------- multiply warps ----------------
    const int half = warp & 1;
    const int phase = warp >> 1;
    const int j = lane >> 2;
    const int q = lane & 3;
    const uint16_t* A = reinterpret_cast<const uint16_t*>(p.a);
    uint32_t cnt0 = 0;   // stages of this CTA before the current segment
    bool ok = true;

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
      const int nst = w.st_end - w.st_begin;

      for (int r = static_cast<int>((static_cast<uint32_t>(phase) - cnt0) & (PH - 1)); r < nst; r += PH) {
        const uint32_t cnt = cnt0 + static_cast<uint32_t>(r);
        const uint32_t slot = cnt % RING;
        const int st = w.st_begin + r;
        // activations first (global memory, L2-resident), then the stage's barrier
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
        ok &= mbar_wait(&ctl->full[slot], (cnt / RING) & 1u, abort_flag, st_word, 12);
        const uint8_t* stage = ring + slot * kSkinnyStagePitch;
        // ---- decode and multiply, one 16-row block at a time
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
          uint4 codes[2];
          uint32_t szw[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int row = row_lo + mt * 16 + h * 8;
            codes[h] = *reinterpret_cast<const uint4*>(stage + q * 2048 + row * 16);
            if constexpr (WF == WF_U4_SZ) {
              const int si = p.sz_per_kb ? (q >> 1) : 0;
              szw[h] = reinterpret_cast<const uint32_t*>(stage + kCodeBytes + si * 512)[row];
            } else if constexpr (WF == WF_FP4_E8M0) {
              szw[h] = reinterpret_cast<const uint32_t*>(stage + kCodeBytes)[row];
            } else {
              szw[h] = 0;
            }
          }
          uint32_t wa[16], wb[16];
          skinny_decode<WF, kBf16>(p, codes[0], szw[0], q, wa);
          skinny_decode<WF, kBf16>(p, codes[1], szw[1], q, wb);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint32_t* b = reinterpret_cast<const uint32_t*>(&av[nt][0]);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              mma_m16n8k16<kBf16>(acc[mt][nt], wa[2 * i], wb[2 * i], wa[2 * i + 1], wb[2 * i + 1], b[2 * i], b[2 * i + 1]);
          }
        }
        // every lane has read its part of the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->empty[slot]);
      }
      cnt0 += static_cast<uint32_t>(nst);

      // ---- add the phases' partial sums in a fixed order
      skinny_consumer_sync();   // the previous segment's readers are done with the buffer
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
      skinny_consumer_sync();
      const int n_tok = NT * 8;
      for (int o = threadIdx.x; o < n_tok * kTileRows; o += kSkinnyConsumers) {
        const int tok = o >> 7;
        const int row = o & (kTileRows - 1);
        float v = 0.f;
#pragma unroll
        for (int ph = 0; ph < PH; ++ph) v += red[(ph * kSkinnyTokens + tok) * kSkinnyRedStride + row];
        skinny_store(p, w, tok, row, v);
      }
    }
    (void)ok;
  }

  // ---------------- teardown ----------------
  if (*abort_flag) {
    // give copies that may still be in flight time to land before the CTA's
    // shared memory goes away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  __syncthreads();
}

}  // namespace b200dq
