// Memory-bound path for at most 16 tokens (decode shapes): C[m, n] = sum_k A[m, k] * W[n, k]
// with W dequantised in registers from the same packed image the tcgen05 kernel streams.
//
// With so few tokens the tcgen05 pipeline (TMA -> registers -> TMEM -> MMA, a chain of
// barrier hand-offs per k-block) is latency-bound far below HBM speed. This kernel is built
// around the memory stream instead: four producer threads keep a deep shared-memory ring
// full (one cp.async.bulk per packed stage plus one tiled TMA of the activations of the
// same 128 k), so the bytes in flight per SM do not depend on what the compute warps are
// doing; 16 consumer warps decode and multiply with warp-level mma.sync.m16n8k16 (weights
// are the 16-row operand, tokens the 8-column one). The reference's counterpart is its
// split-K SIMT GEMV (examples/dequantize_gemm/example_dequant_gemv_fp16xint4.py:21-136,
// examples/gemv/example_gemv.py:58-96). 4-bit integer weights (with or without scales)
// and e2m1 weights with e8m0 block scales take this path.
//
// Work split: the same stream-K schedule, segments and scratch format as the tcgen05
// kernel (token tile 16). A tile cut between CTAs is finished inside the kernel: every CTA
// writes its partial sums, counts itself in on the tile's counter, and the last one adds the
// partial sums in ascending CTA order (no second launch). A ring
// slot holds one stage (128 rows x 128 k of codes, their scale words, and the tokens'
// 128 k). The consumer warps form four teams of four; team t takes the slots whose
// CTA-wide index is t modulo 4, warp r of the team the weight rows [32 r, +32). The four
// warps of one SM sub-partition belong to four different teams, which run out of phase, so
// the load, decode and MMA phases of different slots overlap on the sub-partition's pipes
// (with two teams in lockstep the phases added up instead). The four partial sums of every
// output (one per team) are added in a fixed order through shared memory when the segment
// ends (deterministic). The ring depth is a multiple of 4, so a team meets every phase of
// the barriers of its slots: a parity wait cannot tell "two phases behind" from "done".
//
// Every format is dequantised completely in registers with the routines of the tcgen05
// kernel (decode.cuh), so both kernels multiply the same 16-bit weights and differ only in the
// order of the fp32 additions. (Applying the group scale to per-stage fp32 sums instead --
// one packed fma less per code pair -- was measured 5 % faster at 1 token and slower at 16,
// and it no longer rounds each weight to 16 bits the way the reference's ref_program does; it
// was not kept.)
//
// Fragment mapping. The instruction fixes which lane holds which (row, k) slot: lanes
// 4j..4j+3 hold rows j and j+8, lane l the k slots {2q, 2q+1, 2q+8, 2q+9}, q = l % 4. A
// dot product does not care which real k sits in which slot as long as both operands
// agree, so lane (j, q) loads the 16-byte chunk q of rows j and j+8 (32 consecutive k
// each) and MMA i of 8 uses the lane's real k = 32q + 4i .. 4i+3 for its four slots; the
// activation fragment is then 8 contiguous bytes of the token row.
//
// Shared-memory reads are bank-conflict free: the image stores chunk c of row r at
// 16-byte position r ^ 2c of its slab (pack_kernels.cuh), and the activations arrive
// through a 4-D tensor map {64 k, k-block parity, token, stage} with the 128-byte swizzle,
// which places (token t, parity p) in row 2t + p.
#pragma once
#include "skinny_launch.h"
#include "umma_gemm.cuh"

namespace b200dq {

constexpr int kSkinnyTeams = 4;                         // consumer teams = partial sums per output
constexpr int kSkinnyConsumerWarps = 4 * kSkinnyTeams;
constexpr int kSkinnyConsumers = kSkinnyConsumerWarps * 32;
constexpr int kSkinnyProducerWarps = 4;
constexpr int kSkinnyThreads = kSkinnyConsumers + kSkinnyProducerWarps * 32;
constexpr int kSkinnyRedStride = kTileRows + 4;         // padded row pitch of the reduction buffer (floats)
constexpr int kSkinnyCtlBytes = 1024;
constexpr int kSkinnyMaxSlots = 16;
// Registers per thread after the hand-over (multiples of 8): 128 x 32 + 512 x 112 is exactly
// the 640 x 96 the launch reserved.
constexpr int kSkinnyProducerRegs = 32;
constexpr int kSkinnyConsumerRegs = 112;

// Shared-memory plan of one kernel instance. NT = 8-token column blocks (1 or 2).
template <int NT, int WF>
struct SkinnyRing {
  static constexpr int kTok = NT * 8;
  static constexpr int kWStage = 2 * codes_per_kblock_bytes(WF) + sz_smem_bytes(WF);  // largest packed stage
  static constexpr int kWSlot = (kWStage + 1023) / 1024 * 1024;
  static constexpr int kASlot = kTok * 256;              // activations of the stage: [token][parity][128 B]
  static constexpr int kSlot = kASlot + kWSlot;          // activations first: their swizzle needs a 1 KiB aligned base
  static constexpr int kRedBytes = kSkinnyTeams * kTok * kSkinnyRedStride * 4;
  static constexpr int kFit = (232448 - 1024 /*align*/ - kSkinnyCtlBytes - kRedBytes) / kSlot;
  static constexpr int kSlots = (kFit > kSkinnyMaxSlots ? kSkinnyMaxSlots : kFit) & ~(kSkinnyTeams - 1);
  static constexpr int kSmemBytes = 1024 + kSkinnyCtlBytes + kRedBytes + kSlots * kSlot;
  static_assert(kSlot % 1024 == 0 && kASlot % 1024 == 0, "slot and code bases keep their alignment");
  static_assert(kSlots >= 2 * kSkinnyTeams, "every team needs a slot to work on and one in flight");
};

struct SkinnyCtl {
  uint64_t full[kSkinnyMaxSlots];
  uint64_t empty[kSkinnyMaxSlots];
  int abort_flag;
  int finish_tile;   // this CTA brought the last partial sum of a cut tile
  int others_done;   // the other CTAs' sums of this CTA's cut tile were published before it got there
  long long pending[2];
};
static_assert(sizeof(SkinnyCtl) <= kSkinnyCtlBytes, "control block must fit its slot");

// 4-D tiled load; c0 * element_size must stay a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* tmap, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void skinny_consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kSkinnyConsumers) : "memory");
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

// Warp-wide wait on a ring barrier. The common case (the copy landed long ago) costs one
// probe by the whole warp; otherwise lane 0 alone polls, so that 32 spinning lanes do not
// flood the shared-memory pipe the producers' issues and every arrive go through.
__device__ __forceinline__ bool skinny_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                            DeviceStatus* st, uint32_t site, int lane) {
  if (mbar_test_wait(bar, parity)) return true;
  return mbar_wait_warp(bar, parity, abort_flag, st, site, lane);
}

// `sz` is the row's scale word of the stage; `q` the lane's chunk (uint4: one {scale, zero}
// pair per group; e2m1: one e8m0 byte per chunk of 32 codes).
template <int WF, bool kBf16>
__device__ __forceinline__ void skinny_decode(const GemmParams& p, const uint4& codes, uint32_t sz, int q,
                                              uint32_t (&out)[16]) {
  if constexpr (WF == WF_U4_SZ) decode_u4_chunk<kBf16>(codes, sz, out);
  else if constexpr (WF == WF_U4_RAW) decode_u4_chunk_noscale<kBf16, false>(codes, out);
  else if constexpr (WF == WF_S4_RAW) decode_u4_chunk_noscale<kBf16, true>(codes, out);
  else decode_fp4_chunk<kBf16>(codes, 126 + static_cast<int>((sz >> (8 * q)) & 0xffu) - p.fp4_exp_bias,
                               (p.flags & GF_FP4_SIMPLE) != 0, out);
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
    case OUT_F16: store_everywhere(p, idx, finish_value<__half, false>(p, bits, m, n)); break;
    case OUT_BF16: store_everywhere(p, idx, finish_value<__nv_bfloat16, false>(p, bits, m, n)); break;
    default: store_everywhere(p, idx, finish_value<float, false>(p, bits, m, n)); break;
  }
}

constexpr int kSkinnyFastParts = 4;   // partial sums of a cut tile the finishing CTA holds in registers

// The CTAs that share a tile: the first one and how many.
__device__ __forceinline__ void skinny_cut_plan(const GemmParams& p, long long tile, int& c_first, int& nc) {
  const long long t_begin = tile * p.st_total;
  c_first = static_cast<int>(t_begin / p.span);
  nc = static_cast<int>((t_begin + p.st_total - 1) / p.span) - c_first + 1;
}

// Adds every CTA's published partial sums of a cut tile in ascending CTA order and stores the
// outputs (all consumer threads; the sums come from L2).
template <int kTok>
__device__ __forceinline__ void skinny_finish_tile(const GemmParams& p, long long tile) {
  __threadfence();
  const long long t_begin = tile * p.st_total;
  const int c_first = static_cast<int>(t_begin / p.span);
  const int c_last = static_cast<int>((t_begin + p.st_total - 1) / p.span);
  Segment whole;
  locate_tile(p, tile, whole);
  whole.slot = -1;
  for (int o = threadIdx.x; o < kTok * kTileRows; o += kSkinnyConsumers) {
    const int tok = o >> 7;
    const int row = o & (kTileRows - 1);
    float v = 0.f;
    for (int cta = c_first; cta <= c_last; ++cta) {
      // slot 0 if the tile holds the first segment of that CTA's span, else slot 1
      const int slot = cta * 2 + ((static_cast<long long>(cta) * p.span >= t_begin) ? 0 : 1);
      v += __uint_as_float(__ldcg(p.partial + (static_cast<size_t>(slot) * kSkinnyTokens + tok) * kTileRows + row));
    }
    skinny_store(p, whole, tok, row, v);
  }
}

// ---------------------------------------------------------------------------------------
// NT: 8-token column blocks (1 for M <= 8, else 2).
// ---------------------------------------------------------------------------------------
template <int NT, int WF, int ACT>
__global__ void __launch_bounds__(kSkinnyThreads, 1)
skinny_dequant_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const GemmParams p) {
  static_assert(WF == WF_U4_SZ || WF == WF_U4_RAW || WF == WF_S4_RAW || WF == WF_FP4_E8M0,
                "4-bit weights on 16-bit activations");
  using Ring = SkinnyRing<NT, WF>;
  constexpr bool kBf16 = (ACT == ACT_BF16);
  constexpr int RING = Ring::kSlots;
  constexpr int kTok = Ring::kTok;
  constexpr int kCodeBytes = 2 * codes_per_kblock_bytes(WF);   // 8192: four 2 KiB chunk slabs

  extern __shared__ uint8_t skinny_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(skinny_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;                                                 // RING x (activations | packed stage)
  float* red = reinterpret_cast<float*>(ring + RING * Ring::kSlot);     // [team][token][row (padded)]
  SkinnyCtl* ctl = reinterpret_cast<SkinnyCtl*>(reinterpret_cast<uint8_t*>(red) + Ring::kRedBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &ctl->abort_flag;
  DeviceStatus* st_word = p.status;

  if (threadIdx.x == 0) {
    for (int i = 0; i < RING; ++i) {
      mbar_init(&ctl->full[i], 1);
      mbar_init(&ctl->empty[i], 4);   // the four warps of the slot's team
    }
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kSkinnyConsumerWarps && lane == 0) tma_prefetch_desc(&tmap_a);
  __syncthreads();

  // The launch gives every thread the same register count (what 20 warps can share). The
  // producer warpgroup hands most of its registers back and the consumer warpgroups take
  // them: the consumers' fragments, decoded weights and sums need more than the even split.
  if (warp >= kSkinnyConsumerWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kSkinnyProducerRegs));
    // ---------------- producers ----------------
    // Four issuing threads, one per warp; producer t fills the slots of team t: one bulk copy
    // of the packed stage and one tiled TMA of the activations of its 128 k. The schedule is
    // dense with one token tile, so unit u of the (tile, stage) space is stage u % st_total of
    // K and its packed bytes start at u * stage_bytes: no segment walk needed.
    const uint32_t team = static_cast<uint32_t>(warp - kSkinnyConsumerWarps);
    if (lane == 0) {
      const long long pos0 = static_cast<long long>(blockIdx.x) * p.span;
      const uint32_t n_slots = static_cast<uint32_t>(min(static_cast<long long>(p.span), p.units - pos0));
      uint32_t slot = team, phase = 0;
      for (uint32_t cnt = team; cnt < n_slots; cnt += kSkinnyTeams) {
        if (!mbar_wait(&ctl->empty[slot], phase ^ 1u, abort_flag, st_word, 11)) break;
        uint8_t* dst = ring + slot * Ring::kSlot;
        mbar_arrive_expect_tx(&ctl->full[slot], static_cast<uint32_t>(p.stage_bytes) + Ring::kASlot);
        tma_bulk_g2s(dst + Ring::kASlot, p.wp + static_cast<size_t>(pos0 + cnt) * p.stage_bytes,
                     static_cast<uint32_t>(p.stage_bytes), &ctl->full[slot]);
        tma_load_4d(dst, &tmap_a, 0, 0, 0, static_cast<int>((pos0 + cnt) % p.st_total), &ctl->full[slot]);
        slot += kSkinnyTeams;
        if (slot >= static_cast<uint32_t>(RING)) { slot -= RING; phase ^= 1u; }
      }
    }
  } else {
    // ---------------- consumers ----------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSkinnyConsumerRegs));
    const uint32_t team = static_cast<uint32_t>(warp >> 2);
    const int rq = warp & 3;           // 32-row quarter of the tile
    const int j = lane >> 2;
    const int q = lane & 3;
    const int row_lo = rq * 32 + j;
    // Per-lane byte offsets inside a slot, fixed for the whole kernel, so that every load of
    // the inner loop is base + constant.
    // Activations of (token t, this lane's 32 k): row 2t + (q >> 1) of the stage's block,
    // 16-byte chunks 4 (q & 1) + v, v = 0..3, swizzled with the row index.
    const int a_par = q >> 1;
    const uint32_t a_xor = static_cast<uint32_t>((2 * j + a_par) & 7);
    uint32_t a_off[4];
#pragma unroll
    for (int v = 0; v < 4; ++v)
      a_off[v] = static_cast<uint32_t>(j * 256 + a_par * 128) + (((static_cast<uint32_t>(4 * (q & 1)) + v) ^ a_xor) << 4);
    // Codes: chunk q of row r at q * 2048 + (r ^ chunk_swizzle(q)) * 16. The swizzle touches
    // bits 1-2 of the row only, so the rows j + 8, + 16, + 24 of this lane are the first one
    // plus a constant.
    const uint32_t c_off = static_cast<uint32_t>(Ring::kASlot + q * 2048) +
                           ((static_cast<uint32_t>(row_lo) ^ static_cast<uint32_t>(chunk_swizzle(q))) << 4);
    // Scale words: [word][row], 4 bytes each; with one word per k-block the lane's chunk picks it.
    const uint32_t z_off = static_cast<uint32_t>(Ring::kASlot + kCodeBytes + (p.sz_per_kb ? (q >> 1) * 512 : 0) +
                                                 row_lo * 4);

    uint32_t my_cnt = team;            // CTA-wide index of this team's next slot
    uint32_t slot = team, phase = 0;
    uint32_t cnt0 = 0;                 // slots of this CTA before the current segment
    bool ok = true;

    long long pending0 = -1, pending1 = -1;   // thread 0: cut tiles this CTA completed by surprise
    SegmentWalk walk(p);
    Segment w;
    while (walk.next(p, w)) {
      float acc[2][NT][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[mt][nt][c] = 0.f;

      // A tile cut between CTAs is the sum of the CTAs' partial sums in ascending CTA order
      // (the same order in every launch: deterministic). The CTA that holds the tile's first
      // stages works on them at the END of its span, the others at the START of theirs, so
      // their sums are published before it even begins: thread 0 looks at the tile's counter
      // now (only its own warp waits for the answer) and leaves the verdict for the segment's end.
      // (No thread can still be reading the flag: thread 0 has passed the previous segment's
      // second barrier, which every thread reaches after its read.)
      if (w.slot >= 0 && threadIdx.x == 0) {
        int c_first, nc;
        skinny_cut_plan(p, w.tile, c_first, nc);
        bool done = false;
        if (static_cast<int>(blockIdx.x) == c_first && nc <= kSkinnyFastParts) {
          const unsigned long long seen = *reinterpret_cast<volatile unsigned long long*>(p.tile_ctr + w.tile);
          done = seen == ((p.epoch << 8) | static_cast<unsigned long long>(nc - 1));
          if (done) __threadfence();   // order the look at the counter before the CTA's reads of the sums
        }
        ctl->others_done = done ? 1 : 0;
      }

      const uint32_t nst = static_cast<uint32_t>(w.st_end - w.st_begin);
      for (; my_cnt < cnt0 + nst; my_cnt += kSkinnyTeams) {
        ok &= skinny_wait(&ctl->full[slot], phase, abort_flag, st_word, 13, lane);
        if (ok) {
          const uint8_t* slot_base = ring + slot * Ring::kSlot;
          // ---- the lane's activations: 32 k of token j (and j + 8)
          uint32_t b[NT][16];
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint8_t* src = slot_base + a_off[v];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const uint4 t = *reinterpret_cast<const uint4*>(src + nt * (8 * 256));
              b[nt][4 * v] = t.x; b[nt][4 * v + 1] = t.y; b[nt][4 * v + 2] = t.z; b[nt][4 * v + 3] = t.w;
            }
          }
          const uint8_t* c_src = slot_base + c_off;
          const uint8_t* z_src = slot_base + z_off;
          // ---- decode and multiply, one 16-row block at a time
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            uint4 codes[2];
            uint32_t szw[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              codes[hh] = *reinterpret_cast<const uint4*>(c_src + (mt * 16 + hh * 8) * 16);
              if constexpr (WF == WF_U4_SZ || WF == WF_FP4_E8M0)
                szw[hh] = *reinterpret_cast<const uint32_t*>(z_src + (mt * 16 + hh * 8) * 4);
              else
                szw[hh] = 0;
            }
            uint32_t wa[16], wb[16];
            skinny_decode<WF, kBf16>(p, codes[0], szw[0], q, wa);
            skinny_decode<WF, kBf16>(p, codes[1], szw[1], q, wb);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                mma_m16n8k16<kBf16>(acc[mt][nt], wa[2 * i], wb[2 * i], wa[2 * i + 1], wb[2 * i + 1], b[nt][2 * i],
                                    b[nt][2 * i + 1]);
            }
          }
        }
        // every lane has read its part of the slot
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->empty[slot]);
        slot += kSkinnyTeams;
        if (slot >= static_cast<uint32_t>(RING)) { slot -= RING; phase ^= 1u; }
      }
      cnt0 += nst;

      // ---- add the teams' partial sums of every output in a fixed order. If the other CTAs'
      // sums of a cut tile were published when this segment began, they are added to this CTA's
      // own straight from L2 and the outputs are stored, with nothing of its own written to
      // scratch and no wait. Otherwise every contributor publishes its sums, counts itself in,
      // and whoever counts last adds them all.
      constexpr int kOuts = kTok * kTileRows / kSkinnyConsumers;     // outputs per thread
      constexpr int kFast = kSkinnyFastParts;
      const bool cut = w.slot >= 0;
      const long long t_begin = w.tile * p.st_total;
      int c_first, nc;
      skinny_cut_plan(p, w.tile, c_first, nc);
      // slot 0 if the tile holds the first segment of that CTA's span, else slot 1
      auto slot_of = [&](int cta) { return cta * 2 + ((static_cast<long long>(cta) * p.span >= t_begin) ? 0 : 1); };
      skinny_consumer_sync();   // the previous segment's readers are done with the buffer
      const bool others_done = cut && ctl->others_done != 0;
      uint32_t raw[kOuts][kFast];
      if (others_done) {
#pragma unroll
        for (int jj = 1; jj < kFast; ++jj) {
          if (jj < nc) {
            const uint32_t* src = p.partial + static_cast<size_t>(slot_of(c_first + jj)) * kSkinnyTokens * kTileRows;
#pragma unroll
            for (int i = 0; i < kOuts; ++i) raw[i][jj] = __ldcg(src + threadIdx.x + i * kSkinnyConsumers);
          }
        }
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int row = rq * 32 + mt * 16 + j + (c >> 1) * 8;
            const int tok = nt * 8 + 2 * q + (c & 1);
            red[(team * kTok + tok) * kSkinnyRedStride + row] = acc[mt][nt][c];
          }
      skinny_consumer_sync();
      Segment whole = w;
      whole.slot = -1;
#pragma unroll
      for (int i = 0; i < kOuts; ++i) {
        const int o = threadIdx.x + i * kSkinnyConsumers;
        const int tok = o >> 7;
        const int row = o & (kTileRows - 1);
        float v = 0.f;
#pragma unroll
        for (int t = 0; t < kSkinnyTeams; ++t) v += red[(t * kTok + tok) * kSkinnyRedStride + row];
        if (others_done) {
          v = 0.f + v;      // the general path starts its sum at zero: keep the same roundings
#pragma unroll
          for (int jj = 1; jj < kFast; ++jj)
            if (jj < nc) v += __uint_as_float(raw[i][jj]);
          skinny_store(p, whole, tok, row, v);
        } else {
          skinny_store(p, w, tok, row, v);
        }
      }
      if (cut && !others_done) {
        // Everyone's partial sums are stored; thread 0 makes them visible device-wide (the barrier
        // orders the others' stores before its fence) and counts this CTA in.
        skinny_consumer_sync();
        if (static_cast<int>(blockIdx.x) != c_first) {
          // Not the CTA that normally finishes the tile: nobody waits for the count. Should this
          // CTA turn out to be the last all the same, it finishes the tile when its span is done.
          if (threadIdx.x == 0) {
            __threadfence();
            if (tile_arrive(p.tile_ctr + w.tile, p.epoch, nc)) {
              if (pending0 < 0) pending0 = w.tile; else pending1 = w.tile;
            }
          }
        } else {
          if (threadIdx.x == 0) {
            __threadfence();
            ctl->finish_tile = tile_arrive(p.tile_ctr + w.tile, p.epoch, nc) ? 1 : 0;
          }
          skinny_consumer_sync();
          if (ctl->finish_tile == 1) skinny_finish_tile<kTok>(p, w.tile);
        }
      }
    }
    // tiles this CTA happened to complete without being their usual finisher
    skinny_consumer_sync();
    if (threadIdx.x == 0) { ctl->pending[0] = pending0; ctl->pending[1] = pending1; }
    skinny_consumer_sync();
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (ctl->pending[i] >= 0) skinny_finish_tile<kTok>(p, ctl->pending[i]);
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
