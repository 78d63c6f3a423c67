// Warp-specialised, persistent, TMA-fed tcgen05 GEMM with in-register weight
// dequantisation:  C[M,N] = A[M,K] * dequant(W[N,K])^T.
//
// It replaces, for sm_100a, the kernels the reference generates from
//   examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:16-90   (W4A16),
//   examples/dequantize_gemm/example_dequant_gemm_bf16_mxfp4_hopper.py:80-378 (MXFP4),
//   examples/dequantize_gemm/example_dequant_gemm_w4a8.py:85-149          (W4A8),
//   examples/bitnet-1.58b/kernel_benchmark/tilelang_bitnet_158_int8xint2_prefill.py:72-298,
// which on this architecture lower to mma.sync with a register->smem->ldmatrix
// round trip of the dequantised tile (src/cuda/op/gemm.cc:337-390).
//
// Design. The product is computed transposed so the *weights* are the MMA's
// M side: one CTA tile is 128 weight rows x TN tokens. Dequantised weights never
// touch shared memory: a dequant thread owns one weight row (= one TMEM lane),
// expands its packed bytes to 64 16-bit (or 128 8-bit) K elements in registers
// and writes them with tcgen05.st into a TMEM ring; the MMA reads its A operand
// from TMEM ("TS" form) and its B operand (activations, K-major, 128-byte
// swizzle) from a TMA-filled shared-memory ring. Accumulators (fp32 or int32)
// live in TMEM columns [0, TN).
//
//   warp 0      : packed-weight producer (cp.async.bulk, one stage per k-block)
//   warp 1      : TMEM owner + MMA issuer (one elected lane)
//   warp 2      : activation producer (tiled TMA)
//   warp 3      : idle
//   warps 4-11  : two dequant warpgroups, alternating k-blocks
//   warps 12-15 : epilogue (tcgen05.ld -> convert -> global)
//
// Per k-block (64 16-bit or 128 8-bit K elements = one 128 B swizzle atom):
//   full_w/empty_w : packed weight ring      (TMA -> dequant warps)
//   full_b/empty_b : activation ring         (TMA -> MMA)
//   a_full/a_empty : dequantised TMEM ring   (dequant warps -> MMA)
//   acc_full/acc_empty : accumulator         (MMA -> epilogue)
// Every wait is bounded (ptx.cuh); a wait that gives up sets a status word.
//
// Scheduling is stream-K: the (tile, k-block) space is cut into equal contiguous
// spans, one per CTA, so every SM streams the same number of weight bytes. A
// span's first and last segment may cover only part of a tile; those write fp32
// partial tiles to scratch slots (two per CTA) and a second small kernel adds the
// slots of each split tile in a fixed order (deterministic, no atomics).
#pragma once
#include <type_traits>

#include "decode.cuh"
#include "ptx.cuh"

namespace b200dq {

enum WeightFormat : int {
  WF_U4_SZ = 0,       // uint4, per-group scale + zero term (16-bit activations)
  WF_U4_RAW = 1,      // uint4, weight = q              (no scale)
  WF_S4_RAW = 2,      // uint4 storing q = w + 8        (no scale)
  WF_FP4_E8M0 = 3,    // e2m1 + e8m0 block scale per 32 (bf16 activations)
  WF_I2_I8 = 4,       // 2-bit codes -> int8, minus `code_bias` (int8 activations)
  WF_I4_I8 = 5,       // 4-bit codes -> int8, minus `code_bias` (int8 activations)
};

enum ActType : int { ACT_F16 = 0, ACT_BF16 = 1, ACT_I8 = 2 };
enum OutType : int { OUT_F16 = 0, OUT_BF16 = 1, OUT_F32 = 2, OUT_I32 = 3 };

enum GemmFlags : int {
  GF_TRANS_C = 1,      // write C^T (N x M) instead of C (M x N)
  GF_HAS_BIAS = 2,     // add bias[M][N] (output dtype) in the epilogue
  GF_ROW_SCALE = 4,    // integer path: acc * row_scale[m] * tensor_scale before the cast
};

struct GemmParams {
  const uint8_t* wp;         // packed weights: [n_tiles][kb_total][stage bytes]
  const void* sz;            // scale table (layout depends on the weight format)
  void* c;                   // output
  uint32_t* partial;         // scratch: [grid][2][TN][128] raw fp32/int32 partial tiles
  const void* bias;          // optional bias [M][N]
  const float* row_scale;    // optional per-token factor [M]
  float tensor_scale;        // optional per-tensor factor
  uint32_t code_bias;        // bytewise bias for the integer decoders
  int fp4_exp_bias;          // 127 for OCP e8m0, 0 for a raw exponent byte
  int M, N, K;
  int n_tiles, m_tiles, kb_total;
  int span;                  // k-blocks per CTA (stream-K span length)
  long long units;           // m_tiles * n_tiles * kb_total
  int group_kb;              // k-blocks per scale group (WF_U4_SZ)
  int n_pad;                 // padded N = n_tiles * 128 (row stride of `sz`)
  int ldc;                   // leading dimension of the output
  int flags;
  int out_type;
  DeviceStatus* status;
};

constexpr int kTileRows = 128;        // weight rows per CTA tile (= TMEM lanes)
constexpr int kAccCols = 256;         // first TMEM column of the dequantised ring
constexpr int kASlots = 8;            // TMEM ring slots, 32 columns each
constexpr int kThreads = 512;

__host__ __device__ constexpr int w_stage_bytes(int wf) { return wf == WF_I4_I8 ? 8192 : 4096; }

template <int TN, int WF>
struct RingConfig {
  static constexpr int kBStageBytes = TN * 128;
  static constexpr int kWStageBytes = w_stage_bytes(WF);
  // activation ring and packed-weight ring depths; the sum stays under ~200 KiB
  static constexpr int kNB = TN >= 256 ? 4 : (TN >= 128 ? 6 : 8);
  static constexpr int kNW = (TN >= 256 ? 16 : (TN >= 128 ? 24 : 32)) * 4096 / kWStageBytes;
  static constexpr int kSmemBytes = kNB * kBStageBytes + kNW * kWStageBytes + 1024 /*align*/ + 1024 /*ctl*/;
};

struct SharedCtl {
  uint64_t full_w[32];
  uint64_t empty_w[32];
  uint64_t full_b[8];
  uint64_t empty_b[8];
  uint64_t a_full[kASlots];
  uint64_t a_empty[kASlots];
  uint64_t acc_full;
  uint64_t acc_empty;
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(SharedCtl) <= 1024, "control block must fit its slot");

// One contiguous run of k-blocks inside one tile.
struct Segment {
  int m_tile, n_tile, kb_begin, kb_end;
  int slot;   // -1: the segment is a whole tile and stores to C; else scratch slot index
};

// Walks the segments of this CTA's span; every warp role runs the same walk.
struct SegmentWalk {
  long long pos, end;
  bool first;
  __device__ __forceinline__ SegmentWalk(const GemmParams& p) {
    pos = static_cast<long long>(blockIdx.x) * p.span;
    end = pos + p.span;
    if (end > p.units) end = p.units;
    first = true;
  }
  __device__ __forceinline__ bool next(const GemmParams& p, Segment& s) {
    if (pos >= end) return false;
    const long long tile = pos / p.kb_total;
    s.kb_begin = static_cast<int>(pos - tile * p.kb_total);
    const long long left = end - pos;
    s.kb_end = static_cast<int>(min(static_cast<long long>(p.kb_total), s.kb_begin + left));
    s.m_tile = static_cast<int>(tile % p.m_tiles);
    s.n_tile = static_cast<int>(tile / p.m_tiles);
    const bool whole = (s.kb_begin == 0 && s.kb_end == p.kb_total);
    s.slot = whole ? -1 : (static_cast<int>(blockIdx.x) * 2 + (first ? 0 : 1));
    first = false;
    pos += (s.kb_end - s.kb_begin);
    return true;
  }
};

template <typename OutT>
__device__ __forceinline__ OutT cast_out(float v);
template <> __device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float cast_out<float>(float v) { return v; }
template <> __device__ __forceinline__ int cast_out<int>(float v) { return __float2int_rn(v); }

template <typename OutT>
__device__ __forceinline__ float bias_as_float(const void* bias, size_t idx) {
  return static_cast<float>(reinterpret_cast<const OutT*>(bias)[idx]);
}

// Store NV accumulator values (tokens m0 .. m0+NV-1 of weight row n) to C.
template <typename OutT, bool kIntAcc, int NV>
__device__ __forceinline__ void store_values(const GemmParams& p, const uint32_t* acc, int m0, int n) {
  OutT* c = reinterpret_cast<OutT*>(p.c);
  const bool trans = (p.flags & GF_TRANS_C) != 0;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int m = m0 + j;
    if (m < p.M) {
      const size_t idx = trans ? static_cast<size_t>(n) * p.ldc + m : static_cast<size_t>(m) * p.ldc + n;
      if constexpr (kIntAcc && sizeof(OutT) == 4 && !std::is_same<OutT, float>::value) {
        c[idx] = static_cast<int>(acc[j]);   // exact int32 result
      } else {
        float v;
        if constexpr (kIntAcc) {
          v = static_cast<float>(static_cast<int>(acc[j]));
          if (p.flags & GF_ROW_SCALE) v = v * p.row_scale[m] * p.tensor_scale;
        } else {
          v = __uint_as_float(acc[j]);
        }
        if (p.flags & GF_HAS_BIAS) v += bias_as_float<OutT>(p.bias, static_cast<size_t>(m) * p.N + n);
        c[idx] = cast_out<OutT>(v);
      }
    }
  }
}

template <int TN, int WF, int ACT>
__global__ void __launch_bounds__(kThreads, 1)
umma_dequant_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const GemmParams p) {
  using Ring = RingConfig<TN, WF>;
  constexpr int NB = Ring::kNB;
  constexpr int NW = Ring::kNW;
  constexpr int WSB = Ring::kWStageBytes;
  constexpr bool kInt = (ACT == ACT_I8);
  constexpr int BKE = kInt ? 128 : 64;   // K elements per k-block
  constexpr int NV = TN >= 32 ? 32 : 16; // accumulator columns per tcgen05.ld

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_b = smem;                                   // NB x (TN x 128 B), 1024-aligned stages
  uint8_t* smem_w = smem + NB * Ring::kBStageBytes;         // NW x stage bytes
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem_w + NW * WSB);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &ctl->abort_flag;
  DeviceStatus* st = p.status;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NW; ++i) { mbar_init(&ctl->full_w[i], 1); mbar_init(&ctl->empty_w[i], 4); }
    for (int i = 0; i < NB; ++i) { mbar_init(&ctl->full_b[i], 1); mbar_init(&ctl->empty_b[i], 1); }
    for (int i = 0; i < kASlots; ++i) { mbar_init(&ctl->a_full[i], 4); mbar_init(&ctl->a_empty[i], 1); }
    mbar_init(&ctl->acc_full, 1);
    mbar_init(&ctl->acc_empty, 4);
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  if (warp == 2 && lane == 0) tma_prefetch_desc(&tmap_a);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ---------------- packed-weight producer ----------------
    if (lane == 0) {
      uint32_t kc = 0;
      SegmentWalk walk(p);
      Segment w;
      while (walk.next(p, w)) {
        const uint8_t* src = p.wp + (static_cast<size_t>(w.n_tile) * p.kb_total + w.kb_begin) * WSB;
        for (int kb = w.kb_begin; kb < w.kb_end; ++kb, ++kc, src += WSB) {
          const uint32_t s = kc % NW;
          mbar_wait(&ctl->empty_w[s], ((kc / NW) & 1) ^ 1, abort_flag, st, 1);
          mbar_arrive_expect_tx(&ctl->full_w[s], WSB);
          tma_bulk_g2s(smem_w + s * WSB, src, WSB, &ctl->full_w[s]);
        }
      }
    }
  } else if (warp == 2) {
    // ---------------- activation producer ----------------
    if (lane == 0) {
      uint32_t kc = 0;
      SegmentWalk walk(p);
      Segment w;
      while (walk.next(p, w)) {
        for (int kb = w.kb_begin; kb < w.kb_end; ++kb, ++kc) {
          const uint32_t s = kc % NB;
          mbar_wait(&ctl->empty_b[s], ((kc / NB) & 1) ^ 1, abort_flag, st, 2);
          mbar_arrive_expect_tx(&ctl->full_b[s], Ring::kBStageBytes);
          tma_load_2d(smem_b + s * Ring::kBStageBytes, &tmap_a, kb * BKE, w.m_tile * TN, &ctl->full_b[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc =
          kInt ? make_idesc(2u, 1u, 1u, 128u, TN)
               : make_idesc(1u, ACT == ACT_BF16 ? 1u : 0u, ACT == ACT_BF16 ? 1u : 0u, 128u, TN);
      uint32_t kc = 0, tc = 0;
      SegmentWalk walk(p);
      Segment w;
      while (walk.next(p, w)) {
        mbar_wait(&ctl->acc_empty, (tc & 1) ^ 1, abort_flag, st, 3);
        tc_fence_after_sync();
        for (int kb = w.kb_begin; kb < w.kb_end; ++kb, ++kc) {
          const uint32_t sa = kc % kASlots;
          const uint32_t sb = kc % NB;
          mbar_wait(&ctl->a_full[sa], (kc / kASlots) & 1, abort_flag, st, 4);
          mbar_wait(&ctl->full_b[sb], (kc / NB) & 1, abort_flag, st, 5);
          tc_fence_after_sync();
          const uint32_t a_tmem = tmem_base + kAccCols + sa * 32;
          const uint64_t b_desc = make_smem_desc_sw128(smem_u32(smem_b + sb * Ring::kBStageBytes));
          if (!*abort_flag) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t acc = (kb > w.kb_begin || j > 0) ? 1u : 0u;
              if constexpr (kInt) umma_ts_i8(tmem_base, a_tmem + j * 8, b_desc + j * 2, idesc, acc);
              else umma_ts_f16(tmem_base, a_tmem + j * 8, b_desc + j * 2, idesc, acc);
            }
          }
          tc_commit(&ctl->a_empty[sa]);
          tc_commit(&ctl->empty_b[sb]);
        }
        tc_commit(&ctl->acc_full);
        ++tc;
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ---------------- dequant warpgroups ----------------
    const int dg = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t kc = 0;
    SegmentWalk walk(p);
    Segment w;
    while (walk.next(p, w)) {
      const int row = w.n_tile * kTileRows + row_in_tile;
      int cached_group = -1;
      uint32_t szv = 0;
      for (int kb = w.kb_begin; kb < w.kb_end; ++kb, ++kc) {
        if ((kc & 1) != static_cast<uint32_t>(dg)) continue;
        // scale words come from global/L2; issue the load before the waits
        if constexpr (WF == WF_U4_SZ) {
          const int g = kb / p.group_kb;
          if (g != cached_group) {
            szv = __ldg(reinterpret_cast<const uint32_t*>(p.sz) + static_cast<size_t>(g) * p.n_pad + row);
            cached_group = g;
          }
        } else if constexpr (WF == WF_FP4_E8M0) {
          szv = __ldg(reinterpret_cast<const uint16_t*>(p.sz) + static_cast<size_t>(kb) * p.n_pad + row);
        }
        const uint32_t sw = kc % NW;
        const uint32_t sa = kc % kASlots;
        mbar_wait(&ctl->full_w[sw], (kc / NW) & 1, abort_flag, st, 6);
        const uint4* wsrc = reinterpret_cast<const uint4*>(smem_w + sw * WSB);
        uint32_t regs[32];
        if constexpr (WF == WF_I4_I8) {
          // 64 packed bytes per row and k-block: four 16-byte chunks
          uint4 c[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) c[q] = wsrc[q * 128 + row_in_tile];
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->empty_w[sw]);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            decode_i4_chunk(c[q], p.code_bias, *reinterpret_cast<uint32_t (*)[8]>(&regs[8 * q]));
        } else {
          const uint4 c0 = wsrc[row_in_tile];
          const uint4 c1 = wsrc[128 + row_in_tile];
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->empty_w[sw]);
          uint32_t (&lo)[16] = *reinterpret_cast<uint32_t (*)[16]>(&regs[0]);
          uint32_t (&hi)[16] = *reinterpret_cast<uint32_t (*)[16]>(&regs[16]);
          if constexpr (WF == WF_U4_SZ) {
            decode_u4_chunk<ACT == ACT_BF16>(c0, szv, lo);
            decode_u4_chunk<ACT == ACT_BF16>(c1, szv, hi);
          } else if constexpr (WF == WF_U4_RAW) {
            decode_u4_chunk_noscale<ACT == ACT_BF16, false>(c0, lo);
            decode_u4_chunk_noscale<ACT == ACT_BF16, false>(c1, hi);
          } else if constexpr (WF == WF_S4_RAW) {
            decode_u4_chunk_noscale<ACT == ACT_BF16, true>(c0, lo);
            decode_u4_chunk_noscale<ACT == ACT_BF16, true>(c1, hi);
          } else if constexpr (WF == WF_FP4_E8M0) {
            decode_fp4_chunk(c0, 126 + static_cast<int>(szv & 0xff) - p.fp4_exp_bias, lo);
            decode_fp4_chunk(c1, 126 + static_cast<int>((szv >> 8) & 0xff) - p.fp4_exp_bias, hi);
          } else {
            decode_i2_chunk(c0, p.code_bias, lo);
            decode_i2_chunk(c1, p.code_bias, hi);
          }
        }
        mbar_wait(&ctl->a_empty[sa], ((kc / kASlots) & 1) ^ 1, abort_flag, st, 7);
        tc_fence_after_sync();
        tmem_st_32x32b_x32(tmem_base + lane_addr + kAccCols + sa * 32, regs);
        tc_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->a_full[sa]);
      }
    }
  } else if (warp >= 12) {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t tc = 0;
    SegmentWalk walk(p);
    Segment w;
    while (walk.next(p, w)) {
      const int n = w.n_tile * kTileRows + row_in_tile;
      const bool n_ok = n < p.N;
      mbar_wait(&ctl->acc_full, tc & 1, abort_flag, st, 8);
      tc_fence_after_sync();
#pragma unroll 1
      for (int c = 0; c < TN / NV; ++c) {
        uint32_t acc[NV];
        if constexpr (NV == 32) tmem_ld_32x32b_x32(tmem_base + lane_addr + c * NV, acc);
        else tmem_ld_32x32b_x16(tmem_base + lane_addr + c * NV, acc);
        tc_wait_ld();
        const int m0 = w.m_tile * TN + c * NV;
        if (w.slot >= 0) {
          // partial tile: raw accumulator values, [token][row] so lanes coalesce
          uint32_t* dst = p.partial + (static_cast<size_t>(w.slot) * TN + c * NV) * kTileRows + row_in_tile;
#pragma unroll
          for (int j = 0; j < NV; ++j) dst[j * kTileRows] = acc[j];
        } else if (n_ok) {
          switch (p.out_type) {
            case OUT_F16: store_values<__half, kInt, NV>(p, acc, m0, n); break;
            case OUT_BF16: store_values<__nv_bfloat16, kInt, NV>(p, acc, m0, n); break;
            case OUT_F32: store_values<float, kInt, NV>(p, acc, m0, n); break;
            default: store_values<int, kInt, NV>(p, acc, m0, n); break;
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty);
      ++tc;
    }
  }

  // ---------------- teardown ----------------
  if (*abort_flag) {
    // give copies that may still be in flight time to land before the CTA's
    // shared memory goes away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// Second pass of stream-K: for every tile that was cut between CTAs, add its
// partial tiles in ascending CTA order and write the result. One block per tile,
// one thread per weight row. Integer partials are added as integers (exact).
template <typename OutT, int TN, bool kIntAcc>
__global__ void __launch_bounds__(kTileRows)
streamk_fixup_kernel(const GemmParams p) {
  const long long tile = blockIdx.x;
  const long long t_begin = tile * p.kb_total;
  const long long t_end = t_begin + p.kb_total;
  const int c_first = static_cast<int>(t_begin / p.span);
  const int c_last = static_cast<int>((t_end - 1) / p.span);
  if (c_first == c_last) return;   // whole tile done by one CTA
  const int m_tile = static_cast<int>(tile % p.m_tiles);
  const int n_tile = static_cast<int>(tile / p.m_tiles);
  const int row = threadIdx.x;
  const int n = n_tile * kTileRows + row;
  if (n >= p.N) return;
  for (int j = 0; j < TN; ++j) {
    const int m = m_tile * TN + j;
    if (m >= p.M) break;
    float facc = 0.f;
    int iacc = 0;
    for (int c = c_first; c <= c_last; ++c) {
      // slot 0 if this tile holds the first segment of CTA c's span, else slot 1
      const long long span_begin = static_cast<long long>(c) * p.span;
      const int slot = c * 2 + ((span_begin >= t_begin) ? 0 : 1);
      const uint32_t raw = p.partial[(static_cast<size_t>(slot) * TN + j) * kTileRows + row];
      if constexpr (kIntAcc) iacc += static_cast<int>(raw);
      else facc += __uint_as_float(raw);
    }
    uint32_t bits;
    if constexpr (kIntAcc) bits = static_cast<uint32_t>(iacc);
    else bits = __float_as_uint(facc);
    store_values<OutT, kIntAcc, 1>(p, &bits, m, n);
  }
}

}  // namespace b200dq
