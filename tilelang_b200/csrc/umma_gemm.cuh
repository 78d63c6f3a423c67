// Warp-specialised, persistent, TMA-fed tcgen05 GEMM with in-register weight
// dequantisation:  C[M,N] = A[M,K] * dequant(W[N,K])^T.
//
// It replaces, for sm_100a, the kernels the reference generates from
//   examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:16-90   (W4A16),
//   examples/dequantize_gemm/example_dequant_gemm_bf16_mxfp4_hopper.py:80-378 (MXFP4),
//   examples/dequantize_gemm/example_dequant_gemm_w4a8.py:85-149          (W4A8),
//   examples/dequantize_gemm/example_dequant_gemv_fp16xint4.py:11-155     (small M),
//   examples/bitnet-1.58b/kernel_benchmark/tilelang_bitnet_158_int8xint2_{decode,prefill}.py,
// which on this architecture lower to mma.sync / dp4a with a register->smem->ldmatrix
// round trip of the dequantised tile (src/cuda/op/gemm.cc:337-390).
//
// Design. The product is computed transposed so the *weights* are the MMA's
// M side: one CTA tile is 128 weight rows x TN tokens. Dequantised weights never
// touch shared memory: a dequant thread owns one weight row (= one TMEM lane),
// expands its packed bytes to 64 16-bit (or 128 8-bit) K elements in registers
// and writes them with tcgen05.st into a TMEM ring; the MMA reads its A operand
// from TMEM ("TS" form) and its B operand (activations, K-major, 128-byte
// swizzle) from a TMA-filled shared-memory ring. Accumulators (fp32 or int32)
// live in TMEM columns [0, 256).
//
//   warp 0      : producer: packed weights (cp.async.bulk, one stage = 2 k-blocks
//                 of codes + their scale words) and activations (tiled TMA)
//   warps 1-3   : MMA issuers (one elected lane each); warp 1 owns TMEM.
//                 A single thread issues one tcgen05.mma per ~45 cycles, so for
//                 narrow token tiles NI = 2 or 3 issuers take k-blocks round-robin,
//                 each into its own accumulator; the epilogue adds them.
//   warps 4-11  : two dequant warpgroups, alternating weight stages
//   warps 12-15 : epilogue (tcgen05.ld -> convert -> smem transpose -> 16-byte stores)
//
// k-block = 64 16-bit (128 8-bit) K elements = one 128 B swizzle atom of activations.
//   full_w/empty_w : packed weight ring, per stage      (TMA -> dequant warps)
//   full_b         : activation ring, per k-block       (TMA -> MMA)
//   a_full         : dequantised TMEM ring, per k-block (dequant warps -> MMA)
//   cons           : k-block consumed by the MMA (tcgen05.commit); frees both the
//                    TMEM slot and the activation stage
//   acc_full/acc_empty : accumulators                   (MMA -> epilogue)
// Every wait is bounded (ptx.cuh); a wait that gives up sets a status word.
//
// Scheduling is stream-K: the (tile, stage) space is cut into equal contiguous
// spans, one per CTA, so every SM streams the same number of weight bytes. A
// span's first and last segment may cover only part of a tile; those write raw
// partial tiles to scratch slots (two per CTA) and a second small kernel adds the
// slots of each split tile in a fixed order (deterministic, no atomics).
#pragma once
#include <type_traits>

#include "decode.cuh"
#include "ptx.cuh"

namespace b200dq {

#ifdef B200DQ_PROFILE
#define PROF_DECL(name) long long name = 0
#define PROF_T0(t) long long t = clock64()
#define PROF_ADD(acc, t) do { long long _n = clock64(); acc += _n - t; t = _n; } while (0)
#else
#define PROF_DECL(name)
#define PROF_T0(t)
#define PROF_ADD(acc, t)
#endif

enum WeightFormat : int {
  WF_U4_SZ = 0,       // uint4, per-group scale + zero (16-bit activations)
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
  GF_ROW_SCALE = 4,    // integer path: acc / row_scale[m] / tensor_scale before the cast
  GF_VEC_STORE = 8,    // internal: base and pitch of the output allow 16-byte stores
};

struct GemmParams {
  const uint8_t* wp;         // packed image: [n_tiles][st_total][stage_bytes]
  void* c;                   // output
  uint32_t* partial;         // scratch: [grid][2][TN][128] raw fp32/int32 partial tiles
  const void* bias;          // optional bias [M][N]
  const float* row_scale;    // optional per-token divisor [M]
  float tensor_scale;        // optional per-tensor divisor
  uint32_t code_bias;        // bytewise bias for the integer decoders
  int fp4_exp_bias;          // 127 for OCP e8m0, 0 for a raw exponent byte
  int M, N, K;
  int n_tiles, m_tiles, st_total;   // st_total = weight stages (2 k-blocks each) per tile
  int span;                  // stages per CTA (stream-K span length)
  long long units;           // m_tiles * n_tiles * st_total
  int stage_bytes;           // bytes of one packed stage in global memory
  int sz_per_kb;             // 1 if each k-block of a stage has its own scale word (group 64)
  int ldc;                   // leading dimension of the output
  int flags;
  int out_type;
  DeviceStatus* status;
  unsigned long long* prof;  // optional per-CTA phase timers (profiling builds only)
};

constexpr int kTileRows = 128;        // weight rows per CTA tile (= TMEM lanes)
constexpr int kThreads = 512;
constexpr int kStageBufBytes = 2048;                    // one epilogue staging buffer: 32 n x 32 m x 2 B
constexpr int kStagingBytesPerWarp = 2 * kStageBufBytes;   // double-buffered
constexpr int kMaxSlots = 16;

__host__ __device__ constexpr int codes_per_kblock_bytes(int wf) { return wf == WF_I4_I8 ? 8192 : 4096; }
// scale words carried by one stage in shared memory (upper bound, bytes)
__host__ __device__ constexpr int sz_smem_bytes(int wf) { return wf == WF_U4_SZ ? 1024 : (wf == WF_FP4_E8M0 ? 512 : 0); }
__host__ __device__ constexpr int issuers_for(int tn) { return tn >= 256 ? 1 : (tn >= 128 ? 2 : 3); }

// TMEM plan: accumulators of the NI issuers in columns [0, kAccCols), then a ring
// of kSlots dequantised k-blocks (32 columns each). The activation ring in shared
// memory has at most as many stages, so one "consumed" barrier per slot serves both.
template <int TN, int WF>
struct RingConfig {
  static constexpr int kNI = issuers_for(TN);
  static constexpr int kAccCols = ((kNI * TN + 31) / 32) * 32;
  static constexpr int kSlots = (512 - kAccCols) / 32 > 14 ? 14 : (512 - kAccCols) / 32;
  static constexpr int kBStageBytes = TN * 128;
  static constexpr int kCodeBytes = 2 * codes_per_kblock_bytes(WF);          // per stage
  static constexpr int kWStageSmem = kCodeBytes + sz_smem_bytes(WF);         // smem stride
  static constexpr int kNB = TN >= 256 ? 5 : kSlots;
  static constexpr int kWBudget = TN >= 256 ? 37 * 1024 : (TN >= 128 ? 74 * 1024 : 110 * 1024);
  static constexpr int kNW = kWBudget / kWStageSmem;
  static constexpr int kStaging = 4 * kStagingBytesPerWarp;
  static constexpr int kSmemBytes = kNB * kBStageBytes + kNW * kWStageSmem + kStaging + 1024 /*align*/ + 1024 /*ctl*/;
  static_assert(kSlots >= 8 && kSlots <= kMaxSlots && kNB <= kSlots, "ring depths");
  static_assert(kNW >= 2 && kNW <= 32, "weight ring depth");
  static_assert(kWStageSmem % 128 == 0, "stage stride keeps 128 B alignment");
  static_assert(kSmemBytes <= 232448, "over the 227 KiB shared-memory limit");
};

struct SharedCtl {
  uint64_t full_w[32];
  uint64_t empty_w[32];
  uint64_t full_b[kMaxSlots];
  uint64_t a_full[kMaxSlots];
  uint64_t cons[kMaxSlots];
  uint64_t acc_full;
  uint64_t acc_empty;
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(SharedCtl) <= 1024, "control block must fit its slot");

// One contiguous run of weight stages inside one tile.
struct Segment {
  int m_tile, n_tile, st_begin, st_end;
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
    const long long tile = pos / p.st_total;
    s.st_begin = static_cast<int>(pos - tile * p.st_total);
    const long long left = end - pos;
    s.st_end = static_cast<int>(min(static_cast<long long>(p.st_total), s.st_begin + left));
    // n fastest: the CTAs working at the same time share a few token slabs (which
    // stay in L2) and stream different weight tiles
    s.n_tile = static_cast<int>(tile % p.n_tiles);
    s.m_tile = static_cast<int>(tile / p.n_tiles);
    const bool whole = (s.st_begin == 0 && s.st_end == p.st_total);
    s.slot = whole ? -1 : (static_cast<int>(blockIdx.x) * 2 + (first ? 0 : 1));
    first = false;
    pos += (s.st_end - s.st_begin);
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

// Final value of one output element from its raw accumulator bits.
template <typename OutT, bool kIntAcc>
__device__ __forceinline__ OutT finish_value(const GemmParams& p, uint32_t raw, int m, int n) {
  if constexpr (kIntAcc && std::is_same<OutT, int>::value) {
    return static_cast<int>(raw);   // exact int32 result
  } else {
    float v;
    if constexpr (kIntAcc) {
      v = static_cast<float>(static_cast<int>(raw));
      if (p.flags & GF_ROW_SCALE) v = v / p.row_scale[m] / p.tensor_scale;
    } else {
      v = __uint_as_float(raw);
    }
    if (p.flags & GF_HAS_BIAS) v += bias_as_float<OutT>(p.bias, static_cast<size_t>(m) * p.N + n);
    return cast_out<OutT>(v);
  }
}

// Slow path: direct, predicated global stores (unaligned pitch or transposed output).
template <typename OutT, bool kIntAcc, int NV>
__device__ __forceinline__ void store_values_direct(const GemmParams& p, const uint32_t* acc, int m0, int n) {
  OutT* c = reinterpret_cast<OutT*>(p.c);
  const bool trans = (p.flags & GF_TRANS_C) != 0;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int m = m0 + j;
    if (m < p.M) {
      const size_t idx = trans ? static_cast<size_t>(n) * p.ldc + m : static_cast<size_t>(m) * p.ldc + n;
      c[idx] = finish_value<OutT, kIntAcc>(p, acc[j], m, n);
    }
  }
}

// Fast path: the warp's 32 (n) x NV (m) block is transposed through shared
// memory ([m][n], one warp-private buffer) and leaves as 16-byte stores, each
// covering 8 (or 4) consecutive n of one output row. Needs a 16-byte aligned
// base and row pitch; rows beyond M and 16-byte groups beyond N are skipped.
template <typename OutT, bool kIntAcc, int NV>
__device__ __forceinline__ void store_values_vec(const GemmParams& p, const uint32_t* acc, int m0, int n,
                                                 int n0_warp, uint8_t* sbuf, int lane, bool plain) {
  constexpr int ES = static_cast<int>(sizeof(OutT));
  constexpr int RPP = (kStagingBytesPerWarp / (32 * ES)) < NV ? (kStagingBytesPerWarp / (32 * ES)) : NV;   // rows per pass
  constexpr int VPR = 32 * ES / 16;          // 16-byte vectors per row: 4 (2-byte) or 8 (4-byte)
  constexpr int RPI = 32 / VPR;              // rows covered by one warp-wide vector store
  OutT* s = reinterpret_cast<OutT*>(sbuf);
  OutT* c = reinterpret_cast<OutT*>(p.c);
#pragma unroll
  for (int pass = 0; pass < NV / RPP; ++pass) {
    __syncwarp();   // previous pass's reads are done
    if (plain) {
#pragma unroll
      for (int j = 0; j < RPP; ++j) {
        const uint32_t raw = acc[pass * RPP + j];
        if constexpr (kIntAcc && std::is_same<OutT, int>::value) s[j * 32 + lane] = static_cast<int>(raw);
        else if constexpr (kIntAcc) s[j * 32 + lane] = cast_out<OutT>(static_cast<float>(static_cast<int>(raw)));
        else s[j * 32 + lane] = cast_out<OutT>(__uint_as_float(raw));
      }
    } else {
      const bool n_ok = n < p.N;
#pragma unroll
      for (int j = 0; j < RPP; ++j) {
        const int m = m0 + pass * RPP + j;
        if (n_ok && m < p.M) s[j * 32 + lane] = finish_value<OutT, kIntAcc>(p, acc[pass * RPP + j], m, n);
      }
    }
    __syncwarp();
    const int vcol = lane % VPR;                       // which 16-byte group of the row
    const int ncol = n0_warp + vcol * (16 / ES);
#pragma unroll
    for (int it = 0; it < RPP / RPI; ++it) {
      const int r = it * RPI + lane / VPR;
      const int m = m0 + pass * RPP + r;
      if (m < p.M && ncol < p.N) {
        const uint4 v = *reinterpret_cast<const uint4*>(sbuf + r * 32 * ES + vcol * 16);
        *reinterpret_cast<uint4*>(c + static_cast<size_t>(m) * p.ldc + ncol) = v;
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
  constexpr int WSS = Ring::kWStageSmem;
  constexpr int CPK = codes_per_kblock_bytes(WF);   // code bytes per k-block
  constexpr int NI = Ring::kNI;
  constexpr int NS = Ring::kSlots;       // dequantised TMEM ring slots
  constexpr int kAccCols = Ring::kAccCols;
  constexpr bool kInt = (ACT == ACT_I8);
  constexpr bool kBf16 = (ACT == ACT_BF16);
  constexpr int BKE = kInt ? 128 : 64;   // K elements per k-block
  constexpr int NV = TN >= 32 ? 32 : 16; // accumulator columns per tcgen05.ld

#ifdef B200DQ_PROFILE
  __shared__ long long prof_ts_b[kMaxSlots];   // issue time of the activation load in each stage
#endif
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_b = smem;                                   // NB x (TN x 128 B), 1024-aligned stages
  uint8_t* smem_w = smem_b + NB * Ring::kBStageBytes;       // NW x stage
  uint8_t* smem_o = smem_w + NW * WSS;                      // epilogue staging, 8 KiB per warp
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem_o + Ring::kStaging);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &ctl->abort_flag;
  DeviceStatus* st = p.status;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NW; ++i) { mbar_init(&ctl->full_w[i], 1); mbar_init(&ctl->empty_w[i], 4); }
    for (int i = 0; i < NB; ++i) mbar_init(&ctl->full_b[i], 1);
    for (int i = 0; i < NS; ++i) { mbar_init(&ctl->a_full[i], 4); mbar_init(&ctl->cons[i], 1); }
    mbar_init(&ctl->acc_full, NI);
    mbar_init(&ctl->acc_empty, 4);
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ---------------- producer: two independent streams (weight stages and
    // activation k-blocks) served by one thread; each is issued as soon as its
    // ring has room, polled without blocking so neither delays the other ----
    if (lane == 0) {
      SegmentWalk walk_w(p), walk_b(p);
      Segment sw_seg, sb_seg;
      bool have_w = walk_w.next(p, sw_seg), have_b = walk_b.next(p, sb_seg);
      int st_w = have_w ? sw_seg.st_begin : 0, kb_b = have_b ? sb_seg.st_begin * 2 : 0;
      uint32_t wc = 0;   // weight stages issued
      uint32_t bc = 0;   // k-blocks of activations issued
      uint64_t t_idle = 0;
      uint32_t idle = 0;
      PROF_DECL(pp_w); PROF_DECL(pp_b); PROF_DECL(pp_idle); PROF_DECL(pp_iters);
      PROF_T0(tp);
      while (have_w || have_b) {
        bool progressed = false;

        if (have_w) {
          const uint32_t s = wc % NW;
          if (mbar_test_wait(&ctl->empty_w[s], ((wc / NW) & 1) ^ 1)) {
            mbar_arrive_expect_tx(&ctl->full_w[s], p.stage_bytes);
            const uint8_t* src = p.wp + (static_cast<size_t>(sw_seg.n_tile) * p.st_total + st_w) * p.stage_bytes;
            tma_bulk_g2s(smem_w + s * WSS, src, p.stage_bytes, &ctl->full_w[s]);
            ++wc;
            if (++st_w >= sw_seg.st_end) { have_w = walk_w.next(p, sw_seg); st_w = sw_seg.st_begin; }
            progressed = true;
            PROF_ADD(pp_iters, tp);
          }
        }
        if (have_b) {
          const uint32_t s = bc % NB;
          bool room = bc < static_cast<uint32_t>(NB);
          if (!room) {
            const uint32_t prev = bc - NB;   // k-block that used this stage before
            room = mbar_test_wait(&ctl->cons[prev % NS], (prev / NS) & 1);
          }
          PROF_ADD(pp_idle, tp);
          if (room) {
#ifdef B200DQ_PROFILE
            prof_ts_b[s] = clock64();
#endif
            mbar_arrive_expect_tx(&ctl->full_b[s], Ring::kBStageBytes);
            tma_load_2d(smem_b + s * Ring::kBStageBytes, &tmap_a, kb_b * BKE, sb_seg.m_tile * TN, &ctl->full_b[s]);
            PROF_ADD(pp_w, tp);
            ++bc;
            if (++kb_b >= sb_seg.st_end * 2) { have_b = walk_b.next(p, sb_seg); kb_b = sb_seg.st_begin * 2; }
            progressed = true;
            PROF_ADD(pp_b, tp);
          }
        }

        if (progressed) {
          idle = 0;
        } else if (((++idle) & 0x3f) == 0) {
          // bounded: give up if nothing moved for the wait limit
          if (*abort_flag) break;
          const uint64_t now = globaltimer_ns();
          if (idle == 0x40) t_idle = now;
          else if (now - t_idle > B200DQ_WAIT_LIMIT_NS) { mbar_wait_failed(abort_flag, st, 1); break; }
        }
      }
#ifdef B200DQ_PROFILE
      if (p.prof) { unsigned long long* o = p.prof + blockIdx.x * 32 + 28; o[0] = pp_w; o[1] = pp_b; o[2] = pp_idle; o[3] = pp_iters; }
#endif
    }
  } else if (warp >= 1 && warp <= 3) {
    // ---------------- MMA issuers ----------------
    // The tensor pipe queues only a couple of MMAs, so the issuer must never be
    // away from it for long: the barriers of its next k-block are checked between
    // the second and third MMA of the current one, and ring positions are stepped
    // without divisions.
    const int me = warp - 1;
    if (me < NI && lane == 0) {
      constexpr uint32_t idesc =
          kInt ? make_idesc(2u, 1u, 1u, 128u, TN) : make_idesc(1u, kBf16 ? 1u : 0u, kBf16 ? 1u : 0u, 128u, TN);
      const uint32_t acc_tmem = tmem_base + me * TN;
      const uint32_t b_base = smem_u32(smem_b);
      // ring state of this issuer's next k-block (global k-block counter kc = me, me+NI, ...)
      uint32_t sa = me % NS, pa = 0;   // dequantised slot and its a_full parity
      uint32_t sb = me % NB, pb = 0;   // activation stage and its full_b parity
      uint32_t mine = me;              // global index of this issuer's next k-block
      uint32_t kc_seg = 0;             // global index of the segment's first k-block
      uint32_t tc = 0;
      bool ok = true;
      SegmentWalk walk(p);
      Segment w;
      PROF_DECL(pm_acc); PROF_DECL(pm_a); PROF_DECL(pm_b); PROF_DECL(pm_issue); PROF_DECL(pm_commit); PROF_DECL(pm_lat);
#ifdef B200DQ_PROFILE
      long long pm_latmin = 1ll << 40;
#endif
      PROF_T0(tm);
      while (walk.next(p, w)) {
        ok &= mbar_wait(&ctl->acc_empty, (tc & 1) ^ 1, abort_flag, st, 3);
        tc_fence_after_sync();
        PROF_ADD(pm_acc, tm);
        const uint32_t kc_end = kc_seg + static_cast<uint32_t>(w.st_end - w.st_begin) * 2;
        bool fresh = true;
        bool ready = false;   // barriers of k-block `mine` already passed
        while (mine < kc_end) {
          if (!ready) {
            ok &= mbar_wait(&ctl->a_full[sa], pa, abort_flag, st, 4);
            PROF_ADD(pm_a, tm);
            ok &= mbar_wait(&ctl->full_b[sb], pb, abort_flag, st, 5);
            PROF_ADD(pm_b, tm);
            tc_fence_after_sync();
          }
          const uint32_t a_tmem = tmem_base + kAccCols + sa * 32;
          const uint64_t b_desc = make_smem_desc_sw128(b_base + sb * Ring::kBStageBytes);
          const uint32_t sa_cur = sa;
          // advance ring state to this issuer's next k-block
          mine += NI;
          sa += NI; if (sa >= static_cast<uint32_t>(NS)) { sa -= NS; pa ^= 1; }
          sb += NI; if (sb >= static_cast<uint32_t>(NB)) { sb -= NB; pb ^= 1; }
          if (ok) {
            if constexpr (kInt) {
              umma_ts_i8(acc_tmem, a_tmem, b_desc, idesc, fresh ? 0u : 1u);
              umma_ts_i8(acc_tmem, a_tmem + 8, b_desc + 2, idesc, 1u);
            } else {
              umma_ts_f16(acc_tmem, a_tmem, b_desc, idesc, fresh ? 0u : 1u);
              umma_ts_f16(acc_tmem, a_tmem + 8, b_desc + 2, idesc, 1u);
            }
          }
          ready = false;
          if (mine < kc_end) {
            PROF_ADD(pm_issue, tm);
            ok &= mbar_wait(&ctl->full_b[sb], pb, abort_flag, st, 5);
            PROF_ADD(pm_b, tm);
#ifdef B200DQ_PROFILE
            { const long long lat = clock64() - prof_ts_b[sb]; pm_lat += lat; if (lat < pm_latmin) pm_latmin = lat; }
#endif
            ok &= mbar_wait(&ctl->a_full[sa], pa, abort_flag, st, 4);
            PROF_ADD(pm_a, tm);
            tc_fence_after_sync();
            ready = true;
          }
          if (ok) {
            if constexpr (kInt) {
              umma_ts_i8(acc_tmem, a_tmem + 16, b_desc + 4, idesc, 1u);
              umma_ts_i8(acc_tmem, a_tmem + 24, b_desc + 6, idesc, 1u);
            } else {
              umma_ts_f16(acc_tmem, a_tmem + 16, b_desc + 4, idesc, 1u);
              umma_ts_f16(acc_tmem, a_tmem + 24, b_desc + 6, idesc, 1u);
            }
          }
          fresh = false;
          PROF_ADD(pm_issue, tm);
          tc_commit(&ctl->cons[sa_cur]);
          PROF_ADD(pm_commit, tm);
        }
        if (!fresh) tc_commit(&ctl->acc_full);
        else mbar_arrive(&ctl->acc_full);
        kc_seg = kc_end;
        ++tc;
      }
#ifdef B200DQ_PROFILE
      if (p.prof && me == 0) { unsigned long long* o = p.prof + blockIdx.x * 32; o[0] = pm_acc; o[1] = pm_a; o[2] = pm_b; o[3] = pm_issue; o[4] = kc_seg; o[5] = pm_commit; o[6] = pm_lat; o[7] = pm_latmin; }
#endif
    }
  } else if (warp >= 4 && warp < 12) {
    // ---------------- dequant warpgroups ----------------
    const int dg = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t sc = 0;   // weight stages seen by this CTA
    bool ok = true;
    SegmentWalk walk(p);
    Segment w;
    PROF_DECL(pd_w); PROF_DECL(pd_dec); PROF_DECL(pd_a); PROF_DECL(pd_st); PROF_DECL(pd_n);
    PROF_T0(td);
    while (walk.next(p, w)) {
      for (int sti = w.st_begin; sti < w.st_end; ++sti, ++sc) {
        if ((sc & 1) != static_cast<uint32_t>(dg)) continue;
        const uint32_t sw = sc % NW;
        PROF_ADD(pd_dec, td);
        ok &= mbar_wait(&ctl->full_w[sw], (sc / NW) & 1, abort_flag, st, 6);
        PROF_ADD(pd_w, td);
        const uint8_t* stage = smem_w + sw * WSS;
        const uint4* codes = reinterpret_cast<const uint4*>(stage);
        constexpr int CH = CPK / 2048;   // 16-byte chunks per row and k-block
        uint4 c[2][CH];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int q = 0; q < CH; ++q) c[h][q] = codes[(h * CH + q) * 128 + row_in_tile];
        uint32_t sz0 = 0, sz1 = 0;
        if constexpr (WF == WF_U4_SZ) {
          const uint32_t* szp = reinterpret_cast<const uint32_t*>(stage + Ring::kCodeBytes);
          sz0 = szp[row_in_tile];
          sz1 = p.sz_per_kb ? szp[128 + row_in_tile] : sz0;
        } else if constexpr (WF == WF_FP4_E8M0) {
          sz0 = reinterpret_cast<const uint32_t*>(stage + Ring::kCodeBytes)[row_in_tile];
          sz1 = sz0 >> 16;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->empty_w[sw]);

#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t szv = h == 0 ? sz0 : sz1;
          uint32_t regs[32];
#ifdef B200DQ_EXP_NODECODE
#pragma unroll
          for (int q = 0; q < 32; ++q) regs[q] = c[h][q & 1].x + szv + q;
          if (true) {} else if (false) {
#else
          if constexpr (WF == WF_I4_I8) {
#endif
#pragma unroll
            for (int q = 0; q < 4; ++q)
              decode_i4_chunk(c[h][q], p.code_bias, *reinterpret_cast<uint32_t (*)[8]>(&regs[8 * q]));
          } else {
            uint32_t (&lo)[16] = *reinterpret_cast<uint32_t (*)[16]>(&regs[0]);
            uint32_t (&hi)[16] = *reinterpret_cast<uint32_t (*)[16]>(&regs[16]);
            if constexpr (WF == WF_U4_SZ) {
              decode_u4_chunk<kBf16>(c[h][0], szv, lo);
              decode_u4_chunk<kBf16>(c[h][1], szv, hi);
            } else if constexpr (WF == WF_U4_RAW) {
              decode_u4_chunk_noscale<kBf16, false>(c[h][0], lo);
              decode_u4_chunk_noscale<kBf16, false>(c[h][1], hi);
            } else if constexpr (WF == WF_S4_RAW) {
              decode_u4_chunk_noscale<kBf16, true>(c[h][0], lo);
              decode_u4_chunk_noscale<kBf16, true>(c[h][1], hi);
            } else if constexpr (WF == WF_FP4_E8M0) {
              decode_fp4_chunk(c[h][0], 126 + static_cast<int>(szv & 0xff) - p.fp4_exp_bias, lo);
              decode_fp4_chunk(c[h][1], 126 + static_cast<int>((szv >> 8) & 0xff) - p.fp4_exp_bias, hi);
            } else {
              decode_i2_chunk(c[h][0], p.code_bias, lo);
              decode_i2_chunk(c[h][1], p.code_bias, hi);
            }
          }
          const uint32_t kc = sc * 2 + h;
          const uint32_t sa = kc % NS;
          PROF_ADD(pd_dec, td);
          if (kc >= static_cast<uint32_t>(NS)) {
            const uint32_t prev = kc - NS;
#ifndef B200DQ_EXP_NO_CONS
            ok &= mbar_wait(&ctl->cons[sa], (prev / NS) & 1, abort_flag, st, 7);
#endif
          }
          PROF_ADD(pd_a, td);
          tc_fence_after_sync();
#ifndef B200DQ_EXP_NOST
          tmem_st_32x32b_x32(tmem_base + lane_addr + kAccCols + sa * 32, regs);
          tc_wait_st();
#else
          if (regs[0] == 0x12345678u && regs[17] == 0x9abcdef0u) tmem_st_32x32b_x32(tmem_base + lane_addr + kAccCols + sa * 32, regs);
#endif
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->a_full[sa]);
          PROF_ADD(pd_st, td);
        }
#ifdef B200DQ_PROFILE
        ++pd_n;
#endif
      }
    }
#ifdef B200DQ_PROFILE
    if (p.prof && lane == 0 && quarter == 0) { unsigned long long* o = p.prof + blockIdx.x * 32 + 8 + dg * 8; o[0] = pd_w; o[1] = pd_dec; o[2] = pd_a; o[3] = pd_st; o[4] = pd_n; }
#endif
    (void)ok;
  } else if (warp >= 12) {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    uint8_t* my_stage = smem_o + quarter * kStagingBytesPerWarp;
    const bool use_vec = (p.flags & GF_VEC_STORE) != 0;
    const bool plain = (p.flags & (GF_HAS_BIAS | GF_ROW_SCALE)) == 0;
    uint32_t tc = 0, kc = 0;
    bool ok = true;
    SegmentWalk walk(p);
    Segment w;
    PROF_DECL(pe_wait); PROF_DECL(pe_ld); PROF_DECL(pe_store);
    PROF_T0(te);
    while (walk.next(p, w)) {
      const int n0_warp = w.n_tile * kTileRows + quarter * 32;
      const int n = n0_warp + lane;
      const int nkb = (w.st_end - w.st_begin) * 2;
      // accumulators that received at least one k-block in this segment
      uint32_t valid = 0;
#pragma unroll
      for (int i = 0; i < NI; ++i)
        if (i < nkb) valid |= 1u << ((kc + i) % NI);
      kc += nkb;
      ok &= mbar_wait(&ctl->acc_full, tc & 1, abort_flag, st, 8);
      tc_fence_after_sync();
      PROF_ADD(pe_wait, te);
#pragma unroll 1
      for (int c = 0; c < TN / NV; ++c) {
        uint32_t acc[NV];
        bool have = false;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          if (!(valid & (1u << i))) continue;
          uint32_t part[NV];
          if constexpr (NV == 32) tmem_ld_32x32b_x32(tmem_base + lane_addr + i * TN + c * NV, part);
          else tmem_ld_32x32b_x16(tmem_base + lane_addr + i * TN + c * NV, part);
          tc_wait_ld();
          if (!have) {
#pragma unroll
            for (int j = 0; j < NV; ++j) acc[j] = part[j];
            have = true;
          } else {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
              if constexpr (kInt) acc[j] = static_cast<uint32_t>(static_cast<int>(acc[j]) + static_cast<int>(part[j]));
              else acc[j] = __float_as_uint(__uint_as_float(acc[j]) + __uint_as_float(part[j]));
            }
          }
        }
        PROF_ADD(pe_ld, te);
        const int m0 = w.m_tile * TN + c * NV;
        if (w.slot >= 0) {
          // partial tile: raw accumulator values, [token][row] so lanes coalesce
          uint32_t* dst = p.partial + (static_cast<size_t>(w.slot) * TN + c * NV) * kTileRows + row_in_tile;
#pragma unroll
          for (int j = 0; j < NV; ++j) dst[j * kTileRows] = acc[j];
        } else if (use_vec) {
          if (m0 < p.M && n0_warp < p.N) {
            switch (p.out_type) {
              case OUT_F16: store_values_vec<__half, kInt, NV>(p, acc, m0, n, n0_warp, my_stage, lane, plain); break;
              case OUT_BF16: store_values_vec<__nv_bfloat16, kInt, NV>(p, acc, m0, n, n0_warp, my_stage, lane, plain); break;
              case OUT_F32: store_values_vec<float, kInt, NV>(p, acc, m0, n, n0_warp, my_stage, lane, plain); break;
              default: store_values_vec<int, kInt, NV>(p, acc, m0, n, n0_warp, my_stage, lane, plain); break;
            }
          }
        } else if (n < p.N) {
          switch (p.out_type) {
            case OUT_F16: store_values_direct<__half, kInt, NV>(p, acc, m0, n); break;
            case OUT_BF16: store_values_direct<__nv_bfloat16, kInt, NV>(p, acc, m0, n); break;
            case OUT_F32: store_values_direct<float, kInt, NV>(p, acc, m0, n); break;
            default: store_values_direct<int, kInt, NV>(p, acc, m0, n); break;
          }
        }
        PROF_ADD(pe_store, te);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty);
      ++tc;
    }
#ifdef B200DQ_PROFILE
    if (p.prof && lane == 0 && quarter == 0) { unsigned long long* o = p.prof + blockIdx.x * 32 + 24; o[0] = pe_wait; o[1] = pe_ld; o[2] = pe_store; o[3] = tc; }
#endif
    (void)ok;
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
  const long long t_begin = tile * p.st_total;
  const long long t_end = t_begin + p.st_total;
  const int c_first = static_cast<int>(t_begin / p.span);
  const int c_last = static_cast<int>((t_end - 1) / p.span);
  if (c_first == c_last) return;   // whole tile done by one CTA
  const int n_tile = static_cast<int>(tile % p.n_tiles);
  const int m_tile = static_cast<int>(tile / p.n_tiles);
  const int row = threadIdx.x;
  const int n = n_tile * kTileRows + row;
  if (n >= p.N) return;
  OutT* c = reinterpret_cast<OutT*>(p.c);
  const bool trans = (p.flags & GF_TRANS_C) != 0;
  for (int j = 0; j < TN; ++j) {
    const int m = m_tile * TN + j;
    if (m >= p.M) break;
    float facc = 0.f;
    int iacc = 0;
    for (int cta = c_first; cta <= c_last; ++cta) {
      // slot 0 if this tile holds the first segment of that CTA's span, else slot 1
      const long long span_begin = static_cast<long long>(cta) * p.span;
      const int slot = cta * 2 + ((span_begin >= t_begin) ? 0 : 1);
      const uint32_t raw = p.partial[(static_cast<size_t>(slot) * TN + j) * kTileRows + row];
      if constexpr (kIntAcc) iacc += static_cast<int>(raw);
      else facc += __uint_as_float(raw);
    }
    uint32_t bits;
    if constexpr (kIntAcc) bits = static_cast<uint32_t>(iacc);
    else bits = __float_as_uint(facc);
    const size_t idx = trans ? static_cast<size_t>(n) * p.ldc + m : static_cast<size_t>(m) * p.ldc + n;
    c[idx] = finish_value<OutT, kIntAcc>(p, bits, m, n);
  }
}

}  // namespace b200dq
