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
//   warp 0      : weight producer (cp.async.bulk, one copy per pair of packed stages;
//                 a stage = 2 k-blocks of codes + their scale words)
//   warp 3      : activation producer (tiled TMA, one load per group of 1, 2 or 4 k-blocks)
//   warps 1-2   : MMA issuers (one elected lane each); warp 1 owns TMEM. They take
//                 alternate stages into the one accumulator, ordered by `turn`.
//   warps 4-11  : two dequant warpgroups, alternating weight stages
//   warps 12-15 : epilogue (tcgen05.ld -> convert -> smem transpose -> 16-byte stores)
//
// k-block = 64 16-bit (128 8-bit) K elements = one 128 B swizzle atom of activations.
//   full_w/empty_w : packed weight ring, per pair of stages (TMA -> dequant warps)
//   full_b/empty_b : activation ring, per group             (TMA -> MMA)
//   a_full         : dequantised TMEM ring, per stage, on the barrier of the stage's
//                    first slot                              (dequant warps -> MMA)
//   cons           : a stage (two k-blocks) consumed by the MMA (tcgen05.commit);
//                    frees its two TMEM slots (and, with one k-block per
//                    activation group, the activation stages)
//   turn           : hands the accumulator from the issuer of one stage to the other
//   acc_full/acc_empty : accumulator                        (MMA -> epilogue)
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


enum WeightFormat : int {
  WF_U4_SZ = 0,       // uint4, per-group scale + zero (16-bit activations)
  WF_U4_RAW = 1,      // uint4, weight = q              (no scale)
  WF_S4_RAW = 2,      // uint4 storing q = w + 8        (no scale)
  WF_FP4_E8M0 = 3,    // e2m1 + e8m0 block scale per 32 (bf16 activations; fp16 without block scale)
  WF_I2_I8 = 4,       // 2-bit codes -> int8, minus `code_bias` (int8 activations)
  WF_I4_I8 = 5,       // 4-bit codes -> int8, minus `code_bias` (int8 activations)
  WF_U2_SZ = 6,       // 2-bit codes + per-group scale and zero-point -> f16/bf16: (q - z) * s
  WF_LUT4_S = 7,      // 4-bit index into a 16-entry table (NF4 and other codebooks) * per-group scale
};
constexpr int kLastWeightFormat = WF_LUT4_S;

enum ActType : int { ACT_F16 = 0, ACT_BF16 = 1, ACT_I8 = 2 };
enum OutType : int { OUT_F16 = 0, OUT_BF16 = 1, OUT_F32 = 2, OUT_I32 = 3 };

enum GemmFlags : int {
  GF_TRANS_C = 1,      // write C^T (N x M) instead of C (M x N)
  GF_HAS_BIAS = 2,     // add bias[M][N] (output dtype) in the epilogue
  GF_ROW_SCALE = 4,    // integer path: acc / row_scale[m] / tensor_scale before the cast
  GF_VEC_STORE = 8,    // internal: base and pitch of the output allow 16-byte stores
  GF_FP4_SIMPLE = 16,  // fp4 codes follow the reference's no-subnormal rule 2^(e-1) * (1 + m/2)
};

struct GemmParams {
  const uint8_t* wp;         // packed image: [n_tiles][st_total][stage_bytes]
  const void* a;             // activations (M, K) row-major; read directly by the small-M kernel only
  void* c;                   // output
  uint32_t* partial;         // scratch: [grid][2][TN][128] raw fp32/int32 partial tiles
  const void* bias;          // optional bias [M][N]
  const float* row_scale;    // optional per-token divisor [M]
  float tensor_scale;        // optional per-tensor divisor
  uint32_t code_bias;        // bytewise bias for the integer decoders
  int fp4_exp_bias;          // 127 for OCP e8m0, 0 for a raw exponent byte
  int M, N, K;
  int n_tiles, m_tiles, st_total;   // st_total = weight stages (2 k-blocks each) per tile
  int st_units;              // stages the schedule gives a tile: st_total, or st_total + 1 (a stage past the
                             // end re-reads the last real stage's weights against zero-filled activations)
  int span;                  // stages per CTA (stream-K span length)
  long long units;           // m_tiles * n_tiles * st_total
  int stage_bytes;           // bytes of one packed stage in global memory
  int sz_per_kb;             // 1 if each k-block of a stage has its own scale word (group 64)
  int b_group;               // k-blocks per activation TMA: the tile's group size, or 1 (2-D map only)
  int ldc;                   // leading dimension of the output
  int flags;
  int out_type;
  // grouped (mixture-of-experts) mode: the rows of A and C are sorted by group,
  // group g owns rows [grp_row_prefix[g], grp_row_prefix[g+1]) and its own packed
  // image at wp + g * grp_w_stride; its tiles are numbered from grp_tile_prefix[g]
  const int* grp_row_prefix;     // num_groups + 1 entries, device memory (nullptr: one dense GEMM)
  const int* grp_tile_prefix;    // num_groups + 1 entries, device memory
  long long grp_w_stride;
  int num_groups;
  // Copies of the output on other GPUs (peer memory mapped into this process): every output
  // element is also stored at the same offset behind each of these bases, so a column shard
  // lands in every rank's gathered tensor straight from the epilogue (no separate all-gather).
  void* c_peer[7];
  int n_peers;
  // Small-M kernel only: tiles cut between CTAs are finished inside the kernel. tile_ctr holds one
  // 64-bit word per weight tile, (epoch << 8) | arrivals; a word whose epoch is not this launch's
  // counts as zero, so the array needs no clearing (the epoch is unique per launch).
  // WF_LUT4_S: the 16 table entries in the activation dtype, split into their low and high bytes
  // (entry i's low byte is byte i % 4 of lut_lo[i / 4]) for the byte-permute lookup.
  uint32_t lut_lo[4], lut_hi[4];
  unsigned long long* tile_ctr;
  unsigned long long epoch;
  int dyn_whole;                 // device-planned spans are rounded up to whole tiles (no tile is cut)
  int dyn_grid;                  // > 0: grouped mode planned on the device -- the tile total is read from
                                 // grp_tile_prefix[num_groups] and cut evenly over dyn_grid CTAs (span, units unused)
  int tn;                        // tokens per tile (the kernel's TN)
  DeviceStatus* status;
};

constexpr int kTileRows = 128;        // weight rows per CTA tile (= TMEM lanes)
constexpr int kThreads = 512;
constexpr int kStageBufBytes = 2048;                    // one epilogue staging buffer: 32 n x 32 m x 2 B
constexpr int kStagingBytesPerWarp = kStageBufBytes;      // one 32 x 32 x 2-byte transpose buffer per epilogue warp
constexpr int kMaxSlots = 16;

__host__ __device__ constexpr int codes_per_kblock_bytes(int wf) {
  return wf == WF_I4_I8 ? 8192 : (wf == WF_U2_SZ ? 2048 : 4096);
}
// scale words carried by one stage in shared memory (upper bound, bytes)
__host__ __device__ constexpr int sz_smem_bytes(int wf) {
  return (wf == WF_U4_SZ || wf == WF_U2_SZ || wf == WF_LUT4_S) ? 1024 : (wf == WF_FP4_E8M0 ? 512 : 0);
}

// TMEM plan: accumulators of the NI issuers in columns [0, kAccCols), then a ring
// of kSlots dequantised k-blocks (32 columns each).
// Shared memory: an activation ring of kNBG groups (one TMA each, kGB k-blocks), a
// weight ring of kNWP slots holding a *pair* of packed stages (one bulk copy
// each), and 4 KiB of epilogue staging per epilogue warp.
// accumulators per tile: narrow token tiles give each issuer its own (the epilogue adds
// them), so the two issue streams do not have to take turns
__host__ __device__ constexpr int issuers_for(int tn) { return tn <= 128 ? 2 : 1; }
__host__ __device__ constexpr int group_kblocks_for(int tn) { return tn >= 256 ? 1 : (tn >= 128 ? 2 : 4); }

template <int TN, int WF>
struct RingConfig {
  static constexpr int kNI = issuers_for(TN);
  static constexpr int kGB = group_kblocks_for(TN);
  static constexpr int kAccCols = ((kNI * TN + 31) / 32) * 32;
  // Ring depth in stages (kSlots / 2) is even: stage g then always returns to a `cons` barrier that
  // stages of its own parity -- its own issuer and dequant group -- used before, so both see every
  // phase of the barriers they wait on.
  static constexpr int kSlots = (512 - kAccCols) / 32 >= 12 ? 12 : 8;
  static constexpr int kBSlabBytes = TN * 128;                                // one k-block of activations
  static constexpr int kBGroupBytes = kGB * kBSlabBytes;
  // With two independent issuers (kNI == 2) the ring depth is even: when K is ragged the
  // groups shrink to single k-blocks, stage g then reads slots 2g and 2g + 1 (mod kNBG), and
  // only an even depth gives every slot to the same issuer each time round. An issuer that
  // sees a slot's barrier only every other phase can find it one phase behind, where the
  // parity test answers "complete" for a load that has not landed.
  static constexpr int kNBG = TN >= 256 ? (WF == WF_I4_I8 ? 5 : 6) : 4;
  static constexpr int kCodeBytes = 2 * codes_per_kblock_bytes(WF);           // per stage
  static constexpr int kWStageMax = kCodeBytes + sz_smem_bytes(WF);           // largest packed stage
  static constexpr int kWPairSmem = 2 * kWStageMax;                           // ring slot: two stages back to back
  static constexpr int kStaging = 4 * kStagingBytesPerWarp;
  static constexpr int kFixed = kNBG * kBGroupBytes + kStaging + 1024 /*align*/ + 1024 /*ctl*/;
  static constexpr int kNWPfit = (232448 - kFixed) / kWPairSmem;
  static constexpr int kNWP = kNWPfit > 8 ? 8 : kNWPfit;
  static constexpr int kSmemBytes = kFixed + kNWP * kWPairSmem;
  static_assert(kSlots >= 8 && kSlots <= kMaxSlots && kSlots % 4 == 0 && kAccCols + kSlots * 32 <= 512, "TMEM ring depth");
  static_assert(kGB > 1 || (kNI == 1 && kNBG <= kSlots), "single-k-block groups reuse the cons barriers");
  static_assert(kGB != 2 || 2 * kNBG <= kSlots, "two-k-block groups reuse the cons barriers");
  static_assert(kNI == 1 || kNBG % 2 == 0, "two issuers need an even activation ring");
  static_assert(kNWP >= 1, "weight ring depth");
  static_assert(kWStageMax % 128 == 0, "stage keeps 128 B alignment");
  static_assert(kSmemBytes <= 232448, "over the 227 KiB shared-memory limit");
};

struct SharedCtl {
  uint64_t full_w[8];
  uint64_t empty_w[8];
  uint64_t full_b[8];
  uint64_t empty_b[8];
  uint64_t a_full[kMaxSlots];
  uint64_t cons[kMaxSlots];
  uint64_t acc_full;
  uint64_t acc_empty;
  uint64_t turn[2];   // the two issuers hand the shared accumulator back and forth
  uint32_t tmem_base;
  int abort_flag;
  int others_done[2];   // epilogue: the other CTA's sums of this segment's cut tile are already published
};
static_assert(sizeof(SharedCtl) <= 1024, "control block must fit its slot");

// One contiguous run of weight stages inside one tile.
struct Segment {
  int n_tile, st_begin, st_end;
  int row0;      // first row of A / C of the tile
  int row_end;   // one past the last valid row (M, or the end of the tile's group)
  size_t wp_off; // byte offset of the tile's packed image (group) inside wp
  int slot;      // -1: the segment is a whole tile and stores to C; else scratch slot index
  long long tile;  // index of the tile in the (tile, stage) space
};

// Tile index -> rows, weight tile and image. Dense: tiles are ordered n-fastest so
// the CTAs working at the same time share a few token slabs (which stay in L2) and
// stream different weight tiles. Grouped: the same inside each group, groups in order.
__device__ __forceinline__ void locate_tile(const GemmParams& p, long long tile, Segment& s) {
  if (p.num_groups > 0) {
    int lo = 0, hi = p.num_groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.grp_tile_prefix[mid] <= tile) lo = mid; else hi = mid;
    }
    const int local = static_cast<int>(tile - p.grp_tile_prefix[lo]);
    s.n_tile = local % p.n_tiles;
    s.row0 = p.grp_row_prefix[lo] + (local / p.n_tiles) * p.tn;
    s.row_end = p.grp_row_prefix[lo + 1];
    s.wp_off = static_cast<size_t>(lo) * static_cast<size_t>(p.grp_w_stride);
  } else {
    s.n_tile = static_cast<int>(tile % p.n_tiles);
    s.row0 = static_cast<int>(tile / p.n_tiles) * p.tn;
    s.row_end = p.M;
    s.wp_off = 0;
  }
}

// Units (tile, stage pairs) of the problem and units per CTA: the host's plan, or, when the
// group sizes are known only on the device, an even cut of the tile total found there.
__device__ __forceinline__ void plan_of(const GemmParams& p, long long& units, long long& span) {
  if (p.dyn_grid > 0) {
    units = static_cast<long long>(p.grp_tile_prefix[p.num_groups]) * p.st_units;
    span = (units + p.dyn_grid - 1) / p.dyn_grid;
    if (p.dyn_whole) span = (span + p.st_units - 1) / p.st_units * p.st_units;
  } else {
    units = p.units;
    span = p.span;
  }
}

// Registers one more published partial tile of a cut tile; true for the CTA that brings the last of
// `expected`. The counter word carries the launch's epoch, a stale word counts as zero.
__device__ __forceinline__ bool tile_arrive(unsigned long long* ctr, unsigned long long epoch, int expected) {
  unsigned long long old = *reinterpret_cast<volatile unsigned long long*>(ctr);
  while (true) {
    const unsigned long long want = ((old >> 8) == epoch) ? old + 1ull : ((epoch << 8) | 1ull);
    const unsigned long long prev = atomicCAS(ctr, old, want);
    if (prev == old) return static_cast<int>(want & 0xffull) == expected;
    old = prev;
  }
}

// The CTAs that share a tile: the first one and how many.
__device__ __forceinline__ void cut_plan(const GemmParams& p, long long tile, int& c_first, int& nc, long long& span) {
  long long units;
  plan_of(p, units, span);
  const long long t_begin = tile * p.st_units;
  c_first = static_cast<int>(t_begin / span);
  nc = static_cast<int>((t_begin + p.st_units - 1) / span) - c_first + 1;
}

// Walks the segments of this CTA's span; every warp role runs the same walk.
struct SegmentWalk {
  long long pos, end;
  bool first;
  __device__ __forceinline__ SegmentWalk(const GemmParams& p) {
    long long units, span;
    plan_of(p, units, span);
    pos = static_cast<long long>(blockIdx.x) * span;
    end = pos + span;
    if (end > units) end = units;
    first = true;
  }
  __device__ __forceinline__ bool next(const GemmParams& p, Segment& s) {
    if (pos >= end) return false;
    const long long tile = pos / p.st_units;
    s.st_begin = static_cast<int>(pos - tile * p.st_units);
    const long long left = end - pos;
    s.st_end = static_cast<int>(min(static_cast<long long>(p.st_units), s.st_begin + left));
    locate_tile(p, tile, s);
    s.tile = tile;
    const bool whole = (s.st_begin == 0 && s.st_end == p.st_units);
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

// One output element to the local output and to every peer copy.
template <typename OutT>
__device__ __forceinline__ void store_everywhere(const GemmParams& p, size_t idx, OutT v) {
  reinterpret_cast<OutT*>(p.c)[idx] = v;
  for (int d = 0; d < p.n_peers; ++d) reinterpret_cast<OutT*>(p.c_peer[d])[idx] = v;
}

// Slow path: direct, predicated global stores (unaligned pitch or transposed output).
template <typename OutT, bool kIntAcc, int NV>
__device__ __forceinline__ void store_values_direct(const GemmParams& p, const uint32_t* acc, int m0, int m_end, int n) {
  OutT* c = reinterpret_cast<OutT*>(p.c);
  const bool trans = (p.flags & GF_TRANS_C) != 0;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int m = m0 + j;
    if (m < m_end) {
      const size_t idx = trans ? static_cast<size_t>(n) * p.ldc + m : static_cast<size_t>(m) * p.ldc + n;
      const OutT v = finish_value<OutT, kIntAcc>(p, acc[j], m, n);
      c[idx] = v;
      for (int d = 0; d < p.n_peers; ++d) reinterpret_cast<OutT*>(p.c_peer[d])[idx] = v;
    }
  }
}

// Fast path: the warp's 32 (n) x NV (m) block is transposed through shared
// memory ([m][n], one warp-private buffer) and leaves as 16-byte stores, each
// covering 8 (or 4) consecutive n of one output row. Needs a 16-byte aligned
// base and row pitch; rows beyond M and 16-byte groups beyond N are skipped.
template <typename OutT, bool kIntAcc, int NV>
__device__ __forceinline__ void store_values_vec(const GemmParams& p, const uint32_t* acc, int m0, int m_end, int n,
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
        if (n_ok && m < m_end) s[j * 32 + lane] = finish_value<OutT, kIntAcc>(p, acc[pass * RPP + j], m, n);
      }
    }
    __syncwarp();
    const int vcol = lane % VPR;                       // which 16-byte group of the row
    const int ncol = n0_warp + vcol * (16 / ES);
#pragma unroll
    for (int it = 0; it < RPP / RPI; ++it) {
      const int r = it * RPI + lane / VPR;
      const int m = m0 + pass * RPP + r;
      if (m < m_end && ncol < p.N) {
        const uint4 v = *reinterpret_cast<const uint4*>(sbuf + r * 32 * ES + vcol * 16);
        const size_t off = static_cast<size_t>(m) * p.ldc + ncol;
        *reinterpret_cast<uint4*>(c + off) = v;
        for (int d = 0; d < p.n_peers; ++d) *reinterpret_cast<uint4*>(reinterpret_cast<OutT*>(p.c_peer[d]) + off) = v;
      }
    }
  }
}

template <int TN, int WF, int ACT>
__global__ void __launch_bounds__(kThreads, 1)
umma_dequant_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const GemmParams p) {
  using Ring = RingConfig<TN, WF>;
  constexpr int NBG = Ring::kNBG;        // activation groups in the ring
  constexpr int GB = Ring::kGB;          // k-blocks per activation group (compile-time maximum)
  constexpr int NWP = Ring::kNWP;        // weight-stage pairs in the ring
  constexpr int WPS = Ring::kWPairSmem;
  constexpr int CPK = codes_per_kblock_bytes(WF);   // code bytes per k-block
  constexpr int NI = Ring::kNI;
  constexpr int NS = Ring::kSlots;       // dequantised TMEM ring slots
  constexpr int kAccCols = Ring::kAccCols;
  constexpr bool kInt = (ACT == ACT_I8);
  constexpr bool kBf16 = (ACT == ACT_BF16);
  constexpr int BKE = kInt ? 128 : 64;   // K elements per k-block
  constexpr int NV = TN >= 32 ? 32 : 16; // accumulator columns per tcgen05.ld

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_b = smem;                                   // NBG x (GB x TN x 128 B), 1024-aligned slabs
  uint8_t* smem_w = smem_b + NBG * Ring::kBGroupBytes;      // NWP x pair of stages
  uint8_t* smem_o = smem_w + NWP * WPS;                     // epilogue staging, 4 KiB per warp
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem_o + Ring::kStaging);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &ctl->abort_flag;
  DeviceStatus* st = p.status;
  // k-blocks per activation group at run time: GB, or 1 when K is not a whole number
  // of k-blocks per row (then only the 2-D tensor map is valid)
  const int gsz = p.b_group;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NWP; ++i) { mbar_init(&ctl->full_w[i], 1); mbar_init(&ctl->empty_w[i], 8); }
    for (int i = 0; i < NBG; ++i) { mbar_init(&ctl->full_b[i], 1); mbar_init(&ctl->empty_b[i], gsz == 4 ? 2 : 1); }
    for (int i = 0; i < NS; ++i) mbar_init(&ctl->a_full[i], 4);
    for (int i = 0; i < NS / 2; ++i) mbar_init(&ctl->cons[i], 1);
    mbar_init(&ctl->acc_full, NI);
    mbar_init(&ctl->acc_empty, 4);
    mbar_init(&ctl->turn[0], 1);
    mbar_init(&ctl->turn[1], 1);
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  if (warp == 3 && lane == 0) tma_prefetch_desc(&tmap_a);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ---------------- weight producer: one bulk copy per pair of packed stages ----
    if (lane == 0) {
      uint32_t wc = 0;   // pairs issued
      SegmentWalk walk(p);
      Segment w;
      while (walk.next(p, w)) {
        for (int sti = w.st_begin; sti < w.st_end; sti += 2, ++wc) {
          const int n = min(2, w.st_end - sti);
          const uint32_t s = wc % NWP;
          mbar_wait(&ctl->empty_w[s], ((wc / NWP) & 1) ^ 1, abort_flag, st, 1);
          const uint32_t bytes = static_cast<uint32_t>(n) * p.stage_bytes;
          mbar_arrive_expect_tx(&ctl->full_w[s], bytes);
          const uint8_t* tile_w = p.wp + w.wp_off + static_cast<size_t>(w.n_tile) * p.st_total * p.stage_bytes;
          if (sti + n <= p.st_total) {
            tma_bulk_g2s(smem_w + s * WPS, tile_w + static_cast<size_t>(sti) * p.stage_bytes, bytes, &ctl->full_w[s]);
          } else {
            // the pair reaches the extra stage past the tile's end: the last real stage stands in for it
            for (int j = 0; j < n; ++j) {
              const int real = min(sti + j, p.st_total - 1);
              tma_bulk_g2s(smem_w + s * WPS + j * p.stage_bytes, tile_w + static_cast<size_t>(real) * p.stage_bytes,
                           static_cast<uint32_t>(p.stage_bytes), &ctl->full_w[s]);
            }
          }
        }
      }
    }
  } else if (warp == 3) {
    // ---------------- activation producer: one TMA per group of k-blocks ----
    if (lane == 0) {
      uint32_t gc = 0;   // groups issued
      SegmentWalk walk(p);
      Segment w;
      while (walk.next(p, w)) {
        const int kb_end = w.st_end * 2;
        for (int kb = w.st_begin * 2; kb < kb_end; kb += gsz, ++gc) {
          const uint32_t s = gc % NBG;
          if (GB == 1 || (GB == 2 && gsz == 2)) {
            // groups that lie inside one stage (one or two k-blocks): the MMA's `cons`
            // commit of the stage that used this slot before also frees the slot (no second
            // commit); prev_kb = first k-block of that group in CTA-wide counting
            if (gc >= static_cast<uint32_t>(NBG)) {
              const uint32_t prev_kb = (gc - NBG) * static_cast<uint32_t>(GB);
              mbar_wait(&ctl->cons[(prev_kb % NS) >> 1], (prev_kb / NS) & 1, abort_flag, st, 2);
            }
          } else {
            mbar_wait(&ctl->empty_b[s], ((gc / NBG) & 1) ^ 1, abort_flag, st, 2);
          }
          mbar_arrive_expect_tx(&ctl->full_b[s], static_cast<uint32_t>(gsz) * Ring::kBSlabBytes);
          if (GB == 1 || gsz == 1)
            tma_load_2d(smem_b + s * Ring::kBGroupBytes, &tmap_a, kb * BKE, w.row0, &ctl->full_b[s]);
          else
            tma_load_3d(smem_b + s * Ring::kBGroupBytes, &tmap_a, 0, w.row0, kb, &ctl->full_b[s]);
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ---------------- MMA issuers ----------------
    // Both issuers feed the one accumulator and take alternate *stages* (two k-blocks,
    // eight MMAs). While one issues, the other is already through the waits, the commits
    // and the loop round trip of its next stage; a single thread cannot fit those under the
    // few MMAs the tensor pipe queues (measured: 1085 -> 1381 TFLOP/s at 4096 tokens).
    // `turn` orders the two threads' MMAs: the issuer of stage g arrives on the other's
    // barrier after its last MMA (fence before the arrive, fence after the wait).
    const int me = warp - 1;
    if (lane == 0) {
      constexpr uint32_t idesc =
          kInt ? make_idesc(2u, 1u, 1u, 128u, TN) : make_idesc(1u, kBf16 ? 1u : 0u, kBf16 ? 1u : 0u, 128u, TN);
      const uint32_t acc_tmem = tmem_base + (NI == 2 ? static_cast<uint32_t>(me) * TN : 0u);
      const uint32_t b_base = smem_u32(smem_b);
      uint32_t g0 = 0;        // stages of this CTA before the current segment (both issuers count all)
      uint32_t gc0 = 0;       // activation groups issued before this segment
      uint32_t tc = 0;        // segments seen
      uint32_t my_turns = 0;  // waits done on turn[me]
      // ring position of my next stage's first k-block (k-block 2 * stage): +4 per own stage
      uint32_t sa = (2u * static_cast<uint32_t>(me)) % NS, pa = 0;
      const uint32_t gshift = gsz == 4 ? 2u : (gsz == 2 ? 1u : 0u);   // gsz is 1, 2 or 4
      const uint32_t gmask = static_cast<uint32_t>(gsz) - 1u;
      bool ok = true;
      SegmentWalk walk(p);
      Segment w;
      while (walk.next(p, w)) {
        const int nst = w.st_end - w.st_begin;
        // my stages of the segment: those whose CTA-wide index g0 + i has my parity
        for (int i = static_cast<int>((static_cast<uint32_t>(me) ^ g0) & 1u); i < nst; i += 2) {
          const bool first_ever = (g0 + static_cast<uint32_t>(i)) == 0u;
          // activation groups of the stage's two k-blocks (segment-relative k-blocks 2i, 2i + 1)
          const uint32_t grp0 = gc0 + (static_cast<uint32_t>(2 * i) >> gshift);
          const uint32_t grp1 = gc0 + (static_cast<uint32_t>(2 * i + 1) >> gshift);
          const uint32_t sb0 = grp0 % NBG, sb1 = grp1 % NBG;
          ok &= mbar_wait(&ctl->a_full[sa], pa, abort_flag, st, 4);
          ok &= mbar_wait(&ctl->full_b[sb0], (grp0 / NBG) & 1u, abort_flag, st, 5);
          if (grp1 != grp0) ok &= mbar_wait(&ctl->full_b[sb1], (grp1 / NBG) & 1u, abort_flag, st, 5);
          // `turn` before `acc_empty`: with one-stage tiles an issuer looks at acc_empty only every other
          // phase, and only the other issuer's hand-over tells it that the phase in between is complete
          if (NI == 1 && !first_ever) {
            ok &= mbar_wait(&ctl->turn[me], my_turns & 1u, abort_flag, st, 9);
            ++my_turns;
          }
          if (i < NI) ok &= mbar_wait(&ctl->acc_empty, (tc & 1u) ^ 1u, abort_flag, st, 3);   // my first stage here
          tc_fence_after_sync();
          if (ok) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t a_tmem = tmem_base + kAccCols + (sa + h) * 32;
              const uint32_t slab = static_cast<uint32_t>(2 * i + h) & gmask;
              const uint64_t b_desc = make_smem_desc_sw128(b_base + (h == 0 ? sb0 : sb1) * Ring::kBGroupBytes +
                                                           slab * Ring::kBSlabBytes);
#pragma unroll
              for (int m = 0; m < 4; ++m) {
                const uint32_t accum = (i < NI && h == 0 && m == 0) ? 0u : 1u;   // first MMA into this accumulator
                if constexpr (kInt) umma_ts_i8(acc_tmem, a_tmem + 8 * m, b_desc + 2 * m, idesc, accum);
                else umma_ts_f16(acc_tmem, a_tmem + 8 * m, b_desc + 2 * m, idesc, accum);
              }
            }
          }
          if constexpr (NI == 1) {
            tc_fence_before_sync();
            mbar_arrive(&ctl->turn[me ^ 1]);
          }
          tc_commit(&ctl->cons[sa >> 1]);
          if (GB > 1 && !(GB == 2 && gsz == 2)) {
            // hand the activation groups back (two-k-block groups ride on `cons`): a group of four k-blocks serves two stages and
            // takes one arrival from each (or both from this one when the segment ends here)
            tc_commit(&ctl->empty_b[sb0]);
            if (grp1 != grp0) tc_commit(&ctl->empty_b[sb1]);
            if (gsz == 4 && (i & 1) == 0 && i == nst - 1) mbar_arrive(&ctl->empty_b[sb0]);
          }
          if (NI == 1 ? (i == nst - 1) : (i + 2 >= nst)) tc_commit(&ctl->acc_full);   // my last stage here
          sa += 4; if (sa >= static_cast<uint32_t>(NS)) { sa -= NS; pa ^= 1u; }
        }
        // a one-stage segment leaves the other issuer without work: it still owes its arrival
        // (after the epilogue has drained the previous segment, so it cannot run ahead and put
        // two arrivals into one phase)
        if (NI == 2 && nst == 1 && ((static_cast<uint32_t>(me) ^ g0) & 1u) != 0u) {
          ok &= mbar_wait(&ctl->acc_empty, (tc & 1u) ^ 1u, abort_flag, st, 3);
          mbar_arrive(&ctl->acc_full);
        }
        g0 += static_cast<uint32_t>(nst);
        gc0 += (static_cast<uint32_t>(2 * nst) + gmask) >> gshift;
        ++tc;
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ---------------- dequant warpgroups: one stage of every pair each ----
    // Group dg takes the stages whose CTA-wide index has parity dg, i.e. always the stages of
    // issuer dg, whose `cons` barriers it therefore sees in every phase. (Taking "stage dg of
    // the pair" instead swaps the groups between the issuers after every segment with an odd
    // number of stages; a group then meets a `cons` barrier it last saw two phases ago, and
    // if its new issuer is a stage behind, the parity test answers "complete" for the phase
    // before the one it means: the group overwrites operands the MMA has not read.)
    const int dg = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t wc = 0;   // weight pairs seen by this CTA
    uint32_t kc0 = 0;  // global index of the first k-block of the current pair
    uint32_t g0_d = 0; // stages of this CTA before the current segment
    bool ok = true;
    SegmentWalk walk(p);
    Segment w;
    while (walk.next(p, w)) {
      const int d = dg ^ static_cast<int>(g0_d & 1u);   // my place in this segment's pairs
      g0_d += static_cast<uint32_t>(w.st_end - w.st_begin);
      for (int sti = w.st_begin; sti < w.st_end; sti += 2, ++wc) {
        const int n = min(2, w.st_end - sti);
        const uint32_t sw = wc % NWP;
        ok &= mbar_wait(&ctl->full_w[sw], (wc / NWP) & 1, abort_flag, st, 6);
        const bool mine = d < n;
        const uint8_t* stage = smem_w + sw * WPS + d * p.stage_bytes;
        constexpr int CH = CPK / 2048;            // 16-byte chunks per row and k-block
        constexpr int RPC = 32 / CH;              // TMEM columns produced by one chunk
        if (mine) {
          uint32_t sz0 = 0, sz1 = 0;
          if constexpr (WF == WF_U4_SZ || WF == WF_U2_SZ || WF == WF_LUT4_S) {
            const uint32_t* szp = reinterpret_cast<const uint32_t*>(stage + Ring::kCodeBytes);
            sz0 = szp[row_in_tile];
            sz1 = p.sz_per_kb ? szp[128 + row_in_tile] : sz0;
          } else if constexpr (WF == WF_FP4_E8M0) {
            sz0 = reinterpret_cast<const uint32_t*>(stage + Ring::kCodeBytes)[row_in_tile];
          }
          const uint4* codes = reinterpret_cast<const uint4*>(stage);
#pragma unroll
          for (int it = 0; it < 2 * CH; ++it) {
            const int h = it / CH, q = it % CH;
            const uint32_t kc = kc0 + d * 2 + h;
            const uint32_t sa = kc % NS;
            const uint4 cq = codes[it * 128 + (row_in_tile ^ chunk_swizzle(it))];
            if (it == 2 * CH - 1) {
              // every thread of this warp has issued its last read of the stage
              __syncwarp();
              if (lane == 0) mbar_arrive(&ctl->empty_w[sw]);
            }
            uint32_t regs[RPC];
            if constexpr (WF == WF_I4_I8) {
              decode_i4_chunk(cq, p.code_bias, regs);
            } else if constexpr (WF == WF_U2_SZ) {
              decode_u2_chunk<kBf16>(cq, h == 0 ? sz0 : sz1, regs);
            } else if constexpr (WF == WF_LUT4_S) {
              decode_lut4_chunk<kBf16>(cq, h == 0 ? sz0 : sz1, p.lut_lo, p.lut_hi, regs);
            } else if constexpr (WF == WF_U4_SZ) {
              decode_u4_chunk<kBf16>(cq, h == 0 ? sz0 : sz1, regs);
            } else if constexpr (WF == WF_U4_RAW) {
              decode_u4_chunk_noscale<kBf16, false>(cq, regs);
            } else if constexpr (WF == WF_S4_RAW) {
              decode_u4_chunk_noscale<kBf16, true>(cq, regs);
            } else if constexpr (WF == WF_FP4_E8M0) {
              decode_fp4_chunk<kBf16>(cq, 126 + static_cast<int>((sz0 >> (8 * it)) & 0xff) - p.fp4_exp_bias,
                                      (p.flags & GF_FP4_SIMPLE) != 0, regs);
            } else {
              decode_i2_chunk(cq, p.code_bias, regs);
            }
            if (q == 0) {
              if (h == 0 && kc >= static_cast<uint32_t>(NS)) {
                const uint32_t prev = kc - NS;   // first k-block of the stage that used these two slots
                ok &= mbar_wait(&ctl->cons[sa >> 1], (prev / NS) & 1, abort_flag, st, 7);
              }
              tc_fence_after_sync();
            }
            const uint32_t dst = tmem_base + lane_addr + kAccCols + sa * 32 + q * RPC;
            if constexpr (RPC == 32) tmem_st_32x32b_x32(dst, regs);
            else if constexpr (RPC == 16) tmem_st_32x32b_x16(dst, regs);
            else tmem_st_32x32b_x8(dst, regs);
            if (it == 2 * CH - 1) {
              // both k-blocks of the stage are stored: one hand-off per stage, on the
              // barrier of the stage's first slot
              tc_wait_st();
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&ctl->a_full[sa - 1]);
            }
          }
        } else {
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->empty_w[sw]);
        }
        kc0 += 2 * n;
      }
    }
    (void)ok;
  } else if (warp >= 12) {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    uint8_t* my_stage = smem_o + quarter * kStagingBytesPerWarp;
    const bool use_vec = (p.flags & GF_VEC_STORE) != 0;
    const bool plain = (p.flags & (GF_HAS_BIAS | GF_ROW_SCALE)) == 0;
    uint32_t tc = 0;
    uint32_t g0_e = 0;   // stages of this CTA before the current segment
    bool ok = true;
    SegmentWalk walk(p);
    Segment w;
    while (walk.next(p, w)) {
      const int n0_warp = w.n_tile * kTileRows + quarter * 32;
      const int n = n0_warp + lane;
      const int nkb = (w.st_end - w.st_begin) * 2;
      // accumulators that hold anything: both, unless the segment is a single stage
      const int nst_e = w.st_end - w.st_begin;
      const uint32_t valid = (NI == 2 && nst_e == 1) ? (1u << (g0_e & 1u)) : ((1u << NI) - 1u);
      g0_e += static_cast<uint32_t>(nst_e);
      (void)nkb;
      ok &= mbar_wait(&ctl->acc_full, tc & 1, abort_flag, st, 8);
      tc_fence_after_sync();
      // A tile cut between two CTAs: the one that holds its first stages works on them at the end
      // of its span, the other at the start of its own, so the other's partial tile is almost
      // always published by now. Then this CTA adds it to its accumulator on the way out and
      // stores the finished outputs (the fix-up pass skips the tile); otherwise it publishes its
      // own partial tile as every contributor does, and the fix-up pass adds them.
      // (Only at the 256-token tile: with two accumulators per tile the extra registers spill and
      // the narrow tiles' short epilogues do not hide the L2 reads -- measured slower there.)
      constexpr bool kFinishInKernel = (TN == 256);
      const bool cut = w.slot >= 0;
      bool finish_here = false;
      const uint32_t* other = nullptr;
      int nc_e = 1;
      if (kFinishInKernel && cut && p.tile_ctr != nullptr) {
        int c_first;
        long long span;
        cut_plan(p, w.tile, c_first, nc_e, span);
        if (warp == 12 && lane == 0) {
          bool done = false;
          if (static_cast<int>(blockIdx.x) == c_first && nc_e == 2) {
            const unsigned long long seen = *reinterpret_cast<volatile unsigned long long*>(p.tile_ctr + w.tile);
            done = seen == ((p.epoch << 8) | 1ull);
            if (done) __threadfence();
          }
          ctl->others_done[tc & 1] = done ? 1 : 0;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");     // the four epilogue warps
        finish_here = ctl->others_done[tc & 1] != 0;
        if (finish_here) {
          // the other contributor is CTA c_first + 1, and the tile holds the first segment of its span
          other = p.partial + static_cast<size_t>((c_first + 1) * 2) * TN * kTileRows + row_in_tile;
        }
      }
      auto store_chunk = [&](const uint32_t (&acc)[NV], int c) {
        const int m0 = w.row0 + c * NV;
        if (cut && !finish_here) {
          // partial tile: raw accumulator values, [token][row] so lanes coalesce
          uint32_t* dst = p.partial + (static_cast<size_t>(w.slot) * TN + c * NV) * kTileRows + row_in_tile;
#pragma unroll
          for (int j = 0; j < NV; ++j) dst[j * kTileRows] = acc[j];
        } else if (use_vec) {
          if (m0 < w.row_end && n0_warp < p.N) {
            switch (p.out_type) {
              case OUT_F16: store_values_vec<__half, kInt, NV>(p, acc, m0, w.row_end, n, n0_warp, my_stage, lane, plain); break;
              case OUT_BF16: store_values_vec<__nv_bfloat16, kInt, NV>(p, acc, m0, w.row_end, n, n0_warp, my_stage, lane, plain); break;
              case OUT_F32: store_values_vec<float, kInt, NV>(p, acc, m0, w.row_end, n, n0_warp, my_stage, lane, plain); break;
              default: store_values_vec<int, kInt, NV>(p, acc, m0, w.row_end, n, n0_warp, my_stage, lane, plain); break;
            }
          }
        } else if (n < p.N) {
          switch (p.out_type) {
            case OUT_F16: store_values_direct<__half, kInt, NV>(p, acc, m0, w.row_end, n); break;
            case OUT_BF16: store_values_direct<__nv_bfloat16, kInt, NV>(p, acc, m0, w.row_end, n); break;
            case OUT_F32: store_values_direct<float, kInt, NV>(p, acc, m0, w.row_end, n); break;
            default: store_values_direct<int, kInt, NV>(p, acc, m0, w.row_end, n); break;
          }
        }
      };
      // The accumulator goes back to the issuers as soon as its last columns are in
      // registers, before they are stored.
      auto release_acc = [&]() {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->acc_empty);
      };
      if (kFinishInKernel && finish_here) {
        // own sums from tensor memory plus the other CTA's from L2 (requested one chunk ahead),
        // added in ascending CTA order like the fix-up pass: own first
        uint32_t oth[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) oth[j] = __ldcg(other + static_cast<size_t>(j) * kTileRows);
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
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            if constexpr (kInt) acc[j] = static_cast<uint32_t>(static_cast<int>(acc[j]) + static_cast<int>(oth[j]));
            else acc[j] = __float_as_uint((0.f + __uint_as_float(acc[j])) + __uint_as_float(oth[j]));
          }
          if (c + 1 < TN / NV) {
#pragma unroll
            for (int j = 0; j < NV; ++j)
              oth[j] = __ldcg(other + (static_cast<size_t>(c + 1) * NV + j) * kTileRows);
          } else {
            release_acc();
          }
          store_chunk(acc, c);
        }
      } else if constexpr (NI == 1 && NV == 32 && (TN / NV) % 2 == 0) {
        // one accumulator, an even number of 32-column chunks: the load of the next chunk
        // flies under the stores of the current one (two register buffers, loop unrolled by 2)
        uint32_t buf_a[NV], buf_b[NV];
        tmem_ld_32x32b_x32(tmem_base + lane_addr, buf_a);
#pragma unroll 1
        for (int c = 0; c < TN / NV; c += 2) {
          tc_wait_ld();
          tmem_ld_32x32b_x32(tmem_base + lane_addr + (c + 1) * NV, buf_b);
          store_chunk(buf_a, c);
          tc_wait_ld();
          if (c + 2 < TN / NV) tmem_ld_32x32b_x32(tmem_base + lane_addr + (c + 2) * NV, buf_a);
          else release_acc();
          store_chunk(buf_b, c + 1);
        }
      } else {
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
          if (c == TN / NV - 1) release_acc();
          store_chunk(acc, c);
        }
      }
      if (kFinishInKernel && cut && !finish_here && p.tile_ctr != nullptr) {
        // this CTA's partial tile is stored: make it visible device-wide and count it (nobody waits)
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (warp == 12 && lane == 0) {
          __threadfence();
          tile_arrive(p.tile_ctr + w.tile, p.epoch, nc_e);
        }
      }
      ++tc;
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
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// Second pass of stream-K: every tile that was cut between CTAs gets its partial
// tiles added in ascending CTA order. blockIdx.x names the boundary between CTA b
// and CTA b+1; the first boundary that falls strictly inside a tile owns that tile,
// the others return at once, so only split tiles cost anything. blockIdx.y picks a
// few tokens (so the loads of a thread are independent and the pass is not a chain of
// L2 latencies); one thread per weight row. Integer partials are added as integers (exact).
__host__ __device__ constexpr int fixup_tokens_per_block(int tn) { return tn >= 64 ? 8 : (tn >= 32 ? 4 : 2); }

template <typename OutT, int TN, bool kIntAcc>
__global__ void __launch_bounds__(kTileRows)
streamk_fixup_kernel(const GemmParams p) {
  constexpr int TCH = fixup_tokens_per_block(TN);
  long long units, span;
  plan_of(p, units, span);
  if (span == 0 || span % p.st_units == 0) return;          // no tile is cut
  const long long pos = static_cast<long long>(blockIdx.x + 1) * span;
  if (pos >= units) return;
  const long long tile = pos / p.st_units;
  const long long t_begin = tile * p.st_units;
  const long long t_end = t_begin + p.st_units;
  if (pos == t_begin) return;                               // the cut is a tile boundary
  const int c_first = static_cast<int>(t_begin / span);
  if (static_cast<int>(blockIdx.x) != c_first) return;      // an earlier cut owns this tile
  const int c_last = static_cast<int>((t_end - 1) / span);
  if (TN == 256 && p.tile_ctr != nullptr && c_last - c_first == 1) {
    // one arrival out of two: the CTA holding the tile's first stages added the other's partial
    // tile itself and stored the outputs
    const unsigned long long seen = p.tile_ctr[tile];
    if (seen == ((p.epoch << 8) | 1ull)) return;
  }
  Segment seg;
  locate_tile(p, tile, seg);
  const int row = threadIdx.x;
  const int n = seg.n_tile * kTileRows + row;
  const int j0 = blockIdx.y * TCH;
  if (n >= p.N || seg.row0 + j0 >= seg.row_end) return;
  float facc[TCH];
  int iacc[TCH];
#pragma unroll
  for (int jj = 0; jj < TCH; ++jj) { facc[jj] = 0.f; iacc[jj] = 0; }
  for (int cta = c_first; cta <= c_last; ++cta) {
    // slot 0 if this tile holds the first segment of that CTA's span, else slot 1
    const long long span_begin = static_cast<long long>(cta) * span;
    const int slot = cta * 2 + ((span_begin >= t_begin) ? 0 : 1);
    const uint32_t* src = p.partial + (static_cast<size_t>(slot) * TN + j0) * kTileRows + row;
    uint32_t raw[TCH];
#pragma unroll
    for (int jj = 0; jj < TCH; ++jj) raw[jj] = src[jj * kTileRows];
#pragma unroll
    for (int jj = 0; jj < TCH; ++jj) {
      if constexpr (kIntAcc) iacc[jj] += static_cast<int>(raw[jj]);
      else facc[jj] += __uint_as_float(raw[jj]);
    }
  }
  OutT* c = reinterpret_cast<OutT*>(p.c);
  const bool trans = (p.flags & GF_TRANS_C) != 0;
#pragma unroll
  for (int jj = 0; jj < TCH; ++jj) {
    const int m = seg.row0 + j0 + jj;
    if (m < seg.row_end) {
      uint32_t bits;
      if constexpr (kIntAcc) bits = static_cast<uint32_t>(iacc[jj]);
      else bits = __float_as_uint(facc[jj]);
      const size_t idx = trans ? static_cast<size_t>(n) * p.ldc + m : static_cast<size_t>(m) * p.ldc + n;
      const OutT v = finish_value<OutT, kIntAcc>(p, bits, m, n);
      c[idx] = v;
      for (int d = 0; d < p.n_peers; ++d) reinterpret_cast<OutT*>(p.c_peer[d])[idx] = v;
    }
  }
}

}  // namespace b200dq
