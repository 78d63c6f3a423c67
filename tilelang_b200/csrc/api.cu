// C ABI of the library (declared in include/b200dq.h): argument validation,
// tensor-map encoding, stream-K schedule and kernel launch.
//
// Plays the role of the reference's generated host stub + runtime helpers:
// argument checks (docs/compiler_internals/tensor_checks.md:19-60), tensor-map
// creation with validation (src/cuda/runtime.cc:385-560) and the
// init/call/get_last_error convention (tilelang/jit/adapter/wrapper.py:60-86).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <algorithm>
#include <atomic>
#include <mutex>

#include "../../include/b200dq.h"
#include "elementwise.cuh"
#include "pack_kernels.cuh"
#include "umma_gemm.cuh"
#include "skinny_launch.h"
#include "umma_launch.h"
#include "mxf4_launch.h"
#include "peak_launch.h"
#include "int8_skinny_launch.h"

namespace {

using namespace b200dq;

constexpr int kMaxDevices = 32;
constexpr int kAbiVersion = 5;
constexpr int kMinSpan = 8;   // fewest k-blocks worth giving a CTA of its own

thread_local char g_err[1024] = "";

int fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return -1;
}

#define CUDA_OK(expr)                                                                   \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess) return fail("%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

struct DeviceState {
  std::atomic<bool> ready{false};   // set (release) after the fields below, under g_mu
  int sm_count = 0;
  DeviceStatus* status = nullptr;
};

std::mutex g_mu;
DeviceState g_dev[kMaxDevices];
EncodeTiledFn g_encode = nullptr;

// ---- state of b200dq_gemm_static_scratch ------------------------------------
// Scratch for callers that cannot allocate device memory: a fixed array that lives
// in the library's device image (every GPU that loads the library holds it until
// the process exits). 40 MiB covers the stream-K partial tiles of every schedule on
// a part with up to 148 SMs (148 CTAs x 2 slots x 256 tokens x 128 rows x 4 B =
// 38,797,312 B).
constexpr size_t kStaticScratchBytes = 40u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticScratchState {
  std::atomic<bool> ready{false};   // set (release) after the two fields below, under g_mu
  int sm_count = 0;
  void* scratch = nullptr;   // device address of g_static_scratch on this device
};
StaticScratchState g_static_dev[kMaxDevices];

int current_device_state(DeviceState** out) {
  int dev = 0;
  CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail("device index %d out of range", dev);
  if (!g_dev[dev].ready.load(std::memory_order_acquire)) {
    if (b200dq_init() != 0) return -1;
  }
  *out = &g_dev[dev];
  return 0;
}

int token_tile_for(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

struct Schedule {
  int tn, m_tiles, n_tiles, st_total, grid, span;
  int st_units;   // stages the schedule gives a tile: st_total, or one more (see make_schedule)
  bool whole_tiles;   // spans are whole tiles by construction (narrow tiles on tall problems)
  long long units;
  size_t workspace_bytes, slot_bytes;
  bool needs_scratch;   // some tile is cut between CTAs
};

int k_elems_per_kblock(int act_type) { return act_type == ACT_I8 ? 128 : 64; }

// weight stages (2 k-blocks each) that cover K
int stages_for(int K, int act_type) {
  const int per_stage = 2 * k_elems_per_kblock(act_type);
  return (K + per_stage - 1) / per_stage;
}

// scale words per row and stage
int nsz_for(int weight_format, int group_size) {
  if (weight_format == WF_U4_SZ || weight_format == WF_U2_SZ || weight_format == WF_LUT4_S) return group_size == 64 ? 2 : 1;
  if (weight_format == WF_FP4_E8M0) return 1;
  return 0;
}

int stage_bytes_for(int weight_format, int group_size) {
  return 2 * codes_per_kblock_bytes(weight_format) + 512 * nsz_for(weight_format, group_size);
}

int make_schedule(int M, int N, int K, int act_type, int token_tile, int max_ctas, int sm_count, Schedule* s,
                  long long grouped_tiles = -1, bool tile_kernel = true) {
  s->tn = token_tile > 0 ? token_tile : token_tile_for(M);
  if (s->tn != 16 && s->tn != 32 && s->tn != 64 && s->tn != 128 && s->tn != 256)
    return fail("token_tile must be 16, 32, 64, 128 or 256 (got %d)", s->tn);
  s->m_tiles = (M + s->tn - 1) / s->tn;
  s->n_tiles = (N + kTileRows - 1) / kTileRows;
  s->st_total = stages_for(K, act_type);
  const long long tiles = grouped_tiles >= 0 ? grouped_tiles : static_cast<long long>(s->m_tiles) * s->n_tiles;
  if (tiles <= 0) return fail("no tiles to compute");
  // Tiles of at most 128 tokens run two issuers and two dequant groups on alternate stages. When the
  // groups were still paired to the issuers by their place in a weight pair, a tile with an odd number
  // of stages swapped the pairing at every tile boundary, and a group could pass a parity wait one
  // phase early (with tens of such tiles per CTA a bounded wait gave up now and then). Those tiles get
  // one more stage: it re-reads the last real stage's weights against activations beyond K, which the
  // tensor map fills with zeros. The kernel has since been changed to keep group and issuer together
  // by CTA-wide stage parity; the even stage count stays (it also splits a tile's stages evenly).
  s->st_units = s->st_total + ((s->tn <= 128 && tile_kernel) ? (s->st_total & 1) : 0);
  s->units = tiles * s->st_units;
  int cap = sm_count;
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  long long g = s->units / kMinSpan;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  s->span = static_cast<int>((s->units + g - 1) / g);
  // Narrow tiles with plenty of tiles per SM: spans of eight whole tiles, in as many CTAs as that
  // takes (they run in waves). Whole tiles need no scratch and no fix-up pass, no segment has an odd
  // number of stages (see above), and the imbalance of whole-tile waves is about 1 % at this size.
  s->whole_tiles = s->tn <= 128 && tile_kernel && max_ctas <= 0 && tiles >= 16LL * cap;
  if (s->whole_tiles) s->span = 8 * s->st_units;
  s->grid = static_cast<int>((s->units + s->span - 1) / s->span);
  // two partial-tile slots per CTA, then one 64-bit arrival counter per tile (small-M kernel)
  s->slot_bytes = static_cast<size_t>(s->grid) * 2 * s->tn * kTileRows * sizeof(uint32_t);
  s->workspace_bytes = s->slot_bytes + static_cast<size_t>(tiles) * sizeof(unsigned long long);
  s->needs_scratch = (s->span % s->st_units != 0) && s->grid > 1;
  return 0;
}

// Encoded activation tensor maps of this thread's recent calls. Encoding costs a driver
// call of a microsecond or two, which matters next to a 20 us small-M kernel; a map depends
// only on the key below (the descriptor holds the address, not the data).
struct TensorMapKey {
  const void* a;
  int M, K, act_type, box_tokens, kind;   // kind: 0 = tcgen05 kernel (box_tokens x group), 1 = small-M kernel
  int group;
  bool operator==(const TensorMapKey& o) const {
    return a == o.a && M == o.M && K == o.K && act_type == o.act_type && box_tokens == o.box_tokens &&
           kind == o.kind && group == o.group;
  }
};
struct TensorMapEntry {
  TensorMapKey key;
  CUtensorMap map;
  int group_encoded;
  bool valid = false;
};
constexpr int kTensorMapCache = 16;
thread_local TensorMapEntry g_tmap_cache[kTensorMapCache];
thread_local int g_tmap_next = 0;

const TensorMapEntry* tensor_map_lookup(const TensorMapKey& key) {
  for (int i = 0; i < kTensorMapCache; ++i)
    if (g_tmap_cache[i].valid && g_tmap_cache[i].key == key) return &g_tmap_cache[i];
  return nullptr;
}

void tensor_map_remember(const TensorMapKey& key, const CUtensorMap& map, int group_encoded) {
  TensorMapEntry& e = g_tmap_cache[g_tmap_next];
  g_tmap_next = (g_tmap_next + 1) % kTensorMapCache;
  e.key = key;
  e.map = map;
  e.group_encoded = group_encoded;
  e.valid = true;
}

CUtensorMapDataType tensor_map_dtype(int act_type) {
  return act_type == ACT_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
         : act_type == ACT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

// Tensor map of the activations for the tcgen05 kernel. With `group` > 1 k-blocks per load
// the map is 3-D, {k-block element, token row, k-block index}, so one TMA lands `group`
// consecutive k-blocks as separate [row][128 B] slabs; that view needs K to be a whole
// number of k-blocks. Returns the group size actually encoded (1 = plain 2-D map) or -1.
int encode_activation_map(CUtensorMap* map, const void* a, int M, int K, int act_type, int tn, int group) {
  if (g_encode == nullptr) return fail("tensor-map encoder not resolved (b200dq_init not run?)");
  const int esize = (act_type == ACT_I8) ? 1 : 2;
  const int bke = k_elems_per_kblock(act_type);
  if ((reinterpret_cast<uintptr_t>(a) & 15) != 0) return fail("activation pointer must be 16-byte aligned");
  if ((static_cast<long long>(K) * esize) % 16 != 0) return fail("activation row pitch must be a multiple of 16 bytes");
  const TensorMapKey key{a, M, K, act_type, tn, 0, group};
  if (const TensorMapEntry* hit = tensor_map_lookup(key)) {
    *map = hit->map;
    return hit->group_encoded;
  }
  const CUtensorMapDataType dt = tensor_map_dtype(act_type);
  if (group > 1 && K % bke == 0) {
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(bke), static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(K / bke)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(K) * esize, static_cast<cuuint64_t>(bke) * esize};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(bke), static_cast<cuuint32_t>(tn), static_cast<cuuint32_t>(group)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(map, dt, 3, const_cast<void*>(a), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
      tensor_map_remember(key, *map, group);
      return group;
    }
    // fall through to the 2-D map
  }
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * esize};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(bke), static_cast<cuuint32_t>(tn)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, dt, 2, const_cast<void*>(a), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with CUresult %d (M=%d K=%d box=%dx%d)",
                                     static_cast<int>(r), M, K, bke, tn);
  tensor_map_remember(key, *map, 1);
  return 1;
}

// Tensor map of the activations for the small-M kernel: 16-bit elements viewed as
// {64 k, k-block parity, token, stage of 128 k}; one load brings the box
// {64, 2, box_tokens, 1} = one stage of every token, which the 128-byte swizzle lays out
// as [token][parity][128 B] with bank-conflict-free fragment reads
// (skinny_gemm.cuh). K must be a multiple of 128. Returns 0 or -1.
int encode_skinny_activation_map(CUtensorMap* map, const void* a, int M, int K, int act_type, int box_tokens) {
  if (g_encode == nullptr) return fail("tensor-map encoder not resolved (b200dq_init not run?)");
  if ((reinterpret_cast<uintptr_t>(a) & 15) != 0) return fail("activation pointer must be 16-byte aligned");
  if (K % 128 != 0) return fail("the small-M kernel needs K to be a multiple of 128 (got %d)", K);
  const TensorMapKey key{a, M, K, act_type, box_tokens, 1, 2};
  if (const TensorMapEntry* hit = tensor_map_lookup(key)) {
    *map = hit->map;
    return 0;
  }
  cuuint64_t dims[4] = {64, 2, static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(K / 128)};
  cuuint64_t strides[3] = {128, static_cast<cuuint64_t>(K) * 2, 256};
  cuuint32_t box[4] = {64, 2, static_cast<cuuint32_t>(box_tokens), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_encode(map, tensor_map_dtype(act_type), 4, const_cast<void*>(a), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail("cuTensorMapEncodeTiled (small-M view) failed with CUresult %d (M=%d K=%d)", static_cast<int>(r), M, K);
  tensor_map_remember(key, *map, 2);
  return 0;
}

int out_elem_size(int out_type) { return (out_type == OUT_F16 || out_type == OUT_BF16) ? 2 : 4; }

// The epilogue uses 16-byte stores when the output is (M, N) row-major with a
// 16-byte aligned base and pitch; otherwise it falls back to element stores.
bool output_takes_vector_stores(const void* c, int N, int out_type, int flags) {
  if (flags & GF_TRANS_C) return false;
  if ((reinterpret_cast<uintptr_t>(c) & 15) != 0) return false;
  return (static_cast<long long>(N) * out_elem_size(out_type)) % 16 == 0;
}

// The small-M kernel takes dense problems of at most 16 tokens with 4-bit weights on 16-bit
// activations and K a multiple of 128 when the caller leaves the token tile to the library
// (an explicit token_tile = 16 keeps the tcgen05 kernel).
bool takes_skinny_path(const b200dq_gemm_args* a) {
  if (a->num_groups > 0 || a->M > kSkinnyTokens || a->token_tile != 0) return false;
  if (a->act_type != ACT_F16 && a->act_type != ACT_BF16) return false;
  if (a->out_type == OUT_I32) return false;
  if (a->K % 128 != 0) return false;
  if (a->weight_format == WF_FP4_E8M0) return true;
  return a->weight_format == WF_U4_SZ || a->weight_format == WF_U4_RAW || a->weight_format == WF_S4_RAW;
}

// Integer codes on int8 activations with at most 32 tokens go to the decode-shape kernel
// (one launch, no scratch) under the same rule: dense, token tile left to the library.
bool takes_int8_skinny_path(const b200dq_gemm_args* a) {
  if (a->num_groups > 0 || a->M > 32 || a->token_tile != 0) return false;
  if (a->act_type != ACT_I8) return false;
  if (a->K % 16 != 0 || (reinterpret_cast<uintptr_t>(a->a) & 15) != 0) return false;
  return a->weight_format == WF_I2_I8 || a->weight_format == WF_I4_I8;
}

// SM count of the current device once b200dq_init has run on it, else an upper bound that
// needs no device (256 SMs), so that a size query never under-reports.
int sm_count_or_bound() {
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices &&
      g_dev[dev].ready.load(std::memory_order_acquire))
    return g_dev[dev].sm_count;
  return 256;
}

int resolve_encoder() {
  if (g_encode != nullptr) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  CUDA_OK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
  if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return fail("driver has no cuTensorMapEncodeTiled");
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return 0;
}

// Scratch bytes the schedule of a dense call needs on a part with `sm_count` SMs (what
// b200dq_gemm_static_scratch compares with its array; no device needed).
int static_scratch_need(const b200dq_gemm_args* a, int sm_count, size_t* need) {
  if (a->M <= 0 || a->N <= 0 || a->K <= 0)
    return fail("gemm: M, N, K must be positive (got %d, %d, %d)", a->M, a->N, a->K);
  Schedule s;
  if (takes_int8_skinny_path(a)) { *need = 0; return 0; }
  const int tile = takes_skinny_path(a) ? kSkinnyTokens : a->token_tile;
  if (make_schedule(a->M, a->N, a->K, a->act_type, tile, a->max_ctas, sm_count, &s, -1, !takes_skinny_path(a)) != 0) return -1;
  *need = s.needs_scratch ? s.workspace_bytes : 0;
  return 0;
}

// The one implementation behind b200dq_gemm and b200dq_gemm_static_scratch: validation,
// schedule, tensor map, kernel choice and launch. `scratch` receives the stream-K partial
// tiles; `who` prefixes error messages.
int run_gemm(const char* who, const b200dq_gemm_args* a, void* scratch, size_t scratch_bytes, int sm_count,
             DeviceStatus* status, cudaStream_t stream) {
  if (a->a == nullptr || a->wp == nullptr || a->c == nullptr) return fail("%s: null tensor pointer", who);
  if (a->M <= 0 || a->N <= 0 || a->K <= 0)
    return fail("%s: M, N, K must be positive (got %d, %d, %d)", who, a->M, a->N, a->K);
  const int wf = a->weight_format, act = a->act_type;
  const bool int_act = (act == ACT_I8);
  const bool wf_int = (wf == WF_I2_I8 || wf == WF_I4_I8);
  if (wf < WF_U4_SZ || wf > kLastWeightFormat) return fail("%s: unknown weight format %d", who, wf);
  if (act < ACT_F16 || act > ACT_I8) return fail("%s: unknown activation type %d", who, act);
  if (a->out_type < OUT_F16 || a->out_type > OUT_I32) return fail("%s: unknown output type %d", who, a->out_type);
  if (wf_int != int_act) return fail("%s: weight format %d and activation type %d do not go together", who, wf, act);
  if (wf == WF_FP4_E8M0 && act == ACT_I8) return fail("%s: fp4 weights need f16 or bf16 activations", who);
  if ((wf == WF_U4_SZ || wf == WF_U2_SZ || wf == WF_LUT4_S) && (a->group_size <= 0 || a->K % a->group_size != 0))
    return fail("%s: group_size=%d must divide K=%d", who, a->group_size, a->K);
  if ((a->flags & GF_HAS_BIAS) && a->bias == nullptr) return fail("%s: HAS_BIAS set but bias is null", who);
  if ((a->flags & GF_ROW_SCALE) && a->row_scale == nullptr) return fail("%s: ROW_SCALE set but row_scale is null", who);
  if ((reinterpret_cast<uintptr_t>(a->wp) & 15) != 0) return fail("%s: packed weights must be 16-byte aligned", who);
  if (a->num_peers < 0 || a->num_peers > 7) return fail("%s: num_peers=%d outside [0, 7]", who, a->num_peers);
  for (int d = 0; d < a->num_peers; ++d) {
    if (a->c_peers[d] == nullptr) return fail("%s: c_peers[%d] is null", who, d);
    if ((reinterpret_cast<uintptr_t>(a->c_peers[d]) & 15) != (reinterpret_cast<uintptr_t>(a->c) & 15))
      return fail("%s: c_peers[%d] must have the alignment of c (same layout behind every base)", who, d);
  }

  const bool grouped = a->num_groups > 0;
  if (grouped) {
    if (a->group_row_prefix == nullptr || a->group_tile_prefix == nullptr)
      return fail("%s: grouped mode needs group_row_prefix and group_tile_prefix", who);
    if (a->total_tiles == 0) return fail("%s: grouped mode needs total_tiles (or minus an upper bound of it)", who);
    if (a->token_tile == 0) return fail("%s: grouped mode needs an explicit token_tile (the prefix arrays depend on it)", who);
    if (a->flags & (GF_TRANS_C | GF_HAS_BIAS)) return fail("%s: grouped mode supports neither TRANS_C nor bias", who);
  }
  if (takes_int8_skinny_path(a)) {
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.wp = static_cast<const uint8_t*>(a->wp);
    p.a = a->a;
    p.c = a->c;
    p.bias = a->bias;
    p.row_scale = a->row_scale;
    p.tensor_scale = a->tensor_scale;
    p.code_bias = a->code_bias;
    p.M = a->M; p.N = a->N; p.K = a->K;
    p.n_tiles = (a->N + kTileRows - 1) / kTileRows;
    p.st_total = stages_for(a->K, ACT_I8);
    p.st_units = p.st_total;
    p.stage_bytes = stage_bytes_for(wf, a->group_size);
    p.ldc = (a->flags & GF_TRANS_C) ? a->M : a->N;
    p.flags = a->flags & (GF_TRANS_C | GF_HAS_BIAS | GF_ROW_SCALE);
    p.out_type = a->out_type;
    p.status = status;
    p.n_peers = a->num_peers;
    for (int d = 0; d < a->num_peers; ++d) p.c_peer[d] = a->c_peers[d];
    CUDA_OK(launch_int8_skinny_gemm(wf, p, stream));
    return 0;
  }
  const bool skinny = takes_skinny_path(a);
  Schedule s;
  // total_tiles < 0: the group sizes are known on the device only; plan the grid for the bound
  // and let the kernel cut the real total (group_tile_prefix[num_groups]) evenly over it
  const bool dyn = grouped && a->total_tiles < 0;
  const long long plan_tiles = grouped ? (dyn ? -static_cast<long long>(a->total_tiles) : a->total_tiles) : -1;
  if (make_schedule(a->M, a->N, a->K, act, skinny ? kSkinnyTokens : a->token_tile, a->max_ctas, sm_count, &s,
                    plan_tiles, !skinny) != 0) return -1;
  // device-planned: the kernel cuts the real total evenly, so tiles are cut unless the spans are
  // rounded up to whole tiles (the narrow-tile rule above; the grid was sized for the bound)
  if (dyn && s.grid > 1) s.needs_scratch = !s.whole_tiles;
  if (s.needs_scratch) {
    if (scratch == nullptr || scratch_bytes < s.workspace_bytes)
      return fail("%s: workspace too small: need %zu bytes, got %zu", who, s.workspace_bytes, scratch_bytes);
    if ((reinterpret_cast<uintptr_t>(scratch) & 15) != 0) return fail("%s: workspace must be 16-byte aligned", who);
  }

  CUtensorMap tmap;
  int b_group = 1;
  if (skinny) {
    if (encode_skinny_activation_map(&tmap, a->a, a->M, a->K, act, skinny_box_tokens(a->M)) != 0) return -1;
  } else {
    b_group = encode_activation_map(&tmap, a->a, a->M, a->K, act, s.tn, group_kblocks_for(s.tn));
    if (b_group < 0) return -1;
  }
  int flags = a->flags & (GF_TRANS_C | GF_HAS_BIAS | GF_ROW_SCALE | GF_FP4_SIMPLE);
  if (output_takes_vector_stores(a->c, a->N, a->out_type, flags)) flags |= GF_VEC_STORE;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.b_group = b_group;
  p.wp = static_cast<const uint8_t*>(a->wp);
  p.a = a->a;
  p.c = a->c;
  p.partial = static_cast<uint32_t*>(scratch);
  p.bias = a->bias;
  p.row_scale = a->row_scale;
  p.tensor_scale = a->tensor_scale;
  p.code_bias = a->code_bias;
  p.fp4_exp_bias = a->fp4_exp_bias;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.n_tiles = s.n_tiles; p.m_tiles = s.m_tiles; p.st_total = s.st_total; p.st_units = s.st_units;
  p.span = s.span; p.units = s.units;
  p.stage_bytes = stage_bytes_for(wf, a->group_size);
  p.sz_per_kb = ((wf == WF_U4_SZ || wf == WF_U2_SZ || wf == WF_LUT4_S) && a->group_size == 64) ? 1 : 0;
  p.ldc = (a->flags & GF_TRANS_C) ? a->M : a->N;
  p.flags = flags;
  p.out_type = a->out_type;
  p.tn = s.tn;
  p.num_groups = grouped ? a->num_groups : 0;
  p.dyn_grid = dyn ? s.grid : 0;
  p.dyn_whole = (dyn && s.whole_tiles) ? 1 : 0;
  if (wf == WF_LUT4_S) {
    // the table in the activation dtype, low and high bytes apart
    for (int i = 0; i < 16; ++i) {
      const float v = a->code_table[i];
      const uint16_t bits = act == ACT_BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
      p.lut_lo[i >> 2] |= static_cast<uint32_t>(bits & 0xffu) << (8 * (i & 3));
      p.lut_hi[i >> 2] |= static_cast<uint32_t>(bits >> 8) << (8 * (i & 3));
    }
  }
  if (s.needs_scratch) {
    // unique per launch in this process; a counter word left by another launch never matches
    static std::atomic<unsigned long long> launch_epoch{0x5bd1e995ull};
    p.tile_ctr = reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(scratch) + s.slot_bytes);
    p.epoch = launch_epoch.fetch_add(1, std::memory_order_relaxed) & 0x00ffffffffffffffull;
  }
  p.n_peers = a->num_peers;
  for (int d = 0; d < a->num_peers; ++d) p.c_peer[d] = a->c_peers[d];
  p.grp_row_prefix = grouped ? a->group_row_prefix : nullptr;
  p.grp_tile_prefix = grouped ? a->group_tile_prefix : nullptr;
  p.grp_w_stride = grouped ? a->group_weight_stride : 0;
  p.status = status;

  if (skinny) {
    CUDA_OK(launch_skinny_gemm(wf, act, tmap, p, s.grid, stream));
    return 0;
  }
  const cudaError_t e = launch_umma_gemm(wf, act, s.tn, tmap, p, s.grid, stream);
  if (e == cudaSuccess) return 0;
  if (e != cudaErrorInvalidValue) return fail("%s: launch failed: %s", who, cudaGetErrorString(e));
  return fail("%s: no kernel for weight format %d with activation type %d", who, wf, act);
}

}  // namespace

extern "C" {

int b200dq_version(void) { return kAbiVersion; }

const char* b200dq_get_last_error(void) { return g_err; }

int b200dq_init(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  int dev = 0;
  CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail("device index %d out of range", dev);
  if (g_dev[dev].ready.load(std::memory_order_relaxed)) return 0;
  cudaDeviceProp prop;
  CUDA_OK(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10) return fail("b200dq needs an sm_100 GPU, device %d is sm_%d%d", dev, prop.major, prop.minor);
  if (resolve_encoder() != 0) return -1;
  DeviceStatus* st = nullptr;
  CUDA_OK(cudaMalloc(&st, sizeof(DeviceStatus)));
  CUDA_OK(cudaMemset(st, 0, sizeof(DeviceStatus)));
  g_dev[dev].status = st;
  g_dev[dev].sm_count = prop.multiProcessorCount;
  g_dev[dev].ready.store(true, std::memory_order_release);
  return 0;
}

size_t b200dq_gemm_workspace_bytes(int32_t M, int32_t N, int32_t K, int32_t weight_format, int32_t act_type,
                                   int32_t token_tile, int32_t max_ctas) {
  (void)weight_format;
  Schedule s;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (make_schedule(M, N, K, act_type, token_tile, max_ctas, sm_count_or_bound(), &s) != 0) return 0;
  return s.workspace_bytes;
}

size_t b200dq_gemm_workspace_bytes_for(const b200dq_gemm_args* a) {
  if (a == nullptr || a->M <= 0 || a->N <= 0 || a->K <= 0) return 0;
  Schedule s;
  const bool grouped = a->num_groups > 0;
  if (takes_int8_skinny_path(a)) return 0;
  const int tile = takes_skinny_path(a) ? kSkinnyTokens : a->token_tile;
  const long long tiles = grouped ? (a->total_tiles < 0 ? -static_cast<long long>(a->total_tiles) : a->total_tiles) : -1;
  if (make_schedule(a->M, a->N, a->K, a->act_type, tile, a->max_ctas, sm_count_or_bound(), &s, tiles,
                    !takes_skinny_path(a)) != 0) return 0;
  return s.workspace_bytes;
}

size_t b200dq_packed_weight_bytes(int32_t N, int32_t K, int32_t group_size, int32_t weight_format) {
  if (N <= 0 || K <= 0 || weight_format < WF_U4_SZ || weight_format > kLastWeightFormat) return 0;
  const int n_tiles = (N + kTileRows - 1) / kTileRows;
  const bool int8_target = (weight_format == WF_I2_I8 || weight_format == WF_I4_I8);
  const int st_total = stages_for(K, int8_target ? ACT_I8 : ACT_BF16);
  return static_cast<size_t>(n_tiles) * st_total * stage_bytes_for(weight_format, group_size);
}

int b200dq_pack_weights(const void* q_natural, const void* scales, const void* zeros, void* wp, int32_t N, int32_t K,
                        int32_t group_size, int32_t weight_format, int32_t act_type, void* cuda_stream) {
  if (q_natural == nullptr || wp == nullptr) return fail("pack_weights: null pointer");
  if (weight_format < WF_U4_SZ || weight_format > kLastWeightFormat) return fail("pack_weights: unknown weight format %d", weight_format);
  const bool int8_target = (weight_format == WF_I2_I8 || weight_format == WF_I4_I8);
  const int bits = (weight_format == WF_I2_I8 || weight_format == WF_U2_SZ) ? 2 : 4;
  if (N <= 0 || K <= 0) return fail("pack_weights: N and K must be positive");
  if (K % (128 / bits) != 0) return fail("pack_weights: K=%d must be a multiple of %d for %d-bit codes", K, 128 / bits, bits);
  if ((reinterpret_cast<uintptr_t>(q_natural) & 3) != 0 || (reinterpret_cast<uintptr_t>(wp) & 15) != 0)
    return fail("pack_weights: input must be 4-byte and output 16-byte aligned");
  PackParams p;
  memset(&p, 0, sizeof(p));
  p.q = static_cast<const uint32_t*>(q_natural);
  p.wp = static_cast<uint32_t*>(wp);
  p.N = N; p.K = K; p.bits = bits;
  p.mode = int8_target ? 1 : (weight_format == WF_FP4_E8M0 ? 2 : (weight_format == WF_LUT4_S ? 3 : 0));
  p.n_tiles = (N + kTileRows - 1) / kTileRows;
  p.st_total = stages_for(K, int8_target ? ACT_I8 : ACT_BF16);
  p.code_words_per_kb = codes_per_kblock_bytes(weight_format) / 4;
  p.elems_per_kblock = int8_target ? 128 : 64;
  if (weight_format == WF_U4_SZ || weight_format == WF_U2_SZ || weight_format == WF_LUT4_S) {
    if (scales == nullptr) return fail("pack_weights: this weight format needs scales");
    if (act_type != ACT_F16 && act_type != ACT_BF16) return fail("pack_weights: scales must be f16 or bf16");
    if (group_size <= 0 || K % group_size != 0) return fail("pack_weights: group_size=%d must divide K=%d", group_size, K);
    if (!(group_size == 64 || group_size % 128 == 0 || group_size == K))
      return fail("pack_weights: group_size=%d must be 64, a multiple of 128, or K", group_size);
    p.sz_kind = weight_format == WF_LUT4_S ? 3 : 1;
    p.scales = static_cast<const uint16_t*>(scales);
    p.zeros = static_cast<const uint16_t*>(zeros);
    p.bf16 = (act_type == ACT_BF16);
    p.group_size = group_size;
    p.groups = K / group_size;
  } else if (weight_format == WF_FP4_E8M0) {
    if (scales == nullptr) return fail("pack_weights: e2m1 weights need their exponent bytes");
    if (K % 32 != 0) return fail("pack_weights: K=%d must be a multiple of 32", K);
    p.sz_kind = 2;
    p.exps = static_cast<const uint8_t*>(scales);
  }
  p.nsz = nsz_for(weight_format, group_size);
  p.stage_words = stage_bytes_for(weight_format, group_size) / 4;
  const long long total = static_cast<long long>(p.n_tiles) * p.st_total * p.stage_words;
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  pack_image_kernel<<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(p);
  CUDA_OK(cudaGetLastError());
  return 0;
}

int b200dq_gemm(const b200dq_gemm_args* a, void* cuda_stream) {
  if (a == nullptr) return fail("gemm: null argument struct");
  DeviceState* ds = nullptr;
  if (current_device_state(&ds) != 0) return -1;
  return run_gemm("gemm", a, a->workspace, a->workspace_bytes, ds->sm_count, ds->status,
                  static_cast<cudaStream_t>(cuda_stream));
}

int b200dq_gemm_static_scratch(const b200dq_gemm_args* a, void* cuda_stream) {
  if (a == nullptr) return fail("gemm_static_scratch: null argument struct");
  int dev = 0;
  CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail("device index %d out of range", dev);
  StaticScratchState& ss = g_static_dev[dev];
  if (!ss.ready.load(std::memory_order_acquire)) {
    // One-time set-up for this device, with this device current. In host code the
    // array's name is only a stand-in; the kernels need its device address.
    std::lock_guard<std::mutex> lock(g_mu);
    if (!ss.ready.load(std::memory_order_relaxed)) {
      cudaDeviceProp prop;
      CUDA_OK(cudaGetDeviceProperties(&prop, dev));
      if (prop.major != 10) return fail("b200dq needs an sm_100 GPU, device %d is sm_%d%d", dev, prop.major, prop.minor);
      if (resolve_encoder() != 0) return -1;
      void* ptr = nullptr;
      CUDA_OK(cudaGetSymbolAddress(&ptr, g_static_scratch));
      if (ptr == nullptr) return fail("gemm_static_scratch: no device address for the static scratch array");
      ss.scratch = ptr;
      ss.sm_count = prop.multiProcessorCount;
      ss.ready.store(true, std::memory_order_release);
    }
  }
  if (a->num_groups > 0) return fail("gemm_static_scratch: grouped mode is not offered by this entry point");
  size_t need = 0;
  if (static_scratch_need(a, ss.sm_count, &need) != 0) return -1;
  if (need > kStaticScratchBytes)
    return fail("gemm_static_scratch: this problem needs %zu bytes of scratch, the static array holds %zu; "
                "lower max_ctas or use b200dq_gemm with a caller-provided workspace",
                need, kStaticScratchBytes);
  // device-side status reporting needs the word b200dq_init allocates; without it the
  // kernels still bound every wait, they just have nowhere to record one that gave up
  DeviceStatus* status = g_dev[dev].ready.load(std::memory_order_acquire) ? g_dev[dev].status : nullptr;
  return run_gemm("gemm_static_scratch", a, ss.scratch, kStaticScratchBytes, ss.sm_count, status,
                  static_cast<cudaStream_t>(cuda_stream));
}

int b200dq_static_scratch_check(const b200dq_gemm_args* a, int32_t sm_count, size_t* needed_bytes,
                                size_t* capacity_bytes) {
  if (a == nullptr) return fail("static_scratch_check: null argument struct");
  if (sm_count <= 0) return fail("static_scratch_check: sm_count must be positive");
  size_t need = 0;
  if (static_scratch_need(a, sm_count, &need) != 0) return -1;
  if (needed_bytes != nullptr) *needed_bytes = need;
  if (capacity_bytes != nullptr) *capacity_bytes = kStaticScratchBytes;
  if (need > kStaticScratchBytes)
    return fail("gemm_static_scratch: this problem needs %zu bytes of scratch, the static array holds %zu; "
                "lower max_ctas or use b200dq_gemm with a caller-provided workspace",
                need, kStaticScratchBytes);
  return 0;
}

int b200dq_absmax_quant_int8(const void* x, void* q, float* scale, int32_t M, int32_t K, int32_t act_type,
                             void* cuda_stream) {
  if (x == nullptr || q == nullptr || scale == nullptr) return fail("absmax_quant_int8: null pointer");
  if (M <= 0 || K <= 0 || K % 8 != 0) return fail("absmax_quant_int8: M=%d, K=%d (K must be a positive multiple of 8)", M, K);
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (reinterpret_cast<uintptr_t>(q) & 7) != 0)
    return fail("absmax_quant_int8: x must be 16-byte and q 8-byte aligned");
  auto stream = static_cast<cudaStream_t>(cuda_stream);
  if (act_type == ACT_BF16)
    absmax_quant_int8_kernel<__nv_bfloat16><<<M, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<int8_t*>(q), scale, K);
  else if (act_type == ACT_F16)
    absmax_quant_int8_kernel<__half><<<M, 256, 0, stream>>>(static_cast<const __half*>(x), static_cast<int8_t*>(q), scale, K);
  else
    return fail("absmax_quant_int8: input must be f16 or bf16");
  CUDA_OK(cudaGetLastError());
  return 0;
}

int b200dq_moe_combine(const void* y, const int64_t* row_of, const float* weights, void* out, int64_t tokens,
                       int32_t top_k, int32_t H, int32_t act_type, void* cuda_stream) {
  if (y == nullptr || row_of == nullptr || weights == nullptr || out == nullptr) return fail("moe_combine: null pointer");
  if (tokens < 0 || top_k <= 0 || H <= 0 || H % 8 != 0)
    return fail("moe_combine: tokens=%lld, top_k=%d, H=%d (H must be a positive multiple of 8)", static_cast<long long>(tokens), top_k, H);
  if (tokens == 0) return 0;
  if ((reinterpret_cast<uintptr_t>(y) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0)
    return fail("moe_combine: pointers must be 16-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  const long long total = tokens * (H / 8);
  const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 148 * 16));
  const long long* rows = reinterpret_cast<const long long*>(row_of);
  if (act_type == ACT_BF16)
    moe_combine_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(y), rows, weights, static_cast<__nv_bfloat16*>(out), tokens, top_k, H);
  else if (act_type == ACT_F16)
    moe_combine_kernel<__half><<<blocks, 256, 0, stream>>>(static_cast<const __half*>(y), rows, weights, static_cast<__half*>(out), tokens, top_k, H);
  else
    return fail("moe_combine: rows must be f16 or bf16");
  CUDA_OK(cudaGetLastError());
  return 0;
}

int b200dq_unpack_int4_to_int8(const void* packed, void* out, int64_t num_elems, void* cuda_stream) {
  if (packed == nullptr || out == nullptr) return fail("unpack_int4_to_int8: null pointer");
  if (num_elems < 0 || num_elems % 16 != 0) return fail("unpack_int4_to_int8: element count must be a multiple of 16");
  if (num_elems == 0) return 0;
  if ((reinterpret_cast<uintptr_t>(packed) & 7) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0)
    return fail("unpack_int4_to_int8: input must be 8-byte and output 16-byte aligned");
  const long long nvec = num_elems / 16;
  const int blocks = static_cast<int>(std::min<long long>((nvec + 255) / 256, 148 * 16));
  unpack_int4_to_int8_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint2*>(packed), static_cast<uint4*>(out), nvec);
  CUDA_OK(cudaGetLastError());
  return 0;
}

int b200dq_silu_mul(const void* h, void* out, int64_t rows, int32_t H, int32_t act_type, void* cuda_stream) {
  if (h == nullptr || out == nullptr) return fail("silu_mul: null pointer");
  if (rows < 0 || H <= 0 || H % 8 != 0) return fail("silu_mul: rows=%lld, H=%d (H must be a positive multiple of 8)", static_cast<long long>(rows), H);
  if (rows == 0) return 0;
  if ((reinterpret_cast<uintptr_t>(h) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0)
    return fail("silu_mul: pointers must be 16-byte aligned");
  auto stream = static_cast<cudaStream_t>(cuda_stream);
  const long long total = rows * (H / 8);
  const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 148 * 16));
  if (act_type == ACT_BF16)
    silu_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(h), static_cast<__nv_bfloat16*>(out), rows, H);
  else if (act_type == ACT_F16)
    silu_mul_kernel<__half><<<blocks, 256, 0, stream>>>(static_cast<const __half*>(h), static_cast<__half*>(out), rows, H);
  else
    return fail("silu_mul: input must be f16 or bf16");
  CUDA_OK(cudaGetLastError());
  return 0;
}

int b200dq_quant_mxfp4(const void* x, void* codes, void* scale_bytes, int32_t M, int32_t K, int32_t act_type,
                       int32_t sf_blocked, void* cuda_stream) {
  if (x == nullptr || codes == nullptr || scale_bytes == nullptr) return fail("quant_mxfp4: null pointer");
  if (M <= 0 || K <= 0 || K % 32 != 0) return fail("quant_mxfp4: M=%d, K=%d (K must be a positive multiple of 32)", M, K);
  if (sf_blocked && K % 128 != 0) return fail("quant_mxfp4: the blocked scale layout needs K to be a multiple of 128");
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (reinterpret_cast<uintptr_t>(codes) & 3) != 0)
    return fail("quant_mxfp4: x must be 16-byte and codes 4-byte aligned");
  auto stream = static_cast<cudaStream_t>(cuda_stream);
  const long long n_vec = static_cast<long long>(M) * K / 8;
  const unsigned blocks = static_cast<unsigned>((n_vec + 255) / 256);
  if (act_type == ACT_BF16)
    quant_mxfp4_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                                   static_cast<uint32_t*>(codes),
                                                                   static_cast<uint8_t*>(scale_bytes), n_vec, K, sf_blocked);
  else if (act_type == ACT_F16)
    quant_mxfp4_kernel<__half><<<blocks, 256, 0, stream>>>(static_cast<const __half*>(x), static_cast<uint32_t*>(codes),
                                                            static_cast<uint8_t*>(scale_bytes), n_vec, K, sf_blocked);
  else
    return fail("quant_mxfp4: input must be f16 or bf16");
  CUDA_OK(cudaGetLastError());
  return 0;
}

int b200dq_gemm_mxfp4_native(const void* a_codes, const void* a_sf, const void* w_codes, const void* w_sf, void* c,
                             int32_t M, int32_t N, int32_t K, int32_t out_type, void* cuda_stream) {
  if (a_codes == nullptr || a_sf == nullptr || w_codes == nullptr || w_sf == nullptr || c == nullptr)
    return fail("gemm_mxfp4_native: null pointer");
  if (M <= 0 || N <= 0 || K <= 0) return fail("gemm_mxfp4_native: M, N, K must be positive (got %d, %d, %d)", M, N, K);
  if (K % 256 != 0) return fail("gemm_mxfp4_native: K=%d must be a multiple of 256", K);
  if (out_type != OUT_BF16 && out_type != OUT_F16 && out_type != OUT_F32)
    return fail("gemm_mxfp4_native: output must be f16, bf16 or f32");
  for (const void* ptr : {a_codes, a_sf, w_codes, w_sf, static_cast<const void*>(c)})
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return fail("gemm_mxfp4_native: pointers must be 16-byte aligned");
  DeviceState* ds = nullptr;
  if (current_device_state(&ds) != 0) return -1;
  CUtensorMap maps[2];
  const void* bases[2] = {a_codes, w_codes};
  const int rows[2] = {M, N};
  for (int i = 0; i < 2; ++i) {
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(K / 2), static_cast<cuuint64_t>(rows[i])};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(K / 2)};
    cuuint32_t box[2] = {kMxf4BoxBytes, kMxf4BoxRows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(&maps[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(bases[i]), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("gemm_mxfp4_native: cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  }
  Mxf4Params p;
  memset(&p, 0, sizeof(p));
  p.sfa = static_cast<const uint32_t*>(a_sf);
  p.sfw = static_cast<const uint32_t*>(w_sf);
  p.c = c;
  p.M = M; p.N = N; p.K = K;
  p.m_tiles = (M + 127) / 128;
  p.n_tiles = (N + 127) / 128;
  p.k_blocks = K / 256;
  p.out_type = out_type;
  p.status = ds->status;
  CUDA_OK(launch_mxf4_gemm(maps[0], maps[1], p, ds->sm_count, static_cast<cudaStream_t>(cuda_stream)));
  return 0;
}

int b200dq_tensor_peak(int32_t kind, int32_t mmas, double* ops, void* cuda_stream) {
  if (kind < 0 || kind > 2) return fail("tensor_peak: kind must be 0 (bf16), 1 (int8) or 2 (mxfp4)");
  if (mmas <= 0 || mmas > (1 << 22)) return fail("tensor_peak: mmas=%d outside [1, 2^22]", mmas);
  DeviceState* ds = nullptr;
  if (current_device_state(&ds) != 0) return -1;
  CUDA_OK(launch_tensor_peak(kind, mmas, ds->sm_count, ds->status, ops, static_cast<cudaStream_t>(cuda_stream)));
  return 0;
}

int b200dq_grouped_prefixes(const void* counts, int32_t counts_are_int64, int32_t num_groups, int32_t N,
                            int32_t token_tile, int32_t* row_prefix, int32_t* tile_prefix, void* cuda_stream) {
  if (counts == nullptr || row_prefix == nullptr || tile_prefix == nullptr) return fail("grouped_prefixes: null pointer");
  if (num_groups <= 0 || N <= 0) return fail("grouped_prefixes: num_groups and N must be positive");
  if (token_tile != 16 && token_tile != 32 && token_tile != 64 && token_tile != 128 && token_tile != 256)
    return fail("grouped_prefixes: token_tile must be 16, 32, 64, 128 or 256 (got %d)", token_tile);
  grouped_prefix_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      counts, counts_are_int64, num_groups, (N + kTileRows - 1) / kTileRows, token_tile, row_prefix, tile_prefix);
  CUDA_OK(cudaGetLastError());
  return 0;
}

int b200dq_check_status(void* cuda_stream) {
  DeviceState* ds = nullptr;
  if (current_device_state(&ds) != 0) return -1;
  auto stream = static_cast<cudaStream_t>(cuda_stream);
  DeviceStatus h;
  CUDA_OK(cudaMemcpyAsync(&h, ds->status, sizeof(h), cudaMemcpyDeviceToHost, stream));
  CUDA_OK(cudaStreamSynchronize(stream));
  if (h.error == ERR_NONE) return 0;
  CUDA_OK(cudaMemsetAsync(ds->status, 0, sizeof(DeviceStatus), stream));
  CUDA_OK(cudaStreamSynchronize(stream));
  return fail("device status: error %u (1 = a bounded wait gave up), first at block %u wait site %u, %u waits gave up, "
              "site mask 0x%x",
              h.error, h.where >> 8, h.where & 0xff, h.count, h.sites);
}

}  // extern "C"
