/* b200dq — C ABI of the B200 (sm_100a) low-bit dequantize-GEMM library.
 *
 * The reference (tile-ai/tilelang) exposes every JIT-compiled kernel through a
 * three-symbol C convention that its ctypes/Cython adapters bind:
 *     int init(void); int call(<device pointers, scalars>, cudaStream_t);
 *     const char* get_last_error(void);
 * (tilelang/jit/adapter/wrapper.py:60-86, used from
 *  tilelang/jit/adapter/cython/adapter.py:135-139, 338-345). This header keeps
 * that convention with one `call`-style entry point per kernel family.
 *
 * Rules shared by every entry point:
 *   - returns 0 on success, -1 on error; the message is in b200dq_get_last_error();
 *   - never throws, never synchronises the device, never allocates device memory
 *     (scratch is passed in by the caller), launches on the given stream;
 *   - all pointers are device pointers unless stated otherwise; inputs are only
 *     borrowed for the duration of the (asynchronous) launch.
 */
#ifndef B200DQ_H_
#define B200DQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Weight formats of the private, pre-packed device layout (see pack entry points). */
enum b200dq_weight_format {
  B200DQ_WF_U4_SZ = 0,    /* uint4 + per-group scale/zero term; fp16/bf16 activations   */
  B200DQ_WF_U4_RAW = 1,   /* uint4, weight = q (no scale)                               */
  B200DQ_WF_S4_RAW = 2,   /* int4 stored as q + 8, weight = q (no scale)                */
  B200DQ_WF_FP4_E8M0 = 3, /* fp4 codes + one e8m0 exponent byte per 32 K elements (bf16
                           * activations; with fp16 activations the exponent bytes are ignored) */
  B200DQ_WF_I2_I8 = 4,    /* 2-bit codes -> int8 (minus code_bias); int8 activations    */
  B200DQ_WF_I4_I8 = 5,    /* 4-bit codes -> int8 (minus code_bias); int8 activations    */
  B200DQ_WF_U2_SZ = 6,    /* 2-bit codes + per-group scale and zero-point; fp16/bf16 activations
                           * (the int2 / int1 -> f16 decoders of quantize/lop3.py:424-891) */
  B200DQ_WF_LUT4_S = 7    /* 4-bit index into code_table[16] * per-group scale (NF4 and other
                           * codebooks); fp16/bf16 activations                            */
};
enum b200dq_act_type { B200DQ_ACT_F16 = 0, B200DQ_ACT_BF16 = 1, B200DQ_ACT_I8 = 2 };
enum b200dq_out_type { B200DQ_OUT_F16 = 0, B200DQ_OUT_BF16 = 1, B200DQ_OUT_F32 = 2, B200DQ_OUT_I32 = 3 };
enum b200dq_gemm_flags {
  B200DQ_GF_TRANS_C = 1,   /* write C^T (N x M), the orientation of the reference's fp4/w4a8 examples */
  B200DQ_GF_HAS_BIAS = 2,  /* add bias[M][N] (output dtype) before the cast                           */
  B200DQ_GF_ROW_SCALE = 4, /* integer path: acc / row_scale[m] / tensor_scale before the cast          */
  B200DQ_GF_FP4_SIMPLE = 16 /* FP4 codes follow the reference's no-subnormal rule 2^(e-1) * (1 + m/2)
                             * (example_dequant_gemm_fp4_hopper.py:10-29, dequantize_utils.py:57-84)
                             * instead of true e2m1 */
};

/* Replaces init() of tilelang/jit/adapter/wrapper.py:60-70: selects nothing, but
 * raises the dynamic shared-memory limit of every kernel, resolves the driver's
 * tensor-map encoder and allocates the 16-byte device status word of the current
 * device. Idempotent, thread-safe, once per device. */
int b200dq_init(void);

/* Replaces get_last_error() of tilelang/jit/adapter/wrapper.py:72-76. The buffer
 * is thread-local and valid until the next failing call on the same thread. */
const char* b200dq_get_last_error(void);

/* Library ABI version (bumped when a struct below changes). */
int b200dq_version(void);

/* Arguments of the dequantize-GEMM  C[M,N] = A[M,K] * dequant(W[N,K])^T. */
typedef struct b200dq_gemm_args {
  const void* a;            /* activations, row-major (M, K), act_type                          */
  const void* wp;           /* packed image from b200dq_pack_weights                            */
  const void* bias;         /* optional (M, N) bias in the output dtype, or NULL                */
  const float* row_scale;   /* optional per-token divisor (M), or NULL                          */
  void* c;                  /* output (M, N) or, with TRANS_C, (N, M)                           */
  void* workspace;          /* scratch of at least b200dq_gemm_workspace_bytes() bytes          */
  size_t workspace_bytes;
  int32_t M, N, K;
  int32_t group_size;       /* K elements per scale group (U4_SZ); 32 for FP4_E8M0; else ignored */
  int32_t weight_format;    /* enum b200dq_weight_format */
  int32_t act_type;         /* enum b200dq_act_type      */
  int32_t out_type;         /* enum b200dq_out_type      */
  int32_t flags;            /* enum b200dq_gemm_flags    */
  float tensor_scale;       /* used with ROW_SCALE       */
  uint32_t code_bias;       /* bytewise bias of the integer decoders, e.g. 0x02020202 */
  int32_t fp4_exp_bias;     /* 127: OCP e8m0 exponent bytes; 0: raw power-of-two exponents */
  int32_t token_tile;       /* 0 = choose (M <= 16 with uint4 or e2m1 weights on 16-bit activations and
                             * K % 128 == 0 then takes the memory-bound small-M kernel); else 16, 32, 64,
                             * 128 or 256 tokens per CTA tile of the tcgen05 kernel */
  int32_t max_ctas;         /* 0 = one per SM; else an upper bound on the grid */
  /* Grouped mode (mixture of experts; num_groups = 0 for one dense GEMM). Rows of A and C
   * are sorted by group; group g owns rows [group_row_prefix[g], group_row_prefix[g+1]) and
   * the packed image at wp + g * group_weight_stride (all groups share N, K and format).
   * group_tile_prefix[g] = sum over earlier groups of ceil(rows / token_tile) * ceil(N / 128);
   * total_tiles is its last entry. Both prefix arrays are int32 device arrays of
   * num_groups + 1 entries; M is the total number of rows. Same semantics as the grouped
   * GEMM of examples/grouped_gemm/example_grouped_gemm_fwd.py:8-36 with dequantised weights.
   * When the group sizes exist only on the device (a router's counts), fill the prefix
   * arrays with b200dq_grouped_prefixes and pass total_tiles = -(an upper bound of the tile
   * total), e.g. -(ceil(M / token_tile) + num_groups) * ceil(N / 128): the grid is planned
   * for the bound and the kernel cuts the real total, read from group_tile_prefix[num_groups],
   * evenly over it. No host synchronisation is needed then. */
  const int32_t* group_row_prefix;
  const int32_t* group_tile_prefix;
  int64_t group_weight_stride;
  int32_t num_groups;
  int32_t total_tiles;
  /* Copies of the output on other GPUs of the node (0 for none): num_peers device pointers
   * into peer memory that this process can write (peer access enabled, an IPC or symmetric
   * mapping), each the base of a tensor laid out exactly like c. Every output element is stored
   * to c and at the same offset behind every c_peers[i], from the kernel's epilogue: a
   * column-sharded GEMM fills every rank's gathered tensor without a separate all-gather.
   * The stores are complete when the launch is; the ranks still need their own barrier
   * before anyone reads a gathered tensor. The reference is single-GPU and has no counterpart. */
  void* c_peers[7];
  int32_t num_peers;
  /* B200DQ_WF_LUT4_S only: the value of each of the 16 codes (NF4 or any other 4-bit codebook);
   * weight = code_table[q] * scale[row, group], the table rounded to the activation dtype. */
  float code_table[16];
} b200dq_gemm_args;

/* Replaces call(...) of the kernels generated from
 *   examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:16-90,
 *   examples/dequantize_gemm/example_dequant_gemm_bf16_mxfp4_hopper.py:80-378,
 *   examples/dequantize_gemm/example_dequant_gemm_fp4_hopper.py:108-220,
 *   examples/dequantize_gemm/example_dequant_gemm_w4a8.py:85-149,
 *   examples/dequantize_gemm/example_dequant_gemv_fp16xint4.py:11-155,
 *   examples/bitnet-1.58b/kernel_benchmark/tilelang_bitnet_158_int8xint2_{decode,prefill}.py
 * for one B200. */
int b200dq_gemm(const b200dq_gemm_args* args, void* cuda_stream);

/* Scratch bytes b200dq_gemm needs for a dense call of these sizes (stream-K partial
 * tiles). Before b200dq_init has run on the current device the figure is an upper bound
 * that holds for any SM count up to 256. */
size_t b200dq_gemm_workspace_bytes(int32_t M, int32_t N, int32_t K, int32_t weight_format,
                                   int32_t act_type, int32_t token_tile, int32_t max_ctas);

/* The same for a filled-in argument struct; the one to use for grouped calls, whose
 * schedule follows total_tiles (every group rounds up to whole tiles) and not M. The
 * pointers in the struct are not read. */
size_t b200dq_gemm_workspace_bytes_for(const b200dq_gemm_args* args);

/* Device-side row and tile prefixes (num_groups + 1 int32 entries each) of a grouped call
 * from per-group row counts in device memory (int32, or int64 when counts_are_int64 != 0). */
int b200dq_grouped_prefixes(const void* counts, int32_t counts_are_int64, int32_t num_groups, int32_t N,
                            int32_t token_tile, int32_t* row_prefix, int32_t* tile_prefix, void* cuda_stream);

/* Bytes of the packed weight image (codes and scale words) for an (N, K) weight. */
size_t b200dq_packed_weight_bytes(int32_t N, int32_t K, int32_t group_size, int32_t weight_format);

/* Offline layout transform, on the device. Input: natural (N, K*bits/8)
 * little-endian codes (element k in bits [(k % epb)*bits ...] of byte k / epb, the
 * layout of general_compress, examples/dequantize_gemm/quantize/utils.py:50-67)
 * plus, per format:
 *   U4_SZ    : scales and zeros (N, K/group_size) in the activation dtype
 *              (zeros may be NULL = fixed zero-point 8); weight = (q - z) * s, the
 *              reference's "original" zeros mode (quantize/lop3.py:684-689). The image
 *              keeps s * 2^6 (bf16) or s * 2^9 (fp16) in the activation dtype: fp16
 *              scales must stay below 128 in magnitude or they overflow to infinity;
 *   FP4_E8M0 : `scales` = (N, K/32) exponent bytes; zeros unused;
 *   others   : scales and zeros unused (NULL).
 * Output: the tiled, pre-interleaved image the GEMM streams with one bulk copy
 * per stage (two k-blocks of codes followed by their scale words). Plays the role
 * of interleave_weight (quantize/utils.py:71-125) plus the tile re-ordering the
 * reference leaves to TMA/layout inference. K is padded to a whole stage. */
int b200dq_pack_weights(const void* q_natural, const void* scales, const void* zeros, void* wp, int32_t N,
                        int32_t K, int32_t group_size, int32_t weight_format, int32_t act_type,
                        void* cuda_stream);

/* Per-token absmax int8 quantisation of (M, K) f16/bf16 activations: scale[m] =
 * 127 / max|x[m,:]| (max clamped at 1e-5), q = round(x * scale) clamped to [-128, 127].
 * Replaces BitLinear.activation_quant, examples/bitnet-1.58b/utils_quant.py:156-163. */
int b200dq_absmax_quant_int8(const void* x, void* q, float* scale, int32_t M, int32_t K, int32_t act_type,
                             void* cuda_stream);

/* (M, K) f16/bf16 activations -> MXFP4 at block 32 along K: scale_bytes (M, K/32) e8m0 bytes
 * with scale = 2^ceil(log2(amax / 6)) (amax clamped below at 6 * 2^-126), codes (M, K/2) bytes
 * holding the e2m1 codes of x / scale, round to nearest even, the even k in the low nibble; a
 * negative value that rounds to zero keeps its sign bit. K % 32 == 0. Replaces the activation
 * quantiser of examples/deepseek_v4/act_quant.py:112-164 (whose cast to float4_e2m1fn is the
 * same hardware conversion; its torch reference, :249-268, breaks ties downwards instead). */
int b200dq_quant_mxfp4(const void* x, void* codes, void* scale_bytes, int32_t M, int32_t K, int32_t act_type,
                       int32_t sf_blocked, void* cuda_stream);
/* With sf_blocked != 0 (K % 128 == 0) the scale bytes are written in the 128 x 4 blocked layout
 * of b200dq_gemm_mxfp4_native instead of row-major: byte kb % 4 of the uint32 word
 * [m / 128][kb / 4][m % 32][(m % 128) / 32]; the buffer holds ceil(M / 128) * 128 * K / 32 bytes and
 * the rows beyond M must have been zeroed by the caller. */

/* Native MXFP4 GEMM: C[M, N] = A * W^T with both operands as e2m1 codes (M, K/2) and (N, K/2)
 * bytes, row-major, the even k in the low nibble, each with one e8m0 scale per 32 K elements in
 * the 128 x 4 blocked layout above (for W: rows are weight rows, padded with zero words to a
 * multiple of 128), multiplied by tcgen05.mma kind::mxf4.block_scale with fp32 accumulation.
 * K % 256 == 0; out_type f16, bf16 or f32; no scratch. The reference has the pieces
 * (src/tl_templates/cuda/tcgen_05.h:123-178, src/op/tcgen5_meta.h:273-335, the mainloop of
 * examples/deepseek_v4/fp8_fp4_gemm_1d1d_sm100.py:18-185) but no packed-fp4 kind. */
/* Calibration, not a GEMM: launches one CTA per SM that issues `mmas` back-to-back
 * tcgen05.mma instructions of shape 128 x 256 x (32 bytes of K) from shared memory and waits for
 * them. kind 0: bf16 (kind::f16), 1: int8 (kind::i8), 2: MXFP4 (kind::mxf4.block_scale). *ops
 * receives the arithmetic operations of the launch; the caller times it with events on the
 * same stream. The rate is the tensor-pipe ceiling the integer and fp4 results are quoted
 * against. No reference counterpart (its benchmarks quote nominal peaks). */
int b200dq_tensor_peak(int32_t kind, int32_t mmas, double* ops, void* cuda_stream);

int b200dq_gemm_mxfp4_native(const void* a_codes, const void* a_sf, const void* w_codes, const void* w_sf, void* c,
                             int32_t M, int32_t N, int32_t K, int32_t out_type, void* cuda_stream);

/* Mixture-of-experts combine: out[t, :] = sum over s < top_k of weights[t*top_k + s] *
 * y[row_of[t*top_k + s], :], fp32 accumulation in slot order, one rounding to the row type.
 * Deterministic stand-in for the scatter-add of
 * examples/fusedmoe/example_fusedmoe_torch.py:83-91. H % 8 == 0. */
int b200dq_moe_combine(const void* y, const int64_t* row_of, const float* weights, void* out, int64_t tokens,
                       int32_t top_k, int32_t H, int32_t act_type, void* cuda_stream);

/* Signed int4 values, two per byte with the even index in the low nibble (pack_int4,
 * examples/gemm_int4/example_tilelang_gemm_int4.py:59-67) -> one int8 each. Puts packed
 * int4 activations in front of the int8 tensor-core GEMM (tcgen05 has no int4 kind). */
int b200dq_unpack_int4_to_int8(const void* packed, void* out, int64_t num_elems, void* cuda_stream);

/* out[r, c] = silu(h[r, c]) * h[r, H + c] for h of shape (rows, 2H), f16/bf16, fp32 math.
 * The activation between the two expert GEMMs,
 * examples/fusedmoe/example_fusedmoe_torch.py:8-23. */
int b200dq_silu_mul(const void* h, void* out, int64_t rows, int32_t H, int32_t act_type, void* cuda_stream);

/* No counterpart in the reference. The same GEMM as b200dq_gemm (same validation,
 * schedule and kernel choice, small-M kernel included: both run one internal routine) for
 * callers that
 * cannot allocate device memory at all -- code running where cudaMalloc is off
 * limits (inside another framework's allocator callbacks, under a memory pool that
 * owns the whole device, in a process that was handed pre-mapped buffers only). The
 * stream-K partial tiles go to a fixed 40 MiB array compiled into the library's
 * device image instead of `workspace` (args->workspace and workspace_bytes are
 * ignored); every GPU that loads the library holds those 40 MiB until the process
 * exits. Inputs and the output are still the caller's.
 *   - A problem whose schedule needs more than 40 MiB of scratch is rejected with an
 *     error (no schedule on a 148-SM part needs more than 38,797,312 bytes).
 *   - The first call on a device looks up the array's device address and the
 *     device's properties; make that first call outside any stream capture.
 *   - It calls no cudaMalloc, cudaFree or allocating library routine, and it does
 *     not need b200dq_init. If b200dq_init has run on the device, waits that give
 *     up are recorded in its status word; otherwise they are bounded but unrecorded.
 *   - All calls share the one array, which keeps whatever the last call left in it.
 *     Nothing in it has to start at zero (a launch reads only slots it wrote), but two
 *     calls that overlap on the GPU -- different streams, or graphs replayed
 *     concurrently -- race on it: serialise them. */
int b200dq_gemm_static_scratch(const b200dq_gemm_args* args, void* cuda_stream);

/* No counterpart in the reference. The size check of b200dq_gemm_static_scratch alone,
 * for a part with `sm_count` SMs; needs no GPU and launches nothing. Stores the scratch
 * bytes the call's schedule needs and the capacity of the static array (either pointer
 * may be NULL). Returns 0 if the call would fit, -1 (with the same message the entry
 * point gives) if it would be rejected as too large or the sizes are invalid. */
int b200dq_static_scratch_check(const b200dq_gemm_args* args, int32_t sm_count, size_t* needed_bytes,
                                size_t* capacity_bytes);

/* Reads the device status word of the current device (synchronises `stream`).
 * Returns 0 if no kernel recorded an error since the last reset, else -1 with a
 * message naming the wait that gave up; resets the word. */
int b200dq_check_status(void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* B200DQ_H_ */
