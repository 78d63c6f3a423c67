"""CPU oracle for the low-bit dequantize-GEMM path. TEST INFRASTRUCTURE ONLY.

Nothing in the product (``tilelang_b200/``) imports this file; it is used by
``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` as the checker and the timed CPU
reference, never as a fallback.

Every function restates, on CPU with torch/numpy, what the reference
(tile-ai/tilelang) computes in its own torch ``ref_program``s and host-side
packers; the cited lines are paths inside the reference repository. The
restatements are pinned against outputs of the reference's importable helpers
(``tests/golden/*.npz`` made by ``tests/golden/make_golden.py``) and against the
known-answer vectors its tests hold. Parity at the ``bitblas`` boundary of the
BitNet *model* (``examples/bitnet-1.58b/utils_quant.py:51-67``; the package is
neither vendored nor version-pinned in the reference) is unpinned; the in-tree
int8 x int2 kernels (``kernel_benchmark/``) are the specification used here.
"""
from __future__ import annotations

import numpy as np
import torch

# ---------------------------------------------------------------------------
# codecs
# ---------------------------------------------------------------------------

# e2m1 magnitudes, code = s e1 e0 m. quantize/nvfp4.py:18-35 (_FP4_E2M1_VALUES)
# and examples/deepseek_v4/fp8_fp4_gemm_1d1d_sm100.py:217-234 list the same table.
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                        -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def general_compress(w: np.ndarray, source_bits: int = 4) -> np.ndarray:
    """Pack integer codes little-endian within each byte: element k goes to bits
    [(k % epb) * bits, ...) of byte k // epb.
    examples/dequantize_gemm/quantize/utils.py:50-67 (torch) and
    examples/bitnet-1.58b/kernel_benchmark/tilelang_bitnet_158_int8xint2_decode.py:178-194 (numpy)."""
    epb = 8 // source_bits
    w = np.asarray(w).astype(np.int64)
    assert w.shape[-1] % epb == 0
    mask = (1 << source_bits) - 1
    w = (w & mask).reshape(*w.shape[:-1], w.shape[-1] // epb, epb)
    shifts = (np.arange(epb, dtype=np.int64) * source_bits)
    return (w << shifts).sum(-1).astype(np.uint8)


def general_decompress(q: np.ndarray, source_bits: int = 4) -> np.ndarray:
    """Inverse of :func:`general_compress` (unsigned codes)."""
    epb = 8 // source_bits
    q = np.asarray(q).view(np.uint8).astype(np.int64)
    shifts = (np.arange(epb, dtype=np.int64) * source_bits)
    mask = (1 << source_bits) - 1
    out = (q[..., None] >> shifts) & mask
    return out.reshape(*q.shape[:-1], q.shape[-1] * epb).astype(np.uint8)


def interleave_weight(qweight: np.ndarray, nbits: int = 4, target_dtype: str = "float16") -> np.ndarray:
    """The reference's offline permutation for its LOP3 decoders: inside every
    32-bit word, element e moves to bit (e % G) * S + (e // G) * nbits with
    S = 16, G = 2 for a 16-bit target and S = 8, G = 4 for int8, plus the extra
    byte/nibble shuffles for (1-bit, int8), (2-bit, fp16) and (1-bit, fp16).
    examples/dequantize_gemm/quantize/utils.py:71-125."""
    assert target_dtype in ("float16", "int8")
    q = np.ascontiguousarray(qweight).view(np.uint8).view(np.uint32).astype(np.uint64)
    new = np.zeros_like(q)
    bits_stride = 8 if target_dtype == "int8" else 16
    mask = (1 << nbits) - 1
    num_groups = 32 // bits_stride
    elems_per_group = bits_stride // nbits
    for i in range(num_groups):
        for j in range(elems_per_group):
            offset = i * elems_per_group + j
            shift = (offset % num_groups) * bits_stride + (offset // num_groups) * nbits
            new |= ((q >> np.uint64(nbits * offset)) & np.uint64(mask)) << np.uint64(shift)
    new &= np.uint64(0xFFFFFFFF)

    def u(x):
        return np.uint64(x)

    if nbits == 1 and target_dtype == "int8":
        n16 = new & u(0xF0F00F0F)
        n16 |= ((new & u(0x000000F0)) >> u(4)) << u(16)
        n16 |= ((new & u(0x0000F000)) >> u(12)) << u(24)
        n16 |= ((new & u(0x000F0000)) >> u(16)) << u(4)
        n16 |= ((new & u(0x0F000000)) >> u(24)) << u(12)
        new = n16
    elif nbits == 2 and target_dtype == "float16":
        n8 = new & u(0xFF0000FF)
        n8 |= ((new & u(0x0000FF00)) >> u(8)) << u(16)
        n8 |= ((new & u(0x00FF0000)) >> u(16)) << u(8)
        new = n8
    elif nbits == 1 and target_dtype == "float16":
        n8 = new & u(0xF000000F)
        n8 |= ((new & u(0x000000F0)) >> u(4)) << u(8)
        n8 |= ((new & u(0x00000F00)) >> u(8)) << u(16)
        n8 |= ((new & u(0x0000F000)) >> u(12)) << u(24)
        n8 |= ((new & u(0x000F0000)) >> u(16)) << u(4)
        n8 |= ((new & u(0x00F00000)) >> u(20)) << u(12)
        n8 |= ((new & u(0x0F000000)) >> u(24)) << u(20)
        new = n8
    return new.astype(np.uint32).view(np.uint8).reshape(np.asarray(qweight).shape).view(np.int8)


def pack_int4(t: np.ndarray) -> np.ndarray:
    """Signed int4 values in [-8, 7], two per byte, low nibble = even index.
    examples/gemm_int4/example_tilelang_gemm_int4.py:59-67."""
    t = np.asarray(t).astype(np.int16)
    assert t.shape[-1] % 2 == 0
    return ((t[..., ::2] & 0x0F) | ((t[..., 1::2] & 0x0F) << 4)).astype(np.uint8).view(np.int8)


def unpack_u4(qB: torch.Tensor) -> torch.Tensor:
    """byte b -> (b & 15, b >> 4) along K.
    examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:11-13."""
    q = qB.to(torch.uint8)
    return torch.stack((q & 0x0F, q >> 4), dim=-1).reshape(q.shape[0], q.shape[1] * 2)


def sext4(q: torch.Tensor) -> torch.Tensor:
    """Two's-complement sign extension of 4-bit codes: (i4 << 4) >> 4 on int8.
    examples/dequantize_gemm/example_dequant_gemm_w4a8.py:10-21, 68-74."""
    return ((q.to(torch.int16) ^ 8) - 8).to(torch.int8)


def decode_fp4_simple(qB: torch.Tensor, scale_size=None, Scale=None) -> torch.Tensor:
    """The reference's *simple* fp4 -> bf16 decoder: sign, exponent = e + 126,
    mantissa = m << 6 for every code, i.e. 0.5, 0.75, 1, 1.5, 2, 3, 4, 6 with no
    zero and no subnormal; an optional per-block exponent is added and the sum is
    clamped to 255. examples/dequantize_gemm/dequantize_utils.py:57-84."""
    assert qB.dim() == 2 and qB.dtype == torch.uint8
    N, Kb = qB.shape
    f4 = torch.stack((qB & 0x0F, qB >> 4), dim=-1).reshape(N, Kb * 2).to(torch.int16)
    sign = (f4 >> 3) * -32768
    exponent = ((f4 & 6) >> 1) + 126
    if scale_size is not None:
        idx = torch.arange(Kb * 2) // scale_size
        exponent = torch.clamp(exponent + Scale[:, idx].to(torch.int16), max=255)
    mantissa = (f4 & 1) << 6
    return (sign + (exponent << 7) + mantissa).view(torch.bfloat16)


def decode_fp4_twiddled(qB: torch.Tensor) -> torch.Tensor:
    """The reference's *twiddled* layout: every byte pair W = (b[2i] << 8) | b[2i+1]
    holds four true-e2m1 values at bit positions chosen for shift-and-mask
    decoding; the masked pattern times 2^126 is the value.
    examples/dequantize_gemm/dequantize_utils.py:4-54."""
    assert qB.dim() == 2 and qB.dtype == torch.uint8
    N, Kb = qB.shape
    v0 = qB[:, 0::2].to(torch.int32)
    v1 = qB[:, 1::2].to(torch.int32)
    w = ((v0 << 8) | v1).repeat_interleave(4, dim=1)
    pos = torch.arange(Kb * 2) % 4
    mask, m1, m2, m3 = 0b1000000111000000, 0b1000000000000000, 0b0000000110000000, 0b0000000001000000
    r0 = w & mask
    r1 = (w << 3) & mask
    r2 = (w << 6) & mask
    r3 = ((w << 1) & m1) | ((w >> 3) & m2) | ((w >> 7) & m3)
    bits = torch.where(pos == 0, r0, torch.where(pos == 1, r1, torch.where(pos == 2, r2, r3)))
    return (bits & 0xFFFF).to(torch.uint16).view(torch.bfloat16) * (2.0 ** 126)


def decode_fp4_e2m1(qB: torch.Tensor) -> torch.Tensor:
    """True e2m1 in the natural nibble order (low nibble = even k), fp32.
    quantize/nvfp4.py:159-177 (decode_packed_fp4_e2m1) with the LUT of :18-35."""
    codes = unpack_u4(qB).to(torch.int64)
    return torch.from_numpy(E2M1_VALUES)[codes]


def encode_fp4_e2m1(x: np.ndarray) -> np.ndarray:
    """Nearest e2m1 code by the thresholds .25/.75/1.25/1.75/2.5/3.5/5 (a value on a
    threshold takes the larger magnitude); the sign bit is set only for a non-zero
    magnitude. quantize/nvfp4.py:120-138."""
    x = np.nan_to_num(np.asarray(x, dtype=np.float32), nan=0.0, posinf=6.0, neginf=-6.0)
    a = np.abs(x)
    mag = np.zeros(a.shape, dtype=np.uint8)
    for i, t in enumerate([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]):
        mag = np.where(a >= t, i + 1, mag).astype(np.uint8)
    sign = ((x < 0) & (mag != 0)).astype(np.uint8) << 3
    return (mag | sign).astype(np.uint8)


# ---------------------------------------------------------------------------
# dequantisation rules
# ---------------------------------------------------------------------------

def dequant_w4_group(qB: torch.Tensor, scales, zeros, group_size: int, dtype: torch.dtype,
                     zeros_mode: str = "original") -> torch.Tensor:
    """W = (q - z) * s computed in fp32 and rounded once to the activation dtype:
    the reference's "original" zeros mode (quantize/lop3.py:684-689; symmetric case
    z = 8 in quantize/utils.py:29-30), dequantised to in_dtype before the matmul as
    its intrinsics and oracles do. ``zeros=None`` is the fixed zero-point 8;
    ``scales=None`` leaves the raw code q. ``zeros_mode`` "rescale" is q * s - z
    (lop3.py:233-271) and "quantized" (q - qz) * s with integer zero-points
    (lop3.py:326-363), under the same compute-in-fp32, round-once rule."""
    q = unpack_u4(qB).to(torch.float32)
    if scales is None:
        return q.to(dtype)
    g = group_size if group_size and group_size > 0 else q.shape[1]
    s = scales.to(torch.float32).repeat_interleave(g, dim=1)
    z = (zeros.to(torch.float32).repeat_interleave(g, dim=1) if zeros is not None else 8.0)
    if zeros_mode == "rescale":
        return (q * s - z).to(dtype)
    if zeros_mode not in ("original", "quantized"):
        raise ValueError(zeros_mode)
    return ((q - z) * s).to(dtype)


def dequant_mxfp4(qB: torch.Tensor, scale_bytes: torch.Tensor, exp_bias: int = 127, fmt: str = "e2m1",
                  scale_size: int = 32) -> torch.Tensor:
    """bf16 weight = D(code) * 2^(scale - exp_bias), per block of ``scale_size`` K.
    fmt "e2m1": true e2m1, natural nibbles. fmt "twiddled": true e2m1 in the
    reference's twiddled byte layout. fmt "simple": the reference's no-subnormal
    decoder. The reference multiplies by ``2 ** Scale`` with no bias
    (example_dequant_gemm_bf16_mxfp4_hopper.py:397, 420, 444), which is
    ``exp_bias=0``; OCP e8m0 is ``exp_bias=127``."""
    if fmt == "e2m1":
        w = decode_fp4_e2m1(qB)
    elif fmt == "twiddled":
        w = decode_fp4_twiddled(qB).to(torch.float32)
    elif fmt == "simple":
        w = decode_fp4_simple(qB).to(torch.float32)
    else:
        raise ValueError(fmt)
    e = scale_bytes.to(torch.float32) - float(exp_bias)
    mult = torch.pow(torch.tensor(2.0), e).repeat_interleave(scale_size, dim=1)
    return (w * mult).to(torch.bfloat16)


# ---------------------------------------------------------------------------
# ref_programs
# ---------------------------------------------------------------------------

def _matmul_f32(A: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
    return torch.matmul(A.to(torch.float32), W.to(torch.float32).T)


def ref_w4a16_noscale(A: torch.Tensor, qB: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """C = A @ unpack_u4(qB)^T in fp32, cast.
    examples/dequantize_gemm/example_dequant_gemm_fine_grained.py:125-131."""
    B = unpack_u4(qB).to(torch.float16 if A.dtype == torch.float16 else A.dtype)
    return _matmul_f32(A, B).to(out_dtype)


def ref_w4a16(A: torch.Tensor, qB: torch.Tensor, scales, zeros, group_size: int,
              out_dtype: torch.dtype, zeros_mode: str = "original") -> torch.Tensor:
    """Dequantise to the activation dtype, fp32 matmul, cast (group scale/zero rule above)."""
    W = dequant_w4_group(qB, scales, zeros, group_size, A.dtype, zeros_mode)
    return _matmul_f32(A, W).to(out_dtype)


def ref_mxfp4(A: torch.Tensor, qB: torch.Tensor, Scale: torch.Tensor, Bias=None, exp_bias: int = 127,
              fmt: str = "e2m1") -> torch.Tensor:
    """examples/dequantize_gemm/example_dequant_gemm_bf16_mxfp4_hopper.py:381-475
    (ref_program_twiddling / ref_program_simple, with and without bias)."""
    W = dequant_mxfp4(qB, Scale, exp_bias, fmt)
    C = _matmul_f32(A, W)
    if Bias is not None:
        C = C + Bias.to(torch.float32)
    return C.to(torch.bfloat16)


def ref_fp4_noscale(A: torch.Tensor, qB: torch.Tensor, fmt: str = "simple", transpose_out: bool = True):
    """fp16/bf16 x fp4 without scale; the reference's kernel writes C^T (N, M).
    examples/dequantize_gemm/example_dequant_gemm_fp4_hopper.py:32-41, 223-228."""
    if fmt == "simple":
        W = decode_fp4_simple(qB).to(torch.float32)
    else:
        W = decode_fp4_e2m1(qB)
    C = _matmul_f32(A, W.to(A.dtype)).to(A.dtype)
    return C.T.contiguous() if transpose_out else C


def ref_w4a8(A: torch.Tensor, qB: torch.Tensor) -> torch.Tensor:
    """Ct (N, M) int32 = sext4(B) @ A^T. The reference computes it through a float32
    matmul (example_dequant_gemm_w4a8.py:68-82); here the product is exact int64."""
    B = sext4(unpack_u4(qB))
    C = torch.matmul(A.to(torch.int64), B.to(torch.int64).T)
    return C.to(torch.int32).T.contiguous()


def ref_int4_gemm(A_packed: torch.Tensor, B_packed: torch.Tensor) -> torch.Tensor:
    """C int32 = A @ B^T with both operands signed int4, two per byte.
    examples/gemm_int4/example_tilelang_gemm_int4.py:92-101."""
    a = sext4(unpack_u4(A_packed.view(torch.uint8)))
    b = sext4(unpack_u4(B_packed.view(torch.uint8)))
    return torch.matmul(a.to(torch.int64), b.to(torch.int64).T).to(torch.int32)


# ---- BitNet b1.58 ----------------------------------------------------------

def bitnet_weight_quant(weight: torch.Tensor):
    """s = 1 / mean|W| (clamped at 1e-5); W_t = round(W * s).clamp(-1, 1) as int8.
    examples/bitnet-1.58b/utils_quant.py:149-154 (and :16-21)."""
    w = weight.float()
    s = 1 / w.abs().mean().clamp(min=1e-5)
    return (w * s).round().clamp(-1, 1).to(torch.int8), s


def bitnet_activation_quant(x: torch.Tensor, num_bits: int = 8):
    """Per-token absmax: s = 127 / max|x| (clamped at 1e-5); q = round(x * s).clamp(-128, 127).
    examples/bitnet-1.58b/utils_quant.py:156-163."""
    xf = x.float()
    qn, qp = -(2 ** (num_bits - 1)), 2 ** (num_bits - 1) - 1
    s = qp / xf.abs().max(dim=-1, keepdim=True).values.clamp(min=1e-5)
    return (xf * s).round().clamp(qn, qp).to(torch.int8), s


def ref_bitnet_int32(A_q: torch.Tensor, W_t: torch.Tensor) -> torch.Tensor:
    """int32 = A_q @ W_t^T, exact.
    examples/bitnet-1.58b/kernel_benchmark/tilelang_bitnet_158_int8xint2_decode.py:245-258
    checks the kernel against a float32 matmul of the same integers."""
    return torch.matmul(A_q.to(torch.int64), W_t.to(torch.int64).T).to(torch.int32)


def ref_bitnet_linear(A_q, s_act, W_t, s_w, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """out = acc / s_act / s_w, cast (two divisions, in this order).
    examples/bitnet-1.58b/utils_quant.py:165-170 (post_quant_process) and
    :182-197 (forward_fp32_simulated)."""
    acc = ref_bitnet_int32(A_q, W_t).to(torch.float32)
    out = acc / s_act.to(torch.float32).reshape(-1, 1)
    out = out / torch.as_tensor(s_w, dtype=torch.float32)
    return out.to(out_dtype)


# ---- bf16 -> MXFP4 activation quantiser --------------------------------------

def mxfp4_act_quant(x: torch.Tensor, block_size: int = 32, ties: str = "down"):
    """Per row and block: scale = 2^ceil(log2(amax / 6)) with amax clamped below at 6 * 2^-126,
    y = clamp(x / scale, -6, 6), code = nearest e2m1 value (index + 8 for negative y).
    examples/deepseek_v4/act_quant.py:249-268 (``fp4_act_quant_ref``), whose argmin breaks ties
    towards the smaller magnitude (``ties="down"``); its kernel (:112-164) casts to
    float4_e2m1fn, which rounds ties to even (``ties="even"``). Returns (codes (M, K) uint8,
    scale (M, K / block) float32)."""
    M, N = x.shape
    xf = x.float().reshape(M, N // block_size, block_size)
    amax = xf.abs().amax(dim=-1).clamp(min=6.0 * (2.0 ** -126))
    scale = torch.pow(2.0, torch.ceil(torch.log2(amax / 6.0)))
    y = (xf / scale.unsqueeze(-1)).clamp(-6.0, 6.0).reshape(M, N)
    vals = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    d = (y.abs().unsqueeze(-1) - vals).abs()
    idx = d.argmin(dim=-1)                                   # first minimum: the smaller magnitude on a tie
    if ties == "even":
        nxt = (idx + 1).clamp(max=7)
        tie = d.gather(-1, nxt.unsqueeze(-1)).squeeze(-1) == d.gather(-1, idx.unsqueeze(-1)).squeeze(-1)
        idx = torch.where(tie & (idx % 2 == 1) & (nxt != idx), nxt, idx)
    elif ties != "down":
        raise ValueError(ties)
    return torch.where(y < 0, idx + 8, idx).to(torch.uint8), scale


def ref_low_bits_a16(A: torch.Tensor, qB: torch.Tensor, bits: int, scales, zeros, group_size: int, signed: bool,
                     out_dtype=torch.float16) -> torch.Tensor:
    """1- or 2-bit integer weights on 16-bit activations: codes little-endian in each byte
    (general_compress, quantize/utils.py:50-67); weight = q (unsigned), q - 2 (signed 2-bit) or
    2 q - 1 (signed 1-bit) as the reference's decoders produce it (quantize/lop3.py:424-463,
    679-745: sub 1024 [+ add, add -1]), then ``* scale`` (:465-530, 748-810) or
    ``(q - zeros) * scale`` (:532-590 "original"); the weight is rounded to the activation dtype
    before the fp32 matmul, as in the 4-bit ref_programs."""
    N = qB.shape[0]
    per = 8 // bits
    q = qB.to(torch.int32)
    codes = torch.stack([(q >> (bits * i)) & ((1 << bits) - 1) for i in range(per)], dim=-1).reshape(N, -1).float()
    K = codes.shape[1]
    if signed:
        codes = codes - 2.0 if bits == 2 else 2.0 * codes - 1.0
    if scales is not None:
        s = scales.float().repeat_interleave(group_size, dim=1)
        if zeros is not None:
            codes = (codes - zeros.float().repeat_interleave(group_size, dim=1)) * s
        else:
            codes = codes * s
    W = codes.to(A.dtype).float()
    assert K == A.shape[1]
    return torch.matmul(A.float(), W.T).to(out_dtype)


NF4_LEVELS = (-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
              -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
              0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
              0.7229568362236023, 1.0)


def ref_lut4(A: torch.Tensor, qB: torch.Tensor, scales: torch.Tensor, group_size: int, table=NF4_LEVELS,
             out_dtype=torch.bfloat16) -> torch.Tensor:
    """Codebook weights (NF4): weight = table[q] * scale, both rounded to the activation dtype and
    the product rounded once more, as a dequantise-then-matmul ref_program in that dtype does
    (the structure of example_dequant_gemm_fine_grained.py:84-90; the reference has no NF4 code).
    Codes two per byte, even k in the low nibble."""
    q = qB.to(torch.int64)
    codes = torch.stack((q & 15, q >> 4), dim=-1).reshape(qB.shape[0], -1)
    t = torch.tensor(table, dtype=torch.float32).to(A.dtype)
    W = (t[codes].float() * scales.float().repeat_interleave(group_size, dim=1)).to(A.dtype)
    return torch.matmul(A.float(), W.float().T).to(out_dtype)


def ref_mxfp4_native(A: torch.Tensor, qB: torch.Tensor, scale_bytes: torch.Tensor, out_dtype=torch.bfloat16):
    """Both operands MXFP4: the activation is re-quantised per row and 32-block the way the
    reference's kernel does (:func:`mxfp4_act_quant`, ties to even), then
    C = dequant(A_q) @ dequant(W)^T in fp32 -- what a block-scaled fp4 x fp4 tensor-core GEMM
    computes up to the order of the fp32 additions (every product of two e2m1 values and two
    powers of two is exact). The block-scaled mainloop this stands for is
    examples/deepseek_v4/fp8_fp4_gemm_1d1d_sm100.py:18-185 (fp8 x fp4 there)."""
    codes, scale = mxfp4_act_quant(A, 32, ties="even")
    vals = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])
    a = vals[codes.long()] * scale.repeat_interleave(32, dim=1)
    w = dequant_mxfp4(qB, scale_bytes, 127, "e2m1").float()
    return torch.matmul(a, w.T).to(out_dtype)


# ---- MoE -------------------------------------------------------------------

def moe_route(logits: torch.Tensor, top_k: int):
    """softmax over experts then top-k (unsorted), scores are the softmax values.
    examples/fusedmoe/example_fusedmoe_torch.py:26-40."""
    scores = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(scores, top_k, dim=-1, sorted=False)
    return w, idx


def ref_moe_w4a16(x, logits, top_k, w1_q, w1_s, w2_q, w2_s, group_size: int):
    """Per expert y = W2( silu(g) * u ), [g, u] = W1(x) split in halves (gate first),
    each matmul by the W4A16 oracle with the fixed zero-point 8; outputs are
    combined as a score-weighted sum in fp32 and cast to the activation dtype.
    examples/fusedmoe/example_fusedmoe_torch.py:8-23, 65-91;
    examples/grouped_gemm/example_grouped_gemm_fwd.py:8-36."""
    T = x.shape[0]
    E = w1_q.shape[0]
    weights, idx = moe_route(logits, top_k)
    out = torch.zeros(T, w2_q.shape[1], dtype=torch.float32)
    for e in range(E):
        tok, slot = torch.where(idx == e)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        h = ref_w4a16(xe, w1_q[e], w1_s[e], None, group_size, x.dtype)
        half = h.shape[1] // 2
        act = (torch.nn.functional.silu(h[:, :half].float()) * h[:, half:].float()).to(x.dtype)
        y = ref_w4a16(act, w2_q[e], w2_s[e], None, group_size, x.dtype)
        out.index_add_(0, tok, y.float() * weights[tok, slot].unsqueeze(1))
    return out.to(x.dtype)


# ---------------------------------------------------------------------------
# acceptance rule
# ---------------------------------------------------------------------------

def mismatch_ratio(x: torch.Tensor, ref: torch.Tensor, rtol: float = 1e-2, atol: float = 1e-2) -> float:
    """Fraction of elements with |x - ref| > atol + rtol * |ref|; the reference
    accepts up to 1 % of them (tilelang/profiler/__init__.py:104-162,
    tilelang/utils/tensor.py:205-293)."""
    d = (x.double() - ref.double()).abs()
    return float((d > atol + rtol * ref.double().abs()).double().mean())


def max_rel_error(x: torch.Tensor, ref: torch.Tensor, floor_frac: float = 1.0) -> float:
    """max |x - ref| / max(|ref|, floor_frac * rms(ref)): the relative error, measured against
    (a fraction of) the typical output magnitude for elements that happen to fall near zero
    (a plain |x - ref| / |ref| is unbounded there for any rounded output)."""
    r = ref.double()
    floor = floor_frac * float(r.pow(2).mean().sqrt())
    if floor == 0.0:
        return float((x.double() - r).abs().max())
    return float(((x.double() - r).abs() / torch.clamp(r.abs(), min=floor)).max())
