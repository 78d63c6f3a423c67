"""Block-scaled 4-bit float formats: e2m1 codes, UE4M3 / UE8M0 scale codecs, scale-factor
layouts, and the bf16 -> MXFP4 / NVFP4 quantisers (torch, any device).

What the reference keeps in examples/dequantize_gemm/quantize/nvfp4.py (e2m1 encode / pack /
decode :120-177, UE4M3 codec :61-117, the 128-row scale-word swizzle :216-300,
``quantize_bf16_to_nvfp4_blockscaled`` :469-539), examples/deepseek_v4/act_quant.py (the
bf16 -> MXFP4 activation quantiser at block 32: kernel :112-164, torch reference :249-268) and
examples/deepseek_v4/fp8_fp4_gemm_1d1d_sm100.py (``quantize_mxfp4_with_packed_ue8m0`` :264-282,
group-major scale words :198-205), written here from the formats' definitions: every encoder
is a table search over the representable values. ``ops.quant_mxfp4`` is the CUDA version of
:func:`quantize_mxfp4` for activations on the hot path.
"""
from __future__ import annotations

import torch

E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_E2M1_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
E2M1_MAX = 6.0
TIE_RULES = ("up", "down", "even")


# ------------------------------------------------------------------------------------------
# e2m1 codes: bit 3 sign, bits 2..0 index into E2M1_MAGNITUDES
# ------------------------------------------------------------------------------------------

def e2m1_encode(x: torch.Tensor, ties: str = "up", signed_zero: bool = False) -> torch.Tensor:
    """Nearest e2m1 code of every element (uint8, 0..15); magnitudes above 6 saturate, NaN -> 0.

    ``ties`` says where a value exactly between two codes goes: "up" to the larger magnitude
    (the thresholds of nvfp4.py:120-138), "down" to the smaller (an argmin over the value
    table, act_quant.py:215-228), "even" to the code with an even index (what a hardware
    round-to-nearest-even conversion does). ``signed_zero`` keeps the sign bit on a negative
    input that rounds to zero (act_quant.py does; nvfp4.py does not)."""
    if ties not in TIE_RULES:
        raise ValueError(f"ties must be one of {TIE_RULES}")
    v = torch.nan_to_num(x.to(torch.float32), nan=0.0, posinf=E2M1_MAX, neginf=-E2M1_MAX)
    a = v.abs().unsqueeze(-1)
    mids = torch.tensor(_E2M1_MIDPOINTS, dtype=torch.float32, device=x.device)
    above, at = a > mids, a == mids
    if ties == "up":
        passed = above | at
    elif ties == "down":
        passed = above
    else:   # the tie at midpoint i is between codes i and i + 1: take the even one
        odd_below = (torch.arange(7, device=x.device) % 2) == 1
        passed = above | (at & odd_below)
    mag = passed.sum(-1).to(torch.int32)
    neg = v < 0 if signed_zero else (v < 0) & (mag != 0)
    return (mag | (neg.to(torch.int32) << 3)).to(torch.uint8)


def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    """Codes (uint8, one per element) -> float32 values."""
    table = torch.tensor(E2M1_MAGNITUDES + tuple(-m for m in E2M1_MAGNITUDES), dtype=torch.float32, device=codes.device)
    return table[(codes.to(torch.int64) & 15)]


def e2m1_pack(codes: torch.Tensor) -> torch.Tensor:
    """Two codes per byte along the last dimension, the even index in the low nibble."""
    if codes.shape[-1] % 2:
        raise ValueError("e2m1_pack: the last dimension must be even")
    c = codes.to(torch.uint8) & 15
    return (c[..., 0::2] | (c[..., 1::2] << 4)).contiguous()


def e2m1_unpack(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`e2m1_pack`: (..., K/2) bytes -> (..., K) codes."""
    p = packed.contiguous().view(torch.uint8)
    return torch.stack((p & 15, p >> 4), dim=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)


# ------------------------------------------------------------------------------------------
# scale codecs
# ------------------------------------------------------------------------------------------

def _ue4m3_table(device) -> torch.Tensor:
    """Values of the codes 0x00 .. 0x7E (0x7F is NaN), increasing with the code."""
    code = torch.arange(127, dtype=torch.int32, device=device)
    e, m = code >> 3, (code & 7).to(torch.float32)
    normal = torch.ldexp(1.0 + m / 8.0, e - 7)
    return torch.where(e == 0, m * 2.0 ** -9, normal)


def ue4m3_decode(scale_bytes: torch.Tensor) -> torch.Tensor:
    """Unsigned e4m3 scale bytes (bias 7, no sign: bit 7 is ignored) -> float32; 0x7F -> NaN."""
    if scale_bytes.dtype != torch.uint8:
        raise TypeError("ue4m3_decode: uint8 bytes expected")
    idx = scale_bytes.to(torch.int64) & 0x7F
    table = torch.cat((_ue4m3_table(scale_bytes.device), torch.tensor([float("nan")], device=scale_bytes.device)))
    return table[idx]


def ue4m3_encode(values: torch.Tensor, rounding: str = "nearest", min_positive: bool = False) -> torch.Tensor:
    """Non-negative floats -> unsigned e4m3 bytes. "nearest" rounds to the nearest code (ties to
    the larger), "ceil" to the smallest code not below the value; values above 448 saturate at
    0x7E, negatives and NaN give 0. ``min_positive`` keeps a positive value from becoming 0."""
    if rounding not in ("nearest", "ceil"):
        raise ValueError("rounding must be 'nearest' or 'ceil'")
    table = _ue4m3_table(values.device)
    x = torch.nan_to_num(values.to(torch.float32), nan=0.0, posinf=float(table[-1]), neginf=0.0).clamp(0.0, float(table[-1]))
    if rounding == "ceil":
        code = torch.bucketize(x, table, right=False)                    # first code with value >= x
    else:
        code = torch.bucketize(x, (table[:-1] + table[1:]) / 2, right=True)   # midpoints passed, ties up
    code = code.clamp(max=126)
    if min_positive:
        code = torch.where((x > 0) & (code == 0), torch.ones_like(code), code)
    return code.to(torch.uint8)


def pow2_ceil(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= x for positive normal float32 x, by the exponent field
    (act_quant.py:6-23; fp8_fp4_gemm_1d1d_sm100.py ``_ceil_to_ue8m0``)."""
    bits = x.to(torch.float32).contiguous().view(torch.int32)
    e = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return (e.clamp(1, 254) << 23).view(torch.float32)


def ue8m0_byte(scale: torch.Tensor) -> torch.Tensor:
    """The e8m0 byte (biased exponent) of a power-of-two float32 scale."""
    return ((scale.to(torch.float32).contiguous().view(torch.int32) >> 23) & 0xFF).to(torch.uint8)


# ------------------------------------------------------------------------------------------
# scale-factor layouts
# ------------------------------------------------------------------------------------------

def sf_bytes_to_words(scale_bytes: torch.Tensor) -> torch.Tensor:
    """(rows, C) bytes, C a multiple of 4 -> (rows, C/4) uint32 words, byte j of a word in bits
    [8 j, 8 j + 8)."""
    if scale_bytes.dtype != torch.uint8 or scale_bytes.shape[-1] % 4:
        raise ValueError("sf_bytes_to_words: uint8 with a multiple of 4 columns expected")
    return _words_from_bytes(scale_bytes)


def _words_from_bytes(b: torch.Tensor) -> torch.Tensor:
    q = b.to(torch.int64).reshape(*b.shape[:-1], b.shape[-1] // 4, 4)
    w = q[..., 0] | (q[..., 1] << 8) | (q[..., 2] << 16) | (q[..., 3] << 24)
    return w.to(torch.uint32)


def sf_swizzle_128x4(words: torch.Tensor) -> torch.Tensor:
    """Row-major scale words (rows, C) -> the blocked layout the block-scaled tensor-core
    instructions read: inside every block of 128 rows, word (r, c) moves to flat position
    (c * 32 + r % 32) * 4 + r // 32 (nvfp4.py:216-261; the canonical 128 x 4 scale-factor atom).
    Rows are zero-padded to a multiple of 128."""
    if words.dtype != torch.uint32 or words.dim() != 2:
        raise ValueError("sf_swizzle_128x4: 2-D uint32 words expected")
    rows, cols = words.shape
    pad = (-rows) % 128
    w = words.to(torch.int64)
    if pad:
        w = torch.cat((w, torch.zeros(pad, cols, dtype=torch.int64, device=words.device)))
    blocks = w.shape[0] // 128
    r = torch.arange(128, device=words.device).unsqueeze(1)
    c = torch.arange(cols, device=words.device).unsqueeze(0)
    dst = ((c * 32 + r % 32) * 4 + r // 32).reshape(-1)                 # (128 * cols,) a permutation
    out = torch.empty(blocks, 128 * cols, dtype=torch.int64, device=words.device)
    out[:, dst] = w.reshape(blocks, 128 * cols)
    return out.reshape(blocks * 128, cols).to(torch.uint32)


def sf_unswizzle_128x4(words: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`sf_swizzle_128x4` (rows a multiple of 128)."""
    if words.dtype != torch.uint32 or words.dim() != 2 or words.shape[0] % 128:
        raise ValueError("sf_unswizzle_128x4: 2-D uint32 words with a multiple of 128 rows expected")
    rows, cols = words.shape
    blocks = rows // 128
    r = torch.arange(128, device=words.device).unsqueeze(1)
    c = torch.arange(cols, device=words.device).unsqueeze(0)
    src = ((c * 32 + r % 32) * 4 + r // 32).reshape(-1)
    w = words.to(torch.int64).reshape(blocks, 128 * cols)
    return w[:, src].reshape(rows, cols).to(torch.uint32)


def sf_pack_group_major(scale_bytes: torch.Tensor) -> torch.Tensor:
    """(rows, C) e8m0 bytes, C a multiple of 4 -> 1-D uint32 of C/4 x rows words, word (g, r)
    holding bytes 4g .. 4g+3 of row r: all rows of one K group together
    (fp8_fp4_gemm_1d1d_sm100.py:198-205)."""
    return _words_from_bytes(scale_bytes).t().contiguous().reshape(-1)


# ------------------------------------------------------------------------------------------
# quantisers
# ------------------------------------------------------------------------------------------

def quantize_mxfp4(x: torch.Tensor, block: int = 32, ties: str = "even", signed_zero: bool = True):
    """Floating-point (M, K) -> MXFP4: per row and ``block`` consecutive K elements,
    ``scale = 2^ceil(log2(amax / 6))`` (amax clamped below at 6 * 2^-126), codes = nearest
    e2m1 of ``clamp(x / scale, -6, 6)`` (act_quant.py:112-164, 249-268;
    fp8_fp4_gemm_1d1d_sm100.py:264-282 at block 128). Returns ``(packed, scale_bytes, scale)``:
    codes two per byte (M, K/2) uint8, e8m0 bytes (M, K/block) uint8, the scales as float32.
    ``ties="even"`` is what a hardware conversion does (the reference's kernel casts to
    float4_e2m1fn); its torch reference takes the smaller magnitude (``ties="down"``)."""
    if x.dim() != 2 or x.shape[1] % block or block % 2:
        raise ValueError(f"quantize_mxfp4: (M, K) with K a multiple of {block} expected")
    M, K = x.shape
    xb = x.to(torch.float32).reshape(M, K // block, block)
    amax = xb.abs().amax(-1).clamp(min=6.0 * 2.0 ** -126)
    scale = pow2_ceil(amax / E2M1_MAX)
    y = (xb / scale.unsqueeze(-1)).clamp(-E2M1_MAX, E2M1_MAX).reshape(M, K)
    return e2m1_pack(e2m1_encode(y, ties, signed_zero)), ue8m0_byte(scale), scale


def dequantize_mxfp4(packed: torch.Tensor, scale_bytes: torch.Tensor, block: int = 32) -> torch.Tensor:
    """(M, K/2) codes + (M, K/block) e8m0 bytes -> float32 (M, K)."""
    v = e2m1_decode(e2m1_unpack(packed))
    s = torch.pow(2.0, scale_bytes.to(torch.float32) - 127.0)
    return v * s.repeat_interleave(block, dim=1)


def quantize_nvfp4(x: torch.Tensor, return_scale_bytes: bool = False):
    """Floating-point (rows, K), rows a multiple of 128 and K of 256 -> NVFP4 block-scaled
    storage (nvfp4.py:469-539): per 16 consecutive K elements one UE4M3 scale, the smallest
    code not below amax / 6 (a positive amax never gets scale 0; an all-zero block does),
    codes = nearest e2m1 of x / scale with ties to the larger magnitude. Returns
    ``(packed, scale_words)``: codes (rows, K/2) int8 and the scale bytes as uint32 words
    (rows, K/64) in the 128 x 4 blocked layout; with ``return_scale_bytes`` also the row-major
    bytes (rows, K/16)."""
    if x.dim() != 2 or x.shape[0] % 128 or x.shape[1] % 256:
        raise ValueError("quantize_nvfp4: rows must be a multiple of 128 and K of 256")
    rows, K = x.shape
    xb = x.to(torch.float32).reshape(rows, K // 16, 16)
    amax = xb.abs().amax(-1)
    sb = ue4m3_encode(amax / E2M1_MAX, rounding="ceil", min_positive=True)
    sb = torch.where(amax == 0, torch.zeros_like(sb), sb)
    sv = ue4m3_decode(sb).unsqueeze(-1)
    y = torch.where(sv > 0, xb / sv, torch.zeros_like(xb)).reshape(rows, K)
    packed = e2m1_pack(e2m1_encode(y, "up")).view(torch.int8)
    words = sf_swizzle_128x4(_words_from_bytes(sb))
    return (packed, words, sb) if return_scale_bytes else (packed, words)
