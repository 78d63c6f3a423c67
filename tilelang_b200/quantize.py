"""Host-side weight codecs (torch, any device): the natural packed layout of the
reference and converters from its pre-permuted layouts.

These run once per weight, offline; the device layout itself is produced by the
CUDA pack kernel (csrc/pack_kernels.cuh) behind ``ops.pack_*``.
"""
from __future__ import annotations

import torch


def compress_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack integer codes little-endian within each byte: element k goes to bits
    [(k % epb) * bits, ...) of byte k // epb — the reference's ``general_compress``
    (examples/dequantize_gemm/quantize/utils.py:50-67)."""
    epb = 8 // bits
    if codes.shape[-1] % epb:
        raise ValueError(f"last dimension must be a multiple of {epb}")
    c = (codes.to(torch.int32) & ((1 << bits) - 1)).reshape(*codes.shape[:-1], codes.shape[-1] // epb, epb)
    shifts = torch.arange(epb, device=codes.device, dtype=torch.int32) * bits
    return (c << shifts).sum(-1).to(torch.uint8)


def decompress_codes(packed: torch.Tensor, bits: int) -> torch.Tensor:
    """Inverse of :func:`compress_codes` (unsigned codes)."""
    epb = 8 // bits
    p = packed.view(torch.uint8).to(torch.int32)
    shifts = torch.arange(epb, device=packed.device, dtype=torch.int32) * bits
    out = (p.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    return out.reshape(*packed.shape[:-1], packed.shape[-1] * epb).to(torch.uint8)


def _interleave_positions(nbits: int, target_dtype: str):
    """Bit position of element e inside a 32-bit word after the reference's
    ``interleave_weight`` (quantize/utils.py:71-125), including its extra shuffles."""
    stride = 8 if target_dtype == "int8" else 16
    groups = 32 // stride
    per_word = 32 // nbits
    pos = [(e % groups) * stride + (e // groups) * nbits for e in range(per_word)]
    # each source bit of element e lands at pos[e] + b; apply the extra byte/nibble moves
    def move(bitpos: int) -> int:
        if nbits == 1 and target_dtype == "int8":
            nib = bitpos // 4
            table = {1: 4, 3: 6, 4: 1, 6: 3}
            return table.get(nib, nib) * 4 + bitpos % 4
        if nbits == 2 and target_dtype == "float16":
            byte = bitpos // 8
            table = {1: 2, 2: 1}
            return table.get(byte, byte) * 8 + bitpos % 8
        if nbits == 1 and target_dtype == "float16":
            nib = bitpos // 4
            table = {1: 2, 2: 4, 3: 6, 4: 1, 5: 3, 6: 5}
            return table.get(nib, nib) * 4 + bitpos % 4
        return bitpos
    return [[move(p + b) for b in range(nbits)] for p in pos]


def interleave_weight(qweight: torch.Tensor, nbits: int = 4, target_dtype: str = "float16") -> torch.Tensor:
    """The reference's offline permutation (quantize/utils.py:71-125), vectorised."""
    q = qweight.contiguous().view(torch.uint8).view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    out = torch.zeros_like(q)
    for e, bits in enumerate(_interleave_positions(nbits, target_dtype)):
        for b, dst in enumerate(bits):
            out |= ((q >> (nbits * e + b)) & 1) << dst
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out).to(torch.int32)
    return out.view(torch.uint8).reshape(qweight.shape).view(qweight.dtype)


def deinterleave_weight(qweight: torch.Tensor, nbits: int = 4, target_dtype: str = "float16") -> torch.Tensor:
    """Undo :func:`interleave_weight`: back to the natural little-endian code order."""
    q = qweight.contiguous().view(torch.uint8).view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    out = torch.zeros_like(q)
    for e, bits in enumerate(_interleave_positions(nbits, target_dtype)):
        for b, src in enumerate(bits):
            out |= ((q >> src) & 1) << (nbits * e + b)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out).to(torch.int32)
    return out.view(torch.uint8).reshape(qweight.shape).view(qweight.dtype)


def untwiddle_fp4(qB: torch.Tensor) -> torch.Tensor:
    """Reference twiddled e2m1 bytes (dequantize_utils.py:4-54: per byte pair
    W = (b[2i] << 8) | b[2i+1], element0 = bits (15,8,7,6), element1 = (12,5,4,3),
    element2 = (9,2,1,0), element3 = (14,11,10,13) as (s,e1,e0,m)) -> natural
    nibble order (low nibble = even k)."""
    b = qB.view(torch.uint8).to(torch.int32)
    w = (b[..., 0::2] << 8) | b[..., 1::2]

    def bit(i):
        return (w >> i) & 1

    def code(s, e1, e0, m):
        return (bit(s) << 3) | (bit(e1) << 2) | (bit(e0) << 1) | bit(m)

    c0, c1, c2, c3 = code(15, 8, 7, 6), code(12, 5, 4, 3), code(9, 2, 1, 0), code(14, 11, 10, 13)
    lo = (c0 | (c1 << 4)).to(torch.uint8)
    hi = (c2 | (c3 << 4)).to(torch.uint8)
    return torch.stack((lo, hi), dim=-1).reshape(qB.shape)


# ---------------------------------------------------------------------------
# checkpoint adapters: (qweight, scales, qzeros) of common 4-bit formats -> the natural
# layout the kernel factories take (codes (N, K/2), scales and integer zeros (N, K/group)).
# The integer zero-points go with ``zeros_mode="quantized"`` ((q - qz) * s, the reference's
# quantize/lop3.py:326-363); its BitNet checkpoints (examples/bitnet-1.58b/maint/
# create_bitblas_ckpt.py, load_from_quantized.py) are covered by ``BitLinear.from_float``.
# ---------------------------------------------------------------------------

def _unpack_int32_fields(words: torch.Tensor, bits: int, order=None) -> torch.Tensor:
    """(..., W) int32 words -> (..., W * 32 / bits) fields, field f of a word in bits
    [bits * order[f], ...) (``order`` defaults to 0, 1, 2, ...)."""
    per = 32 // bits
    order = list(range(per)) if order is None else order
    w = words.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.tensor([bits * o for o in order], dtype=torch.int64, device=words.device)
    out = (w.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    return out.reshape(*words.shape[:-1], words.shape[-1] * per)


def from_gptq(qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor, bits: int = 4,
              zero_offset: int = 1):
    """AutoGPTQ-style tensors of a (K -> N) linear layer:

    * ``qweight`` int32 (K * bits / 32, N): code of input k, output n in bits
      [bits * (k % 8), ...) of word (k // 8, n);
    * ``scales`` (K / group, N) float16/bfloat16;
    * ``qzeros`` int32 (K / group, N * bits / 32): zero-point of output n in bits
      [bits * (n % 8), ...) of word (group, n // 8), stored minus ``zero_offset``
      (1 in the original format, 0 in its "v2").

    Returns ``(qB, scales_nk, zeros_nk)``: codes (N, K / 2) uint8 with the even k in the low
    nibble, scales (N, K / group) and integer zero-points (N, K / group) uint8, for
    ``matmul(..., group_size=K // scales.shape[0], with_zeros=True, zeros_mode="quantized")``.
    Act-order checkpoints (a ``g_idx`` that is not k // group) must be un-permuted first."""
    if bits != 4:
        raise ValueError("from_gptq: 4-bit checkpoints only")
    K = qweight.shape[0] * 32 // bits
    N = qweight.shape[1]
    codes_kn = _unpack_int32_fields(qweight.t().contiguous(), bits)            # (N, K)
    zeros = _unpack_int32_fields(qzeros, bits)[:, :N] + zero_offset              # (groups, N)
    if int(zeros.max()) > 16 or int(zeros.min()) < 0:
        raise ValueError("from_gptq: zero-points leave [0, 16]; wrong zero_offset?")
    qB = compress_codes(codes_kn.to(torch.uint8), bits)
    assert tuple(qB.shape) == (N, K // 2)
    return qB, scales.t().contiguous(), zeros.t().contiguous().to(torch.uint8)


_AWQ_ORDER = [0, 4, 1, 5, 2, 6, 3, 7]    # nibble of a word that holds output 8 w + j, for j = 0..7


def from_awq(qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor, bits: int = 4):
    """AutoAWQ "GEMM" tensors of a (K -> N) linear layer: ``qweight`` int32 (K, N / 8) and
    ``qzeros`` int32 (K / group, N / 8), eight outputs per word in the interleaved order
    0, 2, 4, 6, 1, 3, 5, 7 (output 8 w + j sits in nibble [0, 4, 1, 5, 2, 6, 3, 7][j] of word w);
    ``scales`` (K / group, N); zero-points are stored as they are. Returns the same triple as
    :func:`from_gptq`."""
    if bits != 4:
        raise ValueError("from_awq: 4-bit checkpoints only")
    codes = _unpack_int32_fields(qweight, bits, _AWQ_ORDER)       # (K, N)
    zeros = _unpack_int32_fields(qzeros, bits, _AWQ_ORDER)        # (groups, N)
    qB = compress_codes(codes.t().contiguous().to(torch.uint8), bits)
    return qB, scales.t().contiguous(), zeros.t().contiguous().to(torch.uint8)


# ---------------------------------------------------------------------------
# scalar decode rules: element-wise restatements, on torch tensors, of the per-element helpers
# the reference's dequantise kernels are generated from
# (examples/dequantize_gemm/quantize/quantization.py). ``val`` holds storage words (uint8 /
# int8 / int32), ``pos`` the index of the field inside the word; every function is a pure tensor
# expression (any device). The device kernels implement the same rules on whole chunks.
# ---------------------------------------------------------------------------

def _field(val: torch.Tensor, nbit: int, pos) -> torch.Tensor:
    bits = val.element_size() * 8
    word = val.to(torch.int64) & ((1 << bits) - 1)
    return (word >> (torch.as_tensor(pos, device=val.device).to(torch.int64) * nbit)) & ((1 << nbit) - 1)


def packed_to_unsigned(val: torch.Tensor, nbit: int, pos, dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """Field ``pos`` of ``nbit`` bits, read unsigned (``_tir_packed_to_unsigned_convert``, :310-318)."""
    return _field(val, nbit, pos).to(dtype)


def packed_to_unsigned_with_zeros(val: torch.Tensor, nbit: int, pos, zero, dtype: torch.dtype = torch.float16):
    """The unsigned field minus an integer zero-point (``..._convert_with_zeros``, :321-330)."""
    return (_field(val, nbit, pos) - torch.as_tensor(zero, device=val.device).to(torch.int64)).to(dtype)


def packed_to_signed(val: torch.Tensor, nbit: int, pos, dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """The field minus 2^(nbit-1): offset-binary storage (``_tir_packed_to_signed_convert``, :298-307)."""
    return (_field(val, nbit, pos) - (1 << (nbit - 1))).to(dtype)


def packed_int_to_int(val: torch.Tensor, nbit: int, pos, dtype: torch.dtype = torch.int8) -> torch.Tensor:
    """The field sign-extended: two's-complement storage (``_tir_packed_int_to_int_convert``,
    :333-343; ``_tir_u32_to_int_to_float``, :111-117, is the same with a float target)."""
    f = _field(val, nbit, pos)
    return torch.where(f >= (1 << (nbit - 1)), f - (1 << nbit), f).to(dtype)


def _f16_from_bits(bits: torch.Tensor) -> torch.Tensor:
    b = bits.to(torch.int32) & 0xFFFF
    return torch.where(b >= 0x8000, b - 0x10000, b).to(torch.int16).view(torch.float16)


def u8_to_f8_e4m3_to_f16(val: torch.Tensor) -> torch.Tensor:
    """A byte read as fp8 e4m3 (fn: no infinities, 0x7f / 0xff are NaN) -> float16, by the bit
    manipulation of ``_tir_u8_to_f8_e4m3_to_f16`` (:250-275): the 7 low bits shifted into place
    with the exponent re-biased (8 added), subnormals (mantissa * 2^-9) normalised by hand."""
    v = val.view(torch.uint8).to(torch.int32)
    sign = (v >> 7) << 15
    e4 = v & 0x40
    normal = ((((v & 63) << 7) | (e4 << 8) | (e4 << 7)) ^ 0x2000)
    m = v & 7
    sub = torch.where(m >= 4, 0x2000 | ((m & 3) << 8),
                      torch.where(m >= 2, 0x1C00 | ((m & 1) << 9), torch.where(m == 1, torch.full_like(m, 0x1800),
                                                                              torch.zeros_like(m))))
    mag = torch.where((v & 0x78) == 0, sub, torch.where((v & 0x7F) == 0x7F, torch.full_like(v, 0x7E00), normal))
    return _f16_from_bits(sign | mag)


def u8_to_f8_e5m2_to_f16(val: torch.Tensor) -> torch.Tensor:
    """A byte read as fp8 e5m2 -> float16: e5m2 is the high byte of the float16 with the same value
    (``_tir_u8_to_f8_e5m2_to_f16``, :278-281)."""
    return _f16_from_bits(val.view(torch.uint8).to(torch.int32) << 8)


def packed_to_fp4_e3m0_to_f16(val: torch.Tensor, pos, nbit: int = 4) -> torch.Tensor:
    """The reference's sign + 3-bit-exponent 4-bit float (``_tir_packed_to_fp4_to_f16``, :206-221):
    0 for exponent 0, else +-2^(e - 7) (exponent field e + 8 of a float16 with zero mantissa)."""
    f4 = _field(val, nbit, pos).to(torch.int32)
    s, e = f4 >> 3, f4 & 7
    bits = ((e | 8) | (s << 5)) << 10
    return torch.where(e == 0, torch.zeros((), dtype=torch.float16, device=val.device), _f16_from_bits(bits))

