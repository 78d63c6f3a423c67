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
