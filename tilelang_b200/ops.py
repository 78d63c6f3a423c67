"""Torch-facing wrappers around the C ABI: offline weight packing and the GEMM call.

Torch is used for device memory and the current stream only; every computation
goes through ``libb200dq.so`` (``_lib.py``). The calling rules follow the
reference adapter: tensors must be contiguous CUDA tensors on one device, the
launch goes on torch's current stream of that device, inputs are borrowed
(tilelang/jit/adapter/base.py:60-79, tilelang/jit/adapter/tvm_ffi.py:242-300).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import (ACT_BF16, ACT_F16, ACT_I8, GF_FP4_SIMPLE, GF_HAS_BIAS, GF_ROW_SCALE, GF_TRANS_C, OUT_BF16, OUT_F16,
                   OUT_F32, OUT_I32, WF_FP4_E8M0, WF_I2_I8, WF_I4_I8, WF_LUT4_S, WF_S4_RAW, WF_U2_SZ, WF_U4_RAW, WF_U4_SZ)

_ACT_OF = {torch.float16: ACT_F16, torch.bfloat16: ACT_BF16, torch.int8: ACT_I8}
_OUT_OF = {torch.float16: OUT_F16, torch.bfloat16: OUT_BF16, torch.float32: OUT_F32, torch.int32: OUT_I32}

_initialised_devices: set[int] = set()
_workspaces: dict[int, torch.Tensor] = {}


def _ensure_init(device: torch.device) -> None:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx in _initialised_devices:
        return
    with torch.cuda.device(idx):
        _lib.check(_lib.load().b200dq_init(), "b200dq_init")
    _initialised_devices.add(idx)


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _check_cuda_contig(name: str, t: torch.Tensor, device: Optional[torch.device] = None) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if device is not None and t.device != device:
        raise ValueError(f"{name} is on {t.device}, expected {device}")


@dataclass
class PackedWeight:
    """A weight in the library's private device layout (see csrc/pack_kernels.cuh)."""

    wp: torch.Tensor                 # uint8 packed image: codes and scale words, stage by stage
    N: int
    K: int
    weight_format: int
    act_type: int
    group_size: int = 0
    code_bias: int = 0
    fp4_exp_bias: int = 127
    fp4_simple: bool = False     # fp4 codes follow the reference's no-subnormal rule
    num_groups: int = 0          # > 0: a stack of per-group images (stack_packed)
    group_stride: int = 0        # bytes between consecutive group images

    @property
    def device(self) -> torch.device:
        return self.wp.device

    def nbytes(self) -> int:
        return self.wp.numel()


def _pack(q: torch.Tensor, scales: Optional[torch.Tensor], zeros: Optional[torch.Tensor], N: int, K: int,
          bits: int, group_size: int, weight_format: int, act_type: int) -> torch.Tensor:
    lib = _lib.load()
    _check_cuda_contig("packed weight codes", q)
    if q.dtype not in (torch.uint8, torch.int8):
        raise TypeError(f"packed weight codes must be uint8/int8, got {q.dtype}")
    if tuple(q.shape) != (N, K * bits // 8):
        raise ValueError(f"packed weight codes must have shape {(N, K * bits // 8)}, got {tuple(q.shape)}")
    _ensure_init(q.device)
    nbytes = lib.b200dq_packed_weight_bytes(N, K, group_size, weight_format)
    wp = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        _lib.check(lib.b200dq_pack_weights(q.data_ptr(), scales.data_ptr() if scales is not None else None,
                                           zeros.data_ptr() if zeros is not None else None, wp.data_ptr(), N, K,
                                           group_size, weight_format, act_type, _stream_ptr(q.device)),
                   "b200dq_pack_weights")
    return wp


ZEROS_MODES = ("original", "rescale", "quantized")


def zeros_for_original_mode(scales: torch.Tensor, zeros: torch.Tensor, zeros_mode: str) -> torch.Tensor:
    """The zero-point tensor that makes the device's ``(q - z) * s`` equal to the weight of the
    given reference mode (examples/dequantize_gemm/quantize/lop3.py:684-689):

    * ``original``: ``(q - z) * s`` -- unchanged;
    * ``rescale``: ``q * s - z`` (:233-271) = ``(q - z / s) * s``, so ``z / s`` computed in fp32
      and rounded once to the activation dtype. In float16 that agrees with the reference's
      ``fma(q, s, -z)`` to about one unit in the last place of the weight; bfloat16 keeps only
      8 significant bits of ``z / s``, a per-group offset of up to 0.4 % of a typical weight
      (the reference has this rule for float16 only);
    * ``quantized``: ``(q - qz) * s`` with integer zero-points (:326-363); ``zeros`` holds one
      integer per (row, group) (any integer dtype, or the activation dtype), exact.
    """
    if zeros_mode == "original":
        return zeros
    if zeros_mode == "rescale":
        return (zeros.float() / scales.float()).to(scales.dtype)
    if zeros_mode == "quantized":
        return zeros.to(scales.dtype)
    raise ValueError(f"zeros_mode must be one of {ZEROS_MODES}, got {zeros_mode!r}")


def pack_w4a16(qweight: torch.Tensor, scales: Optional[torch.Tensor], zeros: Optional[torch.Tensor], N: int, K: int,
               group_size: int, dtype: torch.dtype, signed_storage: bool = False,
               zeros_mode: str = "original") -> PackedWeight:
    """uint4 codes (N, K/2), two per byte with the even k in the low nibble.

    ``scales``/``zeros`` are (N, K/group_size) in ``dtype``; the weight is
    ``(q - z) * s`` (the reference's "original" zeros mode,
    examples/dequantize_gemm/quantize/lop3.py:684-689) or, with ``zeros_mode``, one of its
    other two rules (see :func:`zeros_for_original_mode`). ``zeros=None`` means the
    fixed zero-point 8; ``scales=None`` means the raw code ``q`` (or ``q - 8``
    with ``signed_storage``), as in example_dequant_gemm_fine_grained.py:11-13.
    """
    if dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("W4A16 needs float16 or bfloat16 activations")
    act = _ACT_OF[dtype]
    if scales is None:
        if zeros is not None:
            raise ValueError("zeros without scales is not supported")
        wf = WF_S4_RAW if signed_storage else WF_U4_RAW
        return PackedWeight(_pack(qweight, None, None, N, K, 4, 0, wf, act), N, K, wf, act)
    if group_size in (-1, 0, None):
        group_size = K
    groups = K // group_size
    if zeros is not None and zeros_mode != "original":
        _check_cuda_contig("zeros", zeros, qweight.device)
        if tuple(zeros.shape) != (N, groups) or tuple(scales.shape) != (N, groups):
            raise ValueError(f"scales and zeros must have shape {(N, groups)}")
        zeros = zeros_for_original_mode(scales, zeros, zeros_mode).contiguous()
    for name, t in (("scales", scales), ("zeros", zeros)):
        if t is None:
            continue
        _check_cuda_contig(name, t, qweight.device)
        if t.dtype != dtype or tuple(t.shape) != (N, groups):
            raise ValueError(f"{name} must be {dtype} of shape {(N, groups)}, got {t.dtype} {tuple(t.shape)}")
    wp = _pack(qweight, scales, zeros, N, K, 4, group_size, WF_U4_SZ, act)
    return PackedWeight(wp, N, K, WF_U4_SZ, act, group_size=group_size)


def pack_w2a16(qweight: torch.Tensor, scales: Optional[torch.Tensor], zeros: Optional[torch.Tensor], N: int, K: int,
               group_size: int, dtype: torch.dtype, bits: int = 2, signed: bool = False,
               zeros_mode: str = "original") -> PackedWeight:
    """2-bit codes (N, K/4) or 1-bit codes (N, K/8), little-endian in each byte, for 16-bit
    activations: weight = ``(q - z) * s`` with (N, K/group) scales and zero-points in ``dtype``.
    Without ``zeros`` the zero-point is 0, or with ``signed`` the reference's signed forms:
    ``q - 2`` for 2-bit codes and ``2 q - 1`` for 1-bit codes (quantize/lop3.py:424-463, 679-745);
    without ``scales`` the scale is 1. The image holds 2-bit fields in either case: 1-bit codes
    are widened on the device once, at pack time (a signed bit b becomes the field 2 b with
    zero-point 1), so a 1-bit weight streams 2 bits per element."""
    if dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("16-bit activations only")
    if bits not in (1, 2):
        raise ValueError("pack_w2a16 takes 1- or 2-bit codes")
    if zeros is not None and signed:
        raise ValueError("explicit zero-points go with unsigned codes")
    from . import quantize
    _check_cuda_contig("packed weight codes", qweight)
    dev = qweight.device
    if bits == 1:
        codes = quantize.decompress_codes(qweight.view(torch.uint8), 1)
        if signed:
            codes = codes * 2
        qweight = quantize.compress_codes(codes, 2).contiguous()
    if group_size in (-1, 0, None) or scales is None and zeros is None:
        group_size = K
    groups = K // group_size
    if scales is None:
        scales = torch.ones((N, groups), dtype=dtype, device=dev)
    if zeros is None:
        zeros = torch.full((N, groups), (1.0 if bits == 1 else 2.0) if signed else 0.0, dtype=dtype, device=dev)
    elif zeros_mode != "original":
        zeros = zeros_for_original_mode(scales, zeros, zeros_mode).contiguous()
    for name, t in (("scales", scales), ("zeros", zeros)):
        _check_cuda_contig(name, t, dev)
        if t.dtype != dtype or tuple(t.shape) != (N, groups):
            raise ValueError(f"{name} must be {dtype} of shape {(N, groups)}, got {t.dtype} {tuple(t.shape)}")
    act = _ACT_OF[dtype]
    wp = _pack(qweight.view(torch.uint8), scales, zeros, N, K, 2, group_size, WF_U2_SZ, act)
    return PackedWeight(wp, N, K, WF_U2_SZ, act, group_size=group_size)


# The 16 levels of NF4 (quantiles of a standard normal, normalised to [-1, 1]; Dettmers et al.,
# "QLoRA", 2023, appendix E), index 0..15.
NF4_TABLE = (-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
             -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
             0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
             0.7229568362236023, 1.0)


def pack_lut4(qweight: torch.Tensor, scales: torch.Tensor, N: int, K: int, group_size: int, dtype: torch.dtype,
              table=NF4_TABLE) -> PackedWeight:
    """4-bit codes (N, K/2), even k in the low nibble, that index a 16-entry ``table``:
    weight = ``table[q] * scale[n, k // group_size]`` (NF4 by default; any 4-bit codebook).
    ``scales`` (N, K/group) in ``dtype`` (the per-block absmax of an NF4 checkpoint)."""
    if dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("16-bit activations only")
    if len(table) != 16:
        raise ValueError("the table has 16 entries")
    if group_size in (-1, 0, None):
        group_size = K
    groups = K // group_size
    _check_cuda_contig("scales", scales, qweight.device)
    if scales.dtype != dtype or tuple(scales.shape) != (N, groups):
        raise ValueError(f"scales must be {dtype} of shape {(N, groups)}")
    act = _ACT_OF[dtype]
    wp = _pack(qweight, scales, None, N, K, 4, group_size, WF_LUT4_S, act)
    out = PackedWeight(wp, N, K, WF_LUT4_S, act, group_size=group_size)
    out.code_table = tuple(float(v) for v in table)
    return out


def pack_mxfp4(qweight: torch.Tensor, scale_bytes: Optional[torch.Tensor], N: int, K: int, exp_bias: int = 127,
               fp4_format: str = "e2m1", dtype: torch.dtype = torch.bfloat16) -> PackedWeight:
    """fp4 codes (N, K/2) (even k in the low nibble) + one exponent byte per 32 K.

    ``exp_bias=127`` reads the bytes as OCP e8m0; ``exp_bias=0`` as the raw
    exponent the reference's hopper example applies with ``2**Scale``
    (example_dequant_gemm_bf16_mxfp4_hopper.py:397). ``scale_bytes=None``: no block scale
    (example_dequant_gemm_bf16_fp4_hopper.py, example_dequant_gemm_fp4_hopper.py).
    ``fp4_format``: "e2m1" (true e2m1: 0, .5, 1, 1.5, 2, 3, 4, 6) or "tilelang_simple", the rule
    of the reference's scalar decoders, 2^(e-1) * (1 + m/2) for every code (.5, .75, 1, 1.5, 2, 3,
    4, 6: dequantize_utils.py:57-84, example_dequant_gemm_fp4_hopper.py:10-29).
    ``dtype=torch.float16`` (the fp16 x fp4 example) takes no block scale."""
    if fp4_format not in ("e2m1", "tilelang_simple"):
        raise ValueError("fp4_format must be 'e2m1' or 'tilelang_simple'")
    if dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("fp4 weights need float16 or bfloat16 activations")
    if scale_bytes is None:
        scale_bytes = torch.full((N, K // 32), exp_bias, dtype=torch.uint8, device=qweight.device)
    elif dtype == torch.float16:
        raise ValueError("float16 activations take fp4 weights without a block scale")
    _check_cuda_contig("scale bytes", scale_bytes, qweight.device)
    if scale_bytes.dtype != torch.uint8 or tuple(scale_bytes.shape) != (N, K // 32):
        raise ValueError(f"scale bytes must be uint8 of shape {(N, K // 32)}")
    act = _ACT_OF[dtype]
    wp = _pack(qweight, scale_bytes, None, N, K, 4, 32, WF_FP4_E8M0, act)
    return PackedWeight(wp, N, K, WF_FP4_E8M0, act, group_size=32, fp4_exp_bias=exp_bias,
                        fp4_simple=(fp4_format == "tilelang_simple"))


def pack_int2(qweight: torch.Tensor, N: int, K: int, code_offset: int = 0) -> PackedWeight:
    """2-bit codes (N, K/4), code k in bits [2(k%4), 2(k%4)+1] of byte k//4; weight = code - code_offset."""
    b = code_offset & 0xFF
    return PackedWeight(_pack(qweight, None, None, N, K, 2, 0, WF_I2_I8, ACT_I8), N, K, WF_I2_I8, ACT_I8,
                        code_bias=b | (b << 8) | (b << 16) | (b << 24))


def pack_int4_for_int8(qweight: torch.Tensor, N: int, K: int, code_offset: int = 0) -> PackedWeight:
    """4-bit codes (N, K/2) feeding an int8 MMA; weight = code - code_offset."""
    b = code_offset & 0xFF
    return PackedWeight(_pack(qweight, None, None, N, K, 4, 0, WF_I4_I8, ACT_I8), N, K, WF_I4_I8, ACT_I8,
                        code_bias=b | (b << 8) | (b << 16) | (b << 24))


def workspace_for(device: torch.device, nbytes: int) -> torch.Tensor:
    """A per-device scratch tensor, grown on demand and reused by every call."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[idx] = ws
    return ws


def gemm(A: torch.Tensor, w: PackedWeight, out: Optional[torch.Tensor] = None,
         out_dtype: Optional[torch.dtype] = None, bias: Optional[torch.Tensor] = None,
         row_scale: Optional[torch.Tensor] = None, tensor_scale: float = 1.0, trans_c: bool = False,
         token_tile: int = 0, max_ctas: int = 0, workspace: Optional[torch.Tensor] = None,
         peer_outs: Sequence[int] = ()) -> torch.Tensor:
    """C = A @ dequant(W)^T on the current stream; returns (and, if given, fills) ``out``.
    ``peer_outs``: up to seven device addresses in other GPUs' memory, each the base of a tensor
    laid out like ``out``; the kernel's epilogue stores every element there as well."""
    lib = _lib.load()
    _check_cuda_contig("A", A)
    dev = A.device
    if A.dim() != 2 or A.shape[1] != w.K:
        raise ValueError(f"A must have shape (M, {w.K}), got {tuple(A.shape)}")
    if _ACT_OF.get(A.dtype) != w.act_type:
        raise TypeError(f"A has dtype {A.dtype}, the packed weight expects activation type {w.act_type}")
    if w.wp.device != dev:
        raise ValueError(f"A is on {dev}, the packed weight on {w.wp.device}")
    M = A.shape[0]
    if out is None:
        if out_dtype is None:
            out_dtype = torch.int32 if A.dtype == torch.int8 else A.dtype
        out = torch.empty((w.N, M) if trans_c else (M, w.N), dtype=out_dtype, device=dev)
    else:
        _check_cuda_contig("out", out, dev)
        want = (w.N, M) if trans_c else (M, w.N)
        if tuple(out.shape) != want:
            raise ValueError(f"out must have shape {want}, got {tuple(out.shape)}")
    if out.dtype not in _OUT_OF:
        raise TypeError(f"unsupported output dtype {out.dtype}")
    flags = (GF_TRANS_C if trans_c else 0) | (GF_FP4_SIMPLE if w.fp4_simple else 0)
    if bias is not None:
        _check_cuda_contig("bias", bias, dev)
        if bias.dtype != out.dtype or tuple(bias.shape) != (M, w.N):
            raise ValueError(f"bias must be {out.dtype} of shape {(M, w.N)}")
        flags |= GF_HAS_BIAS
    if row_scale is not None:
        _check_cuda_contig("row_scale", row_scale, dev)
        if row_scale.dtype != torch.float32 or row_scale.numel() != M:
            raise ValueError("row_scale must be float32 with M elements")
        flags |= GF_ROW_SCALE
    if M == 0:
        return out
    _ensure_init(dev)
    need = lib.b200dq_gemm_workspace_bytes(M, w.N, w.K, w.weight_format, w.act_type, token_tile, max_ctas)
    if workspace is None:
        workspace = workspace_for(dev, need)
    elif workspace.numel() * workspace.element_size() < need:
        raise ValueError(f"workspace too small: need {need} bytes")
    args = _lib.GemmArgs(
        a=A.data_ptr(), wp=w.wp.data_ptr(),
        bias=bias.data_ptr() if bias is not None else None,
        row_scale=row_scale.data_ptr() if row_scale is not None else None,
        c=out.data_ptr(), workspace=workspace.data_ptr(),
        workspace_bytes=workspace.numel() * workspace.element_size(),
        M=M, N=w.N, K=w.K, group_size=w.group_size, weight_format=w.weight_format, act_type=w.act_type,
        out_type=_OUT_OF[out.dtype], flags=flags, tensor_scale=float(tensor_scale), code_bias=w.code_bias,
        fp4_exp_bias=w.fp4_exp_bias, token_tile=token_tile, max_ctas=max_ctas)
    table = getattr(w, "code_table", None)
    if table is not None:
        for i, v in enumerate(table):
            args.code_table[i] = v
    if peer_outs:
        if len(peer_outs) > 7:
            raise ValueError("at most seven peer outputs")
        for i, ptr in enumerate(peer_outs):
            args.c_peers[i] = int(ptr)
        args.num_peers = len(peer_outs)
    with torch.cuda.device(dev):
        _lib.check(lib.b200dq_gemm(ctypes.byref(args), _stream_ptr(dev)), "b200dq_gemm")
    return out


def stack_packed(weights: list) -> PackedWeight:
    """Concatenate per-group packed weights (same N, K, format) into one image; group g
    lives at byte offset ``g * stride`` (``stride`` = size of one image)."""
    w0 = weights[0]
    for w in weights:
        if (w.N, w.K, w.weight_format, w.act_type, w.group_size) != (w0.N, w0.K, w0.weight_format, w0.act_type, w0.group_size):
            raise ValueError("all groups must share N, K, format and group size")
    wp = torch.stack([w.wp for w in weights]).contiguous()
    out = PackedWeight(wp.view(-1), w0.N, w0.K, w0.weight_format, w0.act_type, w0.group_size, w0.code_bias,
                       w0.fp4_exp_bias)
    out.num_groups = len(weights)
    out.group_stride = w0.wp.numel()
    return out


def grouped_prefixes(counts, N: int, token_tile: int):
    """Host-side row and tile prefixes of a grouped GEMM from per-group row counts."""
    n_tiles = (N + 127) // 128
    rows, tiles = [0], [0]
    for c in counts:
        rows.append(rows[-1] + int(c))
        tiles.append(tiles[-1] + ((int(c) + token_tile - 1) // token_tile) * n_tiles)
    return rows, tiles


def gemm_grouped(A: torch.Tensor, w: PackedWeight, counts, out: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, token_tile: int = 256) -> torch.Tensor:
    """Grouped GEMM: rows of ``A`` are sorted by group, group g has ``counts[g]`` rows and
    multiplies its own weight ``w`` (from :func:`stack_packed`). ``counts`` is a host
    sequence (the schedule is planned on the host) or an int32/int64 tensor on A's device
    (a router's bincount): then the prefixes are built and the work is cut on the device and
    the host never waits for the counts; they must sum to A's row count (not checked)."""
    lib = _lib.load()
    _check_cuda_contig("A", A)
    dev = A.device
    G = getattr(w, "num_groups", 0)
    if G <= 0 or len(counts) != G:
        raise ValueError(f"counts must have one entry per group ({G})")
    M = A.shape[0]
    if A.shape[1] != w.K or _ACT_OF.get(A.dtype) != w.act_type:
        raise ValueError("A does not match the packed weights")
    if out is None:
        out = torch.empty((M, w.N), dtype=out_dtype or A.dtype, device=dev)
    on_device = isinstance(counts, torch.Tensor) and counts.is_cuda
    if on_device:
        if counts.device != dev or counts.dtype not in (torch.int32, torch.int64) or not counts.is_contiguous():
            raise ValueError("device counts must be a contiguous int32/int64 tensor on A's device")
        if M == 0:
            return out
        _ensure_init(dev)
        prefix = torch.empty(2 * (G + 1), dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.b200dq_grouped_prefixes(counts.data_ptr(), 1 if counts.dtype == torch.int64 else 0, G, w.N,
                                                   token_tile, prefix.data_ptr(), prefix.data_ptr() + 4 * (G + 1),
                                                   _stream_ptr(dev)), "b200dq_grouped_prefixes")
        total_tiles = -((M // token_tile + G) * ((w.N + 127) // 128))          # minus an upper bound
    else:
        rows, tiles = grouped_prefixes(counts, w.N, token_tile)
        if rows[-1] != M:
            raise ValueError(f"counts sum to {rows[-1]}, A has {M} rows")
        if M == 0 or tiles[-1] == 0:
            return out
        _ensure_init(dev)
        prefix = torch.tensor(rows + tiles, dtype=torch.int32).to(dev, non_blocking=True)
        total_tiles = tiles[-1]
    args = _lib.GemmArgs(
        a=A.data_ptr(), wp=w.wp.data_ptr(), bias=None, row_scale=None, c=out.data_ptr(),
        workspace=None, workspace_bytes=0,
        M=M, N=w.N, K=w.K, group_size=w.group_size, weight_format=w.weight_format, act_type=w.act_type,
        out_type=_OUT_OF[out.dtype], flags=0, tensor_scale=1.0, code_bias=w.code_bias, fp4_exp_bias=w.fp4_exp_bias,
        token_tile=token_tile, max_ctas=0,
        group_row_prefix=prefix.data_ptr(), group_tile_prefix=prefix.data_ptr() + 4 * (G + 1),
        group_weight_stride=w.group_stride, num_groups=G, total_tiles=total_tiles)
    # the grouped schedule follows total_tiles, not M: size the scratch from the arguments
    workspace = workspace_for(dev, lib.b200dq_gemm_workspace_bytes_for(ctypes.byref(args)))
    args.workspace, args.workspace_bytes = workspace.data_ptr(), workspace.numel()
    with torch.cuda.device(dev):
        _lib.check(lib.b200dq_gemm(ctypes.byref(args), _stream_ptr(dev)), "b200dq_gemm (grouped)")
    # the prefix tensor must outlive the launch that reads it
    prefix.record_stream(torch.cuda.current_stream(dev))
    return out


def absmax_quant_int8(x: torch.Tensor):
    """Per-token absmax int8 quantisation; returns (q int8 (M, K), scale fp32 (M,))."""
    lib = _lib.load()
    _check_cuda_contig("x", x)
    if x.dim() != 2 or x.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("x must be a 2-D float16/bfloat16 tensor")
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    if M:
        _ensure_init(x.device)
        with torch.cuda.device(x.device):
            _lib.check(lib.b200dq_absmax_quant_int8(x.data_ptr(), q.data_ptr(), s.data_ptr(), M, K, _ACT_OF[x.dtype],
                                                    _stream_ptr(x.device)), "b200dq_absmax_quant_int8")
    return q, s


def quant_mxfp4(x: torch.Tensor, blocked_scales: bool = False):
    """(M, K) float16/bfloat16 -> MXFP4 at block 32: returns (codes (M, K/2) uint8, two e2m1 codes
    per byte, and the e8m0 scale bytes). The CUDA version of
    ``blockscale.quantize_mxfp4(x, 32, ties="even")``. The scale bytes are (M, K/32) row-major,
    or with ``blocked_scales`` (K % 128 == 0) a (ceil(M/128) * 128, K/128) uint32 tensor in the
    128 x 4 blocked layout the native MXFP4 GEMM reads (``blockscale.sf_swizzle_128x4``)."""
    lib = _lib.load()
    _check_cuda_contig("x", x)
    if x.dim() != 2 or x.dtype not in (torch.float16, torch.bfloat16) or x.shape[1] % 32:
        raise ValueError("x must be a 2-D float16/bfloat16 tensor with K a multiple of 32")
    M, K = x.shape
    codes = torch.empty((M, K // 2), dtype=torch.uint8, device=x.device)
    if blocked_scales:
        if K % 128:
            raise ValueError("blocked scales need K to be a multiple of 128")
        rows = (M + 127) // 128 * 128
        sf = (torch.zeros if rows != M else torch.empty)((rows, K // 128), dtype=torch.int32, device=x.device)
    else:
        sf = torch.empty((M, K // 32), dtype=torch.uint8, device=x.device)
    if M:
        _ensure_init(x.device)
        with torch.cuda.device(x.device):
            _lib.check(lib.b200dq_quant_mxfp4(x.data_ptr(), codes.data_ptr(), sf.data_ptr(), M, K, _ACT_OF[x.dtype],
                                              1 if blocked_scales else 0, _stream_ptr(x.device)), "b200dq_quant_mxfp4")
    return codes, (sf.view(torch.uint32) if blocked_scales else sf)


def tensor_peak(kind: str, mmas: int = 16384, repeats: int = 5, device=None) -> float:
    """Measured rate (operations per second) of back-to-back ``tcgen05.mma`` of one kind on this
    GPU: "bf16", "int8" or "mxfp4". Best of ``repeats`` launches timed with events."""
    lib = _lib.load()
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    code = {"bf16": 0, "int8": 1, "mxfp4": 2}[kind]
    _ensure_init(device)
    ops_out = ctypes.c_double(0.0)
    best = float("inf")
    with torch.cuda.device(device):
        for _ in range(repeats + 1):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            _lib.check(lib.b200dq_tensor_peak(code, mmas, ctypes.byref(ops_out), _stream_ptr(device)), "b200dq_tensor_peak")
            stop.record()
            stop.synchronize()
            best = min(best, start.elapsed_time(stop))
    check_status(device)
    return ops_out.value / (best * 1e-3)


def block_mxfp4_scales(scale_bytes: torch.Tensor) -> torch.Tensor:
    """Row-major e8m0 bytes (rows, K/32), K % 128 == 0 -> uint32 words in the 128 x 4 blocked layout
    (rows zero-padded to a multiple of 128) for :func:`gemm_mxfp4_native`. Offline, once per weight."""
    from . import blockscale
    return blockscale.sf_swizzle_128x4(blockscale.sf_bytes_to_words(scale_bytes)).contiguous()


def gemm_mxfp4_native(a_codes: torch.Tensor, a_sf: torch.Tensor, w_codes: torch.Tensor, w_sf: torch.Tensor,
                      out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = A @ W^T on tcgen05.mma kind::mxf4.block_scale. ``a_codes`` (M, K/2) and ``w_codes``
    (N, K/2) uint8 e2m1 codes (even k in the low nibble), ``a_sf`` / ``w_sf`` their e8m0 scales as
    blocked uint32 words (:func:`quant_mxfp4` with ``blocked_scales``, :func:`block_mxfp4_scales`).
    K % 256 == 0."""
    lib = _lib.load()
    for name, t in (("a_codes", a_codes), ("a_sf", a_sf), ("w_codes", w_codes), ("w_sf", w_sf)):
        _check_cuda_contig(name, t, a_codes.device)
    M, Kb = a_codes.shape
    N, K = w_codes.shape[0], 2 * Kb
    if w_codes.shape[1] != Kb or a_codes.dtype != torch.uint8 or w_codes.dtype != torch.uint8:
        raise ValueError("a_codes and w_codes must be uint8 with the same K/2 columns")
    for name, t, rows in (("a_sf", a_sf, M), ("w_sf", w_sf, N)):
        if t.dtype != torch.uint32 or tuple(t.shape) != ((rows + 127) // 128 * 128, K // 128):
            raise ValueError(f"{name} must be uint32 of shape {((rows + 127) // 128 * 128, K // 128)} (blocked layout)")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a_codes.device)
    if M == 0:
        return out
    _ensure_init(a_codes.device)
    with torch.cuda.device(a_codes.device):
        _lib.check(lib.b200dq_gemm_mxfp4_native(a_codes.data_ptr(), a_sf.data_ptr(), w_codes.data_ptr(), w_sf.data_ptr(),
                                                out.data_ptr(), M, N, K, _OUT_OF[out.dtype], _stream_ptr(a_codes.device)),
                   "b200dq_gemm_mxfp4_native")
    return out


def moe_combine(y: torch.Tensor, row_of: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """``out[t] = sum_s weights[t, s] * y[row_of[t, s]]`` (fp32 accumulate, slot order).
    y (rows, H) f16/bf16; row_of (T, k) int64; weights (T, k) float32."""
    lib = _lib.load()
    _check_cuda_contig("y", y)
    _check_cuda_contig("row_of", row_of)
    _check_cuda_contig("weights", weights)
    if row_of.dtype != torch.int64 or weights.dtype != torch.float32 or row_of.shape != weights.shape:
        raise ValueError("moe_combine: row_of must be int64 and weights float32 of the same (tokens, top_k) shape")
    T, k = row_of.shape
    out = torch.empty((T, y.shape[1]), dtype=y.dtype, device=y.device)
    if T:
        _ensure_init(y.device)
        with torch.cuda.device(y.device):
            _lib.check(lib.b200dq_moe_combine(y.data_ptr(), row_of.data_ptr(), weights.data_ptr(), out.data_ptr(), T, k,
                                              y.shape[1], _ACT_OF[y.dtype], _stream_ptr(y.device)), "b200dq_moe_combine")
    return out


def unpack_int4_to_int8(packed: torch.Tensor) -> torch.Tensor:
    """(M, K/2) bytes of signed int4 pairs -> (M, K) int8."""
    lib = _lib.load()
    _check_cuda_contig("packed", packed)
    M, Kb = packed.shape
    out = torch.empty((M, Kb * 2), dtype=torch.int8, device=packed.device)
    if out.numel():
        _ensure_init(packed.device)
        with torch.cuda.device(packed.device):
            _lib.check(lib.b200dq_unpack_int4_to_int8(packed.data_ptr(), out.data_ptr(), out.numel(),
                                                      _stream_ptr(packed.device)), "b200dq_unpack_int4_to_int8")
    return out


def silu_mul(h: torch.Tensor) -> torch.Tensor:
    """silu(h[:, :H]) * h[:, H:] for h of shape (rows, 2H)."""
    lib = _lib.load()
    _check_cuda_contig("h", h)
    if h.dim() != 2 or h.shape[1] % 2 or h.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("h must be a 2-D float16/bfloat16 tensor with an even number of columns")
    rows, H = h.shape[0], h.shape[1] // 2
    out = torch.empty((rows, H), dtype=h.dtype, device=h.device)
    if rows:
        _ensure_init(h.device)
        with torch.cuda.device(h.device):
            _lib.check(lib.b200dq_silu_mul(h.data_ptr(), out.data_ptr(), rows, H, _ACT_OF[h.dtype],
                                           _stream_ptr(h.device)), "b200dq_silu_mul")
    return out


def check_status(device: Optional[torch.device] = None) -> None:
    """Raise if a kernel recorded a device-side error (a bounded wait that gave up)."""
    dev = device or torch.device("cuda", torch.cuda.current_device())
    _ensure_init(dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().b200dq_check_status(_stream_ptr(dev)), "b200dq_check_status")
