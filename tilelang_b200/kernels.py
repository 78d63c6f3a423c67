"""Kernel factories with the call surface of the reference's dequantize-GEMM examples.

A factory takes problem sizes and dtypes and returns a kernel object that is
called on torch CUDA tensors, exactly where a ``tilelang.jit``-compiled kernel is
called in the reference (lazy mode of tilelang/jit/__init__.py:505-550, 574-638;
call semantics of tilelang/jit/adapter/tvm_ffi.py:242-300: with ``out_idx`` the
callee allocates the output with ``torch.empty`` on the first input's device and
returns it, a wrong input count raises ``ValueError``; without ``out_idx`` the
caller passes the output). Tunables of the reference (``block_M``, ``num_stages``,
``threads``, ``split`` ...) are accepted and ignored: tile shapes are fixed by
the hand-written kernel.

Weights arrive in the reference's natural packed layout (two uint4 per byte along
K, low nibble first: example_dequant_gemm_fine_grained.py:11-13,
quantize/utils.py:50-67). The kernels stream a private pre-tiled image, so the
first call with a given weight tensor repacks it on the device
(``ops.pack_*``) and caches the image, keyed by the tensor objects and their versions;
``kernel.pack(...)`` does the same ahead of time.
"""
from __future__ import annotations

from typing import Any, Optional, Sequence

import torch

from . import ops
from .profiler import Profiler, TensorSupplyType

_DTYPES = {
    "float16": torch.float16, "half": torch.float16, "fp16": torch.float16,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "float": torch.float32, "fp32": torch.float32,
    "int8": torch.int8, "uint8": torch.uint8, "int32": torch.int32,
}


def as_torch_dtype(dt: Any) -> torch.dtype:
    """Accepts torch dtypes and the reference's dtype strings ("float16", T.bfloat16 ...)."""
    if isinstance(dt, torch.dtype):
        return dt
    key = str(dt).replace("torch.", "")
    if key in _DTYPES:
        return _DTYPES[key]
    raise ValueError(f"unsupported dtype {dt!r}")


class Param:
    """Shape/dtype of one kernel parameter (the reference's ``KernelParam``)."""

    def __init__(self, name: str, shape: Sequence[int], dtype: torch.dtype):
        self.name, self.shape, self.dtype = name, tuple(shape), dtype

    def __repr__(self) -> str:
        return f"Param({self.name}, {self.shape}, {self.dtype})"


class DequantKernel:
    """A callable on torch tensors, standing where the reference's ``JITKernel`` stands
    (tilelang/jit/kernel.py:40-211, 494-521)."""

    def __init__(self, name: str, params: list[Param], out_idx: Optional[list[int]], impl, pack_fn=None,
                 description: str = ""):
        self.name = name
        self.params = params
        self.out_idx = out_idx
        self._impl = impl
        self._pack_fn = pack_fn
        self._description = description
        self._cache: dict = {}

    # -- reference surface ---------------------------------------------------
    def __call__(self, *inputs):
        n_out = len(self.out_idx) if self.out_idx else 0
        expected = len(self.params) - n_out
        if len(inputs) != expected:
            raise ValueError(f"Expected {expected} inputs, got {len(inputs)} with {len(self.params)} params "
                             f"and out_idx={self.out_idx}")
        return self._impl(self, *inputs)

    def get_profiler(self, tensor_supply_type: TensorSupplyType = TensorSupplyType.Auto) -> Profiler:
        return Profiler(self, tensor_supply_type)

    def get_kernel_source(self) -> str:
        return self._description

    # -- library extras ------------------------------------------------------
    def capture(self, *inputs, before=None, after=None, warmup: int = 2):
        """One call on these (static) input tensors captured in a CUDA graph: returns
        ``(replay, outputs)`` where ``replay()`` re-launches the captured work on the current
        stream and ``outputs`` is what the call returned (the same tensors every replay).
        ``before()`` / ``after(outputs)`` run inside the capture too -- e.g. the copies from and to
        pinned host buffers of a decode step -- so a whole step is one graph launch instead of
        several kernel launches behind the Python call path. The weights are packed and the
        scratch is grown by the warm-up calls, outside the capture."""
        def step():
            if before is not None:
                before()
            out = self(*inputs)
            if after is not None:
                after(out)
            return out

        for _ in range(max(1, warmup)):
            step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                outputs = step()
        torch.cuda.current_stream().wait_stream(side)
        return graph.replay, outputs

    def pack(self, *weight_tensors) -> ops.PackedWeight:
        """Repack the weight tensors into the device layout now (otherwise done on first call)."""
        return self._packed(*weight_tensors)

    def _packed(self, *tensors) -> ops.PackedWeight:
        """The packed image of these weight tensors, repacked unless the cache holds an image
        made from the very same tensor objects at the same version. An entry keeps its source
        tensors alive: a storage address alone does not identify a weight, because the
        allocator hands a freed address to the next tensor of the same size."""
        key = tuple(id(t) if t is not None else None for t in tensors)
        hit = self._cache.get(key)
        if hit is not None:
            sources, versions, packed = hit
            if all(a is b for a, b in zip(sources, tensors)) and versions == self._versions(tensors):
                return packed
        packed = self._pack_fn(*tensors)
        if len(self._cache) >= 16:
            self._cache.clear()
        self._cache[key] = (tuple(tensors), self._versions(tensors), packed)
        return packed

    @staticmethod
    def _versions(tensors):
        return tuple(t._version if t is not None else None for t in tensors)


# ---------------------------------------------------------------------------
# W4A16 / MXFP4: matmul(M, N, K, in_dtype, out_dtype, accum_dtype, num_bits, group_size, ...)
# ---------------------------------------------------------------------------

def matmul(M: int, N: int, K: int, in_dtype, out_dtype, accum_dtype, num_bits: int = 4,
           group_size: Optional[int] = None, with_scaling: Optional[bool] = None, with_zeros: bool = False,
           zeros_mode: str = "original", source_format: Any = "uint", scale_size: int = 32,
           fast_dequant: bool = True, with_bias: bool = False, fp4_format: str = "e2m1",
           scale_exp_bias: int = 127, storage_dtype: Any = "uint8", trans_c: bool = False,
           block_M=None, block_N=None, block_K=None, num_stages=None, threads=None, split=1,
           **ignored) -> DequantKernel:
    """Dequantize-GEMM factory: ``C[M,N] = A[M,K] @ dequant(qB[N,K*num_bits/8])^T``.

    Covers the reference's
    * ``matmul`` of example_dequant_gemm_fine_grained.py:16-30 (no scale: call
      without ``group_size``; inputs ``(A, qB)``),
    * the grouped W4A16 rule of quantize/lop3.py:684-689 (``group_size`` given;
      inputs ``(A, qB, Scale[, Zeros][, Bias])``, scales/zeros of shape (N, K/group)),
    * ``matmul`` of example_dequant_gemm_bf16_mxfp4_hopper.py:83-104
      (``source_format`` "fp4"/"e2m1"/"uint32" with ``scale_size`` 32; inputs
      ``(A, qB, Scale[, Bias])``, Scale (N, K/32) uint8).

    With ``with_scaling=False`` the fp4 weights carry no block scale (inputs ``(A, qB)``): the
    bf16 x fp4 and fp16 x fp4 examples (example_dequant_gemm_bf16_fp4_hopper.py:46-346,
    example_dequant_gemm_fp4_hopper.py:108-220; the latter writes C^T: ``trans_c=True``).
    ``fp4_format``: "e2m1" true e2m1 codes in natural nibble order (default), or
    "tilelang_simple", the no-subnormal rule of the reference's scalar decoders;
    ``scale_exp_bias``: 127 for OCP e8m0 bytes, 0 for the raw ``2**Scale`` of the
    reference's hopper example. ``zeros_mode``: "original" ((q - z) * s), "rescale"
    (q * s - z) or "quantized" ((q - qz) * s with integer zero-points), quantize/lop3.py:684-689;
    all three are an offline rewrite of the zero-point term of the packed image.
    ``in_dtype="int8"`` (with ``out_dtype = accum_dtype = "int32"``) is the integer variant of
    example_dequant_gemm_fine_grained.py:427-428: C = A_int8 @ unpack_u4(qB)^T, exact.
    """
    in_t, out_t, acc_t = as_torch_dtype(in_dtype), as_torch_dtype(out_dtype), as_torch_dtype(accum_dtype)
    if in_t == torch.int8:
        return _matmul_int8_unsigned(M, N, K, out_t, acc_t, group_size or with_scaling or with_zeros or with_bias,
                                     num_bits, str(source_format).lower() == "int")
    if num_bits in (1, 2) and as_torch_dtype(in_dtype) in (torch.float16, torch.bfloat16):
        return _matmul_low_bits(M, N, K, in_t, out_t, acc_t, num_bits, group_size, with_scaling, with_zeros, zeros_mode,
                                str(source_format).lower(), with_bias, trans_c)
    if num_bits != 4:
        raise ValueError("matmul: num_bits must be 4 (or 1 / 2 with float16 / bfloat16 activations)")
    if in_t not in (torch.float16, torch.bfloat16):
        raise ValueError("matmul: in_dtype must be float16, bfloat16 or int8")
    if acc_t != torch.float32:
        raise ValueError("matmul: accumulation is float32 (tcgen05 kind::f16 accumulates in fp32)")
    if zeros_mode not in ops.ZEROS_MODES:
        raise ValueError(f"matmul: zeros_mode must be one of {ops.ZEROS_MODES}")
    if str(source_format).lower() == "nf4":
        return _matmul_nf4(M, N, K, in_t, out_t, group_size, with_bias, trans_c)
    is_fp4 = str(source_format).lower() in ("fp4", "e2m1", "mxfp4", "uint32", "fp")
    if with_scaling is None:
        with_scaling = bool(group_size) or is_fp4
    qk = K * num_bits // 8

    params = [Param("A", (M, K), in_t), Param("B", (N, qk), torch.uint8)]
    if is_fp4:
        if fp4_format not in ("e2m1", "tilelang_simple"):
            raise ValueError("matmul: fp4_format is 'e2m1' (true e2m1) or 'tilelang_simple' (the reference's scalar "
                             "decoders); twiddled bytes go through tilelang_b200.quantize.untwiddle_fp4 first")
        if in_t == torch.float16 and with_scaling:
            raise ValueError("matmul: float16 activations take fp4 weights without a block scale (with_scaling=False)")
        if with_scaling:
            params.append(Param("Scale", (N, K // scale_size), torch.uint8))
            if scale_size != 32:
                raise ValueError("matmul: MXFP4 uses one exponent byte per 32 K elements")
    elif with_scaling:
        g = K if group_size in (None, -1, 0) else group_size
        params.append(Param("Scale", (N, K // g), in_t))
        if with_zeros:
            # "quantized": one integer zero-point per (row, group), any integer dtype
            params.append(Param("Zeros", (N, K // g), torch.uint8 if zeros_mode == "quantized" else in_t))
    if with_bias:
        params.append(Param("Bias", (M, N), out_t))
    params.append(Param("C", (N, M) if trans_c else (M, N), out_t))

    def pack_fn(qB, scale=None, zeros=None):
        if is_fp4:
            return ops.pack_mxfp4(qB.view(torch.uint8), scale, N, K, exp_bias=scale_exp_bias, fp4_format=fp4_format,
                                  dtype=in_t)
        if with_scaling:
            g = K if group_size in (None, -1, 0) else group_size
            return ops.pack_w4a16(qB.view(torch.uint8), scale, zeros, N, K, g, in_t, zeros_mode=zeros_mode)
        return ops.pack_w4a16(qB.view(torch.uint8), None, None, N, K, 0, in_t)

    def impl(kernel: DequantKernel, A, qB, *rest):
        rest = list(rest)
        scale = rest.pop(0) if with_scaling else None
        zeros = rest.pop(0) if (with_scaling and with_zeros and not is_fp4) else None
        bias = rest.pop(0) if with_bias else None
        _check(A, params[0])
        _check(qB, params[1], any_int8=True)
        pw = kernel._packed(qB, scale, zeros)
        return ops.gemm(A, pw, out_dtype=out_t, bias=bias, trans_c=trans_c)

    desc = (f"b200dq umma_dequant_gemm: M={M} N={N} K={K} in={in_t} out={out_t} "
            f"{'mxfp4' if is_fp4 else 'w4a16'} group={group_size} zeros={with_zeros} bias={with_bias}")
    return DequantKernel("matmul", params, [-1], impl, pack_fn, desc)


def matmul_mxfp4_native(M: int, N: int, K: int, in_dtype="bfloat16", out_dtype="bfloat16", accum_dtype="float32",
                        scale_size: int = 32, **ignored) -> DequantKernel:
    """``C[M, N] = quant_mxfp4(A) @ dequant(qB, Scale)^T`` on the block-scaled fp4 tensor-core
    instruction: inputs ``(A, qB, Scale)`` as for ``matmul(..., source_format="fp4")``, but the
    activation is re-quantised to MXFP4 (one e8m0 scale per row and 32 K elements, ties to even:
    the kernel of examples/deepseek_v4/act_quant.py:112-164) and neither operand is dequantised:
    ``tcgen05.mma kind::mxf4.block_scale`` multiplies the codes and applies both scales. Twice the
    tensor rate of the dequantising path at a quarter of the activation bytes, at the price of a
    4-bit activation. The mainloop it stands for is examples/deepseek_v4/
    fp8_fp4_gemm_1d1d_sm100.py:18-185. K must be a multiple of 256. Also callable on an
    activation quantised earlier: ``kernel.quantized(a_codes, a_sf, qB, Scale)``."""
    in_t, out_t, acc_t = as_torch_dtype(in_dtype), as_torch_dtype(out_dtype), as_torch_dtype(accum_dtype)
    if in_t not in (torch.float16, torch.bfloat16) or acc_t != torch.float32 or scale_size != 32:
        raise ValueError("matmul_mxfp4_native: float16/bfloat16 activations, float32 accumulation, scale_size 32")
    if K % 256:
        raise ValueError("matmul_mxfp4_native: K must be a multiple of 256")
    params = [Param("A", (M, K), in_t), Param("B", (N, K // 2), torch.uint8), Param("Scale", (N, K // 32), torch.uint8),
              Param("C", (M, N), out_t)]

    def pack_fn(scale):
        return ops.block_mxfp4_scales(scale)

    def quantized(a_codes, a_sf, qB, scale):
        _check(qB, params[1], any_int8=True)
        _check(scale, params[2])
        return ops.gemm_mxfp4_native(a_codes, a_sf, qB.view(torch.uint8), kernel._packed(scale), out_dtype=out_t)

    def impl(kernel_: DequantKernel, A, qB, scale):
        _check(A, params[0])
        a_codes, a_sf = ops.quant_mxfp4(A, blocked_scales=True)
        return quantized(a_codes, a_sf, qB, scale)

    kernel = DequantKernel("matmul_mxfp4_native", params, [-1], impl, pack_fn,
                           f"b200dq kind::mxf4.block_scale: M={M} N={N} K={K} in={in_t} out={out_t}")
    kernel.quantized = quantized
    return kernel


def _matmul_nf4(M, N, K, in_t, out_t, group_size, with_bias, trans_c) -> DequantKernel:
    """NF4 weights: inputs ``(A, qB, Scale[, Bias])`` with qB (N, K/2) 4-bit indices into the NF4
    table and Scale (N, K/group) the per-block absmax. The reference benchmarks the format
    (W_NF4 A_FP16 in its dequantize_gemm chart) but ships no decoder; ``ops.pack_lut4`` takes any
    16-entry table."""
    g = K if group_size in (None, -1, 0) else group_size
    params = [Param("A", (M, K), in_t), Param("B", (N, K // 2), torch.uint8), Param("Scale", (N, K // g), in_t)]
    if with_bias:
        params.append(Param("Bias", (M, N), out_t))
    params.append(Param("C", (N, M) if trans_c else (M, N), out_t))

    def pack_fn(qB, scale):
        return ops.pack_lut4(qB.view(torch.uint8), scale, N, K, g, in_t)

    def impl(kernel: DequantKernel, A, qB, scale, *rest):
        _check(A, params[0])
        _check(qB, params[1], any_int8=True)
        return ops.gemm(A, kernel._packed(qB, scale), out_dtype=out_t, bias=rest[0] if with_bias else None,
                        trans_c=trans_c)

    return DequantKernel("matmul", params, [-1], impl, pack_fn, f"b200dq umma_dequant_gemm: M={M} N={N} K={K} nf4 group={g}")


def _matmul_low_bits(M, N, K, in_t, out_t, acc_t, num_bits, group_size, with_scaling, with_zeros, zeros_mode,
                     source_format, with_bias, trans_c) -> DequantKernel:
    """1- and 2-bit integer weights on 16-bit activations: the int2 -> f16 and int1 -> f16 decode
    rules of quantize/lop3.py:424-891. ``source_format`` "uint" reads the codes unsigned, "int"
    the reference's signed forms (q - 2; 2 q - 1). Inputs ``(A, qB[, Scale[, Zeros]][, Bias])``
    with qB (N, K * num_bits / 8)."""
    if acc_t != torch.float32:
        raise ValueError("matmul: accumulation is float32")
    if source_format not in ("uint", "int"):
        raise ValueError("matmul: 1- and 2-bit weights are 'uint' or 'int'")
    if with_scaling is None:
        with_scaling = bool(group_size)
    if with_zeros and not with_scaling:
        raise ValueError("matmul: zero-points need scales")
    if with_zeros and source_format == "int":
        raise ValueError("matmul: explicit zero-points go with unsigned codes")
    g = K if group_size in (None, -1, 0) else group_size
    params = [Param("A", (M, K), in_t), Param("B", (N, K * num_bits // 8), torch.uint8)]
    if with_scaling:
        params.append(Param("Scale", (N, K // g), in_t))
        if with_zeros:
            params.append(Param("Zeros", (N, K // g), torch.uint8 if zeros_mode == "quantized" else in_t))
    if with_bias:
        params.append(Param("Bias", (M, N), out_t))
    params.append(Param("C", (N, M) if trans_c else (M, N), out_t))

    def pack_fn(qB, scale=None, zeros=None):
        return ops.pack_w2a16(qB.view(torch.uint8), scale, zeros, N, K, g, in_t, bits=num_bits,
                              signed=(source_format == "int"), zeros_mode=zeros_mode)

    def impl(kernel: DequantKernel, A, qB, *rest):
        rest = list(rest)
        scale = rest.pop(0) if with_scaling else None
        zeros = rest.pop(0) if with_zeros else None
        bias = rest.pop(0) if with_bias else None
        _check(A, params[0])
        _check(qB, params[1], any_int8=True)
        return ops.gemm(A, kernel._packed(qB, scale, zeros), out_dtype=out_t, bias=bias, trans_c=trans_c)

    return DequantKernel("matmul", params, [-1], impl, pack_fn,
                         f"b200dq umma_dequant_gemm: M={M} N={N} K={K} in={in_t} out={out_t} int{num_bits} group={group_size}")


def _matmul_int8_unsigned(M: int, N: int, K: int, out_t: torch.dtype, acc_t: torch.dtype, extras, num_bits: int = 4,
                          signed: bool = False) -> DequantKernel:
    """``C[M, N] int32 = A_int8 @ unpack(qB)^T`` with raw integer codes: the int8 -> int32 variant of
    example_dequant_gemm_fine_grained.py (:427-428 run it with accum int32) for 4-bit codes, and
    the int2 -> int8 and int1 -> int8 decode rules of quantize/lop3.py:893-1047 for 2- and 1-bit
    codes. Unsigned codes are the weight; ``signed`` reads them as q - 8, q - 2 or 2 q - 1.
    1-bit codes are widened to 2-bit fields once, at pack time."""
    if out_t != torch.int32 or acc_t != torch.int32:
        raise ValueError("matmul: int8 activations accumulate and return int32")
    if extras:
        raise ValueError("matmul: the int8 variant takes raw codes only (no scale, zeros or bias)")
    if num_bits not in (1, 2, 4):
        raise ValueError("matmul: num_bits must be 1, 2 or 4")
    params = [Param("A", (M, K), torch.int8), Param("B", (N, K * num_bits // 8), torch.uint8),
              Param("C", (M, N), torch.int32)]

    def pack_fn(qB):
        q = qB.view(torch.uint8)
        if num_bits == 4:
            return ops.pack_int4_for_int8(q, N, K, code_offset=8 if signed else 0)
        if num_bits == 2:
            return ops.pack_int2(q, N, K, code_offset=2 if signed else 0)
        from . import quantize
        codes = quantize.decompress_codes(q, 1)
        return ops.pack_int2(quantize.compress_codes(codes * 2 if signed else codes, 2).contiguous(), N, K,
                             code_offset=1 if signed else 0)

    def impl(kernel: DequantKernel, A, qB):
        _check(A, params[0])
        _check(qB, params[1], any_int8=True)
        return ops.gemm(A, kernel._packed(qB), out_dtype=torch.int32)

    return DequantKernel("matmul", params, [-1], impl, pack_fn, f"b200dq kind::i8 int8 x uint4: M={M} N={N} K={K}")


def _check(t: torch.Tensor, p: Param, any_int8: bool = False) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{p.name}: expected a torch.Tensor")
    if tuple(t.shape) != p.shape:
        raise ValueError(f"{p.name}: expected shape {p.shape}, got {tuple(t.shape)}")
    ok = t.dtype == p.dtype or (any_int8 and t.dtype in (torch.int8, torch.uint8))
    if p.name == "Zeros" and p.dtype == torch.uint8:
        ok = not t.dtype.is_floating_point
    if not ok:
        raise TypeError(f"{p.name}: expected dtype {p.dtype}, got {t.dtype}")


# ---------------------------------------------------------------------------
# small-M entry point of the reference: dequantize_gemv
# ---------------------------------------------------------------------------

def dequantize_gemv(M: int, N: int, K: int, in_dtype, out_dtype, accum_dtype, num_bits: int = 4,
                    storage_dtype: Any = "int8", source_format: str = "uint", n_partition: int = 4,
                    reduce_thread: int = 32, fast_decoding: bool = False, trans_A: bool = False,
                    trans_B: bool = True, group_size: int = -1, with_scaling: bool = False) -> DequantKernel:
    """``kernel(A, qB, C)`` with the caller's preallocated C, as in
    example_dequant_gemv_fp16xint4.py:11-29, 199-205. The reference kernel ignores
    ``group_size``/``with_scaling`` (its body never reads a Scale tensor, :77-155)
    and so does this one: C = A @ q^T with the raw unsigned codes.

    ``fast_decoding=True`` means the caller passes weights already permuted by the
    reference's ``interleave_weight``; they are un-permuted on the device view
    (``tilelang_b200.quantize.deinterleave_weight``) before packing.
    """
    if trans_A or not trans_B:
        raise ValueError("dequantize_gemv: only trans_A=False, trans_B=True (as in the reference)")
    in_t, out_t = as_torch_dtype(in_dtype), as_torch_dtype(out_dtype)
    if source_format != "uint" or num_bits != 4:
        raise ValueError("dequantize_gemv: uint4 weights only")
    params = [Param("A", (M, K), in_t), Param("B", (N, K // 2), torch.int8), Param("C", (M, N), out_t)]

    def pack_fn(qB):
        q = qB
        if fast_decoding:
            from .quantize import deinterleave_weight
            q = deinterleave_weight(qB, 4, "float16")
        return ops.pack_w4a16(q.view(torch.uint8), None, None, N, K, 0, in_t)

    def impl(kernel: DequantKernel, A, qB, C):
        _check(A, params[0])
        _check(qB, params[1], any_int8=True)
        _check(C, params[2])
        ops.gemm(A, kernel._packed(qB), out=C)
        return None

    return DequantKernel("dequantize_gemv", params, None, impl, pack_fn,
                         f"b200dq umma_dequant_gemm (small-M tiles): M={M} N={N} K={K} in={in_t}")


# ---------------------------------------------------------------------------
# W4A8: int8 activations x int4 weights -> int32, transposed output
# ---------------------------------------------------------------------------

def matmul_int8xint4(M: int, N: int, K: int, in_dtype="int8", out_dtype="int32", accum_dtype="int32",
                     num_bits: int = 4, block_M=None, block_N=None, block_K=None, num_stages=None, threads=None,
                     **ignored) -> DequantKernel:
    """``Ct[N, M] int32 = sext4(B) @ A^T`` (example_dequant_gemm_w4a8.py:85-149; decode rule :10-21)."""
    if as_torch_dtype(in_dtype) != torch.int8 or as_torch_dtype(out_dtype) != torch.int32 or num_bits != 4:
        raise ValueError("matmul_int8xint4: int8 activations, 4-bit weights, int32 output")
    params = [Param("A", (M, K), torch.int8), Param("B", (N, K // 2), torch.uint8), Param("Ct", (N, M), torch.int32)]

    def pack_fn(qB):
        # two's-complement nibbles -> offset-8 codes: code = (w + 8) & 15 = nibble ^ 8
        q = qB.view(torch.uint8) ^ 0x88
        return ops.pack_int4_for_int8(q, N, K, code_offset=8)

    def impl(kernel: DequantKernel, A, qB):
        _check(A, params[0])
        _check(qB, params[1], any_int8=True)
        return ops.gemm(A, kernel._packed(qB), out_dtype=torch.int32, trans_c=True)

    return DequantKernel("matmul_int8xint4", params, [2], impl, pack_fn, f"b200dq kind::i8 W4A8: M={M} N={N} K={K}")


def matmul_nt_int4(M: int, N: int, K: int, block_M=None, block_N=None, block_K=None, threads=None) -> DequantKernel:
    """``C[M, N] int32 = A @ B^T`` with both operands signed int4, two per byte
    (examples/gemm_int4/example_tilelang_gemm_int4.py:17-38, compiled there with
    ``out_idx=-1``; check :92-103 is ``rtol=0, atol=0``). A is unpacked to int8 by a
    small kernel, B takes the 4-bit-weights-into-int8-MMA path."""
    if K % 32 != 0:
        raise ValueError("matmul_nt_int4: K must be a multiple of 32")
    params = [Param("A", (M, K // 2), torch.int8), Param("B", (N, K // 2), torch.int8), Param("C", (M, N), torch.int32)]

    def pack_fn(qB):
        return ops.pack_int4_for_int8(qB.view(torch.uint8) ^ 0x88, N, K, code_offset=8)

    def impl(kernel: DequantKernel, A, qB):
        _check(A, params[0], any_int8=True)
        _check(qB, params[1], any_int8=True)
        A8 = ops.unpack_int4_to_int8(A.view(torch.uint8))
        return ops.gemm(A8, kernel._packed(qB), out_dtype=torch.int32)

    return DequantKernel("matmul_nt_int4", params, [-1], impl, pack_fn, f"b200dq kind::i8 int4 x int4: M={M} N={N} K={K}")


# ---------------------------------------------------------------------------
# BitNet b1.58: int8 activations x 2-bit weights -> int32
# ---------------------------------------------------------------------------

def _bitnet_factory(name: str, M: int, N: int, K: int, in_dtype, out_dtype, accum_dtype, fast_decoding: bool,
                    code_offset: int) -> DequantKernel:
    in_t, out_t = as_torch_dtype(in_dtype), as_torch_dtype(out_dtype)
    if in_t != torch.int8:
        raise ValueError(f"{name}: int8 activations only (the reference's float16 variant is not part of this path)")
    if out_t not in (torch.int32, torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"{name}: unsupported output dtype {out_t}")
    params = [Param("A", (M, K), torch.int8), Param("B", (N, K // 4), torch.int8), Param("C", (M, N), out_t)]

    def pack_fn(qB):
        q = qB
        if fast_decoding:
            from .quantize import deinterleave_weight
            q = deinterleave_weight(qB, 2, "int8")
        return ops.pack_int2(q.view(torch.uint8), N, K, code_offset=code_offset)

    def impl(kernel: DequantKernel, A, qB, C):
        _check(A, params[0])
        _check(qB, params[1], any_int8=True)
        _check(C, params[2])
        ops.gemm(A, kernel._packed(qB), out=C)
        return None

    return DequantKernel(name, params, None, impl, pack_fn, f"b200dq kind::i8 int8xint2: M={M} N={N} K={K}")


def bitnet_158_int8xint2_decode(M: int, N: int, K: int, in_dtype="int8", out_dtype="int32", accum_dtype="int32",
                                fast_decoding: bool = True, n_partition: int = 4, reduce_thread: int = 32,
                                code_offset: int = 0) -> DequantKernel:
    """``kernel(A, qW, C)``: C int32 = A @ W^T with 2-bit codes, four per byte.
    examples/bitnet-1.58b/kernel_benchmark/tilelang_bitnet_158_int8xint2_decode.py:66-175;
    with ``fast_decoding`` the weights come through the reference's
    ``general_compress`` + ``interleave_weight(qw, 2, "int8")`` (:178-236, 248-250).
    The reference decodes unsigned codes (:139-144): ``code_offset=0``; the ternary
    mapping code = w + 2 uses ``code_offset=2`` (its ``decode_i2s_to_i8s``, :16-39)."""
    return _bitnet_factory("bitnet_158_int8xint2_decode", M, N, K, in_dtype, out_dtype, accum_dtype, fast_decoding,
                           code_offset)


def bitnet_158_int8xint2_prefill(M: int, N: int, K: int, in_dtype="int8", out_dtype="int32", accum_dtype="int32",
                                 fast_decoding: bool = True, block_row_warps=2, block_col_warps=2,
                                 warp_row_tiles=32, warp_col_tiles=32, chunk=64, code_offset: int = 0) -> DequantKernel:
    """Same contract for large M
    (examples/bitnet-1.58b/kernel_benchmark/tilelang_bitnet_158_int8xint2_prefill.py:72-298)."""
    return _bitnet_factory("bitnet_158_int8xint2_prefill", M, N, K, in_dtype, out_dtype, accum_dtype, fast_decoding,
                           code_offset)


class BitLinear(torch.nn.Module):
    """The BitNet linear layer's inference forward on top of the int8 x int2 kernel:
    per-token absmax int8 quantisation of the activations, ternary GEMM, then
    ``out / s_act / s_w`` (examples/bitnet-1.58b/utils_quant.py:156-170; ``forward`` is
    ``BitLinearBitBLAS.forward``, :199-209: quantise, GEMM, post-scale, bias).
    Weights are ternary codes w + 2 in 2 bits. ``W_t`` is the ternary (N, K) int8 weight and
    ``s_w`` its scale 1 / mean|W_fp| (``weight_quant``, :149-154); ``from_float`` derives both
    from a floating-point weight."""

    def __init__(self, W_t: torch.Tensor, s_w: float, out_dtype: torch.dtype = torch.bfloat16,
                 bias: Optional[torch.Tensor] = None):
        super().__init__()
        from .quantize import compress_codes
        N, K = W_t.shape
        self.N, self.K, self.s_w, self.out_dtype = N, K, float(s_w), out_dtype
        self.in_features, self.out_features = K, N
        codes = compress_codes((W_t.to(torch.int16) + 2).to(torch.uint8), 2)
        self.weight = ops.pack_int2(codes, N, K, code_offset=2)
        self.bias = bias

    @classmethod
    def from_float(cls, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                   bias: Optional[torch.Tensor] = None) -> "BitLinear":
        """Ternarise a floating-point (N, K) weight: s = 1 / mean|W| (clamped at 1e-5),
        W_t = round(W * s).clamp(-1, 1) (utils_quant.py:149-154)."""
        s = 1.0 / weight.float().abs().mean().clamp_(min=1e-5)
        W_t = (weight.float() * s).round().clamp_(-1, 1).to(torch.int8)
        return cls(W_t, float(s), out_dtype, bias)

    def forward_quantized(self, A_q: torch.Tensor, s_act: torch.Tensor) -> torch.Tensor:
        return ops.gemm(A_q, self.weight, out_dtype=self.out_dtype, row_scale=s_act.reshape(-1).float().contiguous(),
                        tensor_scale=self.s_w)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x (..., K) float16/bfloat16 -> (..., N): absmax-quantise every token on the device,
        multiply, rescale; the bias (if any) is added in the output dtype."""
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.K).contiguous()
        A_q, s_act = ops.absmax_quant_int8(x2)
        out = self.forward_quantized(A_q, s_act)
        if self.bias is not None:
            out = out + self.bias.to(out.dtype)
        return out.reshape(*lead, self.N)
