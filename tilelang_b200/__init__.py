"""tilelang_b200 — B200-native low-bit dequantize-GEMM kernels behind the kernel-factory
call surface of tile-ai/tilelang's dequantize_gemm / gemm_int4 / bitnet-1.58b examples."""
from .kernels import (BitLinear, DequantKernel, bitnet_158_int8xint2_decode, bitnet_158_int8xint2_prefill,
                      dequantize_gemv, matmul, matmul_int8xint4, matmul_mxfp4_native, matmul_nt_int4)
from . import blockscale
from .ops import (PackedWeight, check_status, gemm, pack_int2, pack_int4_for_int8, pack_mxfp4, pack_w4a16)
from .profiler import Profiler, TensorSupplyType, do_bench

__all__ = [
    "BitLinear", "DequantKernel", "PackedWeight", "Profiler", "TensorSupplyType",
    "bitnet_158_int8xint2_decode", "bitnet_158_int8xint2_prefill", "blockscale", "check_status", "dequantize_gemv", "do_bench",
    "gemm", "matmul", "matmul_int8xint4", "matmul_mxfp4_native", "matmul_nt_int4", "pack_int2", "pack_int4_for_int8", "pack_mxfp4", "pack_w4a16",
]
