"""GPU parity of the native MXFP4 path (tcgen05.mma kind::mxf4.block_scale, both operands
e2m1 codes with e8m0 scales per 32): the activation quantiser with blocked scale output, then
the GEMM against the oracle that re-quantises the activation the same way and multiplies the
dequantised operands in fp32. Products are exact, so the only difference from the oracle is
the order of the fp32 additions: the fp32 output is held to 1e-4 of max(|ref|, rms), the bf16
output additionally to one rounding (1e-2 is the stated bound; 5e-3 asserted)."""
import pytest
import torch

import tilelang_b200 as tb
from tilelang_b200 import blockscale, ops
from oracle import ref_programs as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def make_weight(N, K, seed):
    qB = torch.randint(0, 256, (N, K // 2), generator=gen(seed), dtype=torch.uint8)
    scale = (torch.randint(-8, 1, (N, K // 32), generator=gen(seed + 1)) + 127).to(torch.uint8)
    return qB, scale


@pytest.mark.parametrize("M,K", [(1, 128), (128, 256), (300, 1024)])
def test_blocked_scale_output_of_the_activation_quantiser(M, K):
    x = (torch.randn(M, K, generator=gen(M)) * 3).to(torch.bfloat16)
    codes_r, sf_r = ops.quant_mxfp4(x.to(DEV))
    codes_b, sf_b = ops.quant_mxfp4(x.to(DEV), blocked_scales=True)
    assert torch.equal(codes_r, codes_b)
    want = ops.block_mxfp4_scales(sf_r.cpu())
    assert torch.equal(sf_b.cpu().view(torch.int32), want.view(torch.int32))


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (128, 128, 1024), (1, 128, 512), (300, 384, 1024),
                                   (77, 200, 768), (512, 14336, 4096)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_native_mxfp4_gemm(M, N, K, out_dtype):
    if out_dtype == torch.float32 and M * N > 1 << 22:
        pytest.skip("large case once, in bf16")
    A = (torch.randn(M, K, generator=gen(10 + M)) * 2).to(torch.bfloat16)
    qB, scale = make_weight(N, K, 20 + N)
    a_codes, a_sf = ops.quant_mxfp4(A.to(DEV), blocked_scales=True)
    w_sf = ops.block_mxfp4_scales(scale).to(DEV)
    C = ops.gemm_mxfp4_native(a_codes, a_sf, qB.to(DEV), w_sf, out_dtype=out_dtype)
    tb.check_status()
    ref32 = R.ref_mxfp4_native(A, qB, scale, torch.float32)
    if out_dtype == torch.float32:
        assert R.max_rel_error(C.cpu(), ref32) <= 1e-4
    else:
        assert R.mismatch_ratio(C.float().cpu(), ref32, 1e-2, 1e-2) <= 0.01
        assert R.max_rel_error(C.float().cpu(), ref32) <= 5e-3
    # second launch, same inputs: identical bits (no split-K, fixed order)
    C2 = ops.gemm_mxfp4_native(a_codes, a_sf, qB.to(DEV), w_sf, out_dtype=out_dtype)
    assert torch.equal(C, C2)


def test_native_mxfp4_against_the_dequantising_kernel():
    """Same quantised operands through the dequantising path (bf16 activations that are exactly
    the de-quantised codes): the two kernels agree to bf16 rounding of the output."""
    M, N, K = 256, 1024, 2048
    A = torch.randn(M, K, generator=gen(3)).to(torch.bfloat16)
    qB, scale = make_weight(N, K, 4)
    codes, sf, _ = blockscale.quantize_mxfp4(A, 32, ties="even")
    A_dq = blockscale.dequantize_mxfp4(codes, sf, 32).to(torch.bfloat16)       # exact in bf16
    kernel = tb.matmul(M, N, K, "bfloat16", "bfloat16", "float32", source_format="fp4", num_bits=4, scale_size=32)
    C_deq = kernel(A_dq.to(DEV), qB.to(DEV), scale.to(DEV))
    a_codes, a_sf = ops.quant_mxfp4(A.to(DEV), blocked_scales=True)
    C_nat = ops.gemm_mxfp4_native(a_codes, a_sf, qB.to(DEV), ops.block_mxfp4_scales(scale).to(DEV))
    tb.check_status()
    assert R.max_rel_error(C_nat.float().cpu(), C_deq.float().cpu()) <= 8e-3
