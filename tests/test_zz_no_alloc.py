"""GPU: the entry point that uses the library's built-in scratch array instead of a
caller-provided workspace, for callers that may not allocate device memory.

Collected last on purpose. It drives ``b200dq_gemm_static_scratch`` straight through
the C ABI and compares it with ``b200dq_gemm`` on the same inputs, twice in a row:
the array is shared by all calls and keeps the previous call's contents, so the
second call shows that stale contents do no harm. Shapes are chosen so that tiles
are split between CTAs, i.e. the scratch is really used.
"""
import ctypes

import pytest
import torch

from tilelang_b200 import _lib, ops

pytestmark = pytest.mark.gpu


def _args(A, pw, out, workspace):
    return _lib.GemmArgs(
        a=A.data_ptr(), wp=pw.wp.data_ptr(), bias=None, row_scale=None, c=out.data_ptr(),
        workspace=workspace.data_ptr() if workspace is not None else None,
        workspace_bytes=workspace.numel() if workspace is not None else 0,
        M=A.shape[0], N=pw.N, K=pw.K, group_size=pw.group_size, weight_format=pw.weight_format,
        act_type=pw.act_type, out_type=_lib.OUT_BF16, flags=0, tensor_scale=1.0, code_bias=0, fp4_exp_bias=127,
        # both entry points on the tcgen05 kernel: an explicit tile of 16 keeps the small-M
        # kernel (which only b200dq_gemm dispatches to) out of the comparison
        token_tile=16 if A.shape[0] <= 16 else 0, max_ctas=0)


@pytest.mark.parametrize("M,N,K", [(16, 3072, 2048), (300, 1280, 2048)])
def test_static_scratch_matches_workspace_entry_point(M, N, K):
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(3)
    group = 128
    qB = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8).to(dev)
    s = (torch.rand(N, K // group, generator=g) * 0.015 + 0.005).to(torch.bfloat16).to(dev)
    z = (torch.rand(N, K // group, generator=g) * 4 + 6).to(torch.bfloat16).to(dev)
    pw = ops.pack_w4a16(qB, s, z, N, K, group, torch.bfloat16)
    need = lib.b200dq_gemm_workspace_bytes(M, N, K, pw.weight_format, pw.act_type, 0, 0)
    assert 0 < need <= 40 << 20
    workspace = torch.empty(need, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    for round_ in range(2):
        A = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
        want = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        a_ref = _args(A, pw, want, workspace)
        _lib.check(lib.b200dq_gemm(ctypes.byref(a_ref), stream), "b200dq_gemm")
        a_new = _args(A, pw, got, None)                      # no workspace at all
        _lib.check(lib.b200dq_gemm_static_scratch(ctypes.byref(a_new), stream), "b200dq_gemm_static_scratch")
        torch.cuda.synchronize()
        ops.check_status(dev)
        # same kernel, same schedule, same summation order: the tolerance of the other
        # GPU tests (rtol = atol = 1e-2) is met with equality
        assert torch.isfinite(got.float()).all()
        assert torch.allclose(got.float(), want.float(), rtol=1e-2, atol=1e-2)
        assert torch.equal(got, want), f"round {round_}: outputs differ"


def test_static_scratch_rejects_oversized_and_bad_arguments():
    lib = _lib.load()
    assert lib.b200dq_gemm_static_scratch(None, None) == -1
    assert "null" in _lib.last_error()
