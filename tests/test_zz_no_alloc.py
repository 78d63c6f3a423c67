"""GPU: the entry point that uses the library's built-in scratch array instead of a
caller-provided workspace, for callers that may not allocate device memory.

Collected last on purpose. It drives ``b200dq_gemm_static_scratch`` straight through
the C ABI and compares it with ``b200dq_gemm`` on the same inputs, twice in a row:
the array is shared by all calls and keeps the previous call's contents, so the
second call shows that stale contents do no harm. Shapes are chosen so that tiles
are split between CTAs, i.e. the scratch is really used, and cover both kernels the
two entry points choose between (the small-M kernel at 1 and 16 tokens, the tcgen05
kernel at 16 tokens with an explicit tile and at 300 tokens). The results are also
held against the CPU oracle, so the pair cannot be wrong together.
"""
import ctypes

import pytest
import torch

from tilelang_b200 import _lib, ops
from oracle import ref_programs as R

GROUP = 128


def _args(A, pw, out, workspace, token_tile=0, max_ctas=0):
    return _lib.GemmArgs(
        a=A.data_ptr(), wp=pw.wp.data_ptr(), bias=None, row_scale=None, c=out.data_ptr(),
        workspace=workspace.data_ptr() if workspace is not None else None,
        workspace_bytes=workspace.numel() if workspace is not None else 0,
        M=A.shape[0], N=pw.N, K=pw.K, group_size=pw.group_size, weight_format=pw.weight_format,
        act_type=pw.act_type, out_type=_lib.OUT_BF16, flags=0, tensor_scale=1.0, code_bias=0, fp4_exp_bias=127,
        token_tile=token_tile, max_ctas=max_ctas)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K,token_tile", [
    (1, 3072, 2048, 0),       # small-M kernel, one 8-token block
    (16, 3072, 2048, 0),      # small-M kernel, two 8-token blocks
    (16, 3072, 2048, 16),     # tcgen05 kernel at its narrowest tile
    (300, 1280, 2048, 0),     # tcgen05 kernel, 256-token tile with a ragged second tile
])
def test_static_scratch_matches_workspace_entry_point_and_oracle(M, N, K, token_tile):
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(3)
    qB_h = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8)
    s_h = (torch.rand(N, K // GROUP, generator=g) * 0.015 + 0.005).to(torch.bfloat16)
    z_h = (torch.rand(N, K // GROUP, generator=g) * 4 + 6).to(torch.bfloat16)
    pw = ops.pack_w4a16(qB_h.to(dev), s_h.to(dev), z_h.to(dev), N, K, GROUP, torch.bfloat16)
    need = lib.b200dq_gemm_workspace_bytes(M, N, K, pw.weight_format, pw.act_type, token_tile, 0)
    assert 0 < need <= 40 << 20
    workspace = torch.empty(need, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    for round_ in range(2):
        A_h = torch.randn(M, K, generator=g).to(torch.bfloat16)
        A = A_h.to(dev)
        want = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        a_ref = _args(A, pw, want, workspace, token_tile)
        _lib.check(lib.b200dq_gemm(ctypes.byref(a_ref), stream), "b200dq_gemm")
        a_new = _args(A, pw, got, None, token_tile)          # no workspace at all
        _lib.check(lib.b200dq_gemm_static_scratch(ctypes.byref(a_new), stream), "b200dq_gemm_static_scratch")
        torch.cuda.synchronize()
        ops.check_status(dev)
        # same kernel, same schedule, same summation order: the tolerance of the other
        # GPU tests (rtol = atol = 1e-2) is met with equality
        assert torch.isfinite(got.float()).all()
        assert torch.allclose(got.float(), want.float(), rtol=1e-2, atol=1e-2)
        assert torch.equal(got, want), f"round {round_}: outputs differ"
        # against the oracle, with the bounds the parity tests use: real-valued zero-points at
        # this short K get 2e-2 on the maximum (q - z is rounded to bf16 before the scale)
        ref = R.ref_w4a16(A_h, qB_h, s_h, z_h, GROUP, torch.bfloat16)
        assert R.mismatch_ratio(got.cpu(), ref, 1e-2, 1e-2) <= 0.01
        assert R.max_rel_error(got.cpu(), ref) <= 2e-2


def _sized_args(M, N, K, token_tile=0, max_ctas=0):
    return _lib.GemmArgs(M=M, N=N, K=K, group_size=GROUP, weight_format=_lib.WF_U4_SZ, act_type=_lib.ACT_BF16,
                         out_type=_lib.OUT_BF16, token_tile=token_tile, max_ctas=max_ctas)


def test_static_scratch_size_check_accepts_and_rejects():
    """The size check the entry point applies, through the helper that needs no GPU."""
    lib = _lib.load()
    need, cap = ctypes.c_size_t(0), ctypes.c_size_t(0)
    # the benchmark weight at 4096 tokens on a 148-SM part: 148 CTAs x 2 slots x 256 x 128 x 4 B of partial
    # tiles and one 8-byte arrival counter per tile (16 x 224 tiles)
    a = _sized_args(4096, 28672, 8192)
    assert lib.b200dq_static_scratch_check(ctypes.byref(a), 148, ctypes.byref(need), ctypes.byref(cap)) == 0
    assert cap.value == 40 << 20 and need.value == 148 * 2 * 256 * 128 * 4 + 16 * 224 * 8
    # a part with more SMs plans more CTAs, whose partial tiles no longer fit the array
    assert lib.b200dq_static_scratch_check(ctypes.byref(a), 192, ctypes.byref(need), ctypes.byref(cap)) == -1
    assert need.value == 192 * 2 * 256 * 128 * 4 + 16 * 224 * 8 > cap.value
    msg = _lib.last_error()
    assert "static array holds" in msg and "max_ctas" in msg
    # ... unless the caller bounds the grid
    a = _sized_args(4096, 28672, 8192, max_ctas=148)
    assert lib.b200dq_static_scratch_check(ctypes.byref(a), 192, ctypes.byref(need), ctypes.byref(cap)) == 0
    # whole tiles per CTA need no scratch at all; small-M calls plan 16-token tiles
    a = _sized_args(256, 128 * 148, 1024)
    assert lib.b200dq_static_scratch_check(ctypes.byref(a), 148, ctypes.byref(need), None) == 0 and need.value == 0
    a = _sized_args(8, 28672, 8192)
    assert lib.b200dq_static_scratch_check(ctypes.byref(a), 148, ctypes.byref(need), None) == 0
    assert need.value == 148 * 2 * 16 * 128 * 4 + 224 * 8


def test_static_scratch_rejects_bad_arguments():
    lib = _lib.load()
    assert lib.b200dq_gemm_static_scratch(None, None) == -1
    assert "null" in _lib.last_error()
    assert lib.b200dq_static_scratch_check(None, 148, None, None) == -1
    a = _sized_args(0, 128, 128)
    assert lib.b200dq_static_scratch_check(ctypes.byref(a), 148, None, None) == -1
    a = _sized_args(16, 128, 128)
    assert lib.b200dq_static_scratch_check(ctypes.byref(a), 0, None, None) == -1
