"""GPU: grouped W4A16 GEMM, the activation kernels and the MoE layer against the oracle."""
import numpy as np
import pytest
import torch

import tilelang_b200 as tb
from tilelang_b200 import moe, ops
from oracle import ref_programs as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def experts(E, N, K, group, seed):
    q = torch.randint(0, 256, (E, N, K // 2), generator=gen(seed), dtype=torch.uint8)
    s = (torch.rand(E, N, K // group, generator=gen(seed + 1)) * 0.015 + 0.005).to(torch.bfloat16)
    packed = ops.stack_packed([ops.pack_w4a16(q[e].to(DEV), s[e].to(DEV), None, N, K, group, torch.bfloat16)
                               for e in range(E)])
    return q, s, packed


@pytest.mark.parametrize("counts,N,K,tile", [
    ([300, 0, 17, 256, 1], 256, 256, 256),       # empty, ragged and exact groups
    ([40, 90, 33], 200, 384, 128),               # N tail, K = 3 groups, 128-token tiles
    ([5, 9, 2, 7], 128, 128, 16),
])
def test_grouped_w4a16_matches_per_group_oracle(counts, N, K, tile):
    E, group = len(counts), 128
    q, s, packed = experts(E, N, K, group, seed=3)
    A = torch.randn(sum(counts), K, generator=gen(9)).to(torch.bfloat16)
    out = ops.gemm_grouped(A.to(DEV), packed, counts, token_tile=tile)
    torch.cuda.synchronize()
    tb.check_status()
    start = 0
    for e, c in enumerate(counts):
        if c:
            ref = R.ref_w4a16(A[start:start + c], q[e], s[e], None, group, torch.bfloat16)
            got = out[start:start + c].cpu()
            assert R.mismatch_ratio(got, ref) <= 0.01
            assert R.max_rel_error(got, ref) <= 1e-2
        start += c


def test_many_one_row_groups_in_a_fresh_process():
    """Eight groups of one row each round up to eight token tiles: the grouped schedule plans more
    CTAs (and more scratch) than a dense call with the same eight rows would. Run in a fresh
    process so that no earlier call has grown the cached workspace; host and device counts."""
    import os
    import subprocess
    import sys
    code = """
import torch
from tilelang_b200 import ops
from oracle import ref_programs as R
E, N, K, group = 8, 256, 2048, 128
g = torch.Generator().manual_seed(3)
q = torch.randint(0, 256, (E, N, K // 2), generator=g, dtype=torch.uint8)
s = (torch.rand(E, N, K // group, generator=g) * 0.015 + 0.005).to(torch.bfloat16)
packed = ops.stack_packed([ops.pack_w4a16(q[e].cuda(), s[e].cuda(), None, N, K, group, torch.bfloat16) for e in range(E)])
A = torch.randn(E, K, generator=g).to(torch.bfloat16)
for counts in ([1] * E, torch.ones(E, dtype=torch.int64, device="cuda")):
    out = ops.gemm_grouped(A.cuda(), packed, counts, token_tile=256).cpu()
    ops.check_status(torch.device("cuda", 0))
    for e in range(E):
        ref = R.ref_w4a16(A[e:e + 1], q[e], s[e], None, group, torch.bfloat16)
        assert R.max_rel_error(out[e:e + 1], ref) <= 1e-2, e
print("GROUPS_OK")
"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=root,
                         env=dict(os.environ, PYTHONPATH=root))
    assert res.returncode == 0 and "GROUPS_OK" in res.stdout, res.stdout[-1500:] + res.stderr[-3000:]


def test_silu_mul_matches_fp32_reference():
    h = torch.randn(77, 2 * 1408, generator=gen(1)).to(torch.bfloat16)
    out = ops.silu_mul(h.to(DEV)).cpu()
    ref = (torch.nn.functional.silu(h[:, :1408].float()) * h[:, 1408:].float()).to(torch.bfloat16)
    # expf on the device vs the host's exp: allow one bf16 ulp
    assert (out.float() - ref.float()).abs().max() <= 2.0 ** -7 * ref.float().abs().max()
    assert (out != ref).float().mean() < 0.01


@pytest.mark.parametrize("M,K,dtype", [(1, 3200, torch.bfloat16), (64, 8640, torch.bfloat16), (33, 3200, torch.float16)])
def test_absmax_quant_int8_bit_exact(M, K, dtype):
    x = torch.randn(M, K, generator=gen(2)).to(dtype)
    q, s = ops.absmax_quant_int8(x.to(DEV))
    q_ref, s_ref = R.bitnet_activation_quant(x)
    assert torch.equal(s.cpu(), s_ref.reshape(-1))
    assert torch.equal(q.cpu(), q_ref)


@pytest.mark.parametrize("M,K,dtype", [(1, 4096, torch.bfloat16), (300, 4096, torch.bfloat16), (33, 256, torch.float16)])
def test_mxfp4_activation_quantiser_bit_exact(M, K, dtype):
    """The CUDA quantiser against the oracle's restatement of act_quant.py with the hardware's
    tie rule: codes and e8m0 bytes must be equal, over scales from 1e-3 to 1e2, with exact
    midpoints, zeros and an all-zero block in the input."""
    x = (torch.randn(M, K, generator=gen(7)) * torch.logspace(-3, 2, M).unsqueeze(1)).to(dtype)
    x[0, :8] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0]).to(dtype)      # midpoints at scale 1
    x[0, 8:32] = 0
    x[-1, 32:64] = 0
    codes, sf = ops.quant_mxfp4(x.to(DEV))
    ref_codes, ref_scale = R.mxfp4_act_quant(x, 32, ties="even")
    assert torch.equal(sf.cpu(), ((ref_scale.view(torch.int32) >> 23) & 0xFF).to(torch.uint8))
    got = codes.cpu()
    unpacked = torch.stack((got & 15, got >> 4), dim=-1).reshape(M, K)
    assert torch.equal(unpacked, ref_codes)


def test_moe_layer_matches_oracle():
    """64-expert layout scaled down: 8 experts, top-2, W1 (2F, H) and W2 (H, F), group 128,
    fp16-range scales, zero-point 8."""
    E, k, T, H, F, group = 8, 2, 96, 256, 128, 128
    x = torch.randn(T, H, generator=gen(1)).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=gen(2))
    w1_q, w1_s, w1_p = experts(E, 2 * F, H, group, seed=10)
    w2_q, w2_s, w2_p = experts(E, H, F, group, seed=20)
    mlp = moe.make_gpu_expert_mlp(w1_p, w2_p, token_tile=32)
    out = moe.moe_forward(x.to(DEV), logits.to(DEV), k, E, mlp).cpu()
    tb.check_status()
    ref = R.ref_moe_w4a16(x, logits, k, w1_q, w1_s, w2_q, w2_s, group)
    assert R.mismatch_ratio(out, ref) <= 0.01
    assert R.max_rel_error(out, ref) <= 2e-2     # two chained GEMMs and a bf16 intermediate


def test_moe_expert_parallel_two_gpus_equals_single_gpu():
    """Experts split over two ranks with NCCL all-to-all dispatch/combine: every rank's
    tokens must come out bit-equal to the single-GPU layer holding all experts."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import os
    import subprocess
    import sys
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ep_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", worker],
                         capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert res.stdout.count("EP_OK") == 2, res.stdout[-2000:]
