"""CPU, two gloo ranks: expert-parallel dispatch / combine against the single-rank oracle,
with the oracle's W4A16 matmul standing in for the grouped GPU GEMM."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ref_programs as R
from tilelang_b200 import moe


def _make(E=4, H=64, F=64, T=24, g=64, seed=0):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=gen).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=gen)
    w1_q = torch.randint(0, 256, (E, 2 * F, H // 2), generator=gen, dtype=torch.uint8)
    w2_q = torch.randint(0, 256, (E, H, F // 2), generator=gen, dtype=torch.uint8)
    w1_s = (torch.rand(E, 2 * F, H // g, generator=gen) * 0.015 + 0.005).to(torch.bfloat16)
    w2_s = (torch.rand(E, H, F // g, generator=gen) * 0.015 + 0.005).to(torch.bfloat16)
    return x, logits, w1_q, w1_s, w2_q, w2_s, g


def _oracle_mlp(w1_q, w1_s, w2_q, w2_s, g, experts):
    def grouped(wq, ws):
        def f(rows, counts):
            outs, start = [], 0
            for e, c in zip(experts, counts):
                outs.append(R.ref_w4a16(rows[start:start + c], wq[e], ws[e], None, g, rows.dtype))
                start += c
            return torch.cat(outs) if outs else rows.new_zeros((0, wq.shape[1]))
        return f

    def act(h):
        half = h.shape[1] // 2
        return (torch.nn.functional.silu(h[:, :half].float()) * h[:, half:].float()).to(h.dtype)

    return moe.ExpertMLP(grouped(w1_q, w1_s), grouped(w2_q, w2_s), act)


def test_single_rank_moe_matches_oracle():
    x, logits, w1_q, w1_s, w2_q, w2_s, g = _make()
    mlp = _oracle_mlp(w1_q, w1_s, w2_q, w2_s, g, list(range(4)))
    out = moe.moe_forward(x, logits, 2, 4, mlp)
    ref = R.ref_moe_w4a16(x, logits, 2, w1_q, w1_s, w2_q, w2_s, g)
    assert torch.allclose(out.float(), ref.float(), rtol=1e-2, atol=1e-2)


def test_expert_ranges_and_sorting():
    assert [list(r) for r in moe.expert_ranges(64, 8)] == [list(range(i * 8, i * 8 + 8)) for i in range(8)]
    assert [len(r) for r in moe.expert_ranges(6, 4)] == [2, 2, 2, 0]
    experts = torch.tensor([[1, 0], [0, 2], [2, 1]])
    order, tok, counts = moe.sort_by_expert(experts, 3)
    assert counts.tolist() == [2, 2, 2] and tok.tolist() == [0, 1, 0, 2, 1, 2]


def test_token_tile_rule_of_the_expert_gemms():
    """128-token tiles only where the schedule hands out whole tiles (16 tiles per SM and more)."""
    # the 64-expert, top-6 layer with 16384 tokens on one GPU: 98304 rows -> both GEMMs on 128
    assert moe.expert_token_tile(98304, 64, 2 * 1408, sms=148) == 128
    assert moe.expert_token_tile(98304, 64, 2048, sms=148) == 128
    # one of eight ranks of the same layer: 12288 rows over 8 experts -> 256
    assert moe.expert_token_tile(12288, 8, 2 * 1408, sms=148) == 256
    assert moe.expert_token_tile(12288, 8, 2048, sms=148) == 256
    # the threshold itself: (rows // 128 + groups) * ceil(N / 128) against 16 * sms
    assert moe.expert_token_tile(128 * 147, 1, 128 * 16, sms=148) == 128
    assert moe.expert_token_tile(128 * 146, 1, 128 * 16, sms=148) == 256


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        E, k = 4, 2
        x, logits, w1_q, w1_s, w2_q, w2_s, g = _make(E=E)
        T = x.shape[0]
        lo, hi = rank * T // world, (rank + 1) * T // world
        mine = list(moe.expert_ranges(E, world)[rank])
        mlp = _oracle_mlp(w1_q, w1_s, w2_q, w2_s, g, mine)
        out = moe.moe_forward_ep(x[lo:hi], logits[lo:hi], k, E, mlp)
        ref = R.ref_moe_w4a16(x, logits, k, w1_q, w1_s, w2_q, w2_s, g)[lo:hi]
        q.put((rank, bool(torch.allclose(out.float(), ref.float(), rtol=1e-2, atol=1e-2))))
    finally:
        dist.destroy_process_group()


def test_two_rank_expert_parallel_matches_oracle():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert dict(q.get(timeout=10) for _ in range(2)) == {0: True, 1: True}
