"""CPU, two gloo ranks: the column-parallel host logic (shard plan, rank-local pack,
all-gather assembly) with the oracle standing in for the GPU kernel."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ref_programs as R
from tilelang_b200.parallel import ColumnParallelDequantLinear, plan_column_shards


def test_plan_covers_everything_in_tile_units():
    for N, p in [(28672, 8), (14336, 8), (3200, 8), (8640, 8), (200, 2), (128, 4), (1000, 3)]:
        shards = plan_column_shards(N, p)
        assert shards[0].start == 0 and shards[-1].stop == N
        for a, b in zip(shards, shards[1:]):
            assert a.stop == b.start
        for s in shards[:-1]:
            assert s.size % 128 == 0 or s.stop == N
    assert [s.size for s in plan_column_shards(28672, 8)] == [3584] * 8
    assert [s.size for s in plan_column_shards(3200, 8)] == [512, 384, 384, 384, 384, 384, 384, 384]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, N, ragged, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        M, K, g = 5, 256, 128
        A = torch.randn(M, K).to(torch.bfloat16)
        codes = torch.randint(0, 16, (N, K))
        qB = torch.from_numpy(R.general_compress(codes.numpy(), 4))
        s = (torch.rand(N, K // g) * 0.015 + 0.005).to(torch.bfloat16)

        def pack_fn(rows):
            return (qB[rows], s[rows])

        def gemm_fn(a, packed):
            return R.ref_w4a16(a, packed[0], packed[1], None, g, torch.bfloat16)

        layer = ColumnParallelDequantLinear(N, pack_fn, gemm_fn, align=128)
        full = layer.forward(A)
        ref = R.ref_w4a16(A, qB, s, None, g, torch.bfloat16)
        ok = torch.equal(full, ref) and layer.forward_sharded(A).shape == (M, layer.shard.size)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("N,ragged", [(512, False), (384, True)])
def test_two_rank_all_gather_matches_single_rank(N, ragged):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, N, ragged, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=10) for _ in range(2))
    assert results == {0: True, 1: True}
