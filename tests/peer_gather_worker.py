"""Worker of the two-GPU test of the peer-store gather (launched by torchrun from
test_gpu_parallel.py): a column-parallel W4A16 GEMM whose epilogue writes each rank's block into
every rank's gathered buffer, compared with NCCL's all-gather of the same blocks and with the
oracle."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tilelang_b200 import ops  # noqa: E402
from tilelang_b200.parallel import PeerGatheredOutput, plan_column_shards  # noqa: E402
from oracle import ref_programs as R  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    N, K, group = 1024, 1024, 128
    g = torch.Generator().manual_seed(3)
    qB = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8)
    s = (torch.rand(N, K // group, generator=g) * 0.015 + 0.005).to(torch.bfloat16)
    z = (torch.rand(N, K // group, generator=g) * 4 + 6).to(torch.bfloat16)
    shard = plan_column_shards(N, world)[rank]
    rows = slice(shard.start, shard.stop)
    pw = ops.pack_w4a16(qB[rows].to(dev), s[rows].contiguous().to(dev), z[rows].contiguous().to(dev), shard.size, K, group,
                        torch.bfloat16)
    for M in (4, 300):          # the small-M kernel and the tcgen05 kernel (split tiles: the fix-up pass stores too)
        A = torch.randn(M, K, generator=g).to(torch.bfloat16)
        out = PeerGatheredOutput(M, shard.size, torch.bfloat16, dev)
        for _ in range(2):      # twice: the second call overwrites a filled buffer
            out.buffer.zero_()
            dist.barrier()
            out.gemm(A.to(dev), pw)
            gathered = out.wait()
            torch.cuda.synchronize()
        c_local = ops.gemm(A.to(dev), pw)
        want = torch.empty(world * M, shard.size, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(want, c_local)
        assert torch.equal(gathered.view(world * M, shard.size), want), f"rank {rank} M={M}: peer stores differ from all_gather"
        full = gathered.permute(1, 0, 2).reshape(M, N).float().cpu()
        ref = R.ref_w4a16(A, qB, s, z, group, torch.bfloat16).float()
        assert R.mismatch_ratio(full, ref, 1e-2, 1e-2) <= 0.01 and R.max_rel_error(full, ref) <= 2e-2
        ops.check_status(dev)
        dist.barrier()
        del out
    print("PEER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
