"""Worker of the two-GPU expert-parallel MoE test: run under torch.distributed.run, one
rank per GPU. Prints one line per rank; `EP_OK` marks bit-equality with the single-GPU layer."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tilelang_b200 import moe, ops
rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(lr); dev = torch.device("cuda", lr)
dist.init_process_group("nccl", device_id=dev)
E, k, T, H, F, g = 16, 4, 512, 512, 256, 128
def ex(e, n, kk, seed):
    gen = torch.Generator().manual_seed(seed * 1000 + e)
    q = torch.randint(0, 256, (n, kk // 2), generator=gen, dtype=torch.uint8).to(dev)
    s = (torch.rand(n, kk // g, generator=gen) * 0.015 + 0.005).to(torch.bfloat16).to(dev)
    return ops.pack_w4a16(q, s, None, n, kk, g, torch.bfloat16)
mine = moe.expert_ranges(E, world)[rank]
mlp_local = moe.make_gpu_expert_mlp(ops.stack_packed([ex(e, 2*F, H, 1) for e in mine]), ops.stack_packed([ex(e, H, F, 2) for e in mine]), 64)
mlp_all = moe.make_gpu_expert_mlp(ops.stack_packed([ex(e, 2*F, H, 1) for e in range(E)]), ops.stack_packed([ex(e, H, F, 2) for e in range(E)]), 64)
gen = torch.Generator().manual_seed(5)
x = torch.randn(T, H, generator=gen).to(torch.bfloat16).to(dev); lg = torch.randn(T, E, generator=gen).to(dev)
tl = T // world
out_ep = moe.moe_forward_ep(x[rank*tl:(rank+1)*tl], lg[rank*tl:(rank+1)*tl], k, E, mlp_local)
out_full = moe.moe_forward(x, lg, k, E, mlp_all)[rank*tl:(rank+1)*tl]
ops.check_status(dev)
print(f"rank {rank}: {'EP_OK' if torch.equal(out_ep, out_full) else 'EP_MISMATCH'} maxdiff={(out_ep.float()-out_full.float()).abs().max().item()}", flush=True)
dist.destroy_process_group()
