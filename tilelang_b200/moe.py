"""Mixture-of-experts MLP on grouped W4A16 dequantize-GEMMs, single GPU and expert-parallel.

The reference has no W4A16 MoE kernel; its semantics come from
examples/fusedmoe/example_fusedmoe_torch.py (routing :26-40: softmax then
``topk(sorted=False)``; expert MLP :8-23: ``down(silu(gate(x)) * up(x))``; dispatch by
argsort/bincount and score-weighted combine :65-91) and from its grouped GEMM
(examples/grouped_gemm/example_grouped_gemm_fwd.py:8-36: rows sorted by expert, one
weight per expert). Here the two grouped GEMMs and the activation between them are this
library's kernels; routing, the row gather and the weighted scatter-add are torch
tensor plumbing around them.

Expert parallelism: experts are split contiguously over the ranks, tokens start out
partitioned by rank; one all-to-all sends every (token, expert) row to the rank that
owns the expert, the local grouped GEMMs run, a second all-to-all returns the rows, and
the token's home rank does the weighted sum. ``torch.distributed`` (NCCL over NVLink on
GPUs, gloo in CPU tests) carries both exchanges.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


def route(logits: torch.Tensor, top_k: int):
    scores = torch.softmax(logits.float(), dim=-1)
    weights, experts = torch.topk(scores, top_k, dim=-1, sorted=False)
    return weights, experts


def sort_by_expert(experts: torch.Tensor, num_experts: int):
    """Flatten (token, slot) pairs and order them by expert (stable). Returns the
    permutation, the token of every sorted row and the per-expert counts."""
    flat = experts.reshape(-1)
    sorted_ids, order = torch.sort(flat, stable=True)
    token_of_row = order // experts.shape[1]
    # counts from the sorted ids (bincount would make the host wait for the largest id)
    edges = torch.searchsorted(sorted_ids, torch.arange(num_experts + 1, device=flat.device, dtype=flat.dtype))
    counts = edges[1:] - edges[:-1]
    return order, token_of_row, counts


class ExpertMLP:
    """``y = W2( silu(g) * u )`` with ``[g, u] = W1(x)`` for rows sorted by expert.

    ``gemm1`` / ``gemm2`` map (rows sorted by expert, per-expert counts) to outputs and
    ``act`` maps the (rows, 2H) intermediate to (rows, H); on a GPU they are
    ``ops.gemm_grouped`` and ``ops.silu_mul``, CPU tests inject stand-ins. ``combine``
    maps (rows, (T, k) row indices, (T, k) weights) to the (T, H) weighted sums
    (``ops.moe_combine`` on a GPU, a torch gather-and-sum otherwise)."""

    def __init__(self, gemm1: Callable, gemm2: Callable, act: Callable, combine: Optional[Callable] = None):
        self.gemm1, self.gemm2, self.act = gemm1, gemm2, act
        self.combine = combine or torch_combine

    def __call__(self, x_sorted: torch.Tensor, counts: Sequence[int]) -> torch.Tensor:
        h = self.gemm1(x_sorted, counts)
        return self.gemm2(self.act(h), counts)


def torch_combine(y: torch.Tensor, row_of: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    return (y[row_of].float() * weights.unsqueeze(-1)).sum(1).to(y.dtype)


def rows_of_tokens(order: torch.Tensor, top_k: int) -> torch.Tensor:
    """(T, k) index of every (token, slot) pair's row in the expert-sorted order."""
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    return inv.view(-1, top_k)


def expert_token_tile(rows: int, num_groups: int, N: int, device=None, sms: Optional[int] = None) -> int:
    """Token tile of a grouped GEMM over ``rows`` rows: 128 when the problem has so many tiles that
    the schedule hands out whole tiles in short spans (at least 16 tiles per SM: no partial tiles,
    no fix-up pass, and an expert's ragged row count wastes half as much padding), else 256.
    ``sms``: the SM count, read from ``device`` when not given."""
    if sms is None:
        sms = torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device()).multi_processor_count
    tiles = (rows // 128 + num_groups) * ((N + 127) // 128)
    return 128 if tiles >= 16 * sms else 256


def make_gpu_expert_mlp(w1_packed, w2_packed, token_tile: Optional[int] = None) -> ExpertMLP:
    """The expert MLP on this library's kernels. ``token_tile=None`` picks the tile per call
    (:func:`expert_token_tile`): on the 64-expert, top-6 layer with 16384 tokens the 128-token tile
    measured 2.49 ms against 3.19 ms for the 256-token tile."""
    from . import ops

    def gemm(w):
        def run(x, counts):
            tt = token_tile or expert_token_tile(x.shape[0], w.num_groups, w.N, x.device)
            return ops.gemm_grouped(x, w, counts, token_tile=tt)
        return run

    return ExpertMLP(gemm(w1_packed), gemm(w2_packed), ops.silu_mul, ops.moe_combine)


def moe_forward(x: torch.Tensor, logits: torch.Tensor, top_k: int, num_experts: int, mlp: ExpertMLP) -> torch.Tensor:
    """Single-device MoE layer: route, gather rows by expert, expert MLP, weighted combine."""
    weights, experts = route(logits, top_k)
    order, token_of_row, counts = sort_by_expert(experts, num_experts)
    x_sorted = x.index_select(0, token_of_row)
    # on a GPU the counts stay on the device: the grouped GEMMs plan their work there
    y = mlp(x_sorted, counts if counts.is_cuda else counts.tolist())
    return mlp.combine(y, rows_of_tokens(order, top_k), weights.contiguous())


def expert_ranges(num_experts: int, world_size: int) -> List[range]:
    per = (num_experts + world_size - 1) // world_size
    return [range(min(r * per, num_experts), min((r + 1) * per, num_experts)) for r in range(world_size)]


def moe_forward_ep(x_local: torch.Tensor, logits_local: torch.Tensor, top_k: int, num_experts: int,
                   local_mlp: ExpertMLP, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Expert-parallel MoE layer. ``x_local`` are this rank's tokens; ``local_mlp`` runs this
    rank's experts (counts are given for the local experts only, in order)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    ranges = expert_ranges(num_experts, world)
    weights, experts = route(logits_local, top_k)
    order, token_of_row, counts = sort_by_expert(experts, num_experts)     # rows sorted by global expert id
    x_sorted = x_local.index_select(0, token_of_row)

    # the full count matrix (every rank learns what it will receive): one collective, one sync
    flat_counts = counts.new_empty(world * num_experts)
    dist.all_gather_into_tensor(flat_counts, counts.contiguous(), group=group)
    all_counts_dev = flat_counts.view(world, num_experts)
    # The one host wait of the layer: the split sizes of the two all-to-alls are host
    # arguments. Only the per-rank totals come to the host (2 * world numbers); the per-expert
    # counts stay on the device and the grouped GEMMs plan their work there.
    my = ranges[rank]
    bounds = torch.tensor([r.start for r in ranges] + [ranges[-1].stop], device=counts.device)
    csum = torch.cat((all_counts_dev.new_zeros(world, 1), all_counts_dev.cumsum(1)), dim=1)    # (world, E + 1)
    per_rank = csum[:, bounds[1:]] - csum[:, bounds[:-1]]                  # [source rank, owner rank] rows
    totals = torch.stack((per_rank[rank], per_rank[:, rank])).cpu()        # what I send to / receive from each rank
    send_rows, recv_rows = totals[0].tolist(), totals[1].tolist()
    mine_dev = all_counts_dev[:, my.start:my.stop]                         # (world, local experts)

    recv = x_sorted.new_empty((sum(recv_rows), x_sorted.shape[1]))
    dist.all_to_all_single(recv, x_sorted.contiguous(), recv_rows, send_rows, group=group)

    # received rows are ordered (source rank, expert); regroup them by expert for the grouped GEMM
    local_ids = torch.arange(len(my), device=recv.device).repeat(world)
    src_expert = torch.repeat_interleave(local_ids, mine_dev.reshape(-1), output_size=sum(recv_rows))
    regroup = torch.argsort(src_expert, stable=True)
    local_counts = mine_dev.sum(0)
    y_grouped = local_mlp(recv.index_select(0, regroup), local_counts if local_counts.is_cuda else local_counts.tolist())
    ungroup = torch.empty_like(regroup)
    ungroup[regroup] = torch.arange(regroup.numel(), device=regroup.device)
    y = y_grouped.index_select(0, ungroup)                                 # back to (source rank, expert) order

    back = y.new_empty((x_sorted.shape[0], y.shape[1]))
    dist.all_to_all_single(back, y.contiguous(), send_rows, recv_rows, group=group)

    return local_mlp.combine(back, rows_of_tokens(order, top_k), weights.contiguous())
