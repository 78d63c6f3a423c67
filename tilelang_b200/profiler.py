"""Parity check and timing helpers with the reference profiler's conventions.

``assert_allclose`` applies the reference's acceptance rule: element-wise
``|x - ref| <= atol + rtol * |ref|`` with at most ``max_mismatched_ratio`` of the
elements allowed to miss (tilelang/profiler/__init__.py:104-162,
tilelang/utils/tensor.py:205-293). ``do_bench`` follows the reference's recipe
(tilelang/profiler/bench.py:68-141, 172-236): a 256 MB buffer is zeroed before
every timed call to flush L2, each call is bracketed by CUDA events, about 25 ms
of warm-up and 100 ms of measurement.
"""
from __future__ import annotations

import enum
from typing import Callable, List, Optional

import torch


class TensorSupplyType(enum.Enum):
    """Input generators of the reference (tilelang/utils/tensor.py:32-40)."""
    Integer = 1
    Uniform = 2
    Normal = 3
    Randn = 4
    Zero = 5
    One = 6
    Auto = 7


def supply_tensor(shape, dtype: torch.dtype, supply: TensorSupplyType, device, gen: Optional[torch.Generator] = None):
    """Same value ranges as tilelang/utils/tensor.py:42-118: Auto/Integer give
    unsigned ints in {0,1,2}, floats U(-1,1), other ints in [-2,2]."""
    is_float = dtype.is_floating_point
    is_unsigned = dtype == torch.uint8
    if supply in (TensorSupplyType.Auto, TensorSupplyType.Integer):
        if supply == TensorSupplyType.Auto and is_float:
            return (torch.rand(shape, device=device, generator=gen) * 2 - 1).to(dtype)
        if is_unsigned:
            return torch.randint(0, 3, shape, device=device, generator=gen, dtype=torch.int32).to(dtype)
        return torch.randint(-2, 3, shape, device=device, generator=gen, dtype=torch.int32).to(dtype)
    if supply == TensorSupplyType.Uniform:
        return (torch.rand(shape, device=device, generator=gen) * 2 - 1).to(dtype)
    if supply in (TensorSupplyType.Normal, TensorSupplyType.Randn):
        return torch.randn(shape, device=device, generator=gen).to(dtype)
    if supply == TensorSupplyType.Zero:
        return torch.zeros(shape, device=device, dtype=dtype)
    if supply == TensorSupplyType.One:
        return torch.ones(shape, device=device, dtype=dtype)
    raise ValueError(supply)


def torch_assert_close(x: torch.Tensor, ref: torch.Tensor, rtol: float = 1e-2, atol: float = 1e-2,
                       max_mismatched_ratio: float = 0.01, name: str = "output") -> None:
    if x.shape != ref.shape:
        raise AssertionError(f"{name}: shape {tuple(x.shape)} != reference {tuple(ref.shape)}")
    xd, rd = x.detach().double().cpu(), ref.detach().double().cpu()
    bad = (xd - rd).abs() > (atol + rtol * rd.abs())
    n_bad, n = int(bad.sum()), bad.numel()
    if n_bad > int(n * max_mismatched_ratio):
        worst = ((xd - rd).abs() - (atol + rtol * rd.abs())).max().item()
        raise AssertionError(f"{name}: {n_bad}/{n} elements ({n_bad / max(n, 1):.3%}) outside rtol={rtol} atol={atol} "
                             f"(allowed {max_mismatched_ratio:.1%}); worst excess {worst:.4g}")


def do_bench(fn: Callable[[], object], warmup: float = 25, rep: float = 100, n_warmup: int = 0, n_repeat: int = 0,
             return_mode: str = "mean", flush_l2: bool = True, quantiles: Optional[List[float]] = None):
    """Milliseconds per call of ``fn`` on the current stream, L2 flushed before each call."""
    fn()
    torch.cuda.synchronize()
    cache = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device="cuda") if flush_l2 else None
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(5):
        if cache is not None:
            cache.zero_()
        fn()
    end.record()
    torch.cuda.synchronize()
    estimate = start.elapsed_time(end) / 5
    nw = n_warmup or max(1, int(warmup / max(estimate, 1e-6)))
    nr = n_repeat or max(1, int(rep / max(estimate, 1e-6)))
    for _ in range(nw):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(nr)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(nr)]
    for i in range(nr):
        if cache is not None:
            cache.zero_()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    times = torch.tensor([s.elapsed_time(e) for s, e in zip(starts, ends)], dtype=torch.float64)
    if quantiles is not None:
        return torch.quantile(times, torch.tensor(quantiles, dtype=torch.float64)).tolist()
    return {"mean": times.mean, "min": times.min, "max": times.max, "median": times.median}[return_mode]().item()


class Profiler:
    """Stands where ``kernel.get_profiler()`` returns the reference's Profiler
    (tilelang/profiler/__init__.py:21-291)."""

    def __init__(self, kernel, supply_type: TensorSupplyType = TensorSupplyType.Auto, seed: int = 0):
        self.kernel = kernel
        self.supply_type = supply_type
        self.seed = seed

    def _get_inputs(self, with_output: bool = False):
        gen = torch.Generator(device="cuda")
        gen.manual_seed(self.seed)
        params = self.kernel.params
        n_out = len(self.kernel.out_idx) if self.kernel.out_idx else 0
        take = params if with_output or n_out == 0 else params[:len(params) - n_out]
        return [supply_tensor(p.shape, p.dtype, self.supply_type, "cuda", gen) for p in take]

    def run_once(self, func: Optional[Callable] = None):
        ins = self._get_inputs()
        return (func or self.kernel)(*ins)

    def assert_allclose(self, reference_program: Callable, input_tensors=None, atol: float = 1e-2, rtol: float = 1e-2,
                        max_mismatched_ratio: float = 0.01):
        ins = input_tensors if input_tensors is not None else self._get_inputs()
        ref = reference_program(*ins)
        out = self.kernel(*ins)
        torch.cuda.synchronize()
        if out is None:      # kernels without out_idx fill their last argument
            out = ins[-1]
        outs = out if isinstance(out, (list, tuple)) else [out]
        refs = ref if isinstance(ref, (list, tuple)) else [ref]
        if len(outs) != len(refs):
            raise AssertionError(f"kernel returned {len(outs)} tensors, reference {len(refs)}")
        for i, (o, r) in enumerate(zip(outs, refs)):
            torch_assert_close(o, r.to(o.device), rtol=rtol, atol=atol, max_mismatched_ratio=max_mismatched_ratio,
                               name=f"output[{i}]")

    def assert_consistent(self, repeat: int = 10):
        """Re-run on the same inputs and demand bit-identical outputs
        (tilelang/profiler/__init__.py:195-212)."""
        ins = self._get_inputs()
        first = self.kernel(*ins)
        first = ins[-1].clone() if first is None else first.clone()
        for _ in range(repeat - 1):
            out = self.kernel(*ins)
            out = ins[-1] if out is None else out
            if not torch.equal(out, first):
                raise AssertionError("kernel output changed between identical runs")

    def do_bench(self, func: Optional[Callable] = None, warmup: int = 25, rep: int = 100, n_warmup: int = 0,
                 n_repeat: int = 0, input_tensors=None, return_mode: str = "mean", **_ignored) -> float:
        ins = input_tensors if input_tensors is not None else self._get_inputs()
        target = func or self.kernel
        return do_bench(lambda: target(*ins), warmup=warmup, rep=rep, n_warmup=n_warmup, n_repeat=n_repeat,
                        return_mode=return_mode)
