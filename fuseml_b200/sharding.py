"""Row sharding over the GPUs of one box.

Every op of a fused chain is independent per row of the activation matrix, so a batch of M
rows is cut into ``world`` contiguous blocks, one per GPU (one process per GPU), with the
weights replicated: no collective is needed on the data path.  Only whole-tensor reductions
(``y.sum()``, ``y.amax()``) need one exchange at the end: each rank reduces its rows (inside the
last fused kernel) and the scalars are combined with an all-reduce — SUM for sums, MAX for
maxima; a global mean is the all-reduced sum divided by the global element count.  The
reference has no distributed code at all; this module is new with the B200 build.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist


def row_range(M: int, world: int, rank: int) -> tuple[int, int]:
    """Rows ``[start, stop)`` of rank ``rank``: contiguous, sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world {world}")
    base, extra = divmod(int(M), world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_rows(x: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """This rank's block of rows (a view, no copy)."""
    a, b = row_range(x.shape[0], world, rank)
    return x[a:b]


def allreduce_scalars(total: torch.Tensor | None = None, maximum: torch.Tensor | None = None,
                      group=None) -> tuple[torch.Tensor | None, torch.Tensor | None]:
    """Combine per-rank partial sums / maxima in fp32 (in place on fp32 copies)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return (None if total is None else total.float(), None if maximum is None else maximum.float())
    out_s = out_m = None
    if total is not None:
        out_s = total.detach().float().clone()
        dist.all_reduce(out_s, op=dist.ReduceOp.SUM, group=group)
    if maximum is not None:
        out_m = maximum.detach().float().clone()
        dist.all_reduce(out_m, op=dist.ReduceOp.MAX, group=group)
    return out_s, out_m


class RowShardedModule:
    """Runs ``fn`` on this rank's rows and finishes global reductions with an all-reduce.

    ``fn(x_local) -> y_local`` or ``-> (y_local, *scalars)``; ``reductions`` names what each
    scalar is (``"sum"``, ``"max"`` or ``"mean"``) so that it can be combined correctly.
    """

    def __init__(self, fn: Callable, reductions: Sequence[str] = (), group=None) -> None:
        for r in reductions:
            if r not in ("sum", "max", "mean"):
                raise ValueError(f"unknown reduction {r!r}")
        self.fn = fn
        self.reductions = tuple(reductions)
        self.group = group

    def __call__(self, x_local: torch.Tensor, global_rows: int | None = None):
        out = self.fn(x_local)
        if not self.reductions:
            return out
        y, *scalars = out
        if len(scalars) != len(self.reductions):
            raise ValueError(f"module returned {len(scalars)} scalars, {len(self.reductions)} reductions declared")
        world = dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1
        combined = []
        for kind, s in zip(self.reductions, scalars):
            if kind == "max":
                combined.append(allreduce_scalars(maximum=s, group=self.group)[1])
            elif kind == "sum":
                combined.append(allreduce_scalars(total=s, group=self.group)[0])
            else:  # mean of equally weighted elements: weight each rank's mean by its share of rows
                if global_rows is None:
                    raise ValueError("a global mean needs global_rows")
                weight = x_local.shape[0] / float(global_rows) if world > 1 else 1.0
                combined.append(allreduce_scalars(total=s.float() * weight, group=self.group)[0])
        return (y, *combined)


def bind_to_device_numa(device_index: int, nvml=None) -> list[int] | None:
    """Pin the calling process to the CPU cores NVML reports as local to CUDA device
    ``device_index`` (its NUMA node), so that pinned host buffers allocated afterwards are
    first-touched next to the GPU that copies from them.  With one process per GPU and every
    process streaming its own batch over PCIe, buffers on the far socket make all ranks share
    the inter-socket link.  Only the process's CPU affinity changes; nothing on the GPU is
    set.  Returns the cores chosen, or None when NVML is not available, reports nothing, or
    none of the reported cores is allowed to this process (the affinity is then left alone).
    ``nvml`` is injectable for tests (an object with the pynvml functions used here)."""
    import os

    if not hasattr(os, "sched_setaffinity"):
        return None
    try:
        if nvml is None:
            import pynvml as nvml  # type: ignore[no-redef]
        nvml.nvmlInit()
        props = torch.cuda.get_device_properties(device_index)
        bus_id = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        handle = nvml.nvmlDeviceGetHandleByPciBusId(bus_id.encode())
        n_cpu = os.cpu_count() or 1
        words = list(nvml.nvmlDeviceGetCpuAffinity(handle, (n_cpu + 63) // 64))
    except Exception:
        return None
    local = {w * 64 + b for w, mask in enumerate(words) for b in range(64) if (int(mask) >> b) & 1}
    allowed = os.sched_getaffinity(0)
    chosen = sorted(local & allowed)
    if not chosen or len(chosen) == len(allowed):
        return None if not chosen else chosen
    os.sched_setaffinity(0, chosen)
    return chosen
