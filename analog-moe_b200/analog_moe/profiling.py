"""Per-kernel device times of a layer step (torch profiler, CUDA activity only) and NVTX ranges.

`ops.NVTX = True` (or AMOE_NVTX=1) puts an NVTX range around every library call.  `kernel_times` is for
runs a kernel profiler cannot attach to (several ranks): it is not a benchmark, since kernels of different
streams overlap in a step and collectives include the time they wait for the other ranks.
"""
from __future__ import annotations

from typing import Callable

import torch


def kernel_times(path: str, run_step: Callable[[int], object], rank: int = 0, world: int = 1, n: int = 3) -> None:
    """Runs `run_step(i)` n times eagerly under the profiler; rank 0 writes to `path` one line per rank with the
    totals of the kernel families, then its own table."""
    from torch.profiler import profile, ProfilerActivity
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for i in range(n):
            run_step(i)
        torch.cuda.synchronize()
    ka = prof.key_averages()

    def tot(pat):
        return sum(e.device_time_total for e in ka if pat in e.key) / n

    line = (f"rank {rank}: cvmm_tc {tot('cvmm_tc'):.0f}  dw_tc {tot('dw_tc'):.0f}  ep_put {tot('ep_put_kernel'):.0f}  "
            f"ep_put_back {tot('ep_put_back'):.0f}  all kernels but nccl "
            f"{sum(e.device_time_total for e in ka if 'nccl' not in e.key) / n:.0f} us per step")
    lines = [line]
    if world > 1:
        import torch.distributed as dist
        lines = [None] * world
        dist.all_gather_object(lines, line)
    if rank == 0:
        with open(path, "w") as f:
            f.write("\n".join(lines) + "\n")
            f.write(ka.table(sort_by="cuda_time_total", row_limit=30, max_name_column_width=80))
