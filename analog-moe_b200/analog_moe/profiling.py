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


def timeline(path: str, run_step: Callable[[int], object], rank: int = 0, n: int = 3) -> None:
    """Runs `run_step(i)` n times under the profiler (every rank, so that collectives meet) and has rank 0 write, for
    the last of them, one line per kernel: start (us from the step's first kernel), duration, stream, name.  For
    steps replayed from a CUDA graph, where no host gap hides the order the device runs them in."""
    from torch.profiler import profile, ProfilerActivity
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for i in range(n):
            run_step(i)
        torch.cuda.synchronize()
    if rank != 0:
        return
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    ev.sort(key=lambda e: e.time_range.start)
    per = len(ev) // n
    last = ev[-per:] if per else ev
    t0 = last[0].time_range.start
    t1 = max(e.time_range.end for e in last)
    iv = sorted((e.time_range.start, e.time_range.end) for e in last)
    busy, (cs, ce) = 0.0, iv[0]
    for s_, e_ in iv[1:]:
        if s_ > ce:
            busy, cs, ce = busy + ce - cs, s_, e_
        else:
            ce = max(ce, e_)
    busy += ce - cs
    with open(path, "w") as f:
        f.write(f"kernels per step {per}, span {t1 - t0:.1f} us, some kernel running {busy:.1f} us\n")
        for e in last:
            f.write(f"{e.time_range.start - t0:9.1f} {e.time_range.end - e.time_range.start:8.1f}  {e.name[:90]}\n")
