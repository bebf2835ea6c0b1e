"""Host-side failure detection for the expert-parallel layer.

Nothing here touches a GPU: a peer that has gone away is noticed on the host, through a key-value store, before the
next kernel or collective is launched, and an exchange whose counts do not add up is refused on every rank at once
instead of being handed to a collective that would wait for rows that never come.
"""
from __future__ import annotations

import time
from typing import Optional

import torch
import torch.distributed as dist


class PeerLostError(RuntimeError):
    """A rank of the group has left or stopped announcing steps."""


class ExchangeMismatchError(RuntimeError):
    """The row counts of an exchange are inconsistent on at least one rank."""


class StepHeartbeat:
    """Every rank writes the number of the step it is about to run under its own key of a c10d store (a FileStore or
    TCPStore shared by the group); `check(step)` returns once every peer has announced that step, and raises
    `PeerLostError` if a peer said it was leaving or stays silent for `timeout_s`.  A rank leaves only between steps
    (`leave()`), with none of its kernels or collectives in flight."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 2.0, prefix: str = "amoe/step"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def announce(self, step: int) -> None:
        self._last = int(step)
        self.store.set(self._key(self.rank), str(int(step)))

    def leave(self) -> None:
        # the last step this rank ran travels with the note: a slower peer still checking that step is not misled
        self.store.set(self._key(self.rank), f"left:{getattr(self, '_last', -1)}")

    def check(self, step: int) -> None:
        deadline = time.monotonic() + self.timeout_s
        for r in range(self.world):
            if r == self.rank:
                continue
            while True:
                val = None
                if self.store.check([self._key(r)]):
                    val = self.store.get(self._key(r)).decode()
                if val is not None and val.startswith("left"):
                    if int(val.partition(":")[2] or -1) >= step:
                        break                       # it ran this step and left afterwards: the next check reports it
                    raise PeerLostError(f"rank {r} left the group before step {step}")
                if val is not None and int(val) >= step:
                    break
                if time.monotonic() > deadline:
                    raise PeerLostError(f"rank {r} did not announce step {step} within {self.timeout_s:.1f} s "
                                        f"(last seen: {val})")
                time.sleep(0.01)


def agree_or_raise(ok: bool, group=None, what: str = "exchange", device: Optional[torch.device] = None) -> None:
    """All ranks learn whether every rank's local check passed (one small all-reduce) and raise together if not: no rank
    walks into the data exchange alone."""
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    if int(flag) == 0:
        raise ExchangeMismatchError(f"{what}: the row counts are inconsistent on at least one rank"
                                    + ("" if ok else " (this one)"))


def counts_consistent(gathered: torch.Tensor, rank: int, local_rows: int) -> bool:
    """gathered [G, G, El] (source, destination, local expert), host tensor: this rank's row of it must account for
    exactly the rows this rank routes, and no count may be negative."""
    if bool((gathered < 0).any()):
        return False
    return int(gathered[rank].sum()) == int(local_rows)
