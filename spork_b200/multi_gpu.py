"""Host-side failure detection for sharded (one process per GPU) runs.

The ranks of an M-sharded GEMM or a head-sharded attention run exchange no data, so a rank that has failed
would otherwise go unnoticed until the result is missing.  Before a launch, every rank publishes its state
under a per-step key of the job's key-value store and reads everyone else's: a rank that reported an error,
or that never reports within the time limit (it crashed or never joined), makes the others stop *before*
they launch anything.  Nothing here touches a GPU; the device-side half of failure detection is the bounded
wait + status word of the kernels.  The reference is single-process and has no counterpart.
"""
from __future__ import annotations

import datetime


class RankFailure(RuntimeError):
    """Raised on every surviving rank when some rank reported a failure or did not report in time."""

    def __init__(self, step, failed: dict[int, str]):
        self.step = step
        self.failed = dict(failed)
        ranks = ", ".join(f"rank {r}: {why}" for r, why in sorted(self.failed.items()))
        super().__init__(f"step {step!r} not started: {ranks}")


class RankHealth:
    """Per-step health exchange over a torch.distributed key-value store."""

    def __init__(self, store, rank: int, world: int, prefix: str = "spork_b200/health"):
        if world < 1 or not (0 <= rank < world):
            raise ValueError(f"bad rank/world: {rank}/{world}")
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def _key(self, step, rank: int) -> str:
        return f"{self.prefix}/{step}/{rank}"

    def report(self, step, error: str | None = None) -> None:
        """Publish this rank's state for `step`: healthy (error is None) or failed with a reason."""
        self.store.set(self._key(step, self.rank), "ok" if error is None else "failed: " + error)

    def check(self, step, timeout_s: float = 30.0) -> None:
        """Wait until every rank has reported for `step`; raise RankFailure unless all are healthy."""
        failed: dict[int, str] = {}
        for r in range(self.world):
            key = self._key(step, r)
            try:
                self.store.wait([key], datetime.timedelta(seconds=timeout_s))
                state = self.store.get(key).decode()
            except Exception:  # the store raises on timeout: the rank never reported
                failed[r] = f"no report within {timeout_s:g} s"
                continue
            if state != "ok":
                failed[r] = state
        if failed:
            raise RankFailure(step, failed)

    def guard(self, step, fn, timeout_s: float = 30.0):
        """Run fn() (this rank's part of `step`, e.g. set-up or a status check), publish whether it raised, then
        check everyone.  Returns fn's result on every rank when all ranks succeeded."""
        try:
            result = fn()
        except Exception as exc:  # publish first so that the other ranks stop, then re-raise here
            self.report(step, f"{type(exc).__name__}: {exc}")
            raise
        self.report(step)
        self.check(step, timeout_s)
        return result


def default_store():
    """The key-value store of the default process group (valid after init_process_group)."""
    import torch.distributed as dist

    return dist.distributed_c10d._get_default_store()
