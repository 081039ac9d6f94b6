"""Failure detection between steps, on the host.

The reference has no timeouts or heartbeats at all. Here every rank publishes a heartbeat
(`hb/<rank>` = last completed step, wall time) in the job's key-value store after each step and,
before launching the next one, checks that every peer has reached the same step within a
tolerance; a missing or stale peer raises `RankFailure` *before* any kernel that waits on that
peer is launched. Device-side waits are bounded as a second line of defence (they record
`kTimeoutPeer` in the status word, which `check_device_status` turns into an exception).
No GPU is ever faulted or hung to test this: tests drive ranks that stop heart-beating.
"""
from __future__ import annotations

import time

import torch.distributed as dist


class RankFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class HeartbeatMonitor:
    def __init__(self, store, rank: int, world_size: int, timeout_s: float = 30.0,
                 poll_s: float = 0.02, prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.timeout_s, self.poll_s, self.prefix = timeout_s, poll_s, prefix

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}")

    def leave(self) -> None:
        """Announce an orderly departure (between steps, nothing in flight)."""
        self.store.set(self._key(self.rank), "left")

    def _read(self, r: int):
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            raw = self.store.get(self._key(r)).decode()
        except Exception:
            return None
        if raw == "left":
            return "left"
        step, ts = raw.split(":")
        return int(step), float(ts)

    def wait_all(self, step: int) -> None:
        """Block until every peer has completed `step`, or raise RankFailure."""
        deadline = time.time() + self.timeout_s
        pending = set(range(self.world)) - {self.rank}
        while pending:
            for r in sorted(pending):
                v = self._read(r)
                if v == "left":
                    raise RankFailure(r, "left the job")
                if v is not None and v[0] >= step:
                    pending.discard(r)
            if not pending:
                return
            if time.time() > deadline:
                r = sorted(pending)[0]
                v = self._read(r)
                raise RankFailure(r, f"no heartbeat for step {step} within {self.timeout_s}s "
                                     f"(last seen: {v})")
            time.sleep(self.poll_s)


def default_store():
    """The TCPStore torch.distributed rendezvoused on (None before init_process_group)."""
    if not dist.is_initialized():
        return None
    return dist.distributed_c10d._get_default_store()


def check_device_status(device=None) -> None:
    """Raise if a bounded device-side wait gave up (synchronises the device)."""
    from ..ops import _lib
    _lib.check_status(device)
