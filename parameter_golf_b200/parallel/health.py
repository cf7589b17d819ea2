"""Host-side failure detection between training steps: heartbeats and failure reports through the process group's store.

The reference turns worker panics and library errors into one error value of its single process
(``parameter-golf-rs/crates/pg-train/src/lib.rs:4019-4023``, ``pg-core/src/error.rs:6-34``) and has no cross-rank
detection. With one process per GPU a rank that raises between steps would leave its peers waiting in their next
collective kernel until the kernel's own bounded wait gives up; here the peers learn of it on the host first:

* every rank posts ``hb/<rank> = "<step>:<unix time>"`` after each step (`beat`);
* a rank that fails posts ``failed = "rank<r>: <reason>"`` (`fail`, or automatically through `guard`);
* before launching a step every rank calls `check`, which raises `PeerFailure` when a failure was posted or when a
  peer that has already beaten once has been silent for longer than ``timeout_s``.

Nothing here touches a GPU: a rank leaves only between steps, with none of its kernels or collectives in flight, and
recovery is a restart from the last full-state checkpoint.
"""
from __future__ import annotations

import contextlib
import time
from typing import Optional


class PeerFailure(RuntimeError):
    """Another rank reported a failure or stopped sending heartbeats."""


class RankHealth:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 120.0, prefix: str = "pgb/health", clock=time.time):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.prefix, self.clock = timeout_s, prefix, clock

    @classmethod
    def from_process_group(cls, timeout_s: float = 120.0) -> Optional["RankHealth"]:
        """Health channel on the default process group's store, or ``None`` when not running distributed."""
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
            return None
        store = dist.distributed_c10d._get_default_store()
        return cls(store, dist.get_rank(), dist.get_world_size(), timeout_s)

    def _key(self, name: str) -> str:
        return f"{self.prefix}/{name}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(f"hb/{self.rank}"), f"{step}:{self.clock():.3f}")

    def fail(self, reason: str) -> None:
        self.store.set(self._key("failed"), f"rank{self.rank}: {reason}")

    def failure(self) -> Optional[str]:
        if self.store.check([self._key("failed")]):
            return self.store.get(self._key("failed")).decode()
        return None

    def check(self) -> None:
        """Raise `PeerFailure` if any rank reported a failure or a peer's heartbeat is older than the timeout."""
        msg = self.failure()
        if msg is not None:
            raise PeerFailure(msg)
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            key = self._key(f"hb/{r}")
            if not self.store.check([key]):
                continue                      # has not finished its first step yet: start-up time is not policed here
            step, ts = self.store.get(key).decode().split(":")
            if now - float(ts) > self.timeout_s:
                raise PeerFailure(f"rank{r} silent for {now - float(ts):.1f}s (last heartbeat at step {step})")

    @contextlib.contextmanager
    def guard(self):
        """Report any exception raised inside the block to the other ranks before re-raising it."""
        try:
            yield
        except PeerFailure:
            raise
        except BaseException as e:          # noqa: BLE001 - the report must also cover KeyboardInterrupt / SystemExit
            # a peer that failed inside the same step usually surfaces here as a broken collective: name the root cause
            peer = None
            try:
                peer = self.failure()
            except Exception:               # noqa: BLE001 - the store itself may be gone
                pass
            if peer is not None and not peer.startswith(f"rank{self.rank}:"):
                raise PeerFailure(peer) from e
            try:
                self.fail(f"{type(e).__name__}: {e}")
            finally:
                raise
