"""Failure detection on the host: peer heartbeats over the job's key-value store, and a non-finite-loss policy.

The reference has neither (its only knob is the distributed-init timeout, mintext/config.py:286 and
mintext/distributed/mesh.py:60-71; recovery is restart + auto-resume, mintext/checkpoint/manager.py:126-133).
Here every rank publishes a heartbeat counter from a background thread; before a step a rank can ask whether all
peers are still alive, and a missing peer becomes a clean ``PeerFailure`` on the survivors instead of a hang inside
the next collective.  Device-side waits are bounded separately (kernels record a status word that
``ops._ext.check_status`` raises on); together they let the launcher restart from the last checkpoint.
"""

from __future__ import annotations

import threading
import time


class PeerFailure(RuntimeError):
    """A peer stopped publishing heartbeats (it exited, hung, or lost its connection to the store)."""


class Heartbeat:
    """``store``: a ``torch.distributed`` store (TCPStore / FileStore / HashStore) shared by all ranks."""

    def __init__(self, store, rank: int, world: int, interval_s: float = 1.0, timeout_s: float = 30.0,
                 prefix: str = "mt_hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = float(interval_s), float(timeout_s), prefix
        # A store client is one socket: the publishing thread gets its own connection (Store.clone) where the store
        # supports it, and a lock serialises the two users otherwise.
        self._lock = threading.Lock()
        try:
            self._pub_store = store.clone()
        except Exception:
            self._pub_store = store
        self._stop = threading.Event()
        self._beat = 0
        self._seen: dict[int, tuple[int, float]] = {}
        self._publish()
        self._thread = threading.Thread(target=self._run, name="mt-heartbeat", daemon=True)
        self._thread.start()

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def _publish(self) -> None:
        self._beat += 1
        with self._lock:
            self._pub_store.set(self._key(self.rank), str(self._beat))

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self._publish()
            except Exception:  # the store is gone: peers will see this rank as failed
                return

    def check(self) -> None:
        """Raise :class:`PeerFailure` naming every peer whose counter has not advanced for ``timeout_s``."""
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                with self._lock:
                    beat = int(self.store.get(self._key(r)).decode()) if self.store.check([self._key(r)]) else 0
            except Exception as e:
                raise PeerFailure(f"rank {self.rank}: heartbeat store unreachable ({e})") from e
            last = self._seen.get(r)
            if last is None or beat != last[0]:
                self._seen[r] = (beat, now)
            elif now - last[1] > self.timeout_s:
                dead.append(r)
        if dead:
            raise PeerFailure(f"rank {self.rank}: no heartbeat from rank(s) {dead} for more than {self.timeout_s:.1f} s")

    def wait_all_alive(self, deadline_s: float) -> None:
        """Block until every peer has published at least once (start-up), or raise after ``deadline_s``."""
        t0 = time.monotonic()
        while True:
            with self._lock:
                missing = [r for r in range(self.world) if r != self.rank and not self.store.check([self._key(r)])]
            if not missing:
                return
            if time.monotonic() - t0 > deadline_s:
                raise PeerFailure(f"rank {self.rank}: rank(s) {missing} never joined within {deadline_s:.1f} s")
            time.sleep(min(0.05, self.interval_s))

    def close(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2 * self.interval_s + 1.0)


class NonFiniteLoss(RuntimeError):
    """The step produced a NaN / Inf loss and the policy is ``abort``."""


def apply_nan_policy(policy: str, loss_value: float, step: int) -> bool:
    """Returns True when the step's update must be skipped.  ``policy``: ``ignore`` (reference behaviour: nothing is
    checked, mintext/utils/pytree.py:16-25 is never called), ``skip`` (drop the update, keep the weights),
    ``abort`` (raise so the launcher restarts from the last checkpoint)."""
    if policy == "ignore" or loss_value == loss_value and abs(loss_value) != float("inf"):
        return False
    if policy == "abort":
        raise NonFiniteLoss(f"non-finite loss {loss_value} at step {step}")
    if policy == "skip":
        return True
    raise ValueError(f"unknown nan_policy '{policy}'")
