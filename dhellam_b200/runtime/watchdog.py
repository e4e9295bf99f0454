"""Host-side failure detection: heartbeats and step agreement over the rendezvous store.

The reference relies on ``--distributed-timeout-minutes`` and NCCL's asynchronous error
handling only (script/run.sh:39, 135).  Here every rank publishes a heartbeat from a
background thread and, before it launches a step, its step number; a rank that stops
(crashed, hung on the host, never joined) is noticed by the others *on the host, before
their next launch*, and they raise ``RankFailure`` instead of entering a collective that
can never complete.  Device-side waits are bounded separately (``runtime/signals.py``).

Nothing here touches a GPU, so the whole module is exercised with CPU ranks.
"""
from __future__ import annotations

import threading
import time
from typing import List, Optional

import torch.distributed as dist


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int], why: str):
        self.ranks = ranks
        super().__init__(f"rank(s) {ranks} {why}")


def default_store():
    from torch.distributed.distributed_c10d import _get_default_store
    return _get_default_store()


class Heartbeat:
    """Publishes ``hb/<rank>`` every ``interval`` seconds; ``dead_ranks`` lists ranks whose
    last beat is older than ``timeout``."""

    def __init__(self, store=None, rank: Optional[int] = None, world: Optional[int] = None, interval: float = 0.2,
                 timeout: float = 2.0, prefix: str = "hb", startup_timeout: float = 60.0):
        self.store = store if store is not None else default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self._stop = threading.Event()
        self._paused = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._beat()
        self._thread.start()
        self._wait_all_started(startup_timeout)

    def _wait_all_started(self, startup_timeout: float):
        """Construction is a rendezvous: a rank that has not published its first beat yet is
        starting up, not dead.  A rank that never joins makes this raise."""
        deadline = time.time() + startup_timeout
        missing = [r for r in range(self.world) if r != self.rank]
        while missing:
            missing = [r for r in missing if not self.store.check([f"{self.prefix}/{r}"])]
            if missing and time.time() > deadline:
                raise RankFailure(missing, f"never joined (no first heartbeat within {startup_timeout} s)")
            if missing:
                time.sleep(0.02)

    def _beat(self):
        self.store.set(f"{self.prefix}/{self.rank}", str(time.time()))

    def _run(self):
        while not self._stop.wait(self.interval):
            if not self._paused.is_set():
                try:
                    self._beat()
                except Exception:
                    return

    def pause(self):
        """Stops beating without stopping the process (fault injection: a hung rank)."""
        self._paused.set()

    def resume(self):
        self._paused.clear()

    def stop(self):
        """Ends the beating thread and waits for it, so that no store call is in flight when the
        caller tears the process group (and with it the store) down."""
        self._stop.set()
        if self._thread.is_alive() and threading.current_thread() is not self._thread:
            self._thread.join(timeout=5.0)

    def dead_ranks(self) -> List[int]:
        now = time.time()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if not self.store.check([f"{self.prefix}/{r}"]):
                    dead.append(r)
                    continue
                t = float(self.store.get(f"{self.prefix}/{r}").decode())
            except Exception:
                dead.append(r)
                continue
            if now - t > self.timeout:
                dead.append(r)
        return dead

    def check(self):
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(dead, f"sent no heartbeat for more than {self.timeout} s")


class StepGate:
    """Every rank announces the step it is about to launch and waits (bounded) until all
    ranks have announced the same step; a stale announcement (a rank replaying an older
    step after a partial restart) is an error, not a hang."""

    def __init__(self, store=None, rank: Optional[int] = None, world: Optional[int] = None, timeout: float = 5.0,
                 heartbeat: Optional[Heartbeat] = None, prefix: str = "step"):
        self.store = store if store is not None else default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.timeout, self.heartbeat, self.prefix = timeout, heartbeat, prefix

    def announce(self, step: int, epoch: int = 0):
        self.store.set(f"{self.prefix}/{self.rank}", f"{epoch}:{step}")

    def agree(self, step: int, epoch: int = 0, poll: float = 0.02):
        """Announces ``step`` and returns once every rank announced it.  Raises
        ``RankFailure`` if a rank is dead, late beyond ``timeout`` or in another epoch."""
        self.announce(step, epoch)
        deadline = time.time() + self.timeout
        pending = set(range(self.world)) - {self.rank}
        while pending:
            for r in list(pending):
                key = f"{self.prefix}/{r}"
                if self.store.check([key]):
                    e, s = (int(x) for x in self.store.get(key).decode().split(":"))
                    if e != epoch:
                        raise RankFailure([r], f"is in restart epoch {e}, this rank is in epoch {epoch}")
                    if s >= step:
                        pending.discard(r)
            if not pending:
                return
            if self.heartbeat is not None:
                dead = [r for r in self.heartbeat.dead_ranks() if r in pending]
                if dead:
                    raise RankFailure(dead, "stopped before reaching step %d" % step)
            if time.time() > deadline:
                raise RankFailure(sorted(pending), f"did not reach step {step} within {self.timeout} s")
            time.sleep(poll)
