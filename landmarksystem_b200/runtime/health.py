"""Failure detection for multi-rank jobs.

The reference has none: a dead rank leaves every other rank blocked in its next NCCL collective until
``COMM_TIMEOUT`` (``landmark/utils/env.py:27``, ``landmark/communicator/comm_context.py:56-62``).
Here every rank publishes a heartbeat (step number + wall clock) in the job's key-value store from a
host thread, and checks its peers' heartbeats *between* steps, i.e. before it launches kernels that
would wait for them.  A peer that stopped beating, exited, or reported an error raises
:class:`PeerFailure` on the survivors, which then leave the step loop cleanly (no collective is left
half-done) and can restart from the last checkpoint.

Device-side waits of the peer-memory kernels are bounded and report through status words instead of
trapping; :class:`StatusWords` gathers those words so that a trainer can poll them off the hot path.

Everything here runs on the host (``torch.distributed`` store / gloo); no GPU is involved.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional

import torch


class PeerFailure(RuntimeError):
    """Raised on a healthy rank when another rank is found dead, stalled or failed."""

    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class HeartbeatMonitor:
    """``store``: any ``torch.distributed.Store`` shared by the job (TCPStore / FileStore / HashStore).

    ``beat(step)`` is cheap (updates a local record); a daemon thread writes it to the store every
    ``interval`` seconds.  ``check()`` reads all peers and raises :class:`PeerFailure` if a peer
    (a) reported a failure, (b) has not written for ``timeout`` seconds, or (c) lags more than
    ``max_step_lag`` steps behind while this rank waits.  ``fail(reason)`` lets a rank that caught an
    exception tell the others before it exits; ``leave()`` announces an orderly departure."""

    def __init__(self, store, rank: int, world: int, interval: float = 0.5, timeout: float = 10.0,
                 max_step_lag: Optional[int] = None, prefix: str = "lmb_hb", clock: Callable[[], float] = time.time):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.max_step_lag = interval, timeout, max_step_lag
        self.prefix, self.clock = prefix, clock
        self._step, self._state = 0, "ok"
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._publish()

    # -- publishing -----------------------------------------------------------------------------------
    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def _publish(self) -> None:
        with self._lock:
            record = f"{self._state}|{self._step}|{self.clock():.3f}"
        self.store.set(self._key(self.rank), record)

    def start(self) -> "HeartbeatMonitor":
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name="lmb-heartbeat", daemon=True)
            self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self._publish()
            except Exception:            # the store itself is gone: nothing left to tell anybody
                return

    def beat(self, step: int) -> None:
        with self._lock:
            self._step = int(step)

    def fail(self, reason: str) -> None:
        with self._lock:
            self._state = "failed:" + reason.replace("|", "/")[:200]
        self._publish()

    def leave(self) -> None:
        with self._lock:
            self._state = "left"
        self._publish()
        self.stop()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1.0)
            self._thread = None

    # -- checking -------------------------------------------------------------------------------------
    def peers(self) -> Dict[int, Dict]:
        out = {}
        for r in range(self.world):
            try:
                if not self.store.check([self._key(r)]):          # get() would block until the key appears
                    raise KeyError(r)
                state, step, stamp = self.store.get(self._key(r)).decode().split("|")
                out[r] = {"state": state, "step": int(step), "time": float(stamp)}
            except Exception:
                out[r] = {"state": "missing", "step": -1, "time": 0.0}
        return out

    def check(self) -> None:
        now = self.clock()
        with self._lock:
            my_step = self._step
        for r, info in self.peers().items():
            if r == self.rank:
                continue
            if info["state"].startswith("failed"):
                raise PeerFailure(r, info["state"])
            if info["state"] == "left":
                raise PeerFailure(r, "left the job")
            if info["state"] == "missing":
                raise PeerFailure(r, "never joined")
            if now - info["time"] > self.timeout:
                raise PeerFailure(r, f"no heartbeat for {now - info['time']:.1f} s (last step {info['step']})")
            if self.max_step_lag is not None and my_step - info["step"] > self.max_step_lag:
                raise PeerFailure(r, f"stalled at step {info['step']} while rank {self.rank} is at {my_step}")

    def guard(self, step: int) -> None:
        """One call per training step: publish progress, then make sure everybody else is alive."""
        self.beat(step)
        self.check()


class StatusWords:
    """Registry of device-side status words (set non-zero by a kernel whose bounded wait expired).
    ``poll()`` reads them all with one device-to-host copy and raises on the first non-zero word."""

    def __init__(self):
        self._words: List = []

    def register(self, name: str, tensor: torch.Tensor, describe: Optional[Callable[[int], str]] = None) -> None:
        self._words.append((name, tensor, describe))

    def poll(self) -> None:
        if not self._words:
            return
        values = torch.stack([w.reshape(-1)[0].to(torch.int64) for _, w, _ in self._words]).tolist()
        for (name, _, describe), code in zip(self._words, values):
            if code:
                detail = describe(code) if describe else f"status {code}"
                raise RuntimeError(f"{name}: {detail}")
