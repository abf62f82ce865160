"""Failure detection on the host: device status words and a store-based heartbeat between ranks.

The reference has no failure detection beyond a gossip flag timeout (fairscale/experimental/nn/data_parallel/gossip/
distributed.py:41,1015-1017) and worker threads that forward exceptions (fairscale/nn/pipe/worker.py:95-100).  Here:

* every device-side wait of the native kernels is bounded and reports through a per-device status word;
  :func:`check_device_status` turns a non-zero word into :class:`CommTimeoutError` on the host, so a kernel that gave
  up waiting for a peer surfaces as an exception instead of as silently wrong data;
* :class:`Heartbeat` lets ranks learn on the host, between steps and before their next launch, that a peer raised,
  left, or stopped making progress: each rank bumps a counter in a ``torch.distributed`` store once per step and posts
  a failure note when it dies with an exception; peers poll the store (never a collective), so detection does not
  depend on a kernel or a collective timing out.
"""

from __future__ import annotations

import contextlib
import time
from typing import Any, Dict, Iterator, List, Optional


class CommTimeoutError(RuntimeError):
    """A native kernel gave up a bounded wait (on an mbarrier, a peer's flag or a barrier) and returned early."""

    def __init__(self, code: int, device: Any):
        self.code = code & 0xFF
        self.site = code >> 8  # which wait gave up (a number from the kernel's source; 0 when the kernel does not say)
        self.device = device
        what = {1: "a bounded device-side wait ran out", 2: "a kernel rejected its arguments"}.get(self.code, "unknown status")
        where = f", wait site {self.site}" if self.site else ""
        super().__init__(f"device {device}: status word {self.code} ({what}{where}); the outputs of the kernels launched since the last check are invalid")


class PeerFailureError(RuntimeError):
    """One or more peers reported a failure or stopped sending heartbeats."""

    def __init__(self, ranks: List[int], reasons: Dict[int, str]):
        self.ranks = ranks
        self.reasons = reasons
        super().__init__("peer failure: " + ", ".join(f"rank {r}: {reasons[r]}" for r in ranks))


def check_device_status(device: Any = None) -> None:
    """Synchronously read (and clear) the status word of ``device``; raise :class:`CommTimeoutError` if a kernel
    reported a problem.  Costs a device synchronisation: call it once per step, not per kernel."""
    from .. import _native

    code = _native.read_status(device)
    if code != 0:
        _poison_workspaces()
        raise CommTimeoutError(code, device if device is not None else "current")


class StatusWatch:
    """Checks the device status word once per step without stalling the device.

    Each :meth:`poll` looks at the value that the previous poll copied to pinned host memory (if that copy has
    finished) and starts the next copy on the current stream, so an error written by a kernel of step *i* surfaces as
    :class:`CommTimeoutError` at step *i + 1* at the latest, with no device synchronisation in between.  The data
    parallel wrappers poll at the end of every backward; after an error the NVLink workspaces of the process are
    marked unusable (their collectives fall back to ``torch.distributed``), because a kernel that gave up early has
    left flags, counters and epochs in an unknown state.
    """

    def __init__(self, device: Any):
        import torch

        self.device = torch.device(device)
        self._host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._event: Optional[Any] = None

    def poll(self) -> None:
        import torch

        from .. import _native

        if self._event is not None and self._event.query():
            code = int(self._host[0])
            self._event = None
            if code != 0:
                _native.status_word(self.device).zero_()
                _poison_workspaces()
                raise CommTimeoutError(code, self.device)
        if self._event is None:
            self._host.copy_(_native.status_word(self.device), non_blocking=True)
            self._event = torch.cuda.Event()
            self._event.record()


_WATCHES: Dict[Any, StatusWatch] = {}


def poll_device_status(device: Any) -> None:
    """Per-step, non-blocking status check of ``device`` (see :class:`StatusWatch`); a no-op for CPU devices."""
    import torch

    dev = torch.device(device)
    if dev.type != "cuda":
        return
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    w = _WATCHES.get(key)
    if w is None:
        w = _WATCHES[key] = StatusWatch(torch.device("cuda", key))
    w.poll()


def _poison_workspaces() -> None:
    from ..parallel import symm

    symm.poison_all()


class Heartbeat:
    """Per-step liveness protocol over a ``torch.distributed`` store (TCPStore, FileStore, HashStore or PrefixStore).

    Usage, on every rank::

        hb = Heartbeat(store, rank, world_size, timeout_s=60)
        for step in range(n):
            with hb.guard():              # an exception inside posts a failure note for the peers, then re-raises
                hb.sync_step(step)        # raises PeerFailureError instead of entering a collective that cannot finish
                train_step()

    Only ``store.add`` and ``store.set`` / ``store.get`` on keys known to exist are used, so no call blocks on a
    missing key.
    """

    def __init__(self, store: Any, rank: int, world_size: int, timeout_s: float = 60.0, poll_s: float = 0.01, prefix: str = "fsb_hb") -> None:
        self.store = store
        self.rank = rank
        self.world_size = world_size
        self.timeout_s = timeout_s
        self.poll_s = poll_s
        self.prefix = prefix

    # ------------------------------------------------------------------ keys
    def _beat_key(self, rank: int) -> str:
        return f"{self.prefix}/beat/{rank}"

    def _fail_key(self, rank: int) -> str:
        return f"{self.prefix}/failed/{rank}"

    def _reason_key(self, rank: int) -> str:
        return f"{self.prefix}/reason/{rank}"

    # ------------------------------------------------------------------ this rank
    def beat(self, step: int) -> None:
        """Publish that this rank has reached ``step`` (steps count from 0 and only grow)."""
        current = self.store.add(self._beat_key(self.rank), 0)
        if step + 1 > current:
            self.store.add(self._beat_key(self.rank), step + 1 - current)

    def fail(self, reason: str) -> None:
        """Tell the peers that this rank is leaving the job."""
        self.store.set(self._reason_key(self.rank), reason[:500])
        self.store.add(self._fail_key(self.rank), 1)

    @contextlib.contextmanager
    def guard(self) -> Iterator[None]:
        try:
            yield
        except PeerFailureError:
            raise  # a reaction to somebody else's failure is not a new failure
        except BaseException as exc:  # noqa: B902  (also KeyboardInterrupt / SystemExit: the rank is going away)
            try:
                self.fail(f"{type(exc).__name__}: {exc}")
            finally:
                raise

    # ------------------------------------------------------------------ peers
    def failed_peers(self) -> Dict[int, str]:
        out: Dict[int, str] = {}
        for r in range(self.world_size):
            if r != self.rank and self.store.add(self._fail_key(r), 0) > 0:
                out[r] = self.store.get(self._reason_key(r)).decode(errors="replace")
        return out

    def check(self) -> None:
        """Raise :class:`PeerFailureError` if any peer has posted a failure (non-blocking)."""
        bad = self.failed_peers()
        if bad:
            raise PeerFailureError(sorted(bad), bad)

    def sync_step(self, step: int) -> None:
        """Publish ``step`` and wait until every peer has reached it too, posted a failure, or has been silent for
        ``timeout_s``.  Returns normally only when all peers are alive at ``step``."""
        self.beat(step)
        deadline = time.monotonic() + self.timeout_s
        waiting = [r for r in range(self.world_size) if r != self.rank]
        while True:
            self.check()
            waiting = [r for r in waiting if self.store.add(self._beat_key(r), 0) < step + 1]
            if not waiting:
                return
            if time.monotonic() > deadline:
                reasons = {r: f"no heartbeat for step {step} within {self.timeout_s} s" for r in waiting}
                raise PeerFailureError(waiting, reasons)
            time.sleep(self.poll_s)


def make_heartbeat(group_store: Optional[Any] = None, timeout_s: float = 60.0, prefix: str = "fsb_hb") -> Heartbeat:
    """Heartbeat over the default process group's store (the one ``init_process_group`` rendezvoused on)."""
    import torch.distributed as dist

    store = group_store if group_store is not None else dist.distributed_c10d._get_default_store()
    return Heartbeat(store, dist.get_rank(), dist.get_world_size(), timeout_s=timeout_s, prefix=prefix)
