"""Host-side failure detection.

The reference has no multi-rank mode, so no failure detection either (its only liveness code is a
stop flag for the visualiser thread, src/bin/infer.rs:356-397). Here:

* `Heartbeat` - every rank publishes a timestamp in the process group's key-value store from a
  background thread; `dead_ranks()` lists peers whose heartbeat is older than the timeout or that
  announced their departure. Trainers call `check()` between steps, i.e. before they launch a
  kernel or collective that would wait for the peer.
* `device_status()` - turns a non-zero kernel status word (a bounded in-kernel wait that gave up)
  into a Python exception, leaving the CUDA context usable.

* `HostFaultInjector` - test hook that makes one rank raise between two steps (no kernel or
  collective of its own in flight), once per marker file, so that restart-from-checkpoint can be
  exercised under a launcher that restarts failed groups.

Nothing here makes a GPU fault, trap or hang; failures are injected on the host (a rank that
raises, exits or stops publishing).
"""
from __future__ import annotations

import os
import threading
import time
from pathlib import Path
from typing import List, Optional

import torch.distributed as dist

STATUS_NAMES = {0: "ok", 1: "smem-full wait timed out", 2: "smem-empty wait timed out",
                3: "tmem-full wait timed out", 4: "tmem-empty wait timed out", 5: "peer flag wait timed out",
                6: "bad argument"}


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int]):
        super().__init__(f"ranks {ranks} stopped responding")
        self.ranks = ranks


class KernelTimeout(RuntimeError):
    pass


class Heartbeat:
    def __init__(self, rank: int, world: int, interval_s: float = 1.0, timeout_s: float = 10.0, store=None,
                 prefix: str = "bdh_hb"):
        self.rank, self.world = rank, world
        self.interval, self.timeout = interval_s, timeout_s
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()
        self.prefix = prefix
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def _publish(self, value: str) -> None:
        self.store.set(self._key(self.rank), value)

    def start(self) -> None:
        self._publish(repr(time.time()))
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self._publish(repr(time.time()))
            except Exception:  # noqa: BLE001 - the store went away: nothing left to tell
                return

    def stop(self, leave: bool = False) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)
        if leave:
            try:
                self._publish("left")
            except Exception:  # noqa: BLE001
                pass

    def dead_ranks(self) -> List[int]:
        now, dead = time.time(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            key = self._key(r)
            try:
                if not self.store.check([key]):
                    continue            # not started yet
                val = self.store.get(key).decode()
            except Exception:  # noqa: BLE001
                dead.append(r)
                continue
            if val == "left" or now - float(val) > self.timeout:
                dead.append(r)
        return dead

    def check(self) -> None:
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(dead)


def device_status(raise_on_error: bool = True) -> int:
    """Read the kernels' status word (synchronises the device)."""
    from ..ops import native
    code = native.status_code()
    if code and raise_on_error:
        native.clear_status()
        raise KernelTimeout(f"kernel status {code}: {STATUS_NAMES.get(code, 'unknown')}")
    return code


class StatusMonitor:
    """Watches the kernels' status word from the training loop without synchronising the device.

    A bounded in-kernel wait that gives up (a peer more than the wait limit late at a cross-rank
    barrier, a pipeline stage that never arrived) makes its kernel return early: a collective then
    leaves its slice unreduced and the optimizer its slice unupdated, so the step's result is wrong
    although nothing faulted. `poll()` is called once per optimizer step: it first looks at the copy
    of the status word it requested on the previous call (ready by now; `KernelTimeout` if non-zero),
    then queues a new 4-byte device-to-host copy behind the step's kernels and returns. A timeout is
    therefore seen at most one step late and costs no synchronisation. `check()` waits for the copy
    in flight (used where the loop synchronises anyway, and at the end of a run). The rank is expected to exit on
    `KernelTimeout`, so that a launcher restarting the group resumes from the last checkpoint.

    `read_async(dst)` must queue a copy of the status word into the pinned int32 tensor `dst` and
    return an object with `query()` / `synchronize()` (a CUDA event); tests pass a host-side fake."""

    def __init__(self, read_async=None):
        self._read_async = read_async
        self._host = None
        self._event = None
        self.enabled = True

    def _default_read(self, dst):
        import torch
        from ..ops import native
        if native.available():
            dst.copy_(torch.ops.bdh.status()[:1], non_blocking=True)      # word 0 holds the first failure code
        else:
            dst.zero_()
        ev = torch.cuda.Event()
        ev.record()
        return ev

    def _raise_if_set(self) -> None:
        code = int(self._host[0])
        self._event = None
        if code:
            from ..ops import native
            try:
                native.clear_status()
            except Exception:  # noqa: BLE001 - reporting the timeout matters more than clearing it
                pass
            raise KernelTimeout(f"kernel status {code}: {STATUS_NAMES.get(code, 'unknown')}; this step's collective or "
                                "GEMM returned early, its results are incomplete")

    def poll(self) -> None:
        if not self.enabled:
            return
        if self._event is not None and self._event.query():
            self._raise_if_set()
        if self._event is None:
            if self._host is None:
                import torch
                pin = self._read_async is None and torch.cuda.is_available()
                self._host = torch.zeros(1, dtype=torch.int32, pin_memory=pin)
            self._event = (self._read_async or self._default_read)(self._host)

    def check(self) -> None:
        if self.enabled and self._event is not None:
            self._event.synchronize()
            self._raise_if_set()


class InjectedFault(RuntimeError):
    pass


class HostFaultInjector:
    """`BDH_INJECT_FAULT="rank=1,step=3,once=/path/to/marker"`: rank 1 raises `InjectedFault` when it
    is about to run step 3 - unless the marker file exists; the file is created first, so a restarted
    job passes the same point. Unset (the default) the injector does nothing."""

    def __init__(self, rank: int, spec: Optional[str] = None):
        spec = os.environ.get("BDH_INJECT_FAULT", "") if spec is None else spec
        self.rank, self.fail_rank, self.fail_step, self.marker = rank, None, None, None
        for part in filter(None, (p.strip() for p in spec.split(","))):
            k, _, v = part.partition("=")
            if k == "rank":
                self.fail_rank = int(v)
            elif k == "step":
                self.fail_step = int(v)
            elif k == "once":
                self.marker = Path(v)
            else:
                raise ValueError(f"BDH_INJECT_FAULT: unknown key {k!r}")

    def before_step(self, step: int) -> None:
        if self.fail_rank != self.rank or self.fail_step != step:
            return
        if self.marker is not None:
            if self.marker.exists():
                return
            self.marker.parent.mkdir(parents=True, exist_ok=True)
            self.marker.write_text(f"rank {self.rank} failed before step {step}\n")
        raise InjectedFault(f"injected host fault on rank {self.rank} before step {step}")
