"""Host-side failure detection: a watchdog thread that bounds every phase of a training step,
a heartbeat store other ranks can poll, and the NaN/Inf skip counter.

The reference arms SIGALRM around init, optimizer step, forward/backward, batch load, metrics
and checkpoint save (``llm_timeout``, training/sensenovalm/utils/timeout.py:44-116; enabled by
SENSENOVALM_ENABLE_TIMEOUT).  A thread does the same without owning the process's only alarm,
and works off the main thread.  Device-side waits are bounded separately, inside the kernels.
"""
from __future__ import annotations

import os
import threading
import time
from contextlib import contextmanager
from typing import Callable, Dict, Optional


class PhaseTimeout(RuntimeError):
    pass


def dump_and_exit(phase: str, late_s: float, code: int = 124) -> None:
    """Hard action for a phase that does not come back (a collective whose peer died, a wedged data worker): writes
    every thread's stack to stderr and ends the process from the watchdog thread, so that the launcher (or the other
    ranks' collective timeouts) sees a dead rank instead of a silent one.  ``os._exit`` skips destructors on purpose:
    a normal exit would wait for the very call that hangs."""
    import faulthandler
    import sys
    sys.stderr.write(f"[watchdog] phase {phase!r} is {late_s:.1f} s past its limit: dumping stacks, exiting {code}\n")
    sys.stderr.flush()
    faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
    sys.stderr.flush()
    os._exit(code)


class Watchdog:
    """``on_timeout(phase, seconds_late)`` runs in the watchdog thread as soon as a phase passes its limit, i.e. also
    while the phase is still hanging; pass :func:`dump_and_exit` (or set ``hard_exit=True`` /
    ``SENSENOVALM_TIMEOUT_EXIT=1``) to end a hung process.  A phase that does come back late raises
    :class:`PhaseTimeout` in the caller."""

    def __init__(self, default_timeout_s: float = 1800.0, on_timeout: Optional[Callable[[str, float], None]] = None,
                 enabled: Optional[bool] = None, hard_exit: Optional[bool] = None):
        env = os.environ.get("SENSENOVALM_ENABLE_TIMEOUT")
        self.enabled = (env is not None and env not in ("0", "false", "False")) if enabled is None else enabled
        self.default = float(os.environ.get("NCCL_TIMEOUT", default_timeout_s))
        if hard_exit is None:
            hard_exit = os.environ.get("SENSENOVALM_TIMEOUT_EXIT", "0") not in ("0", "false", "False", "")
        self.on_timeout = on_timeout if on_timeout is not None else (dump_and_exit if hard_exit else None)
        self._lock = threading.Lock()
        self._phase: Optional[str] = None
        self._deadline = 0.0
        self.expired: Optional[str] = None
        self._stop = threading.Event()
        self._thread = None
        if self.enabled:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def _run(self):
        while not self._stop.wait(0.05):
            with self._lock:
                ph, dl = self._phase, self._deadline
            if ph is not None and time.monotonic() > dl and self.expired is None:
                self.expired = ph
                if self.on_timeout:
                    self.on_timeout(ph, time.monotonic() - dl)

    @contextmanager
    def phase(self, name: str, timeout_s: Optional[float] = None):
        """Bounds the body in time; with ``SNU1_NVTX=1`` the phase is also an NVTX range, so profiler timelines show
        ``load_batch`` / ``fwd_bwd_step`` / ``save_checkpoint`` (the reference exposes ``range_push / range_pop`` on its
        accelerator, accelerator/cuda_accelerator.py:273-285)."""
        nvtx = _nvtx() if os.environ.get("SNU1_NVTX", "0") == "1" else None
        if nvtx is not None:
            nvtx.range_push(name)
        try:
            if not self.enabled:
                yield
                return
            with self._lock:
                self._phase, self._deadline = name, time.monotonic() + (timeout_s or self.default)
            try:
                yield
            finally:
                with self._lock:
                    self._phase = None
                if self.expired == name:
                    self.expired = None
                    raise PhaseTimeout(f"phase {name!r} exceeded its time limit")
        finally:
            if nvtx is not None:
                nvtx.range_pop()

    def close(self):
        self._stop.set()


def _nvtx():
    try:
        import torch
        return torch.cuda.nvtx if torch.cuda.is_available() else None
    except Exception:
        return None


class Heartbeat:
    """Each rank bumps a counter in the rendezvous store; anyone can ask who went silent."""

    def __init__(self, store, rank: int, world: int, prefix: str = "hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def beat(self, step: int):
        self.store.set(f"{self.prefix}/{self.rank}", f"{step}:{time.time()}")

    def silent_ranks(self, max_age_s: float):
        now, out = time.time(), []
        for r in range(self.world):
            key = f"{self.prefix}/{r}"
            try:
                if not self.store.check([key]):      # a rank that never reported (get() would block)
                    out.append(r)
                    continue
                v = self.store.get(key).decode()
                if now - float(v.split(":")[1]) > max_age_s:
                    out.append(r)
            except Exception:
                out.append(r)
        return out
