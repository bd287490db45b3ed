"""Background data loading: worker processes that build packed batches ahead of the training loop, with recovery
when a worker dies, and resumable samplers.

Reference: ``RestartableDataLoader`` and the worker-failure recovery of the trainer
(training/sensenovavl/data/build_dataloader.py:379-400, training/sensenovalm/core/trainer_builder.py:488-526), the
batch samplers with saved state (training/sensenovalm/data/tokenized/batch_sampler.py:24-787) and the "only the
loader rank reads, the others receive" rule (build_dataloader.py:410-517, trainer_builder.py:164-169).

Design: every worker owns a disjoint, deterministic sub-stream (``make_iter(worker_id, num_workers, skip)``), so the
order of batches is a pure function of (seed, number of workers) and a dead worker can be restarted exactly where its
stream stopped: the parent counts what it has taken from each worker and passes that count as ``skip``.  Batches
travel as pickled tensors through a bounded queue (the loader is host-side work; nothing here touches a GPU).
"""
from __future__ import annotations

import multiprocessing as mp
import queue
import random
import time
from typing import Callable, Dict, Iterator, List, Optional, Sequence


def _worker_main(make_iter, wid, nworkers, skip, q, stop):
    try:
        it = make_iter(wid, nworkers, skip)
        for item in it:
            while not stop.is_set():
                try:
                    q.put(("item", wid, item), timeout=0.2)
                    break
                except queue.Full:
                    continue
            if stop.is_set():
                return
        q.put(("end", wid, None))
        # tensors travel through shared memory that the sender must keep open until the receiver has mapped it:
        # stay alive until the parent is done with this worker
        stop.wait()
    except Exception as e:          # reported to the parent, which decides about a restart
        try:
            q.put(("error", wid, repr(e)))
        except Exception:
            pass


class WorkerPoolLoader:
    """Round-robin over ``num_workers`` background streams.

    ``make_iter(worker_id, num_workers, skip)`` must return an iterator that yields worker ``worker_id``'s items from
    position ``skip`` on (picklable items).  A worker that exits with an error or disappears is restarted up to
    ``worker_fail_retry`` times in a row with a growing pause (the reference's ``worker_fail_retry`` /
    ``worker_fail_retry_backoff_s``); the stream continues without losing or repeating an item.
    ``state_dict`` holds the per-worker counts."""

    def __init__(self, make_iter: Callable[[int, int, int], Iterator], num_workers: int = 2, prefetch: int = 4,
                 worker_fail_retry: int = 3, worker_fail_retry_backoff_s: float = 0.2, poll_s: float = 0.5,
                 start_method: str = "spawn"):
        if num_workers < 1:
            raise ValueError("num_workers must be at least 1")
        self.make_iter, self.n, self.prefetch = make_iter, num_workers, prefetch
        self.retry, self.backoff, self.poll_s = worker_fail_retry, worker_fail_retry_backoff_s, poll_s
        self.ctx = mp.get_context(start_method)
        self.taken = [0] * num_workers
        self.restarts = 0
        self._procs: List[Optional[mp.Process]] = [None] * num_workers
        self._queues = [None] * num_workers
        self._stop = None
        self._done = [False] * num_workers

    def _start(self, w: int):
        if self._stop is None:
            self._stop = self.ctx.Event()
        self._queues[w] = self.ctx.Queue(maxsize=self.prefetch)
        p = self.ctx.Process(target=_worker_main, args=(self.make_iter, w, self.n, self.taken[w], self._queues[w], self._stop),
                             daemon=True)
        p.start()
        self._procs[w] = p

    def restart_workers(self):
        """Stops every worker and starts them again at their current positions."""
        self.close()
        self._done = [False] * self.n
        for w in range(self.n):
            self._start(w)

    def __iter__(self):
        if all(p is None for p in self._procs):
            for w in range(self.n):
                self._start(w)
        w, failures = 0, 0
        while not all(self._done):
            if self._done[w]:
                w = (w + 1) % self.n
                continue
            try:
                kind, wid, item = self._queues[w].get(timeout=self.poll_s)
            except queue.Empty:
                if self._procs[w] is not None and not self._procs[w].is_alive():
                    kind, item = "error", "worker process died"
                else:
                    continue
            except (EOFError, OSError):             # the worker's end of the pipe is gone
                kind, item = "error", "worker process died (pipe closed)"
            if kind == "item":
                self.taken[w] += 1
                failures = 0
                yield item
                w = (w + 1) % self.n
            elif kind == "end":
                self._done[w] = True
            else:
                failures += 1
                self.restarts += 1
                if failures > self.retry:
                    self.close()
                    raise RuntimeError(f"data worker {w} failed {failures} times in a row: {item}")
                time.sleep(self.backoff * failures)
                if self._procs[w] is not None and self._procs[w].is_alive():
                    self._procs[w].terminate()
                self._start(w)

    def close(self):
        if self._stop is not None:
            self._stop.set()
        for i, p in enumerate(self._procs):
            if p is not None:
                p.join(timeout=1.0)
                if p.is_alive():
                    p.terminate()
                self._procs[i] = None
        self._stop = None

    def state_dict(self):
        return {"taken": list(self.taken), "num_workers": self.n}

    def load_state_dict(self, sd):
        if sd["num_workers"] != self.n:
            raise ValueError(f"the loader state was saved with {sd['num_workers']} workers, now {self.n}")
        self.taken = list(sd["taken"])


class WeightedResumableSampler:
    """Endless sampler over several datasets: dataset ``d`` is drawn with probability proportional to ``weights[d]``,
    inside a dataset the indices of this rank (``i mod world == rank``) are visited in a per-epoch shuffled order.
    Everything (RNG, epoch and cursor per dataset, consumed count) is in ``state_dict``, so a resumed run yields exactly
    the continuation of the stream."""

    def __init__(self, sizes: Sequence[int], weights: Optional[Sequence[float]] = None, rank: int = 0, world: int = 1,
                 seed: int = 0, shuffle: bool = True):
        self.sizes = list(sizes)
        self.weights = list(weights) if weights is not None else [float(s) for s in sizes]
        self.rank, self.world, self.seed, self.shuffle = rank, world, seed, shuffle
        self.rng = random.Random(seed)
        self.epoch = [0] * len(sizes)
        self.cursor = [0] * len(sizes)
        self.consumed = 0
        self._order: Dict[int, List[int]] = {}

    def _epoch_order(self, d: int) -> List[int]:
        if d not in self._order:
            idx = list(range(self.rank, self.sizes[d], self.world))
            if self.shuffle:
                random.Random(self.seed * 7919 + d * 104729 + self.epoch[d]).shuffle(idx)
            self._order[d] = idx
        return self._order[d]

    def __iter__(self):
        live = [d for d, s in enumerate(self.sizes) if s > self.rank]
        if not live:
            return
        while True:
            d = self.rng.choices(live, weights=[self.weights[j] for j in live], k=1)[0]
            order = self._epoch_order(d)
            if self.cursor[d] >= len(order):
                self.epoch[d] += 1
                self.cursor[d] = 0
                self._order.pop(d, None)
                order = self._epoch_order(d)
            i = order[self.cursor[d]]
            self.cursor[d] += 1
            self.consumed += 1
            yield d, i

    def state_dict(self):
        st = self.rng.getstate()
        return {"rng": [st[0], list(st[1]), st[2]], "epoch": list(self.epoch), "cursor": list(self.cursor),
                "consumed": self.consumed}

    def load_state_dict(self, sd):
        st = sd["rng"]
        self.rng.setstate((st[0], tuple(st[1]), st[2]))
        self.epoch, self.cursor, self.consumed = list(sd["epoch"]), list(sd["cursor"]), int(sd["consumed"])
        self._order.clear()


def broadcast_batches(batch_iter: Optional[Iterator], group=None, src: int = 0):
    """Only rank ``src`` of ``group`` reads data; the others receive every batch (the reference's COMMON_DATA rule).
    The batch travels as one pickled object over the (gloo) group."""
    import torch.distributed as dist
    me = dist.get_rank()
    while True:
        obj = [next(batch_iter) if me == src else None]
        dist.broadcast_object_list(obj, src=src, group=group)
        yield obj[0]
