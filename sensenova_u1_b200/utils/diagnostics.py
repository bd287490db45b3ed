"""Run-time diagnostics of a training job: memory report with allocator-pressure warning, periodic cache release,
process-group warm-up, equality check of replicated weights, and NUMA binding of the rank's host threads.

Roles of the reference's ``sensenovalm/utils/gputest.py:35-175`` (``empty_cache_and_diag``, ``cuda_memory_analyze``,
``warmup_process_group``), ``sensenovalm/utils/parallel.py:166-243`` (``check_parallel_statistic_equality``) and
``sensenovalm/initialize/launch.py:877-916`` (``try_bind_numa``).  Nothing here touches a GPU setting: the NUMA part
only sets this process's CPU affinity, the rest reads counters."""
from __future__ import annotations

import gc
import os
from pathlib import Path
from typing import Callable, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

GiB = float(1 << 30)


class MemoryWatch:
    """Memory line every ``interval`` steps (and on the first five), with a warning when the caching allocator had to
    flush and retry since the last look: that stalls the step on every rank and means the job runs too close to the
    limit."""

    def __init__(self, interval: int = 50, log: Callable[[str], None] = print, stats: Optional[Callable[[], dict]] = None):
        self.interval = int(interval) if interval and interval > 0 else 50
        self.log = log
        self._stats = stats
        self._retries = 0

    def _read(self) -> dict:
        if self._stats is not None:
            return self._stats()
        if not torch.cuda.is_available():
            return {}
        s = torch.cuda.memory_stats()
        return {"allocated": torch.cuda.memory_allocated(), "max_allocated": torch.cuda.max_memory_allocated(),
                "reserved": torch.cuda.memory_reserved(), "max_reserved": torch.cuda.max_memory_reserved(),
                "num_alloc_retries": s.get("num_alloc_retries", 0)}

    def step(self, batch_count: int, tag: str = "") -> Optional[str]:
        """Returns the memory line when one was due."""
        s = self._read()
        line = None
        due = batch_count % self.interval == 0
        if s and (due or batch_count <= 5):
            line = (f"{tag} step {batch_count}: allocated {s['allocated'] / GiB:.3f} GiB (max {s['max_allocated'] / GiB:.3f}), "
                    f"reserved {s['reserved'] / GiB:.3f} GiB (max {s['max_reserved'] / GiB:.3f})").strip()
            self.log(line)
            if self._stats is None and torch.cuda.is_available():
                torch.cuda.reset_peak_memory_stats()
        retries = int(s.get("num_alloc_retries", 0) or 0)
        if retries > self._retries:
            self.log(f"{tag} step {batch_count}: the caching allocator flushed and retried {retries - self._retries} time(s) "
                     "since the last check; memory is tight (fewer kept activations, a smaller micro-batch or a release of "
                     "the cache on every rank at the same step avoids the stalls)".strip())
            self._retries = retries
        if due and batch_count > 0:
            gc.collect()
            if torch.cuda.is_available():
                torch.cuda.empty_cache()          # every rank does it at the same step, so nobody waits for a straggler
        return line


def warmup_process_groups(groups: Iterable, device=None) -> int:
    """One small all-reduce per group, then a barrier: communicators are created (and their buffers allocated) before
    the first step needs the memory.  ``None`` entries (groups a layout does not have) and repeats are skipped; pass
    ``dist.group.WORLD`` for the default group.  Returns the number of groups touched."""
    if not (dist.is_available() and dist.is_initialized()):
        return 0
    n = 0
    buf = torch.ones(64, device=device or ("cuda" if torch.cuda.is_available() and dist.get_backend() == "nccl" else "cpu"))
    seen = set()
    for g in groups:
        if g is None or id(g) in seen:
            continue
        seen.add(id(g))
        if dist.get_world_size(g) > 1:
            dist.all_reduce(buf, group=g)
            n += 1
    dist.barrier()
    return n


def tensor_fingerprint(t: torch.Tensor) -> torch.Tensor:
    """(mean, std) in float64: cheap, order-independent enough, and sensitive to a missed broadcast or update."""
    x = t.detach().to(torch.float64)
    return torch.stack([x.mean(), x.std(unbiased=False) if x.numel() > 1 else x.new_zeros(())])


def check_replicas_equal(named: Iterable[Tuple[str, torch.Tensor]], group=None, rtol: float = 1e-2, atol: float = 1e-2,
                         skip: Sequence[str] = ("bias",), raise_on_mismatch: bool = True) -> List[str]:
    """Tensors that should be identical on every rank of ``group`` (replicated weights of data-parallel ranks, norms
    under tensor parallelism, the routers of expert-parallel ranks) are compared through their fingerprints; one
    gather for all tensors.  Returns the names that differ; raises ``AssertionError`` naming ranks and values by
    default."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return []
    names, prints = [], []
    for name, t in named:
        if any(s in name for s in skip) or t.numel() == 0:
            continue
        names.append(name)
        prints.append(tensor_fingerprint(t))
    if not names:
        return []
    mine = torch.stack(prints).cpu()
    world = dist.get_world_size(group)
    gathered: List[Optional[torch.Tensor]] = [None] * world
    dist.all_gather_object(gathered, mine, group=group)
    bad, detail = [], []
    for r in range(1, world):
        close = torch.isclose(gathered[r], gathered[0], rtol=rtol, atol=atol).all(dim=1)
        for i in (~close).nonzero().flatten().tolist():
            if names[i] not in bad:
                bad.append(names[i])
                detail.append(f"{names[i]}: rank 0 (mean, std) = {gathered[0][i].tolist()}, rank {r} = {gathered[r][i].tolist()}")
    if bad and raise_on_mismatch:
        raise AssertionError("replicated tensors differ across ranks:\n  " + "\n  ".join(detail[:20]))
    return bad


# ---------------------------------------------------------------------------------------------------------------
# NUMA
# ---------------------------------------------------------------------------------------------------------------
def parse_cpulist(text: str) -> List[int]:
    """``0-3,8,10-11`` -> [0, 1, 2, 3, 8, 10, 11]."""
    out: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        out.extend(range(int(lo), int(hi or lo) + 1))
    return out


def gpu_numa_node(pci_bus_id: str, sysfs: str = "/sys") -> Optional[int]:
    """NUMA node of a PCI device (``0000:1b:00.0``), None when the platform does not say."""
    p = Path(sysfs) / "bus" / "pci" / "devices" / pci_bus_id.lower() / "numa_node"
    try:
        n = int(p.read_text().strip())
    except (OSError, ValueError):
        return None
    return n if n >= 0 else None


def numa_cpus(node: int, sysfs: str = "/sys") -> List[int]:
    try:
        return parse_cpulist((Path(sysfs) / "devices" / "system" / "node" / f"node{node}" / "cpulist").read_text())
    except OSError:
        return []


def bind_to_gpu_numa_node(local_rank: int, pci_bus_id: Optional[str] = None, gpus_per_node: Optional[int] = None,
                          sysfs: str = "/sys", set_affinity: Callable = None, allowed: Optional[Iterable[int]] = None) -> Optional[int]:
    """Pins this process's threads to the CPUs of the NUMA node its GPU hangs off (pinned-memory copies and the
    launch thread then stay on the near socket).  The node comes from the GPU's PCI entry; without one, GPUs are dealt
    over the nodes evenly (the reference's rule: ``local_rank // (gpus / nodes)``).  ``allowed``: the CPUs this process may use
    (default: its current affinity); the binding keeps to them and is skipped when fewer than a quarter of them lie on
    the node.  Never raises; returns the node or None when nothing was done."""
    set_affinity = set_affinity or (lambda cpus: os.sched_setaffinity(0, cpus))
    try:
        if pci_bus_id is None and torch.cuda.is_available():
            p = torch.cuda.get_device_properties(local_rank)
            if all(hasattr(p, k) for k in ("pci_domain_id", "pci_bus_id", "pci_device_id")):
                pci_bus_id = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        node = gpu_numa_node(pci_bus_id, sysfs) if pci_bus_id else None
        if node is None:
            nodes = sorted(int(p.name[4:]) for p in (Path(sysfs) / "devices" / "system" / "node").glob("node[0-9]*"))
            n_gpu = gpus_per_node or (torch.cuda.device_count() if torch.cuda.is_available() else 0)
            if len(nodes) < 2 or n_gpu <= len(nodes) or n_gpu % len(nodes):
                return None
            node = nodes[local_rank // (n_gpu // len(nodes))]
        cpus = set(numa_cpus(node, sysfs))
        if allowed is None and hasattr(os, "sched_getaffinity"):
            allowed = os.sched_getaffinity(0)
        if allowed is not None:
            cpus &= set(allowed)                      # a container's CPU set may cover a part of the node only
            if len(cpus) < max(2, len(allowed) // 4):
                return None                           # too few of the node's CPUs are ours: binding would starve the loaders
        if not cpus:
            return None
        set_affinity(cpus)
        return node
    except Exception:
        return None
