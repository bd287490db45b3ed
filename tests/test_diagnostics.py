"""Memory watch, replica check over gloo ranks, NUMA binding against a fake sysfs (CPU)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sensenova_u1_b200.utils.diagnostics import (MemoryWatch, bind_to_gpu_numa_node, check_replicas_equal, gpu_numa_node,
                                                  parse_cpulist, warmup_process_groups)


def test_memory_watch_reports_and_warns_on_allocator_retries():
    lines, stats = [], {"allocated": 2 << 30, "max_allocated": 3 << 30, "reserved": 4 << 30, "max_reserved": 4 << 30,
                        "num_alloc_retries": 0}
    w = MemoryWatch(interval=10, log=lines.append, stats=lambda: dict(stats))
    assert "allocated 2.000 GiB (max 3.000)" in w.step(1, "rank 0") and len(lines) == 1
    assert w.step(7) is None and len(lines) == 1                       # neither early nor due
    stats["num_alloc_retries"] = 3
    assert w.step(10) is not None and len(lines) == 3 and "retried 3 time(s)" in lines[-1]
    w.step(20)
    assert len(lines) == 4                                             # no new retries: the warning is not repeated
    assert MemoryWatch(interval=0).interval == 50


def test_numa_binding_from_sysfs(tmp_path):
    assert parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    sys = tmp_path / "sys"
    (sys / "bus/pci/devices/0000:1b:00.0").mkdir(parents=True)
    (sys / "bus/pci/devices/0000:1b:00.0/numa_node").write_text("1\n")
    (sys / "bus/pci/devices/0000:9b:00.0").mkdir(parents=True)
    (sys / "bus/pci/devices/0000:9b:00.0/numa_node").write_text("-1\n")
    for n, cpus in ((0, "0-3"), (1, "4-7")):
        (sys / f"devices/system/node/node{n}").mkdir(parents=True)
        (sys / f"devices/system/node/node{n}/cpulist").write_text(cpus + "\n")
    assert gpu_numa_node("0000:1B:00.0", str(sys)) == 1 and gpu_numa_node("0000:9b:00.0", str(sys)) is None
    got = []
    assert bind_to_gpu_numa_node(0, "0000:1b:00.0", sysfs=str(sys), set_affinity=got.append, allowed=range(8)) == 1 and got == [{4, 5, 6, 7}]
    # no PCI answer: GPUs are dealt over the nodes evenly (8 GPUs, 2 nodes: ranks 0-3 -> node 0, 4-7 -> node 1)
    assert bind_to_gpu_numa_node(5, "0000:9b:00.0", gpus_per_node=8, sysfs=str(sys), set_affinity=got.append, allowed=range(8)) == 1
    assert bind_to_gpu_numa_node(2, "0000:9b:00.0", gpus_per_node=8, sysfs=str(sys), set_affinity=got.append, allowed=range(8)) == 0 and got[-1] == {0, 1, 2, 3}
    assert bind_to_gpu_numa_node(0, "0000:9b:00.0", gpus_per_node=3, sysfs=str(sys), set_affinity=got.append, allowed=range(8)) is None   # uneven
    assert bind_to_gpu_numa_node(0, "0000:1b:00.0", sysfs=str(sys), set_affinity=got.append, allowed=[0, 1, 2, 3, 4]) is None   # one CPU of ours on that node
    def boom(_):
        raise OSError("not allowed")
    assert bind_to_gpu_numa_node(0, "0000:1b:00.0", sysfs=str(sys), set_affinity=boom, allowed=range(8)) is None            # never raises


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _replica_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        same = {"layers.0.w": torch.randn(64, 32), "norm": torch.ones(32), "head.bias": torch.full((4,), float(rank))}
        n = warmup_process_groups([dist.group.WORLD, None, dist.group.WORLD])      # absent groups and repeats are skipped
        ok = check_replicas_equal(same.items())                       # biases are skipped, the rest is identical
        drift = dict(same)
        drift["layers.0.w"] = same["layers.0.w"] + (0.5 if rank == 1 else 0.0)
        bad = check_replicas_equal(drift.items(), raise_on_mismatch=False)
        try:
            check_replicas_equal(drift.items())
            raised = ""
        except AssertionError as e:
            raised = str(e)
        q.put((rank, n, ok, bad, "layers.0.w" in raised and "rank 1" in raised))
    finally:
        dist.destroy_process_group()


def test_replica_check_over_gloo_ranks():
    ctx = mp.get_context("spawn")
    q, port = ctx.Queue(), _free_port()
    ps = [ctx.Process(target=_replica_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    out = sorted(q.get(timeout=120) for _ in ps)
    for p in ps:
        p.join(60)
    assert out == [(0, 1, [], ["layers.0.w"], True), (1, 1, [], ["layers.0.w"], True)]
