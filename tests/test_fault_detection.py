"""Failure detection on the host: phase watchdog, heartbeats, skipped non-finite steps,
and a collective that times out when a rank never joins (gloo ranks on CPU; no GPU involved)."""
import os
import socket
import sys
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sensenova_u1_b200.utils.watchdog import Heartbeat, PhaseTimeout, Watchdog

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_watchdog_flags_a_slow_phase():
    seen = []
    wd = Watchdog(on_timeout=lambda ph, late: seen.append(ph), enabled=True)
    with wd.phase("fast", 1.0):
        pass
    with pytest.raises(PhaseTimeout):
        with wd.phase("optim_step", 0.1):
            time.sleep(0.4)
    assert seen == ["optim_step"]
    wd.close()


def test_heartbeat_finds_the_silent_rank():
    store = dist.HashStore()
    hb = [Heartbeat(store, r, 3) for r in range(3)]
    hb[0].beat(1); hb[2].beat(1)
    assert hb[0].silent_ranks(max_age_s=5.0) == [1]
    time.sleep(0.2)
    hb[0].beat(2)
    assert hb[0].silent_ranks(max_age_s=0.1) == [1, 2]


def test_non_finite_gradients_skip_the_step():
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.train.optimizer import AdamConfig, ZeroAdamW
    cfg = tiny_mot(num_layers=1)
    store = ParamStore(cfg, dtype=torch.float32, grad_dtype_mat=torch.float32)
    store.init_weights(0)
    opt = ZeroAdamW(store, AdamConfig(lr=1e-2, state_dtype="fp32"))
    before = store.arena["mat"].clone()
    store.grad_arena["mat"].fill_(float("nan"))
    opt.step()
    assert int(opt.skipped) == 1 and torch.equal(before, store.arena["mat"])


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _rank_that_may_never_join(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=3))
    t = torch.ones(4)
    dist.all_reduce(t)                     # step 0: everyone is here
    if rank == 1:
        dist.destroy_process_group()       # leaves between steps, nothing in flight
        return
    t0 = time.time()
    try:
        dist.all_reduce(t)                 # step 1: rank 1 never joins
        res = "no error"
    except Exception as e:                 # the short process-group timeout ends the collective
        res = f"error after {time.time() - t0:.1f}s: {type(e).__name__}"
    open(out, "w").write(res)


def test_collective_times_out_when_a_rank_leaves(tmp_path):
    out = str(tmp_path / "r0.txt")
    mp.spawn(_rank_that_may_never_join, args=(2, _free_port(), out), nprocs=2, join=True)
    assert open(out).read().startswith("error after")
