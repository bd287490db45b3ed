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


# ---------------------------------------------------------------------------
# a phase that never returns is ended by the watchdog thread (opt-in hard exit)
# ---------------------------------------------------------------------------
def test_watchdog_ends_a_hung_phase():
    import subprocess
    code = (
        "import sys, time; sys.path.insert(0, %r)\n"
        "from sensenova_u1_b200.utils.watchdog import Watchdog\n"
        "wd = Watchdog(enabled=True, hard_exit=True)\n"
        "with wd.phase('fwd_bwd_step', 0.2):\n"
        "    time.sleep(60)\n"
        "print('not reached')\n" % ROOT)
    t0 = time.time()
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=50)
    assert r.returncode == 124 and time.time() - t0 < 40
    assert "fwd_bwd_step" in r.stderr and "not reached" not in r.stdout
    assert "time.sleep" in r.stderr or "File" in r.stderr        # the stack dump names where it hung


# ---------------------------------------------------------------------------
# a rank dies between steps; the job is restarted and resumes from the newest complete checkpoint
# ---------------------------------------------------------------------------
def _train_worker(rank, world, port, folder, steps, die_after, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=20))
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.train.checkpoint import CheckpointManager, LoadMask
    from sensenova_u1_b200.train.optimizer import AdamConfig
    from sensenova_u1_b200.train.trainer import Trainer
    cfg = tiny_mot(num_layers=1)
    store = ParamStore(cfg, dtype=torch.float32, grad_dtype_mat=torch.float32, shard_multiple=8 * 128 * world)
    store.init_weights(0)
    tr = Trainer(cfg, store, AdamConfig(lr=1e-2, state_dtype="fp32"))
    mgr = CheckpointManager(folder, checkpoint_every=2, dp_rank=rank, zero_rank=rank)
    step = 0
    res = mgr.try_resume(store, tr.optim, LoadMask.parse("all"))
    if res is not None:
        step = int(res[1][0]["step"])
    losses = {}
    while step < steps:
        loss = tr.train_step([tiny_batch(cfg, seed=100 * step + rank, n_text=64)])["loss"]
        step += 1
        losses[step] = loss
        if mgr.decide(step, steps)[0]:
            mgr.save(step, store, tr.optim, {"step": step})
        if die_after is not None and step == die_after and rank == 1:
            os._exit(17)            # between steps: nothing of this rank is in flight
    torch.save(losses, f"{out}.{rank}")
    dist.destroy_process_group()


def _spawn(world, args):
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_train_worker, args=(r, world) + args) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    return [p.exitcode for p in procs]


def test_killed_rank_then_restart_resumes_and_reproduces_the_losses(tmp_path):
    world, steps = 2, 6
    # uninterrupted run
    codes = _spawn(world, (_free_port(), str(tmp_path / "a"), steps, None, str(tmp_path / "ref")))
    assert codes == [0, 0]
    ref = torch.load(str(tmp_path / "ref.0"))
    # rank 1 dies after step 3 (a checkpoint exists for step 2); rank 0's next collective fails within its timeout
    codes = _spawn(world, (_free_port(), str(tmp_path / "b"), steps, 3, str(tmp_path / "x")))
    assert codes[1] == 17 and codes[0] != 0
    assert (tmp_path / "b" / "2" / "2.step").exists() and not (tmp_path / "b" / "4").exists()
    # restart: auto-resume from step 2, same losses from step 3 on
    codes = _spawn(world, (_free_port(), str(tmp_path / "b"), steps, None, str(tmp_path / "got")))
    assert codes == [0, 0]
    got = torch.load(str(tmp_path / "got.0"))
    assert sorted(got) == [3, 4, 5, 6]
    for k in got:
        assert got[k] == ref[k], (k, got[k], ref[k])


def test_truncated_shard_is_reported_not_loaded(tmp_path):
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.train.checkpoint import CheckpointManager, LoadMask
    cfg = tiny_mot(num_layers=1)
    store = ParamStore(cfg, dtype=torch.float32, with_grads=False)
    store.init_weights(0)
    mgr = CheckpointManager(str(tmp_path / "run"))
    d = mgr.save(5, store)
    f = d / "model_wp0_pp0.pt"
    data = f.read_bytes()
    f.write_bytes(data[: len(data) // 2])                     # the write was cut short
    fresh = ParamStore(cfg, dtype=torch.float32, with_grads=False)
    before = fresh.arena["mat"].clone()
    with pytest.raises(Exception) as e:
        mgr.load(d, fresh, mask=LoadMask(True, False, False, False))
    assert torch.equal(fresh.arena["mat"], before), "a damaged shard must not be half-applied"
    assert "model_wp0_pp0.pt" in str(e.value) or isinstance(e.value, (RuntimeError, EOFError, OSError, ValueError))
