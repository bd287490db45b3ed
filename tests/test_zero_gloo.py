"""ZeRO-1 on CPU/gloo, world_size 2: one SFT step of the tiny MoT must equal the
single-process step on the concatenated data (reference semantics: sum of gradients,
each rank updates its partition, updated weights reach every rank)."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _build(rank_seed):
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.models.params import ParamStore
    cfg = tiny_mot(num_layers=2)
    store = ParamStore(cfg, dtype=torch.float32, grad_dtype_mat=torch.float32, shard_multiple=8 * 128 * 2)
    store.init_weights(0)
    return cfg, store, tiny_batch(cfg, seed=rank_seed, n_text=128)


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sensenova_u1_b200.train.optimizer import AdamConfig
    from sensenova_u1_b200.train.trainer import Trainer
    cfg, store, batch = _build(10 + rank)
    tr = Trainer(cfg, store, AdamConfig(lr=1e-2, state_dtype="fp32"), dp_group=None, host_group=None)
    res = tr.train_step([batch])
    torch.save({"arena": {k: v.clone() for k, v in store.arena.items()}, "loss": res["loss"],
                "pieces": tr.optim.pieces}, out + f".{rank}")
    dist.destroy_process_group()


def test_zero1_two_ranks_matches_single_process(tmp_path):
    world, port = 2, _free_port()
    out = str(tmp_path / "r")
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    r0, r1 = torch.load(out + ".0"), torch.load(out + ".1")
    for k in r0["arena"]:
        assert torch.equal(r0["arena"][k], r1["arena"][k]), "ranks diverged after the all-gather"
    for a in r0["pieces"]:                                          # every bucket is split in two
        for p0, p1 in zip(r0["pieces"][a], r1["pieces"][a]):
            assert p0[1] == p0[3] and p0[4] == p1[3] and p1[4] == p1[2]

    # single process: two micro-batches, same normalisers (mean over "ranks")
    from sensenova_u1_b200.train.optimizer import AdamConfig
    from sensenova_u1_b200.train.trainer import Trainer
    cfg, store, b0 = _build(10)
    _, _, b1 = _build(11)
    tr = Trainer(cfg, store, AdamConfig(lr=1e-2, state_dtype="fp32"))
    ce = (b0.ce_weight_sum + b1.ce_weight_sum) / 2
    gn = (b0.gen_weight_sum + b1.gen_weight_sum) / 2
    store.zero_grads()
    tr._oracle_step(b0, None, ce, gn)
    tr._oracle_step(b1, None, ce, gn)
    tr.optim.grad_divisor = 2.0
    tr.optim.step()
    for k in store.arena:
        err = (store.arena[k] - r0["arena"][k]).abs().max().item()
        assert err < 2e-5, (k, err)
