"""1F1B pipeline over gloo (2 stages, 4 micro-batches): losses and gradients equal the
single-process run of the same micro-batches."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sensenova_u1_b200.parallel.pipeline import one_f_one_b, partition_uniform

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_schedule_shape():
    assert one_f_one_b(2, 0, 4) == [("F", 0), ("F", 1), ("B", 0), ("F", 2), ("B", 1), ("F", 3), ("B", 2), ("B", 3)]
    assert one_f_one_b(2, 1, 4) == [("F", 0), ("B", 0), ("F", 1), ("B", 1), ("F", 2), ("B", 2), ("F", 3), ("B", 3)]
    s = one_f_one_b(4, 0, 8)
    assert [o for o, _ in s[:3]] == ["F"] * 3 and sorted(i for o, i in s if o == "B") == list(range(8))
    assert partition_uniform(42, 4) == [(0, 10), (10, 20), (20, 31), (31, 42)]


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _model():
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.models.params import ParamStore
    cfg = tiny_mot(num_layers=2)
    st = ParamStore(cfg, dtype=torch.float32, with_grads=False)
    st.init_weights(0)
    p = {k: v.clone().requires_grad_(True) for k, v in st.p.items()}
    batches = [tiny_batch(cfg, seed=20 + i, n_text=96) for i in range(4)]
    noises = [torch.randn(b.gen_x16.shape, generator=torch.Generator().manual_seed(i)) for i, b in enumerate(batches)]
    return cfg, p, batches, noises


def _stage_fn(cfg, p, batches, noises, layers, first, last):
    from sensenova_u1_b200.data.batch import KIND_GEN_IMG
    from sensenova_u1_b200.models import oracle

    def fn(x_in, i):
        b = batches[i]
        is_gen = (b.kind == KIND_GEN_IMG) | (b.tile_group.repeat_interleave(128) == 1)
        mask = oracle.dense_mask(b.meta, b.meta)
        if first:
            x, _, _ = oracle.embed_inputs(p, b, cfg, noises[i])
        else:
            x = x_in
        for l in range(*layers):
            x = oracle.decoder_layer(p, l, x, is_gen, b.pos3, mask, cfg)
        if not last:
            return x
        return oracle.head_losses(p, x, b, cfg, noises[i])[0] / len(batches)
    return fn


def _worker(rank, world, port, out, schedule="1f1b"):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sensenova_u1_b200.parallel.pipeline import PipelineStage
    cfg, p, batches, noises = _model()
    ranges = partition_uniform(cfg.num_layers, world)
    st = PipelineStage(_stage_fn(cfg, p, batches, noises, ranges[rank], rank == 0, rank == world - 1), rank, world,
                       rank - 1 if rank > 0 else None, rank + 1 if rank < world - 1 else None,
                       schedule=schedule, params=list(p.values()))
    losses = st.run(len(batches))
    torch.save({"grads": {k: v.grad for k, v in p.items() if v.grad is not None}, "losses": losses,
                "trace": st.trace}, out + f".{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_zero_bubble_order():
    from sensenova_u1_b200.parallel.pipeline import zero_bubble_h1
    for r in range(4):
        o = zero_bubble_h1(4, r, 8)
        assert [x for x in o if x[0] != "W"] == one_f_one_b(4, r, 8)          # same F/B order as 1F1B
        assert sorted(x for x in o if x[0] == "W") == [("W", i) for i in range(8)]
        assert all(o.index(("W", i)) > o.index(("B", i)) for i in range(8))
        # stage r holds back r weight-gradient passes: they fill its cool-down bubble
        tail = o[o.index(("B", 7)) + 1:]
        assert len(tail) == min(r, 8) + 1 and all(op == "W" for op, _ in tail)


@pytest.mark.parametrize("schedule", ["1f1b", "zero_bubble"])
def test_two_stage_pipeline_matches_single_process(tmp_path, schedule):
    out = str(tmp_path / "pp")
    mp.spawn(_worker, args=(2, _free_port(), out, schedule), nprocs=2, join=True)
    r0, r1 = torch.load(out + ".0"), torch.load(out + ".1")
    assert r0["trace"][:2] == [("F", 0), ("F", 1)] and r1["trace"][:2] == [("F", 0), ("B", 0)]
    if schedule == "zero_bubble":
        assert ("W", 0) in r0["trace"] and r1["trace"][-2:] == [("W", 2), ("W", 3)]
    from sensenova_u1_b200.models import oracle
    cfg, p, batches, noises = _model()
    total = 0
    for b, n in zip(batches, noises):
        loss, _ = oracle.training_loss(p, b, cfg, n)
        (loss / len(batches)).backward()
        total += float(loss) / len(batches)
    assert abs(sum(float(l) for l in r1["losses"]) - total) < 1e-5
    for k, v in p.items():
        if v.grad is None:
            continue
        g = r0["grads"].get(k)
        g1 = r1["grads"].get(k)
        got = (g if g is not None else 0) + (g1 if g1 is not None else 0)
        assert torch.allclose(got, v.grad, atol=2e-5, rtol=1e-4), k
