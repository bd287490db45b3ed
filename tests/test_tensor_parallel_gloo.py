"""Tensor-parallel building blocks on gloo (2 ranks): column/row linears (with and without sequence
parallel), the Ulysses all-to-all and vocab-parallel cross entropy against single-process math."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _data():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(16, 32, generator=g)
    w1 = torch.randn(64, 32, generator=g) * 0.1
    w2 = torch.randn(32, 64, generator=g) * 0.1
    tgt = torch.randint(0, 64, (16,), generator=g)
    return x, w1, w2, tgt


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sensenova_u1_b200.parallel import tensor as tp
    x, w1, w2, tgt = _data()
    res = {}
    for sp in (False, True):
        xs = (x.chunk(world)[rank] if sp else x).clone().requires_grad_(True)
        a = w1.chunk(world, 0)[rank].clone().requires_grad_(True)        # column parallel
        b = w2.chunk(world, 1)[rank].clone().requires_grad_(True)        # row parallel
        h = tp.column_parallel_linear(xs, a, sequence_parallel=sp)
        y = tp.row_parallel_linear(F.silu(h), b, sequence_parallel=sp)
        loss = y.pow(2).sum()
        if sp:                                   # each rank holds its sequence slice of y
            loss_all = loss.detach().clone(); dist.all_reduce(loss_all)
        loss.backward()
        res[f"y_{sp}"], res[f"dx_{sp}"], res[f"da_{sp}"], res[f"db_{sp}"] = y.detach(), xs.grad, a.grad, b.grad
    # vocab-parallel CE: logits = x @ w1^T split over the vocabulary
    xs = x.clone().requires_grad_(True)
    ws = w1.chunk(world, 0)[rank].clone().requires_grad_(True)
    ce = tp.vocab_parallel_cross_entropy(F.linear(tp.copy_to_tp(xs), ws), tgt).mean()
    ce.backward()
    res["ce"], res["ce_dx"], res["ce_dw"] = ce.detach(), xs.grad, ws.grad
    # Ulysses: [S_local, heads, D] <-> [S, heads / w, D]
    q = torch.arange(8 * 4 * 2, dtype=torch.float32).view(8, 4, 2)            # full sequence 8, 4 heads
    ql = q.chunk(world, 0)[rank].clone().requires_grad_(True)
    qh = tp.seq_all_to_all(ql, None, True)
    res["a2a_ok"] = bool(torch.equal(qh, q[:, rank * 2:(rank + 1) * 2]))
    back = tp.seq_all_to_all(qh, None, False)
    res["a2a_roundtrip"] = bool(torch.equal(back, ql))
    back.sum().backward()
    res["a2a_grad"] = bool(torch.equal(ql.grad, torch.ones_like(ql)))
    torch.save(res, out + f".{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_tensor_parallel_matches_single_process(tmp_path):
    out = str(tmp_path / "tp")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    r = [torch.load(out + f".{i}") for i in range(2)]
    x, w1, w2, tgt = _data()
    xr, a, b = x.clone().requires_grad_(True), w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    y = F.linear(F.silu(F.linear(xr, a)), b)
    y.pow(2).sum().backward()
    assert torch.allclose(r[0]["y_False"], y, atol=1e-5) and torch.allclose(r[1]["y_False"], y, atol=1e-5)
    assert torch.allclose(r[0]["dx_False"], xr.grad, atol=1e-4)
    assert torch.allclose(torch.cat([r[0]["da_False"], r[1]["da_False"]], 0), a.grad, atol=1e-4)
    assert torch.allclose(torch.cat([r[0]["db_False"], r[1]["db_False"]], 1), b.grad, atol=1e-4)
    # sequence parallel: outputs and input grads are sequence slices
    assert torch.allclose(torch.cat([r[0]["y_True"], r[1]["y_True"]], 0), y, atol=1e-5)
    assert torch.allclose(torch.cat([r[0]["dx_True"], r[1]["dx_True"]], 0), xr.grad, atol=1e-4)
    assert torch.allclose(torch.cat([r[0]["da_True"], r[1]["da_True"]], 0), a.grad, atol=1e-4)
    xr2, w = x.clone().requires_grad_(True), w1.clone().requires_grad_(True)
    ce = F.cross_entropy(F.linear(xr2, w), tgt)
    ce.backward()
    assert abs(float(r[0]["ce"]) - float(ce)) < 1e-5
    assert torch.allclose(r[0]["ce_dx"], xr2.grad, atol=1e-5)
    assert torch.allclose(torch.cat([r[0]["ce_dw"], r[1]["ce_dw"]], 0), w.grad, atol=1e-5)
    for i in range(2):
        assert r[i]["a2a_ok"] and r[i]["a2a_roundtrip"] and r[i]["a2a_grad"]
