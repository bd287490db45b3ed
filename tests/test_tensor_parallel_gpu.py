"""Tensor parallelism inside the CUDA engine: two ranks with half of the heads / FFN units each and peer-memory
all-reduces must reproduce the single-GPU step (2 GPUs); the sharding helpers round-trip on one."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg():
    from sensenova_u1_b200.config import tiny_mot
    return tiny_mot(head_dim=128, patch_size=16, num_layers=2, hidden_size=256, num_heads=4, num_kv_heads=2, ffn_size=1024)


def _batch(cfg, seed):
    from sensenova_u1_b200.data.synthetic import tiny_batch
    return tiny_batch(cfg, seed=seed, n_text=200, image_px=8 * 32, with_und_image=True)


def test_shard_and_merge_round_trip():
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.parallel.tensor_engine import merge_tp_stores, shard_store_tp, tp_local_config
    cfg = _cfg()
    full = ParamStore(cfg, device="cuda", with_grads=False)
    full.init_weights(0, std=0.05)
    parts = [shard_store_tp(full, 2, r, with_grads=False) for r in range(2)]
    loc = tp_local_config(cfg, 2)
    assert parts[0].p["layers.0.wqkv"].shape == (2, loc.q_dim + 2 * loc.kv_dim, cfg.hidden_size)
    assert parts[1].p["layers.1.w2"].shape == (2, cfg.hidden_size, cfg.ffn_size // 2)
    back = merge_tp_stores(parts, cfg, device="cuda")
    for k in full.p:
        assert torch.equal(back.p[k], full.p[k]), k


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import datetime
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.ops import _lib
    from sensenova_u1_b200.parallel.tensor_engine import shard_store_tp, tp_local_config
    from sensenova_u1_b200.train.optimizer import AdamConfig
    from sensenova_u1_b200.train.trainer import Trainer
    cfg = _cfg()
    full = ParamStore(cfg, device=dev, with_grads=False)
    full.init_weights(0, std=0.05)
    store = shard_store_tp(full, world, rank)
    del full
    tr = Trainer(tp_local_config(cfg, world), store, AdamConfig(lr=1e-2, state_dtype="fp32", clip_grad_norm=0.0),
                 tp_group=dist.group.WORLD, max_tokens=1024)
    losses = [tr.train_step([_batch(cfg, 100 + s).pin()])["loss"] for s in range(2)]
    torch.cuda.synchronize()
    _lib.check_status()
    assert tr.engine.tp.calls > 0
    torch.save({"p": {k: v.cpu() for k, v in store.p.items()}, "loss": losses}, out + f".{rank}")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_tensor_parallel_step_matches_single_gpu(tmp_path):
    import torch.multiprocessing as mp
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.parallel.tensor_engine import merge_tp_stores, tp_local_config
    from sensenova_u1_b200.train.optimizer import AdamConfig
    from sensenova_u1_b200.train.trainer import Trainer
    out = str(tmp_path / "w")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    cfg = _cfg()
    parts = []
    res = [torch.load(out + f".{r}") for r in range(2)]
    for r in range(2):
        st = ParamStore(tp_local_config(cfg, 2), device="cpu", with_grads=False)
        for k, v in res[r]["p"].items():
            st.p[k].copy_(v)
        parts.append(st)
    got = merge_tp_stores(parts, cfg)
    # replicated tensors must have stayed identical on both ranks
    for k in ("embed_tokens", "lm_head", "layers.0.attn_norm", "final_norm", "fm_head.w1"):
        assert torch.equal(res[0]["p"][k], res[1]["p"][k]), k
    ref = ParamStore(cfg, device="cuda")
    ref.init_weights(0, std=0.05)
    init = {k: v.clone() for k, v in ref.p.items()}
    tr = Trainer(cfg, ref, AdamConfig(lr=1e-2, state_dtype="fp32", clip_grad_norm=0.0))
    ref_losses = [tr.train_step([_batch(cfg, 100 + s).pin()])["loss"] for s in range(2)]
    for a, b in zip(ref_losses, res[0]["loss"]):
        assert abs(a - b) <= 2e-3 * max(1.0, abs(a)), (ref_losses, res[0]["loss"])
    for a, b in zip(res[0]["loss"], res[1]["loss"]):          # loss sums use atomics: equal up to the last bits
        assert abs(a - b) <= 1e-5 * max(1.0, abs(a))
    for k in ("layers.0.wqkv", "layers.1.w13", "layers.0.wo", "layers.1.w2", "embed_tokens", "lm_head"):
        du = got.p[k].float() - init[k].float().cpu()
        dr = ref.p[k].float().cpu() - init[k].float().cpu()
        cos = ((du * dr).sum() / (du.norm() * dr.norm() + 1e-20)).item()
        assert cos > 0.97, (k, cos)
