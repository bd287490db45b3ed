"""Pipeline parallelism of the CUDA engine (2 GPUs): two stages, four micro-batches, 1F1B over NCCL point-to-point
on two communicators, against the single-GPU step with the same four micro-batches; and the same with two
tensor-parallel ranks per stage when four GPUs are there."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg():
    from sensenova_u1_b200.config import tiny_mot
    return tiny_mot(head_dim=128, patch_size=16, num_layers=4, hidden_size=256, num_heads=4, num_kv_heads=2, ffn_size=1024)


def _batches(cfg, step, n=4):
    from sensenova_u1_b200.data.synthetic import tiny_batch
    return [tiny_batch(cfg, seed=100 * step + i, n_text=200, image_px=8 * 32, with_und_image=True) for i in range(n)]


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, tp, pp, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import datetime
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    from sensenova_u1_b200.ops import _lib
    from sensenova_u1_b200.parallel.pipeline_engine import PipelineTrainer
    from sensenova_u1_b200.train.optimizer import AdamConfig
    cfg = _cfg()
    pt = PipelineTrainer(cfg, tp, pp, dev, AdamConfig(lr=1e-2, state_dtype="fp32", clip_grad_norm=0.0), init_seed=0,
                         init_std=0.05, max_tokens=1024)
    losses = []
    for step in range(2):
        o = pt.step([b.to(dev) for b in _batches(cfg, step)])
        losses.append(float(o["loss"]) if o else None)
    torch.cuda.synchronize()
    _lib.check_status()
    torch.save({"p": {k: v.cpu() for k, v in pt.store.p.items()}, "loss": losses, "layers": pt.layers,
                "trace": pt.stage.trace}, out + f".{rank}")
    dist.barrier()
    dist.destroy_process_group()


def _reference(cfg):
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.train.optimizer import AdamConfig
    from sensenova_u1_b200.train.trainer import Trainer
    ref = ParamStore(cfg, device="cuda")
    ref.init_weights(0, std=0.05)
    init = {k: v.clone().cpu() for k, v in ref.p.items()}
    tr = Trainer(cfg, ref, AdamConfig(lr=1e-2, state_dtype="fp32", clip_grad_norm=0.0))
    losses = [float(tr.step_on_device([b.to("cuda") for b in _batches(cfg, step)])["loss"]) for step in range(2)]
    return ref, init, losses


def _cos(a, b):
    return ((a * b).sum() / (a.norm() * b.norm() + 1e-20)).item()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_stage_pipeline_matches_single_gpu(tmp_path):
    import torch.multiprocessing as mp
    out = str(tmp_path / "w")
    mp.spawn(_worker, args=(2, _free_port(), 1, 2, out), nprocs=2, join=True)
    cfg = _cfg()
    r0, r1 = torch.load(out + ".0"), torch.load(out + ".1")
    assert r0["layers"] == (0, 2) and r1["layers"] == (2, 4)
    assert r0["trace"][:2] == [("F", 0), ("F", 1)] and r1["trace"][:2] == [("F", 0), ("B", 0)]     # 1F1B
    ref, init, losses = _reference(cfg)
    for a, b in zip(losses, r1["loss"]):
        assert abs(a - b) <= 2e-3 * max(1.0, abs(a)), (losses, r1["loss"])
    # stage 0 owns layers 0-1 and the embeddings, stage 1 layers 2-3 and the heads
    for name, (res, local) in {"layers.1.wqkv": (r0, "layers.1.wqkv"), "layers.3.w13": (r1, "layers.1.w13"),
                               "embed_tokens": (r0, "embed_tokens"), "lm_head": (r1, "lm_head"),
                               "vision_gen.merge_w": (r0, "vision_gen.merge_w"), "fm_head.w2": (r1, "fm_head.w2")}.items():
        du = res["p"][local].float() - init[name].float()
        dr = ref.p[name].float().cpu() - init[name].float()
        assert _cos(du, dr) > 0.97, (name, _cos(du, dr))
    # what a stage does not use is not touched
    assert torch.equal(r1["p"]["embed_tokens"], init["embed_tokens"]) and torch.equal(r0["p"]["lm_head"], init["lm_head"])


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_tensor_parallel_stages(tmp_path):
    import torch.multiprocessing as mp
    from sensenova_u1_b200.parallel.tensor_engine import _slices
    out = str(tmp_path / "w")
    mp.spawn(_worker, args=(4, _free_port(), 2, 2, out), nprocs=4, join=True)
    cfg = _cfg()
    res = [torch.load(out + f".{r}") for r in range(4)]
    ref, init, losses = _reference(cfg)
    for a, b in zip(losses, res[2]["loss"]):
        assert abs(a - b) <= 3e-3 * max(1.0, abs(a)), (losses, res[2]["loss"])
    for a, b in zip(res[2]["loss"], res[3]["loss"]):
        assert abs(a - b) <= 1e-5 * max(1.0, abs(a))
    qkv_rows, w13_rows, o_cols, f_cols = _slices(cfg, 2, 1)
    du = res[3]["p"]["layers.0.w13"].float() - init["layers.2.w13"].float().index_select(1, w13_rows)
    dr = (ref.p["layers.2.w13"].float().cpu() - init["layers.2.w13"].float()).index_select(1, w13_rows)
    assert _cos(du, dr) > 0.97
