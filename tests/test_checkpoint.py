"""Training snapshot save / auto-resume and HF safetensors round trip (CPU)."""
import json

import torch

from sensenova_u1_b200.config import tiny_mot
from sensenova_u1_b200.data.synthetic import tiny_batch
from sensenova_u1_b200.models.params import ParamStore
from sensenova_u1_b200.train.checkpoint import CheckpointManager, LoadMask, export_hf, import_hf
from sensenova_u1_b200.train.optimizer import AdamConfig
from sensenova_u1_b200.train.trainer import Trainer


def _trainer(seed=0):
    cfg = tiny_mot(num_layers=1)
    store = ParamStore(cfg, dtype=torch.float32, grad_dtype_mat=torch.float32)
    store.init_weights(seed)
    return cfg, store, Trainer(cfg, store, AdamConfig(lr=1e-2, state_dtype="fp32"))


def test_resume_reproduces_the_loss_curve(tmp_path):
    cfg, store, tr = _trainer()
    batches = [tiny_batch(cfg, seed=s, n_text=64) for s in range(4)]
    for b in batches[:2]:
        tr.train_step([b])
    mgr = CheckpointManager(f"local:{tmp_path}/run", checkpoint_every=2)
    save, kind, stop = mgr.decide(2, 100)
    assert save and kind == "step" and not stop
    d = mgr.save(2, store, tr.optim, train_state={"step": 2}, scheduler_state={"last_epoch": 2})
    assert (d / "2.step").exists() and (d / "model_tp0_pp0.pt").exists() and (d / "optimizer_tp0_pp0_zo0.pt").exists()
    assert (d / "schedulder.pt").exists() and (d / "context.pt").exists()
    ref = [tr.train_step([b])["loss"] for b in batches[2:]]
    # a fresh process: different init, then auto-resume
    cfg2, store2, tr2 = _trainer(seed=99)
    found = CheckpointManager(f"local:{tmp_path}/run").try_resume(store2, tr2.optim)
    assert found is not None and found[1][0]["step"] == 2
    got = [tr2.train_step([b])["loss"] for b in batches[2:]]
    assert got == ref


def test_incomplete_checkpoint_is_ignored_and_snapshots_alternate(tmp_path):
    cfg, store, tr = _trainer()
    mgr = CheckpointManager(str(tmp_path / "run"), snapshot_every=1)
    d0 = mgr.save(1, store, tr.optim, kind="snapshot")
    d1 = mgr.save(2, store, tr.optim, kind="snapshot")
    d2 = mgr.save(3, store, tr.optim, kind="snapshot")
    assert d0.name == "0" and d1.name == "1" and d2 == d0 and not (d0 / "1.step").exists()
    assert mgr.latest() == d0
    (d0 / "3.step").unlink()                      # a crash before the marker was written
    assert mgr.latest() == d1
    assert LoadMask.parse("all").optimizer and not LoadMask.parse(("model",)).optimizer


def test_stop_file_requests_a_final_checkpoint(tmp_path):
    stop = tmp_path / "stop"
    mgr = CheckpointManager(str(tmp_path / "run"), stop_file_path=str(stop))
    assert mgr.decide(5, 100) == (False, "", False)
    stop.write_text("1")
    assert mgr.decide(6, 100) == (True, "step", True)


def test_hf_export_import_roundtrip(tmp_path):
    cfg, store, _ = _trainer()
    store16 = ParamStore(cfg, dtype=torch.bfloat16, with_grads=False)
    store16.copy_from(store)
    wm = export_hf(store16, str(tmp_path / "hf"), max_shard_bytes=1 << 20)
    assert len(set(wm.values())) > 1
    idx = json.loads((tmp_path / "hf" / "model.safetensors.index.json").read_text())
    assert "language_model.model.layers.0.mlp_mot_gen.down_proj.weight" in idx["weight_map"]
    back = import_hf(str(tmp_path / "hf"))
    assert back.cfg.hidden_size == cfg.hidden_size and back.cfg.patch_size == cfg.patch_size
    for k in store16.p:
        assert torch.equal(store16.p[k], back.p[k]), k
