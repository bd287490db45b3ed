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
    assert (d / "2.step").exists() and (d / "model_wp0_pp0.pt").exists() and (d / "optimizer_wp0_pp0_zo0.pt").exists()
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


# ---------------------------------------------------------------------------
# name-keyed shards, expert files, conversion by the reference's own tool
# ---------------------------------------------------------------------------
import importlib.util
import os
import socket
import sys
from pathlib import Path

import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
_REF = next((c for c in (ROOT / "baseline" / "_ref", Path("/root/reference"))
             if (c / "training" / "tools" / "revert2hf.py").is_file()), None)


def _revert2hf():
    spec = importlib.util.spec_from_file_location("ref_revert2hf", _REF / "training" / "tools" / "revert2hf.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _moe_cfg(ep=1):
    return tiny_mot(num_layers=2, num_experts=8, num_experts_per_tok=2, gen_num_experts=4, gen_num_experts_per_tok=2,
                    moe_intermediate_size=64, ep_size=ep)


def test_weight_parallel_shards_reload_at_another_layout(tmp_path):
    cfg, store, tr = _trainer()
    for w in range(2):          # two weight-parallel ranks write their rows
        CheckpointManager(str(tmp_path / "run"), wp_rank=w, wp_size=2).save(7, store)
    d = tmp_path / "run" / "7"
    s0 = torch.load(d / "model_wp0_pp0.pt")
    k = "model.language_model.layers.0.feed_forward_mot_gen.w3.weight"
    assert s0[k].shape == (cfg.ffn_size // 2, cfg.hidden_size)
    assert s0["model.language_model.tok_embeddings.weight"].shape == (cfg.vocab_size, cfg.hidden_size // 2)
    assert s0["model.language_model.layers.0.attention_norm.weight"].shape == (cfg.hidden_size,)
    _, store2, _ = _trainer(seed=5)
    CheckpointManager(str(tmp_path / "run")).load(d, store2, mask=LoadMask(True, False, False, False))
    for name in store.p:
        assert torch.equal(store.p[name], store2.p[name]), name


@pytest.mark.skipif(_REF is None, reason="no copy of the reference's tools/revert2hf.py")
def test_reference_converter_reads_our_training_checkpoint(tmp_path):
    """Dense model written as two weight-parallel shards -> the reference's revert2hf -> the HF tensors."""
    from safetensors import safe_open
    from sensenova_u1_b200.models.params import hf_state_dict
    cfg, store, tr = _trainer()
    for w in range(2):
        CheckpointManager(str(tmp_path / "run"), wp_rank=w, wp_size=2).save(3, store)
    r2h = _revert2hf()
    r2h.convert(str(tmp_path / "run" / "3"), str(tmp_path / "hf"), "neo++_mot")
    got = {}
    for f in sorted((tmp_path / "hf").glob("*.safetensors")):
        with safe_open(str(f), framework="pt") as fh:
            for k in fh.keys():
                got[k] = fh.get_tensor(k)
    want = hf_state_dict(store)
    assert set(got) == set(want), (sorted(set(want) - set(got))[:4], sorted(set(got) - set(want))[:4])
    for k, v in want.items():
        assert torch.equal(got[k], v.reshape(got[k].shape)), k
    assert len(list((tmp_path / "hf").glob("model-*-of-00016.safetensors"))) == 16


def _ep_stores(seed=0):
    out = []
    for r in range(2):
        st = ParamStore(_moe_cfg(ep=2), dtype=torch.float32, with_grads=False, ep_rank=r)
        st.init_weights(seed)
        out.append(st)
    return out


def test_expert_parallel_ranks_keep_their_own_experts_across_resume(tmp_path):
    stores = _ep_stores()
    assert not torch.equal(stores[0].arena["exp"], stores[1].arena["exp"])
    for r, st in enumerate(stores):
        CheckpointManager(str(tmp_path / "run"), dp_rank=r, ep_rank=r).save(4, st)
    d = tmp_path / "run" / "4"
    assert (d / "model_moe_layer0_expert0_wp0.pt").exists() and (d / "model_moe_layer3_expert1_wp0.pt").exists()
    fresh = _ep_stores(seed=77)
    for r, st in enumerate(fresh):
        CheckpointManager(str(tmp_path / "run"), dp_rank=r, ep_rank=r).load(d, st, mask=LoadMask(True, False, False, False))
        assert torch.equal(st.arena["exp"], stores[r].arena["exp"])
        for name in st.p:
            assert torch.equal(st.p[name], stores[r].p[name]), name
    assert not torch.equal(fresh[0].arena["exp"], fresh[1].arena["exp"])


@pytest.mark.skipif(_REF is None, reason="no copy of the reference's tools/revert2hf.py")
def test_reference_converter_reads_our_expert_files(tmp_path):
    from safetensors import safe_open
    from sensenova_u1_b200.models.params import hf_state_dict
    stores = _ep_stores()
    for r, st in enumerate(stores):
        CheckpointManager(str(tmp_path / "run"), dp_rank=r, ep_rank=r).save(4, st)
    _revert2hf().convert(str(tmp_path / "run" / "4"), str(tmp_path / "hf"), "neo++_mot")
    got = {}
    for f in sorted((tmp_path / "hf").glob("*.safetensors")):
        with safe_open(str(f), framework="pt") as fh:
            for k in fh.keys():
                got[k] = fh.get_tensor(k)
    want = {}
    for st in stores:
        want.update(hf_state_dict(st))
    assert set(got) == set(want), (sorted(set(want) - set(got))[:4], sorted(set(got) - set(want))[:4])
    for k, v in want.items():
        assert torch.equal(got[k], v.reshape(got[k].shape)), k
    assert len(list((tmp_path / "hf").glob("moemodel-*.safetensors"))) == 2


def _export_worker(rank, world, port, out):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    st = ParamStore(_moe_cfg(ep=2), dtype=torch.float32, with_grads=False, ep_rank=rank)
    st.init_weights(0)
    export_hf(st, out)
    dist.destroy_process_group()


def test_hf_export_collects_every_ranks_experts(tmp_path):
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "hf")
    mp.spawn(_export_worker, args=(2, port, out), nprocs=2, join=True)
    idx = json.loads((tmp_path / "hf" / "model.safetensors.index.json").read_text())["weight_map"]
    cfg = _moe_cfg(ep=2)
    for e in range(cfg.num_experts):
        assert f"language_model.model.layers.1.mlp.experts.{e}.down_proj.weight" in idx
    for e in range(cfg.gen_num_experts):
        assert f"language_model.model.layers.0.mlp_mot_gen.experts.{e}.gate_proj.weight" in idx
    # a single process (no expert parallelism) imports the merged checkpoint with all experts
    back = import_hf(str(tmp_path / "hf"), dtype=torch.float32, ep_size=1)
    stores = _ep_stores()
    E2 = cfg.num_experts // 2
    w = back.p["layers.1.moe_und.w2"]
    assert torch.equal(w[:E2], stores[0].p["layers.1.moe_und.w2"]) and torch.equal(w[E2:], stores[1].p["layers.1.moe_und.w2"])


# ---------------------------------------------------------------------------
# converter command line: training shards <-> HF directory
# ---------------------------------------------------------------------------
def test_converter_dense_round_trip(tmp_path):
    from sensenova_u1_b200.train import convert
    cfg, store, _ = _trainer()
    store16 = ParamStore(cfg, dtype=torch.bfloat16, with_grads=False)
    store16.copy_from(store)
    for w in range(2):
        CheckpointManager(str(tmp_path / "run"), wp_rank=w, wp_size=2).save(9, store16)
    extras = tmp_path / "released"
    extras.mkdir()
    (extras / "tokenizer_config.json").write_text("{}")
    assert convert.main(["to-hf", "--src", str(tmp_path / "run" / "9"), "--tgt", str(tmp_path / "hf"),
                         "--extras-from", str(extras)]) == 0
    assert (tmp_path / "hf" / "tokenizer_config.json").exists() and (tmp_path / "hf" / "config.json").exists()
    back = import_hf(str(tmp_path / "hf"))
    for k in store16.p:
        assert torch.equal(store16.p[k], back.p[k]), k
    # and back to four training shards, read by the checkpoint manager
    assert convert.main(["to-train", "--src", str(tmp_path / "hf"), "--tgt", str(tmp_path / "init"), "--wp", "4"]) == 0
    assert sorted(p.name for p in (tmp_path / "init").glob("model_wp*")) == [f"model_wp{r}_pp0.pt" for r in range(4)]
    again = ParamStore(cfg, dtype=torch.bfloat16, with_grads=False)
    again.init_weights(123)
    CheckpointManager(str(tmp_path / "x")).load_model(tmp_path / "init", again)
    for k in store16.p:
        assert torch.equal(store16.p[k], again.p[k]), k


def test_converter_copies_understanding_branch_on_request(tmp_path):
    from sensenova_u1_b200.models.params import GEN, UND
    from sensenova_u1_b200.train import convert
    cfg, store, _ = _trainer()
    store16 = ParamStore(cfg, dtype=torch.bfloat16, with_grads=False)
    store16.copy_from(store)
    export_hf(store16, str(tmp_path / "hf"))
    convert.hf_to_training(str(tmp_path / "hf"), str(tmp_path / "init"), wp=1, mot_gen_init="copy")
    got = ParamStore(cfg, dtype=torch.bfloat16, with_grads=False)
    CheckpointManager(str(tmp_path / "x")).load_model(tmp_path / "init", got)
    assert not torch.equal(store16.p["layers.0.wqkv"][GEN], store16.p["layers.0.wqkv"][UND])
    assert torch.equal(got.p["layers.0.wqkv"][GEN], store16.p["layers.0.wqkv"][UND])
    assert torch.equal(got.p["layers.0.wqkv"][UND], store16.p["layers.0.wqkv"][UND])
    assert torch.equal(got.p["vision_gen.patch_w"], store16.p["vision_gen.patch_w"])


def test_converter_moe_experts_split_and_merge(tmp_path):
    from sensenova_u1_b200.train import convert
    cfg = _moe_cfg()
    store = ParamStore(cfg, dtype=torch.bfloat16, with_grads=False)
    store.init_weights(3)
    export_hf(store, str(tmp_path / "hf"))
    convert.hf_to_training(str(tmp_path / "hf"), str(tmp_path / "init"), wp=2, ep=2)
    d = tmp_path / "init"
    assert (d / "model_moe_layer3_expert1_wp0.pt").exists() and not (d / "model_moe_layer0_expert2_wp0.pt").exists()
    # an expert-parallel rank reads its half
    half = ParamStore(_moe_cfg(ep=2), dtype=torch.bfloat16, with_grads=False, ep_rank=1)
    CheckpointManager(str(tmp_path / "x"), dp_rank=1, ep_rank=1).load_model(d, half)
    assert torch.equal(half.p["layers.1.moe_und.w13"], store.p["layers.1.moe_und.w13"][4:])
    assert torch.equal(half.p["layers.1.moe_gen.w2"], store.p["layers.1.moe_gen.w2"][2:])
    # the converter merges the expert-parallel files again
    convert.training_to_hf(str(d), str(tmp_path / "hf2"))
    back = import_hf(str(tmp_path / "hf2"))
    for k in store.p:
        assert torch.equal(store.p[k], back.p[k]), k


def test_pipeline_stage_files_carry_the_models_layer_numbers(tmp_path):
    """A stage that holds layers [1, 2) of a 2-layer model numbers them from 0; its file says layer 1, and a
    tensor-parallel rank reads back exactly its own file."""
    from sensenova_u1_b200.parallel.pipeline_engine import stage_store
    cfg = tiny_mot(num_layers=2)
    full = ParamStore(cfg, dtype=torch.float32, with_grads=False)
    full.init_weights(11)
    st = stage_store(full, 1, 2, with_grads=False)
    mgr = CheckpointManager(str(tmp_path / "run"), pp_rank=1, layer_offset=1)
    d = mgr.save(5, st)
    sd = torch.load(d / "model_wp0_pp1.pt")
    assert any(".layers.1." in k for k in sd) and not any(".layers.0." in k for k in sd)
    back = stage_store(ParamStore(cfg, dtype=torch.float32, with_grads=False), 1, 2, with_grads=False)
    mgr.load_model(d, back)
    assert torch.equal(back.p["layers.0.wqkv"], full.p["layers.1.wqkv"])
    tp = CheckpointManager(str(tmp_path / "run_tp"), tp_rank=1, tp_size=2, pp_rank=0)
    d2 = tp.save(5, st)
    assert (d2 / "model_tp1_pp0.pt").exists()
    again = stage_store(ParamStore(cfg, dtype=torch.float32, with_grads=False), 1, 2, with_grads=False)
    tp.load_model(d2, again)
    assert torch.equal(again.p["layers.0.w2"], st.p["layers.0.w2"])
    with pytest.raises(FileNotFoundError):
        CheckpointManager(str(tmp_path / "run_tp"), tp_rank=0, tp_size=2).load_model(d2, again)


def test_remote_destination_is_mirrored_in_the_background_and_restored_on_a_fresh_machine(tmp_path):
    """A registered storage back-end stands for the remote side (here: another folder, with a slow upload)."""
    import time as _time
    from sensenova_u1_b200.utils import storage

    class Slow(storage.LocalBackend):
        def __init__(self, root):
            self.root, self.uploads = str(root), []

        def _p(self, path):
            return os.path.join(self.root, path.lstrip("/"))

        def upload(self, local_path, remote_path):
            _time.sleep(0.01)
            self.uploads.append(remote_path)
            super().upload(local_path, self._p(remote_path))

        def download(self, remote_path, local_path):
            super().download(self._p(remote_path), local_path)

        def listdir(self, remote_path):
            return super().listdir(self._p(remote_path))

    remote = Slow(tmp_path / "bucket")
    storage.register_backend("fake", remote)
    cfg, store, tr = _trainer()
    batches = [tiny_batch(cfg, seed=s, n_text=64) for s in range(3)]
    tr.train_step([batches[0]])
    mgr = CheckpointManager("fake:run1", checkpoint_every=1, local_work_folder=str(tmp_path / "work"))
    mgr.save(1, store, tr.optim, train_state={"step": 1})
    tr.train_step([batches[1]])
    mgr.save(2, store, tr.optim, train_state={"step": 2})            # confirms save 1 first: its marker goes out
    assert "run1/1/1.step" in remote.uploads and "run1/2/2.step" not in remote.uploads
    assert remote.uploads.index("run1/1/1.step") > remote.uploads.index("run1/1/model_wp0_pp0.pt")
    mgr.close()
    assert remote.uploads[-1] == "run1/2/2.step" and (tmp_path / "bucket" / "run1" / "2" / "optimizer_wp0_pp0_zo0.pt").exists()
    ref = tr.train_step([batches[2]])["loss"]
    # another machine: empty work folder, same remote
    cfg2, store2, tr2 = _trainer(seed=7)
    mgr2 = CheckpointManager("fake:run1", local_work_folder=str(tmp_path / "work2"))
    d, (ts, _, _) = mgr2.try_resume(store2, tr2.optim)
    assert ts["step"] == 2 and d == tmp_path / "work2" / "2"
    assert tr2.train_step([batches[2]])["loss"] == ref
    mgr2.close()

    class Broken(Slow):
        def upload(self, local_path, remote_path):
            if remote_path.endswith("context.pt"):
                raise OSError("disk full")
            super().upload(local_path, remote_path)

    bad = Broken(tmp_path / "bucket2")
    storage.register_backend("fake2", bad)
    mgr3 = CheckpointManager("fake2:run", local_work_folder=str(tmp_path / "work3"))
    mgr3.save(1, store, tr.optim, train_state={"step": 1})
    with pytest.raises(IOError, match="disk full"):
        mgr3.close()
    assert "run/1/1.step" not in bad.uploads                           # an incomplete remote copy never gets its marker


def test_ping_finds_an_unwritable_folder_before_training(tmp_path):
    mgr = CheckpointManager(str(tmp_path / "run"))
    mgr.ping()
    assert list((tmp_path / "run").iterdir()) == []                 # nothing is left behind
    blocker = tmp_path / "file"
    blocker.write_text("x")
    with pytest.raises(OSError):
        CheckpointManager(str(blocker / "run")).ping()              # a path below a file cannot be created


def test_converter_merges_a_tensor_x_pipeline_checkpoint(tmp_path):
    """Four ranks' files (tp 2 x pp 2, each stage trained its own non-layer tensors) -> one HF directory."""
    from sensenova_u1_b200.parallel.pipeline_engine import stage_store
    from sensenova_u1_b200.parallel.tensor_engine import shard_store_tp
    from sensenova_u1_b200.train import convert
    cfg = tiny_mot(num_layers=3)
    full = ParamStore(cfg, dtype=torch.bfloat16, with_grads=False)
    full.init_weights(21)
    ranges = [(0, 1), (1, 3)]                                   # partition_uniform(3, 2): the remainder goes to the last stage
    for p_, (l0, l1) in enumerate(ranges):
        st = stage_store(full, l0, l1, with_grads=False)
        # a stage does not train the other end's tensors: scramble them so that a wrong pick would show
        for name, v in st.p.items():
            tail = name.startswith(("final_norm", "lm_head", "fm_head"))
            if not name.startswith("layers.") and ((p_ == 0 and tail) or (p_ == 1 and not tail)):
                v.add_(1.0)
        for t in range(2):
            part = shard_store_tp(st, 2, t, with_grads=False)
            CheckpointManager(str(tmp_path / "run"), tp_rank=t, tp_size=2, pp_rank=p_, layer_offset=l0).save(4, part, model_cfg=cfg)
    d = tmp_path / "run" / "4"
    assert sorted(f.name for f in d.glob("model_tp*")) == ["model_tp0_pp0.pt", "model_tp0_pp1.pt", "model_tp1_pp0.pt", "model_tp1_pp1.pt"]
    convert.training_to_hf(str(d), str(tmp_path / "hf"))
    back = import_hf(str(tmp_path / "hf"))
    for k in full.p:
        assert torch.equal(full.p[k], back.p[k]), k


def test_ema_shadow_is_saved_and_found_again(tmp_path):
    cfg, store, tr = _trainer()
    mgr = CheckpointManager(str(tmp_path / "run"))
    ema = {"mat": torch.arange(8.0), "vec": torch.ones(3)}
    d = mgr.save(1, store, tr.optim, ema=ema)
    back = mgr.load_ema(d)
    assert set(back) == {"mat", "vec"} and torch.equal(back["mat"], ema["mat"])
    assert CheckpointManager(str(tmp_path / "run"), zero_rank=3).load_ema(d) is None      # another rank's file is not there
