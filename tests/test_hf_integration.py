"""transformers integration of the inference model: Auto-class registration, checkpoint round trip through
``from_pretrained`` / ``save_pretrained``, key names, sampling knobs, offload budgets (CPU)."""
import json

import pytest
import torch

import sensenova_u1_b200 as pkg
from sensenova_u1_b200.config import tiny_mot
from sensenova_u1_b200.models.params import ParamStore, hf_state_dict
from sensenova_u1_b200.train.checkpoint import export_hf


def _ckpt(tmp_path, **kw):
    cfg = tiny_mot(num_layers=2, **kw)
    store = ParamStore(cfg, dtype=torch.bfloat16, with_grads=False)
    store.init_weights(1)
    export_hf(store, str(tmp_path / "hf"))
    return cfg, store, str(tmp_path / "hf")


def test_auto_classes_resolve_to_this_package(tmp_path):
    from transformers import AutoConfig, AutoModel
    cfg, store, path = _ckpt(tmp_path)
    pkg.NEOChatModel                                  # first attribute access registers the classes
    c = AutoConfig.from_pretrained(path)
    assert type(c).__name__ == "NEOChatConfig" and c.llm_config.hidden_size == cfg.hidden_size
    assert c.llm_config.rope_theta_hw == cfg.rope_base_hw and not c.is_moe_llm
    m = AutoModel.from_pretrained(path, torch_dtype=torch.bfloat16, device_map="cpu")
    assert isinstance(m, pkg.NEOChatModel)
    sd = m.state_dict()
    want = hf_state_dict(store)
    assert set(sd) == set(want)
    for k, v in want.items():
        assert torch.equal(sd[k], v.reshape(sd[k].shape)), k
    assert m.num_parameters() == sum(v.numel() for v in want.values())
    # parameters are views of the arenas: no second copy of the weights
    assert sd["language_model.lm_head.weight"].data_ptr() == m.store.p["lm_head"].data_ptr()


def test_save_pretrained_round_trip_and_moe_config(tmp_path):
    cfg, store, path = _ckpt(tmp_path, num_experts=4, num_experts_per_tok=2, gen_num_experts=2, gen_num_experts_per_tok=1,
                             moe_intermediate_size=64)
    m = pkg.NEOChatModel.from_pretrained(path, device_map="cpu")
    assert m.config.is_moe_llm and m.config.llm_config.gen_num_experts == 2
    m.save_pretrained(str(tmp_path / "again"))
    m2 = pkg.NEOChatModel.from_pretrained(str(tmp_path / "again"), device_map={"": "cpu"})
    for (k, a), (_, b) in zip(sorted(m.state_dict().items()), sorted(m2.state_dict().items())):
        assert torch.equal(a, b), k
    raw = json.loads((tmp_path / "again" / "config.json").read_text())
    assert raw["model_type"] == "neo_chat" and raw["llm_config"]["num_experts"] == 4


def test_newer_checkpoint_is_refused(tmp_path):
    cfg, store, path = _ckpt(tmp_path)
    p = tmp_path / "hf" / "config.json"
    raw = json.loads(p.read_text()); raw["sensenova_u1_min_version"] = "99.0.0"; p.write_text(json.dumps(raw))
    with pytest.raises(RuntimeError):
        pkg.NEOChatModel.from_pretrained(path, device_map="cpu")


def test_sampling_filters():
    from sensenova_u1_b200.inference.engine import InferenceEngine as E
    torch.manual_seed(0)
    lg = torch.randn(3, 64)
    assert torch.equal(E._pick_token(lg, None), lg.argmax(-1))
    assert torch.equal(E._pick_token(lg, {"do_sample": False, "temperature": 5.0}), lg.argmax(-1))
    top3 = set(torch.topk(lg[0], 3).indices.tolist())
    seen = {int(E._pick_token(lg[:1], {"do_sample": True, "top_k": 3, "temperature": 2.0})) for _ in range(300)}
    assert seen <= top3 and len(seen) > 1
    # a tiny nucleus keeps only the most likely token
    seen = {int(E._pick_token(lg[:1], {"do_sample": True, "top_p": 1e-6})) for _ in range(50)}
    assert seen == {int(lg[0].argmax())}


def test_offload_budgets_and_phases():
    from sensenova_u1_b200.utils.offload import LayerOffloader, parse_bytes, vram_mode_for_budget
    assert parse_bytes("20GiB") == 20 << 30 and parse_bytes("512MB") == 512_000_000 and parse_bytes(7) == 7
    dev = torch.device("cuda", 0)
    assert vram_mode_for_budget({0: "80GiB"}, 35 << 30, dev) == "full"
    assert vram_mode_for_budget({0: "24GiB"}, 35 << 30, dev) == "fast"
    assert vram_mode_for_budget({0: "9GiB"}, 35 << 30, dev) == "balanced"
    assert vram_mode_for_budget({0: "5GiB"}, 35 << 30, dev) == "low"
    cfg = tiny_mot(num_layers=6)
    store = ParamStore(cfg, dtype=torch.float32, with_grads=False)
    store.init_weights(0)
    probe = LayerOffloader(store, "cpu", "low")
    off = LayerOffloader(store, "cpu", "low", resident_budget_bytes=2 * probe.layer_bytes + 5,
                         gen_resident_budget_bytes=3 * probe.gen_layer_bytes)
    assert off.n_resident == 2 and off.n_gen_resident == 3
    phases = []
    off.on_phase.append(phases.append)
    from sensenova_u1_b200.models.params import GEN, UND
    for l in range(6):                       # prefix: understanding tensors
        w = off.layer_weights(l)
        assert torch.equal(w["wqkv"], store.p[f"layers.{l}.wqkv"][UND])
    off.set_phase("denoise")
    for step in range(2):
        before = off.bytes_streamed
        for l in range(6):
            assert torch.equal(off.layer_weights(l)["w2"], store.p[f"layers.{l}.w2"][GEN])
        streamed = off.bytes_streamed - before
        # pass 0 copies the four non-resident layers once; afterwards only the one outside the generation residency moves
        assert (streamed == 4 * probe.gen_layer_bytes) if step == 0 else (streamed <= probe.gen_layer_bytes)
    assert len(off.gen_cache) == 3 and off.residency()["generation"] == 3 * probe.gen_layer_bytes
    off.set_phase("prefix")
    assert not off.gen_cache and phases == ["denoise", "prefix"]


def test_offload_serves_expert_mixtures_per_branch():
    from sensenova_u1_b200.models.params import GEN, UND
    from sensenova_u1_b200.utils.offload import LayerOffloader
    cfg = tiny_mot(num_layers=2, num_experts=4, num_experts_per_tok=2, gen_num_experts=2, gen_num_experts_per_tok=1,
                   moe_intermediate_size=64)
    store = ParamStore(cfg, dtype=torch.float32, with_grads=False)
    store.init_weights(0)
    off = LayerOffloader(store, "cpu", "low")
    w = off.layer_weights(0)
    assert "moe_und.w13" in w and "moe_gen.w13" not in w and torch.equal(w["moe_und.gate"], store.p["layers.0.moe_und.gate"])
    off.set_phase("denoise")
    w = off.layer_weights(1)
    assert "moe_gen.w2" in w and "moe_und.w2" not in w and torch.equal(w["wo"], store.p["layers.1.wo"][GEN])


def test_offline_snapshot_resolution_wants_complete_snapshots(tmp_path, monkeypatch):
    """A repository id resolves to its newest *complete* snapshot in the local cache; a snapshot that lacks a shard
    named by its index (an interrupted download) is not used."""
    import json
    import os
    import time
    from sensenova_u1_b200.inference.hf import resolve_checkpoint_path, snapshot_is_complete
    monkeypatch.setenv("HF_HUB_CACHE", str(tmp_path))
    snaps = tmp_path / "models--acme--tiny" / "snapshots"
    old, new = snaps / "aaa", snaps / "bbb"
    for d in (old, new):
        d.mkdir(parents=True)
        (d / "config.json").write_text("{}")
    (old / "model.safetensors").touch()
    (new / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {
        "a": "model-00001-of-00002.safetensors", "b": "model-00002-of-00002.safetensors"}}))
    (new / "model-00001-of-00002.safetensors").touch()
    os.utime(new, (time.time() + 10, time.time() + 10))
    assert snapshot_is_complete(old) and not snapshot_is_complete(new)
    assert resolve_checkpoint_path("acme/tiny") == str(old)          # the newer one is incomplete
    (new / "model-00002-of-00002.safetensors").touch()
    assert resolve_checkpoint_path("acme/tiny") == str(new)
    (old / "model.safetensors").unlink()
    (new / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(FileNotFoundError, match="missing weight files"):
        resolve_checkpoint_path("acme/tiny")
    with pytest.raises(FileNotFoundError):
        resolve_checkpoint_path("acme/absent")
    assert resolve_checkpoint_path(str(old)) == str(old)             # a directory is taken as given


def test_model_class_has_the_reference_methods():
    """Public methods of the reference's model class that callers outside the generation loops use."""
    import torch
    import sensenova_u1_b200 as pkg
    from sensenova_u1_b200.config import tiny_mot
    m = pkg.NEOChatModel.from_config(tiny_mot(), device="cpu")
    for name in ("t2i_generate", "it2i_generate", "interleave_gen", "interleave_gen_image_only", "chat", "batch_chat",
                 "generate", "extract_feature", "patchify", "unpatchify", "get_thw_indexes", "get_input_embeddings",
                 "get_output_embeddings", "lm_head"):
        assert hasattr(m, name), name
    assert m.get_input_embeddings().weight.shape == (1024, 256) and m.lm_head.weight.shape == (1024, 256)
    x = torch.randn(2, 3, 32, 48)
    pt = m.patchify(x, 16)
    assert pt.shape == (2, 6, 768) and torch.equal(m.unpatchify(pt, 16, 32, 48), x)
    assert torch.equal(pt, torch.einsum("nchpwq->nhwpqc", x.reshape(2, 3, 2, 16, 3, 16)).reshape(2, 6, 768))
    assert torch.equal(m.patchify(x, 16, channel_first=True),
                       torch.einsum("nchpwq->nhwcpq", x.reshape(2, 3, 2, 16, 3, 16)).reshape(2, 6, 768))
    pkg.main()
