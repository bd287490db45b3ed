import torch

from sensenova_u1_b200.config import tiny_mot
from sensenova_u1_b200.models.params import ParamStore, hf_state_dict
from sensenova_u1_b200.utils.lora import merge_lora
from sensenova_u1_b200.utils.offload import LayerOffloader


def _store():
    cfg = tiny_mot(num_layers=4)
    st = ParamStore(cfg, dtype=torch.float32, with_grads=False)
    st.init_weights(0)
    return cfg, st


def test_lora_merge_hits_fused_slices():
    cfg, st = _store()
    name = "language_model.model.layers.1.self_attn.k_proj_mot_gen"
    before = hf_state_dict(st)[name + ".weight"].clone()
    q_before = hf_state_dict(st)["language_model.model.layers.1.self_attn.q_proj_mot_gen.weight"].clone()
    down, up = torch.randn(4, cfg.hidden_size), torch.randn(cfg.kv_dim, 4)
    n = merge_lora(st, {f"base_model.model.{name}.lora_A.weight": down, f"base_model.model.{name}.lora_B.weight": up,
                        f"base_model.model.{name}.alpha": torch.tensor(8.0)})
    assert n == 1
    after = hf_state_dict(st)[name + ".weight"]
    assert torch.allclose(after, before + (up @ down) * 2.0, atol=1e-5)
    assert torch.equal(hf_state_dict(st)["language_model.model.layers.1.self_attn.q_proj_mot_gen.weight"], q_before)


def test_offloader_streams_the_branch_of_the_phase():
    cfg, st = _store()
    off = LayerOffloader(st, "cpu", "balanced")          # 0 resident layers of 4
    assert off.n_resident == 0
    w = off.layer_weights(2)
    assert torch.equal(w["wqkv"], st.p["layers.2.wqkv"][0]) and w["wqkv"].dim() == 2
    off.set_phase("denoise")
    w = off.layer_weights(2)
    assert torch.equal(w["w2"], st.p["layers.2.w2"][1])
    assert torch.equal(off.layer_weights(3)["attn_norm"], st.p["layers.3.attn_norm"][1])
    full = LayerOffloader(st, "cpu", "full")
    assert full.n_resident == 4 and full.bytes_streamed == 0
    assert torch.equal(full.layer_weights(1)["wo"], st.p["layers.1.wo"][0])


def test_moe_monitor_statistics():
    import torch
    from sensenova_u1_b200.utils.moe_monitor import MoEMonitor
    m = MoEMonitor()
    m.record(0, "und", torch.tensor([4, 4, 4, 4], dtype=torch.int32))
    m.record(1, "und", torch.tensor([16, 0, 0, 0], dtype=torch.int32))
    m.record(1, "und", torch.tensor([16, 0, 0, 0], dtype=torch.int32))      # accumulates over micro-batches
    s = m.summary(reduce=False)
    assert s["moe/und/layer0/above_avg_frac"] == 0.0 and abs(s["moe/und/layer0/entropy"] - 1.0) < 1e-9
    assert s["moe/und/layer1/tokens"] == 32 and s["moe/und/layer1/idle_experts"] == 3
    assert abs(s["moe/und/layer1/above_avg_frac"] - 0.75) < 1e-9 and s["moe/und/layer1/max_over_mean"] == 4.0
    assert abs(s["moe/und/mean_idle_experts"] - 1.5) < 1e-9
    m.reset()
    assert m.summary(reduce=False) == {}


def test_gguf_round_trip_and_param_report(tmp_path):
    import torch
    from sensenova_u1_b200.config import get_config, tiny_mot
    from sensenova_u1_b200.models.params import ParamStore, hf_state_dict
    from sensenova_u1_b200.utils import gguf_loader, param_count
    cfg = tiny_mot()
    a = ParamStore(cfg, device="cpu", dtype=torch.float32, with_grads=False)
    a.init_weights(3, std=0.05)
    path = str(tmp_path / "m.gguf")
    gguf_loader.save_gguf(path, {k: v.contiguous() for k, v in hf_state_dict(a).items()}, quant="Q8_0")
    b = ParamStore(cfg, device="cpu", dtype=torch.float32, with_grads=False)
    missing = gguf_loader.load_gguf(path, b)
    assert not missing
    for k in ("embed_tokens", "layers.0.wqkv", "layers.1.w2", "final_norm"):
        err = (a.p[k] - b.p[k]).abs().max().item()
        assert err < 2e-3, (k, err)                      # 8-bit blocks: about 1/256 of the block maximum
    g = param_count.breakdown(get_config("8b-mot"))
    assert sum(g.values()) == 17_552_340_992
    assert abs(g["llm_generation"] + g["generation_modules"] - 8.186e9) < 2e6
    assert abs(g["shared"] - 1.245e9) < 1e6
    assert "17.552 B" in param_count.report(get_config("8b-mot"))


def test_comparison_sheet():
    import torch
    from sensenova_u1_b200.utils.comparison import comparison_sheet, difference
    x, y = torch.zeros(3, 32, 48), torch.full((3, 40, 32), 0.5)
    sheet = comparison_sheet([x, y], ["a", "b"])
    assert sheet.size[0] == 48 + 32 + 3 * 8 and sheet.size[1] >= 40
    d = difference(x, x + 0.1)
    assert abs(d["mae"] - 0.1) < 1e-6 and 25 < d["psnr"] < 27


def test_prompt_enhancer_backends(monkeypatch):
    import pytest
    from sensenova_u1_b200.inference import prompt_enhance as PE
    calls = []

    def oa(url, headers, json):
        calls.append((url, headers, json))
        return {"choices": [{"message": {"content": " a detailed fox "}}]}

    def an(url, headers, json):
        calls.append((url, headers, json))
        return {"content": [{"type": "text", "text": "long "}, {"type": "text", "text": "prompt"}]}

    monkeypatch.setenv("U1_ENHANCE_API_KEY", "k")
    monkeypatch.setenv("U1_ENHANCE_ENDPOINT", "http://x/v1/chat/completions")
    monkeypatch.setenv("U1_ENHANCE_MODEL", "m")
    e = PE.PromptEnhancer.from_env(transport=oa)
    assert e.enhance("fox") == "a detailed fox"
    assert calls[-1][1]["Authorization"] == "Bearer k" and calls[-1][2]["messages"][1]["content"] == "fox"
    e = PE.PromptEnhancer.from_env(backend="anthropic", transport=an, style="infographic")
    assert e.enhance("chart") == "long prompt" and calls[-1][2]["system"] == PE.STYLES["infographic"]
    monkeypatch.delenv("U1_ENHANCE_API_KEY")
    with pytest.raises(RuntimeError):
        PE.PromptEnhancer.from_env()
    with pytest.raises(ValueError):
        PE.PromptEnhancer(None, style="nope")

    e = PE.PromptEnhancer(PE.ChatCompletionsBackend("http://x", "k", "m", oa), style="edit")
    assert e.enhance("make it night", images=["QUJD"]) == "a detailed fox"
    part = calls[-1][2]["messages"][1]["content"]
    assert part[0]["text"] == "make it night" and part[1]["image_url"]["url"].endswith("QUJD")

    class M:
        def chat(self, tok, px, q, generation_config=None):
            return ""
    assert PE.PromptEnhancer.local(M(), None).enhance("keep me") == "keep me"


def test_train_record_counts_and_acc_perplex():
    import math
    import torch
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.train.metrics import AccPerplex, TrainRecord
    cfg = tiny_mot()
    b = tiny_batch(cfg, seed=0, n_text=64)
    rec = TrainRecord()
    out = rec.update([b, b], skipped_steps=2)
    assert out["num_consumed_tokens"] == 2 * b.n_tokens and out["inf_nan_skip_batches"] == 2
    assert out["num_consumed_text_tokens"] == 2 * b.n_text
    assert out["num_consumed_gen_images"] >= 2 and out["num_consumed_images"] >= out["num_consumed_gen_images"]
    assert out["num_padding_tokens"] == 2 * (b.S - b.n_tokens)
    assert sum(out[f"num_gen_samples_{n}"] for n in ("t2i", "editing", "interleave")) >= 2
    again = TrainRecord(); again.load_state_dict(rec.state_dict())
    assert again.update([b])["num_consumed_tokens"] == 3 * b.n_tokens
    m = AccPerplex(("all", "en"))
    m.update(30, 40, 40 * 1.5, "en")
    got = m.get_metric()
    assert got["acc"] == 0.75 and got["acc/en"] == 0.75 and abs(got["perplexity"] - math.exp(1.5)) < 1e-9
    assert m.get_metric() == {}


def test_step_tflops_counts_the_models_products():
    from sensenova_u1_b200.config import get_config
    from sensenova_u1_b200.train.metrics import step_tflops
    cfg = get_config("8b-mot")
    r = step_tflops(cfg, 16384, 1.0)
    # 8.1 B multiplied parameters per token (one branch) x 6 FLOP + dense causal attention + head: ~1.1 PFLOP per step
    assert 1050 < r["tflops"] < 1200 and r["tflops_hw"] > 1.25 * r["tflops"]
    sparse = step_tflops(cfg, 16384, 1.0, attention_pairs=0.06 * 16384 ** 2)
    assert sparse["tflops"] < r["tflops"]
    assert abs(step_tflops(cfg, 16384, 2.0, world=1)["tflops"] - r["tflops"] / 2) < 1e-6
    moe = step_tflops(get_config("a3b-mot"), 8192, 1.0)
    assert 0 < moe["tflops"] < r["tflops"]


def test_zero_grads_can_leave_the_layer_matrices():
    """``zero_grads(keep_layer_matrices=True)`` clears everything but the decoder layers' matrix gradients (their
    first writer stores); the plain call clears all."""
    import torch
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.models.params import ParamStore
    cfg = tiny_mot(num_layers=2)
    store = ParamStore(cfg, device="cpu")
    for t in store.grad_arena.values():
        t.fill_(1.0)
    store.zero_grads(keep_layer_matrices=True)
    for name in ("layers.0.wqkv", "layers.1.w2", "layers.0.w13", "layers.1.wo"):
        assert bool((store.g[name] == 1).all()), name
    for name in ("embed_tokens", "lm_head", "layers.0.attn_norm", "final_norm"):
        assert float(store.g[name].abs().sum()) == 0.0, name
    store.zero_grads()
    assert all(float(t.abs().sum()) == 0.0 for t in store.grad_arena.values())


def _example(name):
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location(f"example_{name}", os.path.join(root, "examples", name, "inference.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_example_clis_take_the_reference_flags(tmp_path):
    """Argument surfaces of the four example command lines (parsing only: no model is loaded)."""
    t2i = _example("t2i").parse(["--model_path", "x", "--prompt", "p", "--cfg_interval", "0.1", "0.9", "--think",
                                 "--think_output", "t.txt", "--print_think", "--enhance", "--print_enhance",
                                 "--device", "cuda:1", "--dtype", "float16", "--attn_backend", "flash", "--lora_path", "l",
                                 "--gguf_checkpoint", "g.gguf", "--output_dir", "o", "--vram_mode", "fast",
                                 "--max_memory", "0=20GiB", "--fast_vram_budget_gib", "12"])
    assert t2i.cfg_interval == [0.1, 0.9] and t2i.think and t2i.dtype == "float16" and t2i.fast_vram_budget_gib == 12.0
    ed_mod = _example("editing")
    ed = ed_mod.parse(["--jsonl", "e.jsonl", "--image", "a.png", "b.png", "--target_pixels", "1048576", "--no-do_resize",
                       "--input_max_pixels", "auto", "--use-edit-pe", "--print_edit_pe", "--edit_pe_model", "m", "--compare",
                       "--think", "--img_cfg_scale", "1.5"])
    assert ed.image == ["a.png", "b.png"] and ed.do_resize is False and ed.use_edit_pe and ed.compare
    assert ed_mod.input_pixel_budget("auto", 2) == 2048 * 2048 and ed_mod.input_pixel_budget("auto", 4) == 2048 * 2048 // 2
    assert ed_mod.input_pixel_budget("1048576", 3) == 1048576
    assert ed_mod.output_size((1000, 2000), 2048 * 2048, 32) == (2912, 1440)       # 2:1 kept, ~4.19 M pixels
    il = _example("interleave").parse(["--prompt", "p", "--no-think_mode", "--system_message", "s", "--resolution", "16:9",
                                       "--stem", "x", "--image_root", "r", "--max_images", "3", "--profile"])
    assert il.think_mode is False and il.max_rounds == 3 and il.resolution == "16:9" and il.profile
    vqa = _example("vqa").parse(["--jsonl", "q.jsonl", "--do_sample", "--temperature", "0.7", "--top_p", "0.9", "--top_k", "40",
                                 "--repetition_penalty", "1.1", "--output_dir", "o"])
    assert vqa.do_sample and vqa.top_k == 40 and vqa.random_init == "tiny-mot"
    import pytest
    with pytest.raises(SystemExit):
        _example("t2i").parse(["--prompt", "p", "--jsonl", "j"])


def test_cli_jobs_and_helpers(tmp_path):
    import argparse
    import json
    from sensenova_u1_b200.utils import cli
    assert cli.parse_max_memory("0=20GiB; cpu=64GiB") == {0: "20GiB", "cpu": "64GiB"}
    j = tmp_path / "jobs.jsonl"
    j.write_text(json.dumps({"prompt": "a", "width": 512, "id": "first"}) + "\n" + json.dumps({"prompt": "b", "seed": 7}) + "\n")
    a = argparse.Namespace(jsonl=str(j), output_dir=str(tmp_path / "out"), output="x.png")
    jobs = list(cli.iter_jobs(a, dict(prompt=None, width=2048, height=2048, seed=42)))
    assert [(jb["prompt"], jb["width"], jb["seed"]) for jb, _ in jobs] == [("a", 512, 42), ("b", 2048, 7)]
    assert [p.name for _, p in jobs] == ["first.png", "00001.png"] and (tmp_path / "out").is_dir()
    single = list(cli.iter_jobs(argparse.Namespace(jsonl=None, output="x.png"), dict(prompt="p")))
    assert single[0][0]["prompt"] == "p" and single[0][1].name == "x.png"
    j.write_text(json.dumps({"width": 1}) + "\n")
    import pytest
    with pytest.raises(ValueError):
        list(cli.iter_jobs(a, {}))
    assert cli.warn_if_unsupported_resolution(2048, 2048) is None and cli.warn_if_unsupported_resolution(512, 512) is None
    assert "buckets" in cli.warn_if_unsupported_resolution(3000, 3000)


def test_editing_compare_sheet(tmp_path):
    import torch
    sheet = _example("editing").compare_sheet([torch.zeros(3, 64, 96), torch.zeros(3, 32, 32)], torch.zeros(3, 64, 64))
    sheet.save(tmp_path / "c.png")
    assert sheet.size[0] >= 96 + 32 + 64 and sheet.size[1] >= 64


def test_param_inspector_counts_a_checkpoint_from_its_headers(tmp_path, capsys):
    import json
    import torch
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.train.checkpoint import export_hf
    from sensenova_u1_b200.utils import param_count as pc
    cfg = tiny_mot(num_layers=2)
    store = ParamStore(cfg, dtype=torch.bfloat16, with_grads=False)
    store.init_weights(0)
    export_hf(store, str(tmp_path / "hf"), max_shard_bytes=1 << 20)
    res = pc.inspect_checkpoint(str(tmp_path / "hf"))
    by_cfg = pc.breakdown(cfg)
    assert res["total_params"] == sum(by_cfg.values()) and res["total_bytes"] == 2 * res["total_params"]
    g = {k: v["params"] for k, v in res["groups"].items()}
    assert g["shared"] == by_cfg["shared"]
    assert g["generation_transformer"] == by_cfg["generation_modules"] + by_cfg["llm_generation"]
    assert g["understanding_transformer"] == by_cfg["visual_understanding"] + by_cfg["llm_understanding"]
    rules = tmp_path / "rules.json"
    rules.write_text(json.dumps({"heads": ["language_model.lm_head", "fm_modules.fm_head"], "rest": ["language_model", "vision_model", "fm_modules"]}))
    pc.main(["--model_path", str(tmp_path / "hf"), "--custom_groups_json", str(rules), "--show_groups", "heads"])
    out = capsys.readouterr().out
    assert "[heads]" in out and "language_model.lm_head.weight" in out and "rest" in out
    assert pc.group_of("something.embed.weight", pc.DEFAULT_RULES) == "embedding_misc" and pc.si(1_250_000) == "1.250M"


def test_requirement_files_follow_pyproject(tmp_path):
    import importlib.util
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    spec = importlib.util.spec_from_file_location("render_requirements", root / "render_requirements.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.main(["--check"]) == 0                                  # the committed files are current
    (tmp_path / "pyproject.toml").write_text('[project]\nname = "x"\ndependencies = ["a>=1", "b"]\n'
                                             '[project.optional-dependencies]\nextra = ["c"]\n')
    assert mod.main(["--check", "--root", str(tmp_path)]) == 1         # nothing written yet
    assert mod.main(["--root", str(tmp_path)]) == 0
    assert (tmp_path / "requirements.txt").read_text().endswith("a>=1\nb\n")
    assert (tmp_path / "requirements-extra.txt").read_text().endswith("-r requirements.txt\nc\n")
    assert mod.main(["--check", "--root", str(tmp_path)]) == 0


def test_token_picking_applies_the_repetition_penalty_before_sampling():
    import torch
    from sensenova_u1_b200.inference.api import NEOChatModel
    from sensenova_u1_b200.inference.engine import InferenceEngine
    pick = InferenceEngine._pick_token
    logits = torch.tensor([[2.0, 1.9, -1.0, 0.5], [0.1, -0.2, -0.3, -0.25]])
    assert pick(logits, None).tolist() == [0, 0]
    seen = torch.tensor([[True, False, False, False], [True, True, False, False]])
    greedy = {"do_sample": False, "repetition_penalty": 1.5}
    # row 0: 2.0 / 1.5 < 1.9 -> token 1; row 1: 0.1 / 1.5 = 0.067 still the largest; negatives move further down
    assert pick(logits, greedy, seen).tolist() == [1, 0]
    assert pick(logits, greedy, None).tolist() == [0, 0]
    torch.manual_seed(0)
    s = {"do_sample": True, "temperature": 1.0, "top_k": 1, "top_p": 1.0, "repetition_penalty": 1.5}
    assert pick(logits, s, seen).tolist() == [1, 0]                      # top-1 sampling = argmax of the penalised logits
    assert NEOChatModel._sampling({"do_sample": False}) is None
    got = NEOChatModel._sampling({"do_sample": False, "repetition_penalty": 1.05, "top_p": None})
    assert got["repetition_penalty"] == 1.05 and got["do_sample"] is False and got["top_p"] == 1.0


def test_placeholders_expand_over_history_question_and_partial_answer():
    from sensenova_u1_b200.inference import prompts
    img = lambda n: prompts.IMG_START_TOKEN + prompts.IMG_CONTEXT_TOKEN * n + prompts.IMG_END_TOKEN
    hist, q, tail = prompts.expand_conversation([("user", "<image>\nwhat?"), ("assistant", "a cat")], "and <image> here <image>?",
                                                "see <image>", [2, 1, 3, 4])
    assert hist == [("user", img(2) + "\nwhat?"), ("assistant", "a cat")]
    assert q == "and " + img(1) + " here " + img(3) + "?" and tail == "see " + img(4)
    assert prompts.expand_conversation([], "plain", "", []) == ([], "plain", "")
    import pytest
    with pytest.raises(ValueError):
        prompts.expand_conversation([], "<image>", "", [])


def test_prompt_embedding_places_pictures_of_history_question_and_partial_answer():
    """``NEOChatModel._embed_prompt`` on CPU with a stand-in vision front-end: every picture's embeddings land on its own
    run of context tokens, in reading order over earlier turns, the question and the part of the answer that exists."""
    import types
    import torch
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.inference.api import ByteTokenizer, NEOChatModel
    cfg = tiny_mot(patch_size=16, vocab_size=1024)
    H, tp = cfg.hidden_size, cfg.token_pixels
    m = NEOChatModel.__new__(NEOChatModel)
    m.cfg, m.system_message = cfg, None
    m.store = types.SimpleNamespace(p={"embed_tokens": torch.zeros(cfg.vocab_size, H, dtype=torch.bfloat16)}, device=torch.device("cpu"))
    calls = []

    class Vision:
        def vision_embed(self, branch, p16, px, py):
            n = p16.shape[0] // cfg.merge_size ** 2
            calls.append(n)
            return torch.full((n, H), float(len(calls)), dtype=torch.bfloat16)      # picture k embeds as the constant k
    m.engine = Vision()
    tok = ByteTokenizer(cfg.vocab_size)
    img = lambda h, w: torch.zeros(3, h * tp, w * tp)
    ids, x, pos3 = m._embed_prompt(tok, "and <image>?", [img(1, 1), img(1, 3), img(2, 1)],
                                   history=[("user", "<image>\nfirst"), ("assistant", "ok")], tail="see <image>")
    assert calls == [1, 3, 2] and ids.numel() == x.shape[0] == pos3.shape[1]
    marks = x[:, 0].float()
    runs = [int((marks == k).sum()) for k in (1, 2, 3)]
    assert runs == [1, 3, 2]                                                         # one run per picture, right sizes
    order = [int(marks[marks > 0][i]) for i in (0, 1, 4)]
    assert order == [1, 2, 3]                                                        # history first, then question, then tail
    import pytest
    with pytest.raises(ValueError):
        m._embed_prompt(tok, "no placeholder", [img(1, 1)])


def test_chat_adds_picture_tags_only_when_nothing_marks_them():
    import types
    import torch
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.inference.api import ByteTokenizer, NEOChatModel
    cfg = tiny_mot(patch_size=16, vocab_size=1024)
    H, tp = cfg.hidden_size, cfg.token_pixels
    m = NEOChatModel.__new__(NEOChatModel)
    m.cfg, m.system_message = cfg, None
    m.store = types.SimpleNamespace(p={"embed_tokens": torch.zeros(cfg.vocab_size, H, dtype=torch.bfloat16)}, device=torch.device("cpu"))
    seen = {}

    class Engine:
        def vision_embed(self, branch, p16, px, py):
            return torch.ones(p16.shape[0] // cfg.merge_size ** 2, H, dtype=torch.bfloat16)

        def prefill(self, docs, reserve_image_tokens=0, docs_embeds=None, docs_pos3=None):
            seen["ids"] = docs[0]
            return ["layout"], torch.zeros(1, H)

        def decode(self, lay, h, max_new_tokens, stop_ids=(), sampling=None, prompt_ids=None):
            seen.update(sampling=sampling, max_new_tokens=max_new_tokens, prompt=prompt_ids)
            return [[ord("o"), ord("k"), stop_ids[0]]]
    m.engine = Engine()
    tok = ByteTokenizer(cfg.vocab_size)
    img = torch.zeros(3, tp, 2 * tp)
    text = lambda: bytes(int(t) for t in seen["ids"].tolist() if int(t) < 256).decode(errors="ignore")
    assert m.chat(tok, img, "what?", generation_config={"max_new_tokens": 9, "repetition_penalty": 1.1}) == "ok"
    assert seen["max_new_tokens"] == 9 and seen["sampling"]["repetition_penalty"] == 1.1 and seen["sampling"]["do_sample"] is False
    assert seen["prompt"] is not None and "what?" in text()
    n_ctx = lambda: int((seen["ids"] == m.img_context_token_id).sum())
    assert n_ctx() == 2                                                   # the tag was added for the unmarked picture
    out, hist = m.chat(tok, [img, img], "and the second?", history=[("<image>\nfirst <image>", "two")], return_history=True)
    assert out == "ok" and n_ctx() == 4 and hist[-1] == ("and the second?", "ok")   # history marks both: nothing added
    assert m.chat(tok, None, "hi", system_message="SYS") == "ok" and "SYS" in text() and seen["sampling"] is None


def test_interleaved_generation_loop_with_a_stand_in_engine():
    """Two rounds: text that asks for a picture, the picture, then text to the end; the generated picture re-enters the
    context through the understanding branch and the sampling knobs of ``generation_config`` reach the decoder."""
    import types
    import torch
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.inference import prompts
    from sensenova_u1_b200.inference.api import ByteTokenizer, NEOChatModel, _encode
    cfg = tiny_mot(patch_size=16, vocab_size=1024)
    H, tp = cfg.hidden_size, cfg.token_pixels
    m = NEOChatModel.__new__(NEOChatModel)
    m.cfg, m.system_message = cfg, None
    m.store = types.SimpleNamespace(p={"embed_tokens": torch.zeros(cfg.vocab_size, H, dtype=torch.bfloat16)}, device=torch.device("cpu"))
    tok = ByteTokenizer(cfg.vocab_size)
    img_start, eos = int(_encode(tok, prompts.IMG_START_TOKEN)[-1]), int(_encode(tok, prompts.IM_END)[-1])
    log = {"prefill": [], "decode": [], "denoise": []}

    class Engine:
        def vision_embed(self, branch, p16, px, py):
            return torch.ones(p16.shape[0] // cfg.merge_size ** 2, H, dtype=torch.bfloat16)

        def prefill(self, docs, reserve_image_tokens=0, docs_embeds=None, docs_pos3=None):
            log["prefill"].append(int((docs[0] == m.img_context_token_id).sum()))
            return ["layout"], torch.zeros(1, H)

        def decode(self, lay, h, max_new_tokens, stop_ids=(), sampling=None, prompt_ids=None):
            log["decode"].append(sampling)
            first = len(log["decode"]) == 1
            return [[ord("a"), img_start] if first else [ord("b"), eos]]

        def denoise(self, samples, size, *a):
            log["denoise"].append((len(samples[0]), size))
            return torch.zeros(1, 3, size[1], size[0])
    m.engine = Engine()
    text, pics = m.interleave_gen(tok, "draw", image_size=(2 * tp, tp), max_rounds=3, think_mode=True,
                                  generation_config={"do_sample": True, "temperature": 0.7, "max_new_tokens": 5})
    assert len(pics) == 1 and pics[0].shape == (3, tp, 2 * tp) and log["denoise"] == [(2, (2 * tp, tp))]
    assert log["prefill"] == [0, 2]                      # the second round's context holds the generated picture (2 tokens)
    assert all(s and s["do_sample"] and s["temperature"] == 0.7 for s in log["decode"])
    assert text.startswith("a") and "[image]" in text and "b" in text.split("[image]")[-1]


def test_reference_helper_names_resolve():
    import sensenova_u1_b200.utils as u
    for name in ("InferenceProfiler", "parse_max_memory", "save_compare", "load_gguf_checkpoint", "build_rules", "format_param_count",
                 "add_offload_args", "load_model_and_tokenizer", "load_and_merge_lora_weight_from_safetensors",
                 "best_available_device", "seed_all_accelerators", "infer_input_device", "format_bytes"):
        assert callable(getattr(u, name)), name
    assert u.VRAM_MODE_OPTIONS == ("full", "fast", "balanced", "low") and u.DEFAULT_VRAM_MODE == "full"
    assert u.format_bytes(2_500_000_000) == "2.500GB" and u.format_bytes(12) == "12B" and u.format_param_count(17_552_000_000) == "17.552B"
    assert u.vram_mode_to_prefetch_count("full") == 0 and isinstance(u.vram_mode_keeps_generation_resident("fast"), bool)
    assert u.parse_max_memory("0=20GiB,cpu=64GiB") == {0: "20GiB", "cpu": "64GiB"} and u.best_available_device() in ("cuda", "cpu")
    import pytest
    with pytest.raises(AttributeError):
        u.no_such_helper
