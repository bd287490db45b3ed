"""Annotation records -> samples: condition dropping, task flags, mixing, sharding, resume."""
import json
import pytest
import random

import torch

from sensenova_u1_b200.data.multimodal import (CfgDrop, ConversationDataset, prepare_generation_record,
                                                record_to_sample)
from sensenova_u1_b200.inference import prompts

tok = lambda s: [ord(c) % 251 + 4 for c in s]
img = lambda path, gen: torch.full((3, 64, 64), 1.0 if gen else -1.0)


def _t2i():
    return {"conversations": [{"from": "human", "value": "a red fox"},
                              {"from": "gpt", "value": "<think>plan</think><image>"}], "image": "fox.png"}


def _it2i():
    return {"conversations": [{"from": "human", "value": "<image>\nmake it night"},
                              {"from": "gpt", "value": "<image>"}], "images": ["a.png", "b.png"]}


def test_t2i_text_drop_removes_prompt_and_thinking():
    rec, info = prepare_generation_record(_t2i(), "mm_t2i", CfgDrop(txt=1.0), random.Random(0))
    assert rec["conversations"][0]["value"] == "" and rec["conversations"][-1]["value"] == "<image>"
    assert info["dropped_text"] and info["gen_flags"] == [1]
    rec, info = prepare_generation_record(_t2i(), "mm_t2i", CfgDrop(txt=0.0), random.Random(0))
    assert rec["conversations"][0]["from"] == "system" and not info["dropped_text"]
    assert rec["conversations"][0]["value"] == prompts.SYSTEM_MESSAGE_FOR_GEN


def test_editing_drops():
    rec, info = prepare_generation_record(_it2i(), "mm_it2i", CfgDrop(txt=1.0, img=0.0), random.Random(0))
    assert rec["conversations"][0]["value"] == "<image>" and info["dropped_text"] and info["gen_flags"] == [0, 1]
    rec, info = prepare_generation_record(_it2i(), "mm_it2i", CfgDrop(txt=0.0, img=1.0), random.Random(0))
    assert rec["images"] == ["b.png"] and "<image>" not in rec["conversations"][0]["value"]
    assert info["gen_flags"] == [1] and not info["dropped_text"]
    # joint policy: exactly one case is drawn
    rec, info = prepare_generation_record(_it2i(), "mm_it2i", CfgDrop(txtimg=1.0, independent=False), random.Random(0))
    assert rec["images"] == ["b.png"] and rec["conversations"][0]["value"] == "" and info["dropped_text"]
    rec, info = prepare_generation_record(_it2i(), "mm_it2i", CfgDrop(), random.Random(0))
    assert rec["conversations"][0]["from"] == "system" and len(rec["images"]) == 2


def test_sample_segments_and_losses():
    rec, info = prepare_generation_record(_it2i(), "mm_it2i", CfgDrop(), random.Random(0))
    s = record_to_sample(rec, "mm_it2i", tok, img, info)
    kinds = [g.kind for g in s.segments]
    assert kinds.count("und_image") == 1 and kinds.count("gen_image") == 1 and s.task == 4
    gen = [g for g in s.segments if g.kind == "gen_image"][0]
    assert gen.loss and float(gen.pixels[0, 0, 0]) == 1.0
    und = [g for g in s.segments if g.kind == "und_image"][0]
    assert not und.loss and float(und.pixels[0, 0, 0]) == -1.0
    # with the text dropped no text token is a target
    rec, info = prepare_generation_record(_it2i(), "mm_it2i", CfgDrop(txt=1.0), random.Random(0))
    s = record_to_sample(rec, "mm_it2i", tok, img, info)
    assert not any(g.loss for g in s.segments)


def test_interleave_duplicates_all_but_last_generated_image():
    rec = {"conversations": [{"from": "human", "value": "story"},
                             {"from": "gpt", "value": "one <image> two <image>"}], "images": ["1.png", "2.png"]}
    rec, info = prepare_generation_record(rec, "mm_interleave_gen", CfgDrop(), random.Random(0))
    assert info["gen_flags"] == [1, 1] and info["dup_for_und"] == [1, 0]
    s = record_to_sample(rec, "mm_interleave_gen", tok, img, info)
    g = [x for x in s.segments if x.kind == "gen_image"]
    assert g[0].duplicate_for_und and not g[1].duplicate_for_und


def test_dataset_mixing_sharding_and_resume(tmp_path):
    a, b = tmp_path / "a.jsonl", tmp_path / "b.jsonl"
    a.write_text("\n".join(json.dumps({"conversations": [{"from": "human", "value": f"q{i}"},
                                                          {"from": "gpt", "value": f"a{i}"}]}) for i in range(10)))
    b.write_text("\n".join(json.dumps(_t2i()) for _ in range(4)) + "\n{broken json\n")
    meta = {"text": {"annotation": str(a), "repeat_time": 3.0},
            "t2i": {"annotation": str(b), "data_type": "mm_t2i", "repeat_time": 1.0}}
    seen = []
    for rank in range(2):
        ds = ConversationDataset(meta, tok, img, rank=rank, world=2, seed=1, repeat=False)
        samples = list(ds)
        seen.append(len(samples))
        assert ds.skipped <= 1
    assert sum(seen) == 14                      # every valid record exactly once across the two ranks
    ds = ConversationDataset(meta, tok, img, seed=2)
    it = iter(ds)
    first = [next(it) for _ in range(5)]
    sd = json.loads(json.dumps(ds.state_dict()))   # must survive serialisation
    nxt = [next(it) for _ in range(3)]
    ds2 = ConversationDataset(meta, tok, img, seed=2)
    ds2.load_state_dict(sd)
    it2 = iter(ds2)
    again = [next(it2) for _ in range(3)]
    for x, y in zip(nxt, again):
        assert [g.kind for g in x.segments] == [g.kind for g in y.segments]
        assert all(torch.equal(p.ids, q.ids) for p, q in zip(x.segments, y.segments) if p.ids is not None)


# ---------------------------------------------------------------------------
# the data section of a config as one validated object
# ---------------------------------------------------------------------------
def test_data_options_defaults_budgets_and_schedules():
    from sensenova_u1_b200.data.options import DataOptions
    o = DataOptions.from_config(dict(seq_len=28672, micro_num=8, min_pixels=65536, max_pixels=4194304,
                                     max_pixels_gen=1048576, rampup_batch_size="2 2 10", loss_reduction="square",
                                     use_packed_ds="true", cfg_txt_uncond_drop_prob=0.1))
    assert o.token_pixels == 32 and o.packed_tokens == 28672 and o.extra == {"cfg_txt_uncond_drop_prob": 0.1}
    # one image: the configured bounds; generation images have their own upper bound
    assert o.pixel_budget(False) == (65536, 4194304) and o.pixel_budget(True) == (65536, 1048576)
    # eight images share the sequence: (28672 - 3072) tokens / 8 = 3200 tokens = 3,276,800 pixels each
    assert o.pixel_budget(False, 8) == (65536, 3276800) and o.pixel_budget(True, 8) == (65536, 1048576)
    assert o.pixel_budget(False, 1000)[1] == 65536                 # never below the minimum
    # ramp-up: 2, 2 more every 10 steps, capped by micro_num
    assert [o.batch_size_at(s) for s in (0, 9, 10, 25, 30, 500)] == [2, 2, 4, 6, 8, 8]
    assert DataOptions.from_config({}).batch_size_at(123, 4) == 4
    assert abs(o.loss_weight(16) - 0.25) < 1e-12 and o.loss_weight(0) == 0.0
    assert DataOptions.from_config(dict(loss_reduction="sample")).loss_weight(4) == 0.25


def test_data_options_mixing_weights_and_refusals():
    from sensenova_u1_b200.data.options import DataOptions
    o = DataOptions.from_config(dict(llm_data_weights=0.2, mm_cc_data_weights=0.25))
    w = o.mixing_weights(["paired", "paired", "cc"], [100, 300, 50])
    # multimodal share 0.8: caption pairs 0.25 * 0.8 = 0.2, the rest 0.6 split 1:3 by length
    assert [round(x, 6) for x in w] == [0.15, 0.45, 0.2]
    # a kind without datasets hands its share to the others
    w = o.mixing_weights(["paired", "paired"], [1, 1])
    assert abs(sum(w) - 0.8) < 1e-9 and abs(w[0] - w[1]) < 1e-12
    for bad in (dict(use_packed_ds=False), dict(group_by_length=True), dict(dynamic_image_version="v2"),
                dict(strict_mode=True), dict(loss_reduction="mean"), dict(rampup_batch_size="4 2"),
                dict(mm_cc_data_weights=0.7, mm_plain_pair_data_weights=0.6), dict(min_pixels=10, max_pixels=5)):
        with pytest.raises(ValueError):
            DataOptions.from_config(bad)
    # keys of the fixed-tile pipeline and keys nobody reads are accepted
    DataOptions.from_config(dict(force_image_size=448, use_thumbnail=True, pad2square=False, max_dynamic_patch=12,
                                 use_bos=True, use_eos=True, split_data_chunk=None, conv_style="sensenovalm-v3"))


def test_dataset_min_length_weights_and_epochs(tmp_path):
    import json
    from sensenova_u1_b200.data.multimodal import ConversationDataset
    rows_a = [{"conversations": [{"from": "human", "value": "q " * n}, {"from": "gpt", "value": "a"}]} for n in (1, 40, 60)]
    rows_b = [{"conversations": [{"from": "human", "value": "hello there " * 20}, {"from": "gpt", "value": "b"}]}]
    for name, rows in (("a", rows_a), ("b", rows_b)):
        (tmp_path / f"{name}.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    meta = {n: {"annotation": str(tmp_path / f"{n}.jsonl"), "root": str(tmp_path), "data_type": "vqa"} for n in "ab"}
    tok = lambda s: list(s.encode())
    ds = ConversationDataset(meta, tok, lambda *a: None, min_length=100, max_epochs=1, weights=[1.0, 0.0])
    got = list(ds)
    # one pass over file "a" (file "b" has weight 0 and is never drawn); its shortest record is below min_length
    assert len(got) == 2 and ds.short == 1
    with pytest.raises(ValueError):
        ConversationDataset(meta, tok, lambda *a: None, weights=[1.0])


def test_batch_skipper_and_its_config_key():
    from sensenova_u1_b200.data.options import BatchSkipper, DataOptions
    sk = BatchSkipper("3,10-12")
    assert [b for b in range(15) if sk(b)] == [3, 10, 11, 12] and not BatchSkipper("")(0)
    with pytest.raises(ValueError):
        BatchSkipper("5,2")
    assert DataOptions.from_config({"skip_batches": "1-2"}).skip_batches == "1-2"
    with pytest.raises(ValueError):
        DataOptions.from_config({"skip_batches": "4-1"})


def test_video_and_caption_pair_records_go_through_the_dataset(tmp_path):
    import json
    import numpy as np
    from PIL import Image
    from sensenova_u1_b200.data.multimodal import ConversationDataset, default_image_loader, plain_pair_to_sample
    frames = (np.random.default_rng(0).random((10, 96, 128, 3)) * 255).astype("uint8")
    np.save(tmp_path / "clip.npy", frames)
    Image.new("RGB", (96, 64), (10, 120, 30)).save(tmp_path / "a.png")
    (tmp_path / "video.jsonl").write_text(json.dumps({"video": "clip.npy", "conversations": [
        {"from": "human", "value": "<video>\nWhat happens?"}, {"from": "gpt", "value": "It moves."}]}) + "\n")
    (tmp_path / "cc.jsonl").write_text(json.dumps({"image": "a.png", "caption": "a green field"}) + "\n" + json.dumps(
        {"image": "a.png", "conversations": [{"from": "human", "value": "<image>\n"}, {"from": "gpt", "value": "grass"}]}) + "\n")
    meta = {"vid": {"annotation": str(tmp_path / "video.jsonl"), "root": str(tmp_path), "repeat_time": 1},
            "cc": {"annotation": str(tmp_path / "cc.jsonl"), "root": str(tmp_path), "dataset_type": "cc", "repeat_time": 1}}
    tok = lambda s: list(s.encode())
    ds = ConversationDataset(meta, tok, default_image_loader(min_pixels=1024), repeat=False, min_num_frame=4, max_num_frame=4,
                             frame_max_pixels=64 * 64)
    samples = list(ds)
    assert ds.skipped == 0 and len(samples) == 3
    vid = next(s for s in samples if sum(g.kind == "und_image" for g in s.segments) == 4)
    px = next(g.pixels for g in vid.segments if g.kind == "und_image")
    assert px.shape[1] % 32 == 0 and px.shape[2] % 32 == 0 and px.shape[1] * px.shape[2] <= 64 * 64
    caps = [s for s in samples if s is not vid]
    for s in caps:                                      # plain style: picture, then the caption with loss, no chat markup
        assert [g.kind for g in s.segments] == ["und_image", "text"] and s.segments[1].loss
        assert not bytes(s.segments[1].ids.tolist()).startswith(b"<|im_start|>")
    texts = sorted(bytes(s.segments[1].ids.tolist()).decode() for s in caps)
    assert texts[0].startswith("a green field") and texts[1].startswith("grass")
    with pytest.raises(ValueError):
        plain_pair_to_sample({"caption": "x"}, tok, default_image_loader())


def test_chat_options_follow_the_reference_text_preparation():
    import random
    import torch
    from sensenova_u1_b200.data.multimodal import ChatOptions, apply_chat_options, record_to_sample
    from sensenova_u1_b200.inference import prompts
    tok = lambda s: list(s.encode())
    text = lambda smp: b"".join(bytes(g.ids.tolist()) for g in smp.segments if g.kind == "text").decode()
    loss_text = lambda smp: b"".join(bytes(g.ids.tolist()) for g in smp.segments if g.kind == "text" and g.loss).decode()
    rec = {"conversations": [{"from": "system", "value": "Be brief.\n" + prompts.REASON_PROMPT},
                             {"from": "human", "value": "2+2?"}, {"from": "gpt", "value": "<think>\nadd\n</think>\n\n4"},
                             {"from": "human", "value": "and 3+3?"}, {"from": "gpt", "value": "6"},
                             {"from": "tool", "value": "ignored"}]}
    tag = record_to_sample(rec, "", tok, None, chat=ChatOptions("tag"), rng=random.Random(0))
    t = text(tag)
    assert prompts.REASON_PROMPT not in t and "<|im_start|>system\nBe brief.<|im_end|>" in t and "ignored" not in t
    assert "<|im_start|>assistant\n<think>\nadd\n</think>\n\n4<|im_end|>" in t                # own reasoning: no empty block
    assert "<|im_start|>assistant\n<think>\n\n</think>\n\n6<|im_end|>" in t                    # empty block before a plain answer
    assert loss_text(tag) == "<think>\nadd\n</think>\n\n4<|im_end|>\n6<|im_end|>\n"            # the empty block carries no loss
    # "sys": a sample with reasoning gets the sentence in its system message; one without is left alone
    conv, thinking = apply_chat_options([{"from": "human", "value": "q"}, {"from": "gpt", "value": "<think>\nx\n</think>\n\na"}],
                                        ChatOptions("sys"), random.Random(1))
    assert thinking and conv[0] == {"from": "system", "value": prompts.REASON_PROMPT}
    plain = record_to_sample({"conversations": [{"from": "human", "value": "q"}, {"from": "gpt", "value": "a"}]}, "", tok, None,
                             chat=ChatOptions("sys"), rng=random.Random(1))
    assert text(plain) == "<|im_start|>user\nq<|im_end|>\n<|im_start|>assistant\na<|im_end|>\n"
    # a dropped text condition gets no empty block; rm_all_think_token strips reasoning; identity sentence by ratio
    dropped = record_to_sample({"conversations": [{"from": "human", "value": ""}, {"from": "gpt", "value": "x"}]}, "", tok, None,
                               info={"dropped_text": True}, chat=ChatOptions("tag"), rng=random.Random(0))
    assert "<think>" not in text(dropped)
    conv, _ = apply_chat_options(rec["conversations"], ChatOptions("tag", rm_all_think_token=True), random.Random(0))
    assert conv[2]["value"] == "add\n\n4" and conv[0]["value"] == "Be brief."
    conv, _ = apply_chat_options([{"from": "human", "value": "q"}], ChatOptions("tag", st_prompt_ratio=1.0), random.Random(0))
    assert conv[0] == {"from": "system", "value": prompts.DEFAULT_IDENTITY_PROMPT}
    moved = [apply_chat_options([{"from": "human", "value": "<image>\nlook"}], ChatOptions(image_token_position_random="end"),
                                random.Random(s))[0][0]["value"] for s in range(8)]
    assert set(moved) == {"<image>\nlook", "look\n<image>"}
    # an assistant turn marked as input is context
    ctx = record_to_sample({"conversations": [{"from": "human", "value": "q"}, {"from": "gpt", "value": "given", "is_input": True},
                                              {"from": "gpt", "value": "new"}]}, "", tok, None, chat=ChatOptions("sys"), rng=random.Random(0))
    assert loss_text(ctx) == "new<|im_end|>\n"
