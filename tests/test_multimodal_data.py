"""Annotation records -> samples: condition dropping, task flags, mixing, sharding, resume."""
import json
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
