"""The four interleaved / visual-reasoning benchmarks: per-benchmark inference protocols and judging.

Every protocol talks to an ``Engine`` (four calls: draw from text, edit pictures, answer about pictures, interleaved
text + pictures), so the same code runs the in-process model, a served model or a test double.

* RealUnify "GEU"  one picture + ``edit_prompt`` + ``evaluation_prompt`` + answer letter.  ``step``: edit the picture,
                   then answer the question about the edited picture; ``interleave``: answer directly, drawing while
                   thinking; the text after ``</think>`` is scored (Realunify/inference_realunify.py:501-720)
* RealUnify "UEG"  a JSON list (``index``, ``new_prompt``, ``question_list``).  ``understand_t2i``: the model rewrites the
                   prompt as text, then draws it; ``interleave``; ``t2i``: draws the part of ``new_prompt`` after the
                   "Here is the prompt for image generation:" marker.  A judge answers the yes/no questions about the
                   last picture; a sample scores 1 only if all agree with the key
                   (Realunify/inference_realunify_ueg.py:122-372, calculate_score_ueg.py:73-180)
* UniMMMU          ``messages`` in chat form with 1-3 pictures; ``i2t`` (answer only) or ``interleave``; task fields are
                   carried over for the benchmark's own scorer (Unimmmu/inference_unimmmu.py:467-756)
* BabyVision       ``meta_data.jsonl`` (``taskId``, ``image``, ``question``, ``ansType`` blank / choice, ``options``,
                   ``choiceAns`` / ``blankAns``, ``type``, ``subtype``); answer inside ``<answer></answer>``; judged by
                   rule extraction, then a judge compares with the key (BabyVision/infer_babyvision.py:281-341, 546-600,
                   eval_babyvision.py:20-318)
* OpenING          ``test_data.jsonl`` with ``conversations[0].input`` / ``[1].output`` lists of {text, image}; the model
                   must produce as many (text, picture) steps as the key; results are written per ``total_uid`` in the
                   benchmark's own layout; a judge rates seven criteria 0-10
                   (OpenING/infer_opening.py:185-420, 709-880, eval_opening.py:37-400)
"""
from __future__ import annotations

import copy
import json
import os
import re
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

from evaluation.benchmarks import rules
from evaluation.common.judge import parse_json_block

OPENING_CRITERIA = ("Correctness", "Image-Text Coherency", "Multi-step Consistency", "Content Quality",
                    "Human Preference Alignment", "Completeness", "Content Richness")
UEG_TASKS = ("world_knowledge", "commonsense_reasoning", "logical_reasoning", "mathematical_reasoning",
             "scientific_reasoning", "code_to_image")


# ---------------------------------------------------------------------------------------------------------------
# engine
# ---------------------------------------------------------------------------------------------------------------
class LocalEngine:
    """The in-process model behind the four calls.  ``s`` holds the sampling flags of the command line."""

    def __init__(self, model, tok, **s):
        self.model, self.tok, self.s = model, tok, s

    def _kw(self, *names):
        return {k: self.s[k] for k in names if k in self.s}

    def _und(self, images, min_pixels=None, max_pixels=None):
        from sensenova_u1_b200.inference.images import load_image_native
        kw = {k: v for k, v in (("min_pixels", min_pixels), ("max_pixels", max_pixels)) if v}
        return [load_image_native(im, factor=self.model.cfg.token_pixels, normalize="imagenet", **kw) for im in images]

    def t2i(self, prompt: str, size):
        from sensenova_u1_b200.inference.images import to_pil
        img = self.model.t2i_generate(self.tok, prompt, image_size=tuple(size), batch_size=1,
                                      **self._kw("cfg_scale", "cfg_norm", "cfg_interval", "num_steps", "timestep_shift", "seed"))
        return to_pil(img[0])

    def edit(self, prompt: str, images, size):
        from sensenova_u1_b200.inference.images import to_pil
        img = self.model.it2i_generate(self.tok, prompt, self._und(images), image_size=tuple(size), **self._kw(
            "cfg_scale", "img_cfg_scale", "cfg_norm", "cfg_interval", "num_steps", "timestep_shift", "seed"))
        return to_pil(img[0])

    def ask(self, question: str, images=(), max_new_tokens: int = 512, min_pixels=None, max_pixels=None, **gen) -> str:
        pv = self._und(images, min_pixels, max_pixels) if images else None
        return self.model.chat(self.tok, pv, question, generation_config={"max_new_tokens": max_new_tokens, **gen})

    def interleave(self, prompt: str, images, size, system: Optional[str] = None, think: bool = True,
                   max_new_tokens: int = 4096, max_images: Optional[int] = None):
        from sensenova_u1_b200.inference.images import to_pil
        text, pics = self.model.interleave_gen(self.tok, prompt, self._und(images), image_size=tuple(size),
                                               system_message=system, think_mode=think, max_new_tokens=max_new_tokens,
                                               max_images=max_images, **self._kw(
                                                   "cfg_scale", "img_cfg_scale", "cfg_norm", "cfg_interval", "num_steps",
                                                   "timestep_shift", "seed"))
        return text, [to_pil(p) for p in pics]


def interleave_system() -> str:
    """System message of interleaved answers (think mode / non-think mode rules) the released checkpoints know."""
    from sensenova_u1_b200.inference.prompts import SYSTEM_MESSAGE_FOR_INTERLEAVE
    return SYSTEM_MESSAGE_FOR_INTERLEAVE


def final_answer(text: str) -> str:
    """What follows the last ``</think>``; the whole text when there is no think block."""
    return text.split("</think>")[-1].strip() if "</think>" in text else text.strip()


def target_size(img, target: Optional[int], min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    """(W, H) of the pictures drawn for an input picture: a forced square, or the input's own size inside the pixel
    budget, sides multiples of 32."""
    if target:
        return target, target
    from sensenova_u1_b200.inference.images import smart_resize
    h, w = smart_resize(img.height, img.width, 32, min_pixels, max_pixels)
    return w, h


def _open(path):
    from PIL import Image
    return Image.open(path).convert("RGB")


def _save_all(pics, folder: Path, stem: str) -> List[str]:
    folder.mkdir(parents=True, exist_ok=True)
    out = []
    for k, im in enumerate(pics):
        p = folder / f"{stem}_gen_{k}.png"
        im.save(p)
        out.append(str(p.resolve()))
    return out


class Suite:
    name = ""
    id_field = "hash_uid"
    result_file = "results.jsonl"
    modes: Tuple[str, ...] = ()

    def add_args(self, ap) -> None:
        pass

    def load(self, a) -> List[dict]:
        raise NotImplementedError

    def run_one(self, eng, item: dict, a, out_dir: Path) -> Optional[dict]:
        raise NotImplementedError

    # judging: records of ``run_one`` -> records the scorer reads
    needs_judge = False

    def judge(self, client, rec: dict, a) -> dict:
        return rec

    def summarize(self, records: Sequence[dict], a) -> dict:
        return rules.SCORERS[self.name](records)


# ---------------------------------------------------------------------------------------------------------------
class RealUnify(Suite):
    name = "realunify"
    result_file = "realunify_results.jsonl"
    modes = ("step", "interleave")

    def add_args(self, ap):
        ap.add_argument("--data_path", default="evaluation/data/realunify/GEU_step.jsonl")
        ap.add_argument("--image_root", default=None, help="prefix of relative picture paths (default: the data file's folder)")

    def load(self, a):
        from evaluation.gen.suites import read_jsonl
        return read_jsonl(a.data_path)

    def run_one(self, eng, it, a, out_dir):
        uid, task = str(it.get("hash_uid", "unknown")), it.get("task_type", "unknown")
        src = _resolve(a, it.get("input_image", ""))
        if not os.path.exists(src):
            raise FileNotFoundError(f"input picture {src}")
        img = _open(src)
        size = target_size(img, a.target_image_size, a.min_pixels, a.max_pixels)
        img = img.resize(size)
        folder = out_dir / "images" / task
        base = {"task_type": task, "answer": it.get("answer", ""), "hash_uid": uid, "index": it.get("index", -1),
                "question": it.get("question", ""), "option": it.get("option", []), "edit_prompt": it.get("edit_prompt", ""),
                "evaluation_prompt": it.get("evaluation_prompt", ""), "inference_mode": a.inference_mode}
        if a.inference_mode == "step":
            edited = eng.edit(it.get("edit_prompt", ""), [img], size)
            folder.mkdir(parents=True, exist_ok=True)
            ep = folder / f"{uid}_edited.png"
            edited.save(ep)
            resp = eng.ask("<image>\n" + it.get("evaluation_prompt", ""), [edited], max_new_tokens=512)
            return {**base, "image": [os.path.abspath(src), str(ep.resolve())], "model_response": resp,
                    "generated_image": [os.path.abspath(src), str(ep.resolve())],
                    "conversations": [{"from": "human", "value": "<image>\n" + it.get("edit_prompt", "")},
                                      {"from": "gpt", "value": "<image>\n"},
                                      {"from": "human", "value": "<image>\n" + it.get("evaluation_prompt", "")},
                                      {"from": "gpt", "value": resp}]}
        system = interleave_system()
        text, pics = eng.interleave(it.get("evaluation_prompt", ""), [img], size, system=system, think=True)
        paths = _save_all(pics, folder, uid)
        return {**base, "image": [os.path.abspath(src)] + paths, "model_response": final_answer(text),
                "generated_images": paths, "full_generated_text": text,
                "conversations": [{"from": "system", "value": system},
                                  {"from": "human", "value": "<image>\n" + it.get("evaluation_prompt", "")},
                                  {"from": "gpt", "value": text}]}


def ueg_raw_prompt(new_prompt: str) -> str:
    """The drawing prompt inside a UEG ``new_prompt``: after the marker sentence, up to the first blank line."""
    marker = "Here is the prompt for image generation:"
    t = new_prompt[new_prompt.find(marker) + len(marker):] if marker in new_prompt else new_prompt
    return t.split("\n\n", 1)[0].strip()


class RealUnifyUEG(Suite):
    name = "realunify_ueg"
    result_file = "ueg_results.jsonl"
    modes = ("understand_t2i", "interleave", "t2i")
    needs_judge = True
    ASK = ("Please answer the following question based on the image:\nQuestion: {q}\n\n"
           "You should only reply yes or no, and do not provide any other extra content.")

    def add_args(self, ap):
        ap.add_argument("--data_path", default="evaluation/data/realunify/UEG_step.json")

    def load(self, a):
        data = json.loads(Path(a.data_path).read_text(encoding="utf-8"))
        return [dict(d, hash_uid=str(d["index"])) for d in data]

    def run_one(self, eng, it, a, out_dir):
        uid, task = it["hash_uid"], it.get("task_type", "unknown")
        side = a.target_image_size or 1024
        folder = out_dir / "images" / task
        folder.mkdir(parents=True, exist_ok=True)
        base = {"index": it.get("index", -1), "task_type": task, "question_list": it.get("question_list", []),
                "hash_uid": uid, "inference_mode": a.inference_mode, "new_prompt": it.get("new_prompt", "")}
        if a.inference_mode == "interleave":
            raw = ueg_raw_prompt(it["new_prompt"])
            text, pics = eng.interleave(raw, [], (side, side), system=interleave_system(), think=True)
            paths = _save_all(pics, folder, uid)
            return {**base, "image": paths, "generated_images": paths, "generated_image": paths[-1] if paths else "",
                    "model_response": final_answer(text), "mid_output": text, "full_generated_text": text}
        if a.inference_mode == "understand_t2i":
            prompt = eng.ask(it["new_prompt"], (), max_new_tokens=512)       # the model rewrites the prompt first
            mid = prompt + "\n\n<image>"
        else:
            prompt, mid = ueg_raw_prompt(it["new_prompt"]), "<image>"
        p = folder / f"{uid}_gen.png"
        eng.t2i(prompt, (side, side)).save(p)
        return {**base, "image": [str(p.resolve())], "generated_images": [str(p.resolve())], "generated_image": str(p.resolve()),
                "model_response": prompt if a.inference_mode == "understand_t2i" else "<image>", "mid_output": mid}

    def judge(self, client, rec, a):
        img = rec.get("generated_image")
        if isinstance(img, list):
            img = img[-1] if img else None
        if not img or not os.path.exists(img):
            return {**rec, "score": 0, "judge_outputs": [{"error": "no picture"}]}
        outs, score = [], 1
        for qa in rec.get("question_list", []):
            raw = client.ask(self.ASK.format(q=qa["question"]), [img], None, temperature=0.2, max_tokens=16)
            low = raw.lower()
            got = "no" if "no" in low else ("yes" if "yes" in low else "")
            outs.append({"question": qa["question"], "gt_answer": qa["answer"], "judge_raw_response": raw,
                         "judge_parsed_answer": got, "correct": got == qa["answer"]})
            if got != qa["answer"]:
                score = 0
                break                                              # all-or-nothing: the first miss decides
        return {**rec, "score": score, "judge_outputs": outs}

    def summarize(self, records, a):
        per = {t: [0, 0] for t in UEG_TASKS}
        for r in records:
            if r.get("task_type") in per:
                per[r["task_type"]][1] += 1
                per[r["task_type"]][0] += int(r.get("score") == 1)
        c, n = sum(v[0] for v in per.values()), sum(v[1] for v in per.values())
        return {"per_task": {t: {"correct": v[0], "total": v[1], "accuracy": v[0] / v[1] if v[1] else 0.0} for t, v in per.items()},
                "total": {"correct": c, "total": n, "accuracy": c / n if n else 0.0}}


# ---------------------------------------------------------------------------------------------------------------
def chat_prompt_and_images(item: dict) -> Tuple[str, List[str]]:
    """First text part and all picture URLs of the user turns of a chat-form ``messages`` field."""
    texts, pics = [], []
    for m in item.get("messages", []):
        if m.get("role") != "user":
            continue
        c = m.get("content", [])
        if isinstance(c, str):
            texts.append(c)
            continue
        for part in c:
            if isinstance(part, dict) and part.get("type") == "text" and part.get("text"):
                texts.append(part["text"])
            elif isinstance(part, dict) and part.get("type") == "image_url" and part.get("image_url", {}).get("url"):
                pics.append(part["image_url"]["url"])
    return (texts[0] if texts else ""), pics


class UniMMMU(Suite):
    name = "unimmmu"
    result_file = "unimmmu_results.jsonl"
    modes = ("i2t", "interleave")

    def add_args(self, ap):
        ap.add_argument("--data_path", default="evaluation/data/unimmmu/unimmmu_direct.jsonl")
        ap.add_argument("--image_root", default=None)

    def load(self, a):
        from evaluation.gen.suites import read_jsonl
        return read_jsonl(a.data_path)

    def run_one(self, eng, it, a, out_dir):
        uid, task = str(it.get("hash_uid", "unknown")), it.get("task", "unknown")
        prompt, pics = chat_prompt_and_images(it)
        paths = [p for p in (_resolve(a, u) for u in pics) if os.path.exists(p)]
        if not paths:
            raise FileNotFoundError(f"sample {uid}: none of its {len(pics)} pictures exists")
        rec = {"task": task, "id": it.get("id", ""), "hash_uid": uid, "gt_text": it.get("gt_text", ""),
               "reasoning_imgs": it.get("reasoning_imgs", []), "inference_mode": a.inference_mode}
        if task == "geometry":                                   # the benchmark's geometry scorer reads these
            rec.update({k: it.get(k, [] if k == "gt_auxiliary_imgs" else "")
                        for k in ("task_type", "reasoning_qs", "auxiliary_qs", "gt_auxiliary_imgs")})
        q = "<image>\n" * len(paths) + prompt
        if a.inference_mode == "i2t":
            rec["model_response"] = eng.ask(q, [_open(p) for p in paths], max_new_tokens=512, min_pixels=a.min_pixels,
                                            max_pixels=a.max_pixels)
            return rec
        imgs = []
        for p in paths:
            im = _open(p)
            imgs.append(im.resize(target_size(im, a.target_image_size, a.min_pixels, a.max_pixels)))
        text, out = eng.interleave(prompt, imgs, imgs[0].size, system=interleave_system(), think=True)
        rec.update(model_response=final_answer(text), full_generated_text=text,
                   generated_images=_save_all(out, out_dir / "images" / task, uid))
        return rec

    def summarize(self, records, a):
        rows = [dict(r, response=r.get("model_response", ""), answer=r.get("gt_text", "")) for r in records]
        return rules.unimmmu_summary(rows)


# ---------------------------------------------------------------------------------------------------------------
_ANSWER_RULES = [re.compile(r"<answer>\s*(.*?)\s*</answer>", re.I | re.S), re.compile(r"\\boxed\{([^}]*)\}", re.S),
                 re.compile(r"(?:final answer|correct answer)\s*[:：]\s*(.+)", re.I),
                 re.compile(r"(?:so|thus|therefore)\s+the answer is\s*[:：]?\s*(.+)", re.I),
                 re.compile(r"(?:the answer|answer|correct answer)\s+is\s*[:：]?\s*(.+)", re.I)]


def _clean_answer(v) -> Optional[str]:
    if v is None:
        return None
    v = re.sub(r"</?answer>", "", str(v), flags=re.I).strip()
    v = re.sub(r"^(?:final answer|answer)\s*[:：]\s*", "", v, flags=re.I).strip().strip("\"'").strip()
    return re.sub(r"\s+", " ", v).strip() or None


def rule_answer(response: str) -> Optional[str]:
    """The last explicit conclusion of a response, by pattern; None when no pattern fits."""
    for pat in _ANSWER_RULES:
        found = pat.findall(response or "")
        if found:
            c = _clean_answer(found[-1])
            if c and c.lower() not in ("given", "none", "null", "unknown"):
                return c
    return None


def tagged_answer(text: Optional[str]) -> Optional[str]:
    """``<answer>...</answer>`` if present, else the last line after ``</think>``, else the last line."""
    if text is None:
        return None
    m = re.findall(r"<answer>\s*(.*?)\s*</answer>", text, flags=re.S | re.I)
    if m:
        return m[-1].strip()
    tail = re.split(r"</think>", text, flags=re.I)[-1]
    lines = [l.strip() for l in (tail if tail.strip() else text).splitlines() if l.strip()]
    if not lines:
        return None
    return re.sub(r"\s*```$", "", re.sub(r"^```[\w-]*\s*", "", lines[-1])).strip() or None


class BabyVision(Suite):
    name = "babyvision"
    id_field = "taskId"
    result_file = "babyvision_results.jsonl"
    modes = ("vqa",)
    needs_judge = True
    GEN = {"max_new_tokens": 32768, "do_sample": False, "temperature": 0, "top_p": 0.95, "repetition_penalty": 1.05}
    PIXELS = (262144, 16777216)
    JUDGE = ("You judge answers. Decide whether the extracted answer means the same as the ground truth; match the "
             "format of the ground truth as closely as possible; an empty answer is wrong.\n\nQuestion: {q}\n\n"
             "Extracted Answer: {a}\n\nGround Truth: {gt}\n\nReply with JSON only: {{\"is_correct\": true}} or "
             "{{\"is_correct\": false}}")
    EXTRACT = ("You extract and judge answers. From the model response take the final answer (the last explicit "
               "conclusion; null if there is none), then decide whether it means the same as the ground truth.\n\n"
               "Question: {q}\n\nModel Response: {r}\n\nGround Truth: {gt}\n\nReply with JSON only: "
               "{{\"extracted_answer\": \"<string-or-null>\", \"is_correct\": true}} (or false)")

    def add_args(self, ap):
        ap.add_argument("--data_path", default="evaluation/data/babyvision/meta_data.jsonl")
        ap.add_argument("--image_root", default=None)
        ap.add_argument("--extractor", default="rule_then_llm", choices=["rule_then_llm", "llm", "rule_only"])

    def load(self, a):
        from evaluation.gen.suites import read_jsonl
        return read_jsonl(a.data_path)

    @staticmethod
    def question_and_key(it: dict) -> Tuple[str, str]:
        if it["ansType"] == "blank":
            q, key = it["question"], str(it["blankAns"])
        else:
            q = it["question"] + "\nChoices:\n" + "\n".join(f"({chr(65 + i)}) {c}" for i, c in enumerate(it["options"]))
            c = str(it["choiceAns"]).strip()
            key = (chr(64 + int(c)) if 1 <= int(c) <= 26 else chr(65 + int(c))) if c.isdigit() else c
        return q + "\nPut your final answer inside <answer></answer>.", key

    def run_one(self, eng, it, a, out_dir):
        src = _resolve(a, it["image"])
        if not os.path.exists(src):
            raise FileNotFoundError(src)
        q, key = self.question_and_key(it)
        resp = eng.ask(q, [_open(src)], min_pixels=self.PIXELS[0], max_pixels=self.PIXELS[1], **self.GEN)
        return {"taskId": it["taskId"], "type": it["type"], "subtype": it["subtype"], "ansType": it["ansType"],
                "question": q, "answer": key, "model_response": resp, "extracted_answer": tagged_answer(resp)}

    def judge(self, client, rec, a):
        q, gt, resp = rec.get("question", ""), rec.get("answer", ""), rec.get("model_response", "")
        extractor = getattr(a, "extractor", "rule_then_llm")
        found = rule_answer(resp) if extractor != "llm" else None
        if found is None and extractor == "rule_only":
            return {**rec, "extracted_answer": None, "LLMJudgeResult": False}
        if found is not None:
            p = parse_json_block(client.ask(self.JUDGE.format(q=q, a=found, gt=gt), (), None, max_tokens=64)) or {}
        else:
            p = parse_json_block(client.ask(self.EXTRACT.format(q=q, r=resp, gt=gt), (), None, max_tokens=256)) or {}
            found = _clean_answer(p.get("extracted_answer"))
        return {**rec, "extracted_answer": found, "LLMJudgeResult": bool(p.get("is_correct", False)),
                "Type": rec.get("type"), "Subtype": rec.get("subtype")}


# ---------------------------------------------------------------------------------------------------------------
_STEP_DELIMS = r"<IMG>|<image>|\[image\]|<image_?\d+>|</image_?\d+>|<IMG_?\d+>|</IMG_?\d+>"


def split_steps(text: str) -> List[str]:
    """Text between the pictures of an interleaved answer."""
    text = (text or "").replace("**", "").strip()
    parts = [p.strip() for p in re.split(_STEP_DELIMS, text, flags=re.I) if p.strip()]
    return parts or [text]


def align_steps(texts: List[str], names: List[str], n: int) -> Tuple[List[str], List[Optional[str]]]:
    k = min(n, max(len(texts), len(names), 1))
    return ([texts[i] if i < len(texts) else "" for i in range(k)], [names[i] if i < len(names) else None for i in range(k)])


class OpenING(Suite):
    name = "opening"
    id_field = "total_uid"
    result_file = "opening_results.jsonl"
    modes = ("think", "no_think")
    needs_judge = True
    SYSTEM = ("You rate an interleaved text-and-picture answer (OUTPUT) to a task (INPUT). Give an integer 0-10 for each "
              "criterion: " + ", ".join(OPENING_CRITERIA) + ". Answer with JSON only: {\"<criterion>\": {\"Score\": n, "
              "\"Justification\": \"...\"}, ...} with all seven criteria.")

    def add_args(self, ap):
        ap.add_argument("--meta_path", default="evaluation/data/opening")
        ap.add_argument("--data_file_name", default="test_data.jsonl")
        ap.add_argument("--max_new_tokens", type=int, default=4096)
        ap.add_argument("--max_generation_pixels", type=int, default=2048 * 2048)
        ap.add_argument("--image_width", type=int, default=None)
        ap.add_argument("--image_height", type=int, default=None)
        ap.add_argument("--retry_short_outputs", type=int, default=0, help="extra tries when fewer steps than the key come back")
        ap.add_argument("--opening_step_prompt_style", default="none", choices=["none", "can_be", "must_exact"])
        ap.add_argument("--uid_file", default=None)

    def load(self, a):
        from evaluation.gen.suites import read_jsonl
        keep = None
        if getattr(a, "uid_file", None):
            keep = {l.strip() for l in Path(a.uid_file).read_text().splitlines() if l.strip()}
        return [d for d in read_jsonl(Path(a.meta_path) / a.data_file_name) if keep is None or d["total_uid"] in keep]

    @staticmethod
    def io(it: dict):
        i, o = it["conversations"][0]["input"], it["conversations"][1]["output"]
        return [x["text"].strip() for x in i], [x.get("image") for x in i], [x["text"].strip() for x in o], [x.get("image") for x in o]

    @staticmethod
    def prompt(in_text: List[str], n: int, style: str = "none") -> str:
        parts = [t.replace("<BEGIN>", "").strip() for t in in_text]
        pre = {"can_be": f"The number of generated text-image pairs can be {n}: ",
               "must_exact": f"The number of generated text-image pairs must be exactly {n}. "
                             f"Please generate exactly {n} interleaved text-image pairs: "}.get(style, "")
        if pre:
            parts = [pre + parts[0]] + parts[1:] if parts else [pre]
        return "\n".join(parts)

    def _path(self, a, p):
        if not p or os.path.isabs(p):
            return p
        for cand in (Path(a.meta_path) / p, Path(a.meta_path) / "OpenING" / p):
            if cand.exists():
                return str(cand)
        return str(Path(a.meta_path) / p)

    def _size(self, a, inputs, out_paths) -> Tuple[int, int]:
        from sensenova_u1_b200.inference.images import smart_resize
        if a.image_width and a.image_height:
            return max(32, a.image_width // 32 * 32), max(32, a.image_height // 32 * 32)
        mx = max(32 * 32, a.max_generation_pixels)
        ref = inputs[0] if inputs else next((_open(p) for p in out_paths if p and os.path.exists(p)), None)
        w, h = ref.size if ref is not None else (1024, 1024)
        hh, ww = smart_resize(h, w, 32, min(512 * 512, mx), mx)
        return ww, hh

    def run_one(self, eng, it, a, out_dir):
        uid = it["total_uid"]
        in_text, in_img, out_text, out_img = self.io(it)
        n = len(out_text)
        if n == 0:
            raise ValueError(f"{uid}: the key has no output steps")
        inputs = [_open(self._path(a, p)) for p in in_img if p and os.path.exists(self._path(a, p))]
        size = self._size(a, inputs, [self._path(a, p) for p in out_img])
        prompt = self.prompt(in_text, n, a.opening_step_prompt_style)
        best = None
        for _ in range(max(1, a.retry_short_outputs + 1)):
            text, pics = eng.interleave(prompt, inputs, size, system=interleave_system(), think=a.inference_mode == "think",
                                        max_new_tokens=a.max_new_tokens, max_images=n)
            names = [f"{uid}-o-{k}.jpg" for k in range(min(len(pics), n))]
            texts, imgs = align_steps(split_steps(final_answer(text) or text), names, n)
            score = min(len(texts), n) + len(names)
            if best is None or score > best[0]:
                best = (score, texts, imgs, pics[:n])
            if len(texts) >= n and len(names) >= n:
                break
        _, texts, imgs, pics = best
        out_dir.mkdir(parents=True, exist_ok=True)
        for k, im in enumerate(pics):
            tmp = out_dir / f"{uid}-o-{k}.jpg.tmp"
            im.convert("RGB").save(tmp, format="JPEG")
            os.replace(tmp, out_dir / f"{uid}-o-{k}.jpg")
        saved = copy.deepcopy(it)                                   # the benchmark's own layout: one JSON per sample
        saved["conversations"][1]["output"] = [{"text": t.strip(), "image": i} for t, i in zip(texts, imgs)]
        tmp = out_dir / f"{uid}.json.tmp"
        tmp.write_text(json.dumps(saved, ensure_ascii=False, indent=4), encoding="utf-8")
        os.replace(tmp, out_dir / f"{uid}.json")
        return {"total_uid": uid, "steps_expected": n, "steps_text": len(texts), "steps_image": sum(i is not None for i in imgs),
                "output_json": f"{uid}.json"}

    def judge(self, client, rec, a):
        run = Path(a.run_dir)
        d = json.loads((run / rec["output_json"]).read_text(encoding="utf-8"))
        in_text, in_img, out_text, out_img = self.io(d)
        pics = [self._path(a, p) for p in in_img if p and os.path.exists(self._path(a, p))]
        pics += [str(run / p) for p in out_img if p and (run / p).exists()]
        q = "INPUT: " + "\n".join(t.replace("<BEGIN>", "") for t in in_text) + "\nOUTPUT: " + \
            ("\n".join(out_text) if any(out_text) else "None") + \
            f"\n(The first {sum(1 for p in in_img if p)} pictures belong to the INPUT, the rest to the OUTPUT.)" \
            "\nPlease only output the json result: "
        p = parse_json_block(client.ask(q, pics, self.SYSTEM, max_tokens=1024)) or {}
        score = {}
        for c in OPENING_CRITERIA:
            v = p.get(c)
            v = v.get("Score") if isinstance(v, dict) else v
            if not isinstance(v, (int, float)) or not 0 <= v <= 10:
                raise ValueError(f"{rec['total_uid']}: no valid score for {c!r}")
            score[c] = v
        return {**rec, "model": getattr(a, "model_tag", "model"), "score": score}


def _resolve(a, p: str) -> str:
    if not p or os.path.isabs(p) or p.startswith("data:"):
        return p
    root = getattr(a, "image_root", None) or str(Path(getattr(a, "data_path", ".")).resolve().parent)
    return os.path.join(root, p)


SUITES: Dict[str, Suite] = {s.name: s for s in (RealUnify(), RealUnifyUEG(), UniMMMU(), BabyVision(), OpenING())}
