"""The five image-generation benchmarks as data readers + judging protocols.

Each suite knows three things about its benchmark: how the prompt files are laid out and which picture (name, size)
belongs to which prompt; how one picture is judged; how the judged records turn into the benchmark's table (the
arithmetic is in ``evaluation/benchmarks/rules.py``).  ``evaluation/gen/run_benchmark.py`` drives them.

* BizGenEval   one JSONL; ``aspect_ratio`` per line, long side 2048 rounded to 32; a checklist judged in one call,
               answers as JSON ``{"1": {"result": ...}}`` (evaluation/gen/bizgeneval/gen_images_bizgeneval.py:41-111,
               eval_images_bizgeneval.py:211-300)
* IGenBench    a folder of ``<id>.json`` (``t2i_prompt``, ``evaluation[].question / question_type``); 2048 x 2048;
               one call per question, JSON ``{"answer": 0 | 1}`` (gen_images_igenbench.py:56-112,
               eval_images_igenbench.py:149-254)
* LongText     ``text_prompts.jsonl`` / ``text_prompts_zh.jsonl`` (``prompt``, ``text``, ``category``, ``length``); the
               text in the picture is read back and matched as a bag of words / characters
               (gen_images_longtext.py:54-128, eval_images_longtext.py:37-236)
* CVTG-2K      ``<root>/{CVTG,CVTG-Style}/<area>_combined.json`` = ``{key: prompt}``; pictures under
               ``<subset>/<area>/<key>.png``; target words are the quoted spans of the prompt (eval_cvtg.py:41-197).
               The reference reads the pictures with PaddleOCR and adds CLIP / aesthetic scores from local models
               (unified_metrics_eval.py); here a vision-language endpoint reads the text, the other two columns are
               filled when a record carries them.
* TIIF-Bench   a folder of JSONL files (``type``, ``short_description``, ``long_description``, ``yn_question_list``,
               ``yn_answer_list``); pictures under ``<type>/<model>/<short|long>_description/<index>.png``; the questions
               of one picture are asked in one call, one ``yes`` / ``no`` line each (tiif/eval_tiif.py:174-243,
               tiif/eval/eval_with_vlm_mp.py:86-190)
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple

from evaluation.benchmarks import rules
from evaluation.common.judge import parse_json_block

# width x height by aspect ratio, ~4 M pixels, sides multiples of 32
RESOLUTIONS: Dict[str, Tuple[int, int]] = {
    "1:1": (2048, 2048), "16:9": (2720, 1536), "9:16": (1536, 2720), "3:2": (2496, 1664), "2:3": (1664, 2496),
    "4:3": (2368, 1760), "3:4": (1760, 2368), "1:2": (1440, 2880), "2:1": (2880, 1440), "1:3": (1152, 3456),
    "3:1": (3456, 1152)}


@dataclass
class Job:
    """One picture to draw."""
    key: str
    prompt: str
    size: Tuple[int, int]
    out: str                                  # path below the output folder
    meta: Dict[str, Any] = field(default_factory=dict)


def read_jsonl(path) -> List[dict]:
    with open(path, encoding="utf-8") as f:
        return [json.loads(l) for l in f if l.strip()]


def parse_ratio(v) -> Optional[Tuple[int, int]]:
    """``"4:3"``, ``"2400x1800"`` or a pair; None when it is none of these."""
    try:
        if isinstance(v, str):
            parts = re.split(r"[x:]", v.lower())
            if len(parts) != 2:
                return None
            a, b = int(parts[0]), int(parts[1])
        elif isinstance(v, (list, tuple)) and len(v) >= 2:
            a, b = int(v[0]), int(v[1])
        else:
            return None
    except (TypeError, ValueError):
        return None
    return (a, b) if a > 0 and b > 0 else None


def size_for_ratio(ratio: Tuple[int, int], long_side: int = 2048, factor: int = 32) -> Tuple[int, int]:
    rnd = lambda x: max(factor, int(round(x / factor)) * factor)
    w, h = ratio
    return (rnd(long_side), rnd(long_side * h / w)) if w >= h else (rnd(long_side * w / h), rnd(long_side))


def to_bool(v) -> Optional[bool]:
    if isinstance(v, bool):
        return v
    if isinstance(v, int) and v in (0, 1):
        return bool(v)
    if isinstance(v, str):
        t = v.strip().strip('"').lower()
        if t in ("true", "1", "yes", "pass", "supported"):
            return True
        if t in ("false", "0", "no", "fail", "unsupported"):
            return False
    return None


def lenient_json(text: str) -> Optional[dict]:
    """Judges write Python literals now and then (``True`` / ``None``); try the text as it is, then repaired."""
    out = parse_json_block(text or "")
    if out is not None:
        return out
    fixed = re.sub(r"\bNone\b", "null", re.sub(r"\bFalse\b", "false", re.sub(r"\bTrue\b", "true", text or "")))
    return parse_json_block(fixed)


class Suite:
    name = ""
    # sampling defaults of the benchmark's launcher script, overridable on the command line
    defaults: Dict[str, Any] = {}
    summary_file = "summary.json"

    def add_args(self, ap) -> None:
        pass

    def jobs(self, a) -> List[Job]:
        raise NotImplementedError

    def tasks(self, a, image_dir: Path) -> List[dict]:
        """Items to judge: ``id``, ``image`` and whatever ``judge`` needs.  Prompts without a picture are left out."""
        out = []
        for j in self.jobs(a):
            p = image_dir / j.out
            if p.exists():
                out.append({"id": j.key, "image": str(p), "prompt": j.prompt, **j.meta})
        return out

    def judge(self, client, t: dict) -> dict:
        raise NotImplementedError

    def summarize(self, records: Sequence[dict], a) -> dict:
        return rules.SCORERS[self.name](records)


# ---------------------------------------------------------------------------------------------------------------
class BizGenEval(Suite):
    name = "bizgeneval"
    summary_file = "bizgeneval_summary.json"
    FOCUS = {"attribute": "visual attributes: exact colours, counts, relative sizes, shapes, line styles, fonts",
             "layout": "layout: positions, alignment, ordering, containment and spacing of the regions and elements",
             "text": "rendered text: every character, number and symbol must read exactly as stated",
             "knowledge": "domain knowledge: the picture must show what is factually correct for the statement",
             "chart": "charts: values, axes, legends, series and their relations as stated"}
    SYSTEM = ("You are a strict evaluator of {focus}. For each numbered statement decide whether it is true of the "
              "picture. Use only what is visible; if a statement cannot be confirmed, it is false. Answer with JSON "
              "only, one entry per statement number: {{\"1\": {{\"result\": true, \"reason\": \"...\"}}, \"2\": ...}}.")

    def add_args(self, ap):
        ap.add_argument("--data_path", default="evaluation/data/bizgeneval/test.jsonl")

    def _items(self, a):
        return [dict(r, _prompt_id=i) for i, r in enumerate(read_jsonl(a.data_path))]

    def jobs(self, a):
        out = []
        for it in self._items(a):
            ratio = parse_ratio(it.get("aspect_ratio")) or (1, 1)
            meta = {k: it.get(k) for k in ("domain", "dimension", "eval_tag", "questions", "easy_qidxs", "hard_qidxs")}
            meta["dataset_id"] = it.get("id")
            out.append(Job(str(it["_prompt_id"]), it["prompt"], size_for_ratio(ratio), f"{it['_prompt_id']:04d}.png", meta))
        return out

    def tasks(self, a, image_dir):
        out = []
        for j in self.jobs(a):
            for name in (j.out, j.out.replace(".png", "_0.png")):
                if (image_dir / name).exists():
                    out.append({"id": j.key, "image": str(image_dir / name), "prompt": j.prompt, **j.meta})
                    break
        return out

    def judge(self, client, t):
        tag = str(t.get("eval_tag") or t.get("dimension") or "").strip()
        qs = list(t.get("questions") or [])
        if tag not in self.FOCUS or not qs:
            raise ValueError(f"item {t['id']}: no checklist or unknown eval_tag {tag!r}")
        user = "Statements:\n" + "\n".join(f"{i}. {q}" for i, q in enumerate(qs, 1)) + \
               f"\nReturn exactly {len(qs)} entries with keys " + ", ".join(str(i) for i in range(1, len(qs) + 1)) + "."
        raw = client.ask(user, [t["image"]], self.SYSTEM.format(focus=self.FOCUS[tag]), max_tokens=4096)
        parsed = lenient_json(raw)
        if parsed is None:           # a cut-off answer: take the verdicts in order
            found = re.findall(r'"result"\s*:\s*(true|false|True|False|"true"|"false"|1|0)', raw)
            parsed = {str(i): {"result": to_bool(v)} for i, v in enumerate(found[:len(qs)], 1)} if len(found) >= len(qs) else {}
        checks = []
        for i in range(1, len(qs) + 1):
            rec = parsed.get(str(i))
            checks.append(bool(to_bool(rec.get("result"))) if isinstance(rec, dict) else False)   # missing = failed
        return {"checks": checks, "domain": t.get("domain", ""), "dimension": t.get("dimension", ""),
                "easy_qidxs": t.get("easy_qidxs"), "hard_qidxs": t.get("hard_qidxs"), "raw": raw}


# ---------------------------------------------------------------------------------------------------------------
class IGenBench(Suite):
    name = "igenbench"
    summary_file = "igenbench_summary.json"
    QUESTION = ("Look at the infographic and answer the yes/no question about it. Answer 1 only when the picture "
                "clearly satisfies the requirement; anything unclear, partial, unreadable or missing is 0 (a blank or "
                "broken picture is 0 as well).\n\nQuestion: {q}\n\nAnswer with JSON only: "
                "{{\"analysis\": \"what is visible\", \"answer\": \"0 or 1\"}}")

    def add_args(self, ap):
        ap.add_argument("--data_dir", default="evaluation/data/igenbench")
        ap.add_argument("--max_items", type=int, default=None)

    def _items(self, a):
        files = sorted((int(p.stem), p) for p in Path(a.data_dir).glob("*.json") if p.stem.isdigit())
        if getattr(a, "max_items", None):
            files = files[:a.max_items]
        return [json.loads(p.read_text(encoding="utf-8")) for _, p in files]

    def jobs(self, a):
        out = []
        for it in self._items(a):
            ev = [e for e in it.get("evaluation") or [] if str(e.get("question") or "").strip()]
            meta = {"chart_type": it.get("chart_type"), "questions": [e["question"].strip() for e in ev],
                    "question_types": [str(e.get("question_type") or "unknown").strip() for e in ev]}
            out.append(Job(str(int(it["id"])), it["t2i_prompt"], RESOLUTIONS["1:1"], f"{int(it['id']):04d}.png", meta))
        return out

    def judge(self, client, t):
        checks, raws = [], []
        for q in t["questions"]:
            raw = client.ask(self.QUESTION.format(q=q), [t["image"]], None, max_tokens=1024)
            p = lenient_json(raw) or {}
            v = to_bool(p.get("answer", p.get("result", p.get("score"))))
            if v is None:
                m = re.search(r'"(?:answer|result|score)"\s*:\s*"?(true|false|1|0)', raw, flags=re.I)
                if not m:
                    raise ValueError(f"item {t['id']}: unreadable verdict {raw[:80]!r}")
                v = to_bool(m.group(1))
            checks.append(bool(v))
            raws.append(raw)
        return {"checks": checks, "question_types": t["question_types"], "chart_type": t.get("chart_type"), "raw": raws}


# ---------------------------------------------------------------------------------------------------------------
READ_PROMPT = ("Recognize the text in the image, only reply with the text content, but avoid repeating previously "
               "mentioned content. If no text is recognized, please reply with 'No text recognized'.")
_NOISE = ("addCriterion", "No text recognized.", "No text recognized")


def read_text(client, image: str) -> str:
    s = client.ask(READ_PROMPT, [image], None, max_tokens=1024)
    for k in _NOISE:
        s = s.replace(k, "")
    return s.strip()


class LongText(Suite):
    name = "longtext"
    summary_file = "longtext_summary.json"

    def add_args(self, ap):
        ap.add_argument("--data_path", default=None)
        ap.add_argument("--lang", "--mode", dest="lang", default="en", choices=["en", "zh"])
        ap.add_argument("--aspect_ratio", default="1:1", choices=sorted(RESOLUTIONS))

    def _path(self, a):
        return a.data_path or f"evaluation/data/longtext/text_prompts{'_zh' if a.lang == 'zh' else ''}.jsonl"

    def jobs(self, a):
        out = []
        for i, it in enumerate(read_jsonl(self._path(a))):
            pid = int(it.get("prompt_id", i))
            meta = {"target_texts": it.get("text", ""), "category": it.get("category", ""), "length": it.get("length", "")}
            out.append(Job(str(pid), it["prompt"], RESOLUTIONS[a.aspect_ratio], f"{pid:04d}.png", meta))
        return out

    def judge(self, client, t):
        return {"target_texts": t["target_texts"], "read_text": read_text(client, t["image"]),
                "category": t.get("category", ""), "length": t.get("length", "")}

    def summarize(self, records, a):
        s = rules.longtext_summary(records, a.lang)
        s["benchmark"] = f"longtext_{a.lang}"
        by_len: Dict[str, List[dict]] = {}
        for r in records:
            by_len.setdefault(str(r.get("length", "")), []).append(r)
        s["by_length"] = {k: {"count": len(v), "score": rules.longtext_summary(v, a.lang)["score"]} for k, v in sorted(by_len.items())}
        return s


# ---------------------------------------------------------------------------------------------------------------
class CVTG(Suite):
    name = "cvtg"
    summary_file = "CVTG_results.json"
    defaults = {"cfg_scale": 7.0, "timestep_shift": 1.0}

    def add_args(self, ap):
        ap.add_argument("--benchmark_root", default="evaluation/data/cvtg")
        ap.add_argument("--image_size", "--resolution", dest="image_size", type=int, default=2048)
        ap.add_argument("--subsets", default="CVTG,CVTG-Style")
        ap.add_argument("--areas", default="2,3,4,5")
        ap.add_argument("--target_keys", default=None)

    def jobs(self, a):
        keep = {k.strip() for k in a.target_keys.split(",") if k.strip()} if a.target_keys else None
        out = []
        for sub in [s.strip() for s in a.subsets.split(",") if s.strip()]:
            for area in [int(x) for x in a.areas.split(",") if x.strip()]:
                data = json.loads((Path(a.benchmark_root) / sub / f"{area}_combined.json").read_text(encoding="utf-8"))
                for key, prompt in data.items():
                    if keep is None or key in keep:
                        out.append(Job(f"{sub}/{area}/{key}", prompt, (a.image_size, a.image_size),
                                       f"{sub}/{area}/{key}.png", {"subset": sub, "area": area}))
        if not out:
            raise ValueError("no CVTG prompts found: check --benchmark_root, --subsets, --areas, --target_keys")
        return out

    def judge(self, client, t):
        return {"prompt": t["prompt"], "read_text": read_text(client, t["image"]), "area": t["area"], "subset": t["subset"]}


# ---------------------------------------------------------------------------------------------------------------
class TIIF(Suite):
    name = "tiif"
    summary_file = "tiif_summary.json"
    defaults = {"cfg_norm": "global"}
    ASK = ("Examine the picture and answer these yes-or-no questions.\nQuestions:\n{qs}\n"
           "One line per question, in the same order, each line starting with \"yes\" or \"no\" followed by a short "
           "reason. Give exactly as many lines as there are questions and nothing else.")

    def add_args(self, ap):
        ap.add_argument("--input_folder", "--jsonl_dir", dest="input_folder", default="evaluation/data/tiif/testmini_prompts")
        ap.add_argument("--specific_file", default=None)
        ap.add_argument("--resolution", type=int, default=1024)
        ap.add_argument("--model_tag", "--eval_model", dest="model_tag", default="sensenova-u1",
                        help="folder level that names the generating model")
        ap.add_argument("--sample_idx_file", default=None, help="JSON {type: [line indices]}: judge a subset")

    def _files(self, a):
        d = Path(a.input_folder)
        return [d / a.specific_file] if a.specific_file else sorted(d.glob("*.jsonl"))

    def jobs(self, a):
        out = []
        pick = json.loads(Path(a.sample_idx_file).read_text()) if getattr(a, "sample_idx_file", None) else None
        for f in self._files(a):
            for idx, it in enumerate(read_jsonl(f)):
                if pick is not None and idx not in pick.get(it["type"], []):
                    continue
                for kind in ("short_description", "long_description"):
                    meta = {"attribute": it["type"], "type": kind.split("_")[0], "questions": it.get("yn_question_list", []),
                            "gt_answers": it.get("yn_answer_list", []), "file": f.name, "line_idx": idx}
                    out.append(Job(f"{it['type']}/{kind}/{idx}", it[kind], (a.resolution, a.resolution),
                                   f"{it['type']}/{a.model_tag}/{kind}/{idx}.png", meta))
        return out

    def judge(self, client, t):
        qs = [q.strip() for q in t["questions"]]
        raw = client.ask(self.ASK.format(qs="\n".join(qs)), [t["image"]], "You are a professional image critic.",
                         temperature=1.0, max_tokens=2048)
        preds = [m.group(1).lower() for line in raw.strip().splitlines() if line.strip()
                 for m in [re.search(r"(yes|no)", line, flags=re.I)] if m]
        if len(preds) != len(qs):
            raise ValueError(f"{len(preds)} answers for {len(qs)} questions")
        return {"attribute": t["attribute"], "type": t["type"], "gt_answers": t["gt_answers"], "model_pred": preds, "raw": raw}


SUITES: Dict[str, Suite] = {s.name: s for s in (BizGenEval(), IGenBench(), LongText(), CVTG(), TIIF())}
