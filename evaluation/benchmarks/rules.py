"""Scoring and aggregation rules, one function per benchmark.

The arithmetic follows the reference's drivers (cited per function); judging itself (asking a VLM yes/no questions,
reading text out of pictures, rating answers) is done by the shared drivers of this folder's parent and arrives here as
fields of the records."""
from __future__ import annotations

import difflib
import re
from collections import Counter, defaultdict
from statistics import mean
from typing import Callable, Dict, Iterable, List, Optional, Sequence


def _group_mean(records: Sequence[dict], key: str, fields: Sequence[str]) -> Dict[str, dict]:
    groups: Dict[str, List[dict]] = defaultdict(list)
    for r in records:
        groups[str(r.get(key, ""))].append(r)
    return {g: {"count": len(items), **{f: mean(float(i[f]) for i in items) for f in fields}}
            for g, items in sorted(groups.items())}


# ---------------------------------------------------------------------------------------------------------
# BizGenEval: a checklist per picture; accuracy = passed / asked, error score = max(0, 1 - alpha * failures) with
# alpha 0.1 overall and 0.2 on the "easy" and "hard" subsets of the questions; means over pictures, by domain and
# by dimension (evaluation/gen/bizgeneval/eval_images_bizgeneval.py:27, 128-166, 385-415).
# ---------------------------------------------------------------------------------------------------------
BIZGEN_ERROR_ALPHA = 0.1


def _biz_item(checks: Sequence[Optional[bool]], qidxs: Optional[Sequence[int]], alpha: float) -> dict:
    idx = list(qidxs) if qidxs is not None else list(range(1, len(checks) + 1))
    if not idx:
        return {"accuracy": 0.0, "error_score": 0.0, "errors": 0, "n_questions": 0}
    errors = sum(1 for q in idx if not (1 <= q <= len(checks) and checks[q - 1] is True))
    return {"accuracy": (len(idx) - errors) / len(idx), "error_score": max(0.0, 1.0 - alpha * errors), "errors": errors,
            "n_questions": len(idx)}


def bizgeneval_summary(records: Iterable[dict]) -> dict:
    """Records: ``checks`` (list of True / False / None per question), optional ``easy_qidxs`` / ``hard_qidxs``
    (1-based question numbers), ``domain``, ``dimension``."""
    rows = []
    for r in records:
        o = _biz_item(r["checks"], None, BIZGEN_ERROR_ALPHA)
        e = _biz_item(r["checks"], r.get("easy_qidxs") or [], BIZGEN_ERROR_ALPHA * 2)
        h = _biz_item(r["checks"], r.get("hard_qidxs") or [], BIZGEN_ERROR_ALPHA * 2)
        rows.append({"domain": r.get("domain", ""), "dimension": r.get("dimension", ""), "accuracy": o["accuracy"],
                     "error_score": o["error_score"], "easy_accuracy": e["accuracy"], "easy_error_score": e["error_score"],
                     "hard_accuracy": h["accuracy"], "hard_error_score": h["error_score"], "n_questions": o["n_questions"]})
    f = ("accuracy", "error_score")
    out = {"benchmark": "bizgeneval", "items": len(rows), "error_alpha": BIZGEN_ERROR_ALPHA}
    for k in ("accuracy", "error_score", "easy_accuracy", "easy_error_score", "hard_accuracy", "hard_error_score"):
        out[("overall_" + k) if k in f else k] = mean(r[k] for r in rows) if rows else 0.0
    out["by_domain"], out["by_dimension"] = _group_mean(rows, "domain", f), _group_mean(rows, "dimension", f)
    return out


# ---------------------------------------------------------------------------------------------------------
# IGenBench (infographics): factual questions per picture; score = mean per-picture accuracy, q_acc = correct / asked
# over all questions, strict = share of pictures with every question right, accuracy per question type
# (evaluation/gen/igenbench/eval_images_igenbench.py:90-110, 404-425).
# ---------------------------------------------------------------------------------------------------------
def igenbench_summary(records: Iterable[dict]) -> dict:
    """Records: ``checks`` (True / False per question) and ``question_types`` (same length; optional)."""
    per, ok_t, n_t = [], Counter(), Counter()
    correct = total = 0
    for r in records:
        checks = [c is True for c in r["checks"]]
        if not checks:
            continue
        types = r.get("question_types") or ["unknown"] * len(checks)
        for c, t in zip(checks, types):
            n_t[t] += 1
            ok_t[t] += int(c)
        correct += sum(checks)
        total += len(checks)
        per.append({"accuracy": sum(checks) / len(checks), "strict": all(checks), "chart_type": r.get("chart_type", "")})
    return {"benchmark": "igenbench", "items": len(per), "score": mean(p["accuracy"] for p in per) if per else 0.0,
            "q_acc": correct / total if total else 0.0, "i_acc_strict": mean(float(p["strict"]) for p in per) if per else 0.0,
            "correct_questions": correct, "total_questions": total,
            "question_type_acc": {t: ok_t[t] / n_t[t] for t in sorted(n_t)}, "question_type_counts": dict(n_t)}


# ---------------------------------------------------------------------------------------------------------
# LongText: the words (English) or characters (Chinese) of the requested text that the judge read back from the
# picture, as a multiset intersection; the score pools matches over pictures (evaluation/gen/longtext/
# eval_images_longtext.py:140-200).
# ---------------------------------------------------------------------------------------------------------
_KEEP = r"一-龥a-zA-Z0-9àâäéèêëîïôöùûüçÀÂÄÉÈÊËÎÏÔÖÙÛÜÇ"


def longtext_clean(s: str, mode: str = "en") -> str:
    if mode == "en":
        return re.sub(r"\s+", " ", re.sub(rf"[^{_KEEP}\s]", "", s)).strip().lower()
    return "".join(re.findall(rf"[{_KEEP}]", s)).strip()


def longtext_match(gt: str, read: str, mode: str = "en"):
    a, b = (gt.split(), read.split()) if mode == "en" else (list(gt), list(read))
    return sum((Counter(a) & Counter(b)).values()), len(a)


def longtext_summary(records: Iterable[dict], mode: str = "en") -> dict:
    """Records: ``target_texts`` (string or list) and ``read_text``; optional ``category``."""
    rows = []
    for r in records:
        gt = r["target_texts"]
        gt = " ".join(map(str, gt)) if isinstance(gt, (list, tuple)) else str(gt)
        m, n = longtext_match(longtext_clean(gt, mode), longtext_clean(str(r.get("read_text", "")), mode), mode)
        rows.append({"matched": m, "total_gt": n, "score": m / n if n else 0.0, "category": r.get("category", "")})
    pooled = lambda items: (sum(i["matched"] for i in items) / max(1, sum(i["total_gt"] for i in items)))
    groups: Dict[str, List[dict]] = defaultdict(list)
    for r in rows:
        groups[r["category"]].append(r)
    return {"benchmark": f"longtext-{mode}", "items": len(rows), "score": pooled(rows) if rows else 0.0,
            "by_category": {k: {"count": len(v), "score": pooled(v)} for k, v in sorted(groups.items())}}


# ---------------------------------------------------------------------------------------------------------
# CVTG-2K: the quoted words of the prompt against the words read from the picture: word accuracy (exact presence)
# and NED = mean over words of 1 - edit distance / max length to the closest read word
# (evaluation/gen/cvtg/unified_metrics_eval.py:176-235); the CLIP / aesthetic columns of the reference need extra
# model weights and are left to the caller (``extra`` fields are averaged if present).
# ---------------------------------------------------------------------------------------------------------
def _ned(a: str, b: str) -> float:
    from ..common.metrics import edit_distance
    return 1 - edit_distance(a, b) / (max(len(a), len(b)) + 1e-5)


def cvtg_words(prompt: str) -> List[str]:
    return [w for m in re.findall(r"'(.*?)'", prompt) for w in m.lower().split()]


def cvtg_summary(records: Iterable[dict]) -> dict:
    """Records: ``prompt`` (target words are the single-quoted spans) or ``target_texts``, and ``read_text``;
    optional ``area`` (number of text regions: the benchmark's split) and numeric ``clip_score`` / ``aesthetic``."""
    rows = []
    for r in records:
        gt = [w for t in r["target_texts"] for w in str(t).lower().split()] if r.get("target_texts") else cvtg_words(r["prompt"])
        pred = str(r.get("read_text", "")).lower().split() or [""]
        acc = sum(1 for w in gt if w in pred)
        neds = []
        for w in gt:
            best = difflib.get_close_matches(w, pred, n=1, cutoff=0)
            neds.append(_ned(w, best[0]) if best else 0.0)
        rows.append({"area": str(r.get("area", "")), "total": len(gt), "acc": acc, "neds": neds,
                     **{k: float(r[k]) for k in ("clip_score", "aesthetic") if k in r}})

    def agg(items):
        tw = sum(i["total"] for i in items)
        neds = [x for i in items for x in i["neds"]]
        out = {"count": len(items), "word_accuracy": sum(i["acc"] for i in items) / tw if tw else 0.0,
               "ned": mean(neds) if neds else 0.0}
        for k in ("clip_score", "aesthetic"):
            vals = [i[k] for i in items if k in i]
            if vals:
                out[k] = mean(vals)
        return out
    groups: Dict[str, List[dict]] = defaultdict(list)
    for r in rows:
        groups[r["area"]].append(r)
    return {"benchmark": "cvtg", "items": len(rows), **agg(rows), "by_area": {k: agg(v) for k, v in sorted(groups.items())}}


# ---------------------------------------------------------------------------------------------------------
# TIIF-Bench: yes/no questions per picture, accuracy per (attribute, prompt-length type) as correct / asked with
# case-insensitive comparison of the judge's answers (evaluation/gen/tiif/eval/summary_results.py:51-130).
# ---------------------------------------------------------------------------------------------------------
# the benchmark's taxonomy: three tiers, nine dimensions, each a set of attribute files
# (evaluation/gen/tiif/eval/summary_dimension_results.py:44-140; overall = mean of the nine dimension scores)
_ATTR, _REL = ("color", "texture"), ("2d", "3d")
_REASON = ("numeracy", "comparison", "differentiation", "negation")
TIIF_DIMENSIONS: Dict[str, Dict[str, List[str]]] = {
    "Basic": {"Attribute": ["shape+color", "color+texture", "texture+color", "shape+texture"],
              "Relation": ["2d_spatial_relation", "3d_spatial_relation", "action+2d", "action+3d"],
              "Reasoning": ["numeracy", "negation", "differentiation", "comparison"]},
    "Advanced": {"Attribute+Relation": [f"action+{a}" for a in _ATTR] + [f"{a}+{r}" for a in ("color", "shape", "texture") for r in _REL],
                 "Attribute+Reasoning": [f"{q}+{a}" for q in _REASON for a in _ATTR],
                 "Relation+Reasoning": [f"{q}+{r}" for q in _REASON for r in _REL],
                 "Text Generation": ["text"], "Style Control": ["style"]},
    "Real_World": {"Complex": ["real_world"]}}


def tiif_summary(records: Iterable[dict]) -> dict:
    """Records: ``gt_answers`` and ``model_pred`` (lists of "yes" / "no"), ``attribute``, ``type`` ("short" / "long")."""
    cells: Dict[tuple, List[int]] = defaultdict(lambda: [0, 0])
    for r in records:
        key = (str(r.get("attribute", "")), str(r.get("type", "")))
        for g, p in zip(r["gt_answers"], r["model_pred"]):
            cells[key][1] += 1
            cells[key][0] += int(str(g).strip().lower() == str(p).strip().lower())
    table = {f"{a}/{t}": {"accuracy": c / n if n else 0.0, "correct": c, "total": n} for (a, t), (c, n) in sorted(cells.items())}
    by_type: Dict[str, List[float]] = defaultdict(list)
    for (a, t), (c, n) in cells.items():
        if n:
            by_type[t].append(c / n)
    acc = {(a, t): c / n for (a, t), (c, n) in cells.items() if n}
    groups, nine = {}, {"short": [], "long": []}
    for tier, dims in TIIF_DIMENSIONS.items():
        tier_attrs = [a for attrs in dims.values() for a in attrs]
        for name, attrs in [("Overall", tier_attrs)] + list(dims.items()):
            row = {}
            for t in ("short", "long"):
                vals = [acc[(a, t)] for a in attrs if (a, t) in acc]
                row[t] = mean(vals) if vals else None
                if name != "Overall" and vals:
                    nine[t].append(row[t])
            groups[f"{tier}/{name}"] = row
    overall = {t: (mean(v) if v else None) for t, v in nine.items()}        # mean of the nine dimension scores
    return {"benchmark": "tiif", "cells": table, "mean_by_type": {t: mean(v) for t, v in sorted(by_type.items())},
            "dimensions": groups, "overall": overall}


# ---------------------------------------------------------------------------------------------------------
# RealUnify / UniMMMU (multiple choice): the answer letter inside <answer>...</answer> if present, otherwise the first
# A-D letter of the response; accuracy per task type (evaluation/interleave/Realunify/calculate_score.py:16-107).
# ---------------------------------------------------------------------------------------------------------
def choice_letter(response: str) -> str:
    if not response:
        return ""
    m = re.search(r"<answer>(.*?)</answer>", response, re.DOTALL)
    cand = m.group(1).strip() if m else response.strip()
    c = re.search(r"[A-D]", cand, re.IGNORECASE)
    return c.group(0).upper() if c else ""


def realunify_summary(records: Iterable[dict]) -> dict:
    """Records: ``model_response`` / ``response`` (string or list), ``answer`` (letter), ``task_type``."""
    stats: Dict[str, List[int]] = defaultdict(lambda: [0, 0])
    for r in records:
        resp = r.get("model_response", r.get("response", ""))
        if isinstance(resp, list) and resp:
            resp = resp[0]
        s = stats[str(r.get("task_type", "unknown"))]
        s[1] += 1
        s[0] += int(choice_letter(str(resp)) == str(r.get("answer", "")).strip().upper())
    by = {t: {"correct": c, "total": n, "acc": c / n if n else 0.0} for t, (c, n) in sorted(stats.items())}
    tot = sum(n for _, n in stats.values())
    return {"benchmark": "realunify", "by_task": by, "overall_acc": sum(c for c, _ in stats.values()) / tot if tot else 0.0,
            "total": tot}


def unimmmu_summary(records: Iterable[dict]) -> dict:
    """UniMMMU mixes multiple-choice tasks with tasks judged by a model; records carry ``task`` and either
    ``correct`` (bool, from the judge) or ``response`` + ``answer`` (a letter).  Accuracy per task and overall
    (evaluation/interleave/Unimmmu/calculate_score.py defers to the benchmark's own repository for the arithmetic;
    this is the per-task accuracy those scripts report)."""
    stats: Dict[str, List[int]] = defaultdict(lambda: [0, 0])
    for r in records:
        ok = r["correct"] if "correct" in r else choice_letter(str(r.get("response", ""))) == str(r.get("answer", "")).strip().upper()
        s = stats[str(r.get("task", "unknown"))]
        s[1] += 1
        s[0] += int(bool(ok))
    by = {t: {"correct": c, "total": n, "acc": c / n if n else 0.0} for t, (c, n) in sorted(stats.items())}
    tot = sum(n for _, n in stats.values())
    return {"benchmark": "unimmmu", "by_task": by, "overall_acc": sum(c for c, _ in stats.values()) / tot if tot else 0.0,
            "task_mean_acc": mean(v["acc"] for v in by.values()) if by else 0.0, "total": tot}


# ---------------------------------------------------------------------------------------------------------
# BabyVision: overall accuracy of the judged answers, accuracy per Type and per Type/Subtype
# (evaluation/interleave/BabyVision/compute_score.py:13-45).
# ---------------------------------------------------------------------------------------------------------
BABYVISION_TYPES = {"Fine-grained Discrimination": "1", "Visual Tracking": "2", "Spatial Perception": "3",
                    "Visual Pattern Recognition": "4"}


def babyvision_summary(records: Iterable[dict]) -> dict:
    """Records: ``LLMJudgeResult`` (or ``correct``), ``Type``, ``Subtype``."""
    recs = list(records)
    ok = lambda r: bool(r.get("LLMJudgeResult", r.get("correct", False)))
    types: Dict[str, List[int]] = defaultdict(lambda: [0, 0])
    subs: Dict[str, List[int]] = defaultdict(lambda: [0, 0])
    for r in recs:
        t, st = str(r.get("Type", "")), str(r.get("Subtype", ""))
        for d, k in ((types, t), (subs, BABYVISION_TYPES.get(t, "0") + t + "/" + st)):
            d[k][1] += 1
            d[k][0] += int(ok(r))
    acc = lambda d: {k: {"accuracy": c / n if n else 0.0, "correct": c, "total": n} for k, (c, n) in sorted(d.items())}
    ta, sa = acc(types), acc(subs)
    return {"benchmark": "babyvision", "overall_accuracy": sum(map(ok, recs)) / len(recs) if recs else 0.0,
            "type_average_accuracy": mean(v["accuracy"] for v in ta.values()) if ta else 0.0,
            "subtype_average_accuracy": mean(v["accuracy"] for v in sa.values()) if sa else 0.0, "by_type": ta, "by_subtype": sa}


# ---------------------------------------------------------------------------------------------------------
# OpenING: a judge model rates every answer on several named criteria (0-10); entries without a usable score are
# dropped, the rest are averaged per model and criterion, models ranked by the mean over criteria
# (evaluation/interleave/OpenING/summarize_GPT_scores.py:23-157).
# ---------------------------------------------------------------------------------------------------------
def opening_summary(records: Iterable[dict]) -> dict:
    """Records: ``model`` ({"id", "name"} or a string) and ``score`` ({criterion: number} or {"scores": {...}})."""
    per: Dict[str, Dict[str, List[float]]] = defaultdict(lambda: defaultdict(list))
    names, dropped, kept = {}, 0, 0
    for r in records:
        sc = r.get("score")
        if isinstance(sc, dict) and isinstance(sc.get("scores"), dict):
            sc = sc["scores"]
        model = r.get("model", "")
        mid = model.get("id", "") if isinstance(model, dict) else str(model)
        names[mid] = model.get("name", mid) if isinstance(model, dict) else str(model)
        vals = {k: v for k, v in (sc or {}).items() if isinstance(v, (int, float))} if isinstance(sc, dict) else {}
        if not vals:
            dropped += 1
            continue
        kept += 1
        for k, v in vals.items():
            per[mid][k].append(float(v))
    table = {}
    for mid, crit in per.items():
        row = {k: mean(v) for k, v in sorted(crit.items())}
        row["overall"] = mean(row.values()) if row else 0.0
        table[names.get(mid, mid)] = row
    ranking = sorted(table, key=lambda m: -table[m]["overall"])
    return {"benchmark": "opening", "entries": kept, "dropped": dropped, "models": table, "ranking": ranking}


SCORERS: Dict[str, Callable] = {
    "bizgeneval": bizgeneval_summary, "igenbench": igenbench_summary, "longtext": longtext_summary, "cvtg": cvtg_summary,
    "tiif": tiif_summary, "realunify": realunify_summary, "unimmmu": unimmmu_summary, "babyvision": babyvision_summary,
    "opening": opening_summary,
}
