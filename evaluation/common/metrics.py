"""Scoring functions shared by the benchmark drivers (pure Python, no model).

* text rendering (CVTG / LongText style, reference evaluation/gen/cvtg/unified_metrics_eval.py and
  evaluation/gen/longtext/eval_images_longtext.py): word accuracy and normalised edit distance between
  the text that should appear in the picture and what a reader (OCR model or VLM judge) found;
* checklist benchmarks (BizGenEval / IGenBench / TIIF style): per-dimension pass rates;
* understanding (reference evaluation/understanding): exact match, multiple choice, ANLS;
* interleaved reasoning benchmarks (BabyVision / Unimmmu / RealUnify, reference
  evaluation/interleave/*/calculate_score.py): accuracy overall and per category.
"""
from __future__ import annotations

import re
import unicodedata
from collections import defaultdict
from typing import Dict, Iterable, List, Optional, Sequence


def normalize_text(s: str) -> str:
    s = unicodedata.normalize("NFKC", s).lower()
    s = re.sub(r"[^\w\s]", " ", s, flags=re.UNICODE)
    return re.sub(r"\s+", " ", s).strip()


def edit_distance(a: Sequence, b: Sequence) -> int:
    if len(a) < len(b):
        a, b = b, a
    prev = list(range(len(b) + 1))
    for i, ca in enumerate(a, 1):
        cur = [i]
        for j, cb in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (ca != cb)))
        prev = cur
    return prev[-1]


def normalized_edit_distance(pred: str, target: str) -> float:
    """1 - NED in [0, 1] (1 = identical after normalisation)."""
    p, t = normalize_text(pred), normalize_text(target)
    if not p and not t:
        return 1.0
    return 1.0 - edit_distance(p, t) / max(len(p), len(t))


def word_accuracy(pred: str, targets: Sequence[str]) -> float:
    """Share of target words found in the predicted text (each predicted word is used once)."""
    want = [w for t in targets for w in normalize_text(t).split()]
    if not want:
        return 1.0
    have: Dict[str, int] = defaultdict(int)
    for w in normalize_text(pred).split():
        have[w] += 1
    hit = 0
    for w in want:
        if have[w] > 0:
            have[w] -= 1
            hit += 1
    return hit / len(want)


def text_rendering_scores(records: Iterable[dict]) -> Dict[str, float]:
    """``records``: {"target_texts": [...], "read_text": str}.  Mean word accuracy, mean 1-NED and the
    share of pictures with every word right."""
    acc, ned, perfect, n = 0.0, 0.0, 0, 0
    for r in records:
        if "read_text" not in r:
            continue
        a = word_accuracy(r["read_text"], r["target_texts"])
        acc += a
        ned += normalized_edit_distance(r["read_text"], " ".join(r["target_texts"]))
        perfect += a == 1.0
        n += 1
    return {"n": n, "word_accuracy": acc / max(n, 1), "one_minus_ned": ned / max(n, 1), "all_words_right": perfect / max(n, 1)}


def checklist_scores(records: Iterable[dict]) -> Dict[str, float]:
    """``records``: {"dimension": str, "checks": [bool | None, ...]}.  A sample's score is the share of its
    checks that passed (unparsed answers count as failed); dimensions are macro-averaged."""
    per: Dict[str, List[float]] = defaultdict(list)
    for r in records:
        checks = r.get("checks")
        if not checks:
            continue
        per[r.get("dimension", "all")].append(sum(1 for c in checks if c) / len(checks))
    out = {f"dim/{k}": sum(v) / len(v) for k, v in sorted(per.items())}
    out["n"] = sum(len(v) for v in per.values())
    out["overall"] = sum(out[f"dim/{k}"] for k in per) / max(len(per), 1)
    return out


def rating_scores(records: Iterable[dict], key: str = "score") -> Dict[str, float]:
    """Mean judge rating overall and per dimension (OpenING-style 0-10 ratings)."""
    per: Dict[str, List[float]] = defaultdict(list)
    for r in records:
        if r.get(key) is not None:
            per[r.get("dimension", "all")].append(float(r[key]))
    out = {f"dim/{k}": sum(v) / len(v) for k, v in sorted(per.items())}
    allv = [x for v in per.values() for x in v]
    out["n"], out["overall"] = len(allv), sum(allv) / max(len(allv), 1)
    return out


def exact_match(pred: str, answers: Sequence[str]) -> float:
    p = normalize_text(pred)
    return float(any(p == normalize_text(a) for a in answers))


def relaxed_match(pred: str, answers: Sequence[str]) -> float:
    """The answer appears as a whole word sequence in the prediction, or numbers agree within 5 %."""
    p = normalize_text(pred)
    for a in answers:
        na = normalize_text(a)
        if na and re.search(r"(?<!\w)" + re.escape(na) + r"(?!\w)", p):
            return 1.0
        try:
            x, y = float(pred.strip().rstrip("%")), float(a.strip().rstrip("%"))
            if abs(x - y) <= 0.05 * abs(y):
                return 1.0
        except ValueError:
            pass
    return 0.0


def anls(pred: str, answers: Sequence[str], threshold: float = 0.5) -> float:
    best = max((normalized_edit_distance(pred, a) for a in answers), default=0.0)
    return best if best >= threshold else 0.0


def accuracy_by_category(records: Iterable[dict], key: str = "correct") -> Dict[str, float]:
    per: Dict[str, List[float]] = defaultdict(list)
    for r in records:
        if key in r and r[key] is not None:
            per[r.get("category", "all")].append(float(r[key]))
    out = {f"cat/{k}": sum(v) / len(v) for k, v in sorted(per.items())}
    allv = [x for v in per.values() for x in v]
    out["n"], out["accuracy"] = len(allv), sum(allv) / max(len(allv), 1)
    return out


def format_table(scores: Dict[str, float], title: str = "") -> str:
    w = max((len(k) for k in scores), default=4)
    lines = [title] if title else []
    for k, v in scores.items():
        lines.append(f"{k:<{w}}  {v:.4f}" if isinstance(v, float) else f"{k:<{w}}  {v}")
    return "\n".join(lines)
