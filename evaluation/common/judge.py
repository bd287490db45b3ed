"""Judge side of the benchmarks: a client for an OpenAI-style chat endpoint that answers questions
about (image, text) pairs, parsers for its answers, and a resumable parallel runner.

Role of the reference's evaluation/gen/common/judge.py:19-110 (client with retry and back-off) and of
the per-benchmark loops that call it (e.g. evaluation/gen/tiif/eval/eval_with_vlm_mp.py,
evaluation/gen/bizgeneval/eval_images_bizgeneval.py); one implementation here serves every benchmark.

Configuration: ``JUDGE_API_BASE`` (or ``OPENAI_BASE_URL``), ``JUDGE_API_KEY`` (or ``OPENAI_API_KEY``),
``JUDGE_MODEL``.  The endpoint may be this framework's own server.
"""
from __future__ import annotations

import base64
import json
import os
import re
import threading
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence
from urllib import request
from urllib.error import HTTPError, URLError


def image_data_url(path) -> str:
    p = Path(path)
    kind = {"jpg": "jpeg"}.get(p.suffix.lower().lstrip("."), p.suffix.lower().lstrip(".") or "png")
    return f"data:image/{kind};base64," + base64.b64encode(p.read_bytes()).decode()


class JudgeError(RuntimeError):
    pass


class JudgeClient:
    def __init__(self, api_base: Optional[str] = None, api_key: Optional[str] = None, model: Optional[str] = None,
                 timeout: float = 240.0, max_retries: int = 6, backoff_base: float = 2.0, backoff_cap: float = 60.0,
                 sleep: Callable[[float], None] = time.sleep):
        self.api_base = (api_base or os.environ.get("JUDGE_API_BASE") or os.environ.get("OPENAI_BASE_URL") or "").rstrip("/")
        self.api_key = api_key or os.environ.get("JUDGE_API_KEY") or os.environ.get("OPENAI_API_KEY") or ""
        self.model = model or os.environ.get("JUDGE_MODEL") or ""
        if not self.api_base or not self.model:
            raise ValueError("judge endpoint not configured: set JUDGE_API_BASE and JUDGE_MODEL")
        self.timeout, self.max_retries = timeout, max_retries
        self.backoff_base, self.backoff_cap, self._sleep = backoff_base, backoff_cap, sleep
        self.requests = 0
        self.retries = 0

    def ask(self, question: str, images: Sequence = (), system: Optional[str] = None, temperature: float = 0.0,
            max_tokens: int = 1024) -> str:
        """One chat completion; ``images`` are file paths or ready ``data:`` / http URLs."""
        content: Any = question
        if images:
            urls = [i if isinstance(i, str) and (i.startswith("data:") or i.startswith("http")) else image_data_url(i)
                    for i in images]
            content = [{"type": "text", "text": question}] + [{"type": "image_url", "image_url": {"url": u}} for u in urls]
        messages = ([{"role": "system", "content": system}] if system else []) + [{"role": "user", "content": content}]
        body = json.dumps({"model": self.model, "temperature": temperature, "max_tokens": max_tokens,
                           "messages": messages}).encode()
        headers = {"Content-Type": "application/json"}
        if self.api_key:
            headers["Authorization"] = "Bearer " + self.api_key
        url = self.api_base + ("/chat/completions" if self.api_base.endswith("/v1") else "/v1/chat/completions")
        err: Optional[Exception] = None
        for attempt in range(self.max_retries + 1):
            self.requests += 1
            try:
                with request.urlopen(request.Request(url, data=body, headers=headers, method="POST"),
                                     timeout=self.timeout) as resp:
                    data = json.loads(resp.read().decode())
                msg = data["choices"][0]["message"]["content"]
                if isinstance(msg, list):
                    msg = "".join(p.get("text", "") for p in msg if isinstance(p, dict))
                return str(msg)
            except HTTPError as e:
                if not (e.code == 429 or 500 <= e.code < 600):
                    raise JudgeError(f"judge refused the request: HTTP {e.code}") from e
                err = e
            except (URLError, TimeoutError, ConnectionError, KeyError, ValueError) as e:
                err = e
            if attempt < self.max_retries:
                self.retries += 1
                self._sleep(min(self.backoff_cap, self.backoff_base ** attempt))
        raise JudgeError(f"judge request failed after {self.max_retries + 1} attempts: {err}")


# ------------------------------------------------------------------------------------------------
# answer parsing
# ------------------------------------------------------------------------------------------------
def parse_yes_no(text: str) -> Optional[bool]:
    """First clear yes / no of an answer (judges are asked to start with it); None if neither."""
    m = re.search(r"\b(yes|no)\b", text.strip().lower())
    return None if m is None else m.group(1) == "yes"


def parse_score(text: str, lo: float = 0.0, hi: float = 10.0) -> Optional[float]:
    """A numeric rating: ``score: 7``, ``7/10``, ``"score": 7.5`` or a bare number; None if out of range."""
    t = text.strip()
    for pat in (r"score\W{0,4}(-?\d+(?:\.\d+)?)", r"(-?\d+(?:\.\d+)?)\s*/\s*\d+", r"^\W*(-?\d+(?:\.\d+)?)\W*$",
                r"(-?\d+(?:\.\d+)?)"):
        m = re.search(pat, t, flags=re.I | re.M)
        if m:
            v = float(m.group(1))
            return v if lo <= v <= hi else None
    return None


def parse_json_block(text: str) -> Optional[dict]:
    """The first JSON object of an answer (plain, or inside a ```json fence)."""
    m = re.search(r"```(?:json)?\s*(\{.*?\})\s*```", text, flags=re.S)
    cand = [m.group(1)] if m else []
    depth, start = 0, None
    for i, ch in enumerate(text):
        if ch == "{":
            if depth == 0:
                start = i
            depth += 1
        elif ch == "}" and depth:
            depth -= 1
            if depth == 0 and start is not None:
                cand.append(text[start:i + 1])
                break
    for c in cand:
        try:
            out = json.loads(c)
            if isinstance(out, dict):
                return out
        except ValueError:
            continue
    return None


def parse_choice(text: str, letters: str = "ABCDEFGH") -> Optional[str]:
    """The option letter a model settled on: ``Answer: B``, ``(C)``, ``**D**`` or a bare letter at the end."""
    t = text.strip()
    m = re.search(r"answer\s*(?:is|:)?\s*\(?\*{0,2}([%s])\*{0,2}\)?(?![a-z])" % letters, t, flags=re.I)
    if m:
        return m.group(1).upper()
    found = re.findall(r"(?<![A-Za-z])\(?([%s])\)?(?![A-Za-z])" % letters, t)
    return found[-1].upper() if found else None


# ------------------------------------------------------------------------------------------------
# resumable results + parallel runner
# ------------------------------------------------------------------------------------------------
class ResultLog:
    """Append-only JSONL keyed by ``id``: a restarted run skips what is already there."""

    def __init__(self, path):
        self.path = Path(path)
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.done: Dict[str, dict] = {}
        self._lock = threading.Lock()
        if self.path.exists():
            for line in self.path.read_text().splitlines():
                try:
                    r = json.loads(line)
                    self.done[str(r["id"])] = r
                except (ValueError, KeyError):
                    continue               # a line cut off by a crash

    def __contains__(self, key) -> bool:
        return str(key) in self.done

    def add(self, rec: dict) -> None:
        with self._lock:
            self.done[str(rec["id"])] = rec
            with self.path.open("a") as f:
                f.write(json.dumps(rec, ensure_ascii=False) + "\n")

    def records(self) -> List[dict]:
        return list(self.done.values())


def run_parallel(items: Iterable[dict], fn: Callable[[dict], dict], log: ResultLog, workers: int = 8,
                 on_error: str = "record") -> List[dict]:
    """Applies ``fn`` to every item whose ``id`` is not in ``log`` yet.  An item that raises is recorded with
    an ``error`` field (``on_error="record"``) so that one bad sample does not end the evaluation."""
    todo = [it for it in items if it["id"] not in log]

    def guarded(it):
        try:
            out = fn(it)
        except Exception as e:
            if on_error != "record":
                raise
            out = {"error": f"{type(e).__name__}: {e}"}
        return {"id": it["id"], **out}

    with ThreadPoolExecutor(max_workers=max(1, workers)) as pool:
        for fut in as_completed([pool.submit(guarded, it) for it in todo]):
            log.add(fut.result())
    return log.records()


def merge_shards(paths: Sequence, out_path) -> int:
    """Joins per-rank result files (later files win on duplicate ids); returns the record count."""
    merged: Dict[str, dict] = {}
    for p in paths:
        merged.update(ResultLog(p).done)
    Path(out_path).parent.mkdir(parents=True, exist_ok=True)
    with open(out_path, "w") as f:
        for k in sorted(merged, key=lambda s: (len(s), s)):
            f.write(json.dumps(merged[k], ensure_ascii=False) + "\n")
    return len(merged)
