"""HTTP client of the API nodes: OpenAI-style routes of ``sensenova_u1_b200.serving.server`` or of a
hosted endpoint (role of the reference's apps/comfyui/api_client.py:60-289 and config.py:1-31).

Configuration (``config.py``): environment or a ``.env`` file; ``SENSENOVA_BASE_URL`` / ``SN_BASE_URL`` (default
http://127.0.0.1:8000), ``SENSENOVA_API_KEY`` / ``SN_API_KEY`` (optional bearer token), ``SENSENOVA_RETRIES``.
"""
from __future__ import annotations

import base64
import os
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

IMAGE_SIZE_OPTIONS = ("2048x2048|1:1", "2752x1536|16:9", "1536x2752|9:16", "2496x1664|3:2", "1664x2496|2:3",
                      "2368x1760|4:3", "1760x2368|3:4", "2272x1824|5:4", "1824x2272|4:5", "3072x1376|21:9",
                      "1344x3136|9:21", "1024x1024|1:1", "512x512|1:1")


class ApiError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"HTTP {status}: {message}")
        self.status = status


@dataclass
class ChatResult:
    text: str
    usage: Dict[str, Any] = field(default_factory=dict)
    raw: Dict[str, Any] = field(default_factory=dict)
    images: List[bytes] = field(default_factory=list)      # pictures of an interleaved answer


@dataclass
class ImageResult:
    images: List[bytes]
    urls: List[str]
    raw: Dict[str, Any]


def parse_size(option: str) -> str:
    """``"2048x2048|1:1"`` -> ``"2048x2048"`` (the aspect label is for the menu only)."""
    size = option.split("|", 1)[0].strip().lower()
    w, h = size.split("x")
    if int(w) % 32 or int(h) % 32:
        raise ValueError(f"image sides must be multiples of 32, got {size}")
    return size


class ApiClient:
    def __init__(self, base_url: str, api_key: str = "", retries: int = 2, session=None):
        self.base_url = base_url.rstrip("/")
        self.api_key = api_key
        self.retries = max(0, int(retries))
        self._session = session

    @classmethod
    def from_env(cls) -> "ApiClient":
        try:
            from .config import load_config
        except ImportError:                 # direct import in tests
            from config import load_config  # type: ignore
        c = load_config()
        return cls(c.base_url, c.api_key, c.retries)

    # -- transport -----------------------------------------------------------------------------
    def _post(self, route: str, body: dict, timeout: float) -> dict:
        import requests
        sess = self._session or requests
        headers = {"Content-Type": "application/json"}
        if self.api_key:
            headers["Authorization"] = "Bearer " + self.api_key
        last: Optional[Exception] = None
        for attempt in range(self.retries + 1):
            try:
                r = sess.post(self.base_url + route, json=body, headers=headers, timeout=timeout)
            except Exception as e:                       # connection refused / timeout: retry
                last = e
            else:
                if r.status_code < 400:
                    return r.json()
                detail = r.text[:500]
                if r.status_code < 500 and r.status_code != 429:
                    raise ApiError(r.status_code, detail)        # the request itself is wrong: do not retry
                last = ApiError(r.status_code, detail)
            if attempt < self.retries:
                time.sleep(min(2.0 ** attempt * 0.25, 4.0))
        raise last if isinstance(last, ApiError) else ApiError(0, f"request failed: {last}")

    # -- routes --------------------------------------------------------------------------------
    def chat(self, text: str, system_prompt: str = "", model: str = "sensenova-u1", temperature: float = 0.7,
             top_p: float = 1.0, max_tokens: int = 2048, timeout: float = 120, image_urls=(),
             interleave: bool = False, **extra) -> ChatResult:
        content: Any = text
        if image_urls:
            content = [{"type": "text", "text": text}] + [{"type": "image_url", "image_url": {"url": u}}
                                                          for u in image_urls]
        messages = ([{"role": "system", "content": system_prompt}] if system_prompt else []) + [
            {"role": "user", "content": content}]
        body = {"model": model, "messages": messages, "temperature": temperature, "top_p": top_p,
                "max_tokens": max_tokens, "interleave": interleave, **extra}
        raw = self._post("/v1/chat/completions", body, timeout)
        msg = raw["choices"][0]["message"]["content"]
        images: List[bytes] = []
        if isinstance(msg, list):                        # interleaved answer: text parts + data-URL pictures
            texts = []
            for part in msg:
                if part.get("type") == "text":
                    texts.append(part.get("text", ""))
                elif part.get("type") == "image_url":
                    url = part["image_url"]["url"]
                    if url.startswith("data:"):
                        images.append(base64.b64decode(url.split(",", 1)[1]))
            msg = "\n".join(texts)
        return ChatResult(msg, raw.get("usage", {}), raw, images)

    def generate_image(self, prompt: str, model: str = "sensenova-u1", size: str = "2048x2048", n: int = 1,
                       timeout: float = 300, **extra) -> ImageResult:
        raw = self._post("/v1/images/generations", {"model": model, "prompt": prompt, "size": size, "n": n, **extra},
                         timeout)
        return self._image_result(raw, timeout)

    def edit_image(self, prompt: str, images_b64: List[str], n: int = 1, timeout: float = 300, **extra) -> ImageResult:
        raw = self._post("/v1/images/edits", {"prompt": prompt, "image": images_b64, "n": n, **extra}, timeout)
        return self._image_result(raw, timeout)

    def _image_result(self, raw: dict, timeout: float) -> ImageResult:
        images, urls = [], []
        for d in raw.get("data", []):
            if d.get("b64_json"):
                images.append(base64.b64decode(d["b64_json"]))
            elif d.get("url"):
                import requests
                urls.append(d["url"])
                images.append(requests.get(d["url"], timeout=timeout).content)
        if not images:
            raise ApiError(200, "the response carries no image")
        return ImageResult(images, urls, raw)
