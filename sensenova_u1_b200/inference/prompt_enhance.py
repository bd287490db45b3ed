"""Prompt enhancement: expand a short user prompt into a detailed text-to-image prompt with a
language model before generation (``--enhance`` in the example CLIs).

Back-ends, chosen by ``U1_ENHANCE_BACKEND`` or explicitly (same knobs as the reference,
src/sensenova_u1/prompt_enhance/enhancer.py:18-133):

* ``chat_completions``  any OpenAI-compatible ``/chat/completions`` endpoint,
* ``anthropic``         an Anthropic ``/v1/messages`` endpoint,
* ``local``             the loaded NEO-unify model itself through its ``chat`` call: no network and
                        no second model in memory (not in the reference).

The HTTP back-ends take a ``transport(url, headers, json) -> dict`` callable (default: ``requests``),
which is how the tests drive them without a network.
"""
from __future__ import annotations

import os
from typing import Callable, Dict, Optional

ENV = "U1_ENHANCE_"
STYLES: Dict[str, str] = {
    "default": (
        "You rewrite short image requests into one detailed prompt for a text-to-image model. Keep every "
        "subject, attribute, count and piece of quoted text the user asked for. Add concrete visual detail: "
        "composition, viewpoint, lighting, materials, colour palette, background and mood. Do not add new "
        "subjects that change the meaning. Answer with the rewritten prompt only, in the user's language."),
    "edit": (
        "You rewrite a short image-editing instruction into one precise instruction for an image-editing model. "
        "Look at the attached image(s): name the object or region to change, say exactly what it becomes, and list "
        "what must stay as it is (identity, pose, background, lighting, text). Answer with the instruction only."),
    "caption": (
        "Describe the attached image in one dense paragraph usable as a text-to-image prompt: subjects, their "
        "attributes and positions, setting, lighting, style and any visible text (quoted). No preamble."),
    "infographic": (
        "You turn a short request into a detailed prompt for an information graphic: state the title, the "
        "sections and their order, the exact text of every label (in quotes), the chart or diagram types, "
        "the layout grid, the colour scheme and the typography. Answer with the prompt only."),
}


def _requests_transport(url: str, headers: Dict[str, str], json: dict, timeout: float = 120.0) -> dict:
    import requests
    r = requests.post(url, headers=headers, json=json, timeout=timeout)
    r.raise_for_status()
    return r.json()


class ChatCompletionsBackend:
    def __init__(self, endpoint: str, api_key: str, model: str, transport: Optional[Callable] = None):
        self.endpoint, self.api_key, self.model = endpoint, api_key, model
        self.transport = transport or _requests_transport

    def complete(self, system: str, user: str, images=()) -> str:
        content = user if not images else [{"type": "text", "text": user}] + [
            {"type": "image_url", "image_url": {"url": "data:image/png;base64," + b}} for b in images]
        body = {"model": self.model, "messages": [{"role": "system", "content": system},
                                                  {"role": "user", "content": content}]}
        out = self.transport(self.endpoint, {"Authorization": f"Bearer {self.api_key}",
                                             "Content-Type": "application/json"}, body)
        return out["choices"][0]["message"]["content"].strip()


class AnthropicBackend:
    def __init__(self, endpoint: str, api_key: str, model: str, transport: Optional[Callable] = None,
                 max_tokens: int = 2048):
        self.endpoint, self.api_key, self.model, self.max_tokens = endpoint, api_key, model, max_tokens
        self.transport = transport or _requests_transport

    def complete(self, system: str, user: str, images=()) -> str:
        content = user if not images else [{"type": "image", "source": {"type": "base64", "media_type": "image/png",
                                                                         "data": b}} for b in images] + [
            {"type": "text", "text": user}]
        body = {"model": self.model, "max_tokens": self.max_tokens, "system": system,
                "messages": [{"role": "user", "content": content}]}
        out = self.transport(self.endpoint, {"x-api-key": self.api_key, "anthropic-version": "2023-06-01",
                                             "Content-Type": "application/json"}, body)
        return "".join(p.get("text", "") for p in out["content"] if p.get("type") == "text").strip()


class LocalBackend:
    """Uses the already loaded model (``NEOChatModel.chat``)."""

    def __init__(self, model, tokenizer, max_new_tokens: int = 512):
        self.model, self.tok, self.max_new_tokens = model, tokenizer, max_new_tokens

    def complete(self, system: str, user: str, images=()) -> str:
        px = None
        if images:
            import base64
            import io
            from PIL import Image
            from .images import load_image_native
            px = [load_image_native(Image.open(io.BytesIO(base64.b64decode(b))).convert("RGB"),
                                    factor=self.model.cfg.token_pixels) for b in images]
            user = "<image>\n" * len(px) + user
        return self.model.chat(self.tok, px, system + "\n\n" + user,
                               generation_config={"max_new_tokens": self.max_new_tokens}).strip()


def backend_from_env(backend: Optional[str] = None, endpoint: Optional[str] = None, api_key: Optional[str] = None,
                     model: Optional[str] = None, transport: Optional[Callable] = None):
    E = os.environ.get
    backend = (backend or E(ENV + "BACKEND") or "chat_completions").lower()
    endpoint = endpoint or E(ENV + "ENDPOINT")
    model = model or E(ENV + "MODEL")
    api_key = api_key or E(ENV + "API_KEY")
    if backend not in ("chat_completions", "anthropic"):
        raise ValueError(f"unsupported enhance backend {backend!r}; supported: chat_completions, anthropic, local")
    if not api_key:
        raise RuntimeError(f"prompt enhancement over HTTP needs an API key: set {ENV}API_KEY or pass api_key=")
    if not endpoint or not model:
        raise RuntimeError(f"set {ENV}ENDPOINT and {ENV}MODEL (or pass endpoint= / model=)")
    cls = ChatCompletionsBackend if backend == "chat_completions" else AnthropicBackend
    return cls(endpoint, api_key, model, transport)


class PromptEnhancer:
    def __init__(self, backend, style: str = "default"):
        if style not in STYLES:
            raise ValueError(f"unknown enhance style {style!r}; supported: {sorted(STYLES)}")
        self.backend, self.style = backend, style

    @classmethod
    def from_env(cls, style: str = "default", **kw) -> "PromptEnhancer":
        return cls(backend_from_env(**kw), style)

    @classmethod
    def local(cls, model, tokenizer, style: str = "default") -> "PromptEnhancer":
        return cls(LocalBackend(model, tokenizer), style)

    def enhance(self, prompt: str, images=()) -> str:
        """``images``: base64-encoded PNG/JPEG strings (editing instructions, captions); text-only styles
        ignore them.  The U1.5 caption / edit-prompt scripts of the reference
        (src/sensenova_u1_5/{caption,edit_pe,image_pe}.py) are these two styles."""
        out = self.backend.complete(STYLES[self.style], prompt, tuple(images))
        return out or prompt                      # an empty answer must not erase the request
