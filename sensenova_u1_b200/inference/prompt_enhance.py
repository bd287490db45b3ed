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

    def complete(self, system: str, user: str) -> str:
        body = {"model": self.model, "messages": [{"role": "system", "content": system},
                                                  {"role": "user", "content": user}]}
        out = self.transport(self.endpoint, {"Authorization": f"Bearer {self.api_key}",
                                             "Content-Type": "application/json"}, body)
        return out["choices"][0]["message"]["content"].strip()


class AnthropicBackend:
    def __init__(self, endpoint: str, api_key: str, model: str, transport: Optional[Callable] = None,
                 max_tokens: int = 2048):
        self.endpoint, self.api_key, self.model, self.max_tokens = endpoint, api_key, model, max_tokens
        self.transport = transport or _requests_transport

    def complete(self, system: str, user: str) -> str:
        body = {"model": self.model, "max_tokens": self.max_tokens, "system": system,
                "messages": [{"role": "user", "content": user}]}
        out = self.transport(self.endpoint, {"x-api-key": self.api_key, "anthropic-version": "2023-06-01",
                                             "Content-Type": "application/json"}, body)
        return "".join(p.get("text", "") for p in out["content"] if p.get("type") == "text").strip()


class LocalBackend:
    """Uses the already loaded model (``NEOChatModel.chat``)."""

    def __init__(self, model, tokenizer, max_new_tokens: int = 512):
        self.model, self.tok, self.max_new_tokens = model, tokenizer, max_new_tokens

    def complete(self, system: str, user: str) -> str:
        return self.model.chat(self.tok, None, system + "\n\n" + user,
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

    def enhance(self, prompt: str) -> str:
        out = self.backend.complete(STYLES[self.style], prompt)
        return out or prompt                      # an empty answer must not erase the request
