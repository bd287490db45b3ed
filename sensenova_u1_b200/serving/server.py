"""HTTP serving of the unified model behind OpenAI-style routes.

The reference ships only a client for an external LightLLM server (examples/serving/client.py:204-356:
``/v1/chat/completions`` for VQA and interleaved streams, ``/v1/images/generations`` for T2I,
``/v1/images/edits`` for editing).  Here the server is part of the framework: one process per GPU,
requests enter a queue, a single worker thread owns the GPU (the engine is not re-entrant: it reuses
one fixed workspace and one KV arena) and drains the queue; text-to-image requests with equal
sampler settings that wait together are merged into ONE batched denoise (the packed sampler runs
many samples per step at no extra launches).

    python -m sensenova_u1_b200.serving.server --model_path CKPT --port 8000
    python -m sensenova_u1_b200.serving.server --random_init tiny --port 8000     # no checkpoint needed
"""
from __future__ import annotations

import base64
import io
import queue
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class _Job:
    kind: str                      # "t2i" | "edit" | "chat" | "interleave"
    args: Dict[str, Any]
    done: threading.Event = field(default_factory=threading.Event)
    result: Any = None
    error: Optional[str] = None
    t_enqueue: float = field(default_factory=time.time)


def _png_b64(img) -> str:
    from ..inference.images import to_pil
    buf = io.BytesIO()
    to_pil(img).save(buf, format="PNG")
    return base64.b64encode(buf.getvalue()).decode()


def _decode_image(b64: str, factor: int, min_pixels: Optional[int] = None, max_pixels: Optional[int] = None):
    """Base64 picture (plain or data URL) -> understanding input inside the pixel budget (the native-resolution
    defaults, or the request's ``min_pixels`` / ``max_pixels``)."""
    from PIL import Image
    from ..inference.images import load_image_native
    if "," in b64 and b64.strip().startswith("data:"):
        b64 = b64.split(",", 1)[1]
    kw = {k: int(v) for k, v in (("min_pixels", min_pixels), ("max_pixels", max_pixels)) if v}
    return load_image_native(Image.open(io.BytesIO(base64.b64decode(b64))).convert("RGB"), factor=factor, **kw)


class GenerationService:
    """Queue + GPU worker.  ``model`` needs the public generation calls of ``NEOChatModel``
    (t2i_generate, it2i_generate, interleave_gen, chat); anything with that surface works, which is
    how the CPU tests drive it."""

    def __init__(self, model, tokenizer, max_batch: int = 4, batch_wait_s: float = 0.01):
        self.model, self.tok = model, tokenizer
        self.max_batch, self.batch_wait_s = max_batch, batch_wait_s
        self.q: "queue.Queue[_Job]" = queue.Queue()
        self.stats = {"requests": 0, "batches": 0, "merged": 0, "errors": 0, "busy_s": 0.0}
        self._stop = threading.Event()
        self.worker = threading.Thread(target=self._loop, name="snu1-gpu-worker", daemon=True)
        self.worker.start()

    # ---- client side -------------------------------------------------------------
    def submit(self, kind: str, timeout: float = 3600.0, **args):
        job = _Job(kind, args)
        self.q.put(job)
        if not job.done.wait(timeout):
            raise TimeoutError(f"{kind} request timed out after {timeout}s in the queue")
        if job.error:
            raise RuntimeError(job.error)
        return job.result

    def close(self):
        self._stop.set()
        self.q.put(_Job("stop", {}))
        self.worker.join(timeout=5)

    # ---- worker ------------------------------------------------------------------
    @staticmethod
    def _merge_key(j: _Job):
        a = j.args
        return (a.get("width"), a.get("height"), a.get("num_steps"), a.get("cfg_scale"), a.get("timestep_shift"),
                a.get("cfg_norm"), a.get("prompt"), a.get("think", False))

    def _loop(self):
        while not self._stop.is_set():
            job = self.q.get()
            if job.kind == "stop":
                break
            group = [job]
            if job.kind == "t2i":
                # identical prompt + settings, different seeds (n > 1 fan-out or retries): one batched call
                deadline = time.time() + self.batch_wait_s
                held = []
                while len(group) < self.max_batch:
                    try:
                        nxt = self.q.get(timeout=max(0.0, deadline - time.time()))
                    except queue.Empty:
                        break
                    if nxt.kind == "t2i" and self._merge_key(nxt) == self._merge_key(job):
                        group.append(nxt)
                    else:
                        held.append(nxt)
                for h in held:
                    self.q.put(h)
            t0 = time.time()
            try:
                self._run(group)
            except Exception as e:            # the worker must survive a bad request
                self.stats["errors"] += 1
                for j in group:
                    j.error = f"{type(e).__name__}: {e}"
            self.stats["busy_s"] += time.time() - t0
            self.stats["requests"] += len(group)
            self.stats["batches"] += 1
            self.stats["merged"] += len(group) - 1
            for j in group:
                j.done.set()

    def _run(self, group: List[_Job]):
        m, tok, a = self.model, self.tok, group[0].args
        kind = group[0].kind
        if kind == "t2i":
            n = sum(j.args.get("n", 1) for j in group)
            out = m.t2i_generate(tok, a["prompt"], cfg_scale=a.get("cfg_scale", 4.0),
                                 timestep_shift=a.get("timestep_shift", 3.0), cfg_norm=a.get("cfg_norm", "none"),
                                 image_size=(a.get("width", 1024), a.get("height", 1024)),
                                 num_steps=a.get("num_steps", 50), batch_size=n, seed=a.get("seed", 0),
                                 think_mode=a.get("think", False))
            think = None
            if a.get("think", False):
                out, think = out
            i = 0
            for j in group:
                k = j.args.get("n", 1)
                j.result = {"images": [out[i + x] for x in range(k)], "think": think}
                i += k
        elif kind == "edit":
            out = m.it2i_generate(tok, a["prompt"], a["images"], cfg_scale=a.get("cfg_scale", 4.0),
                                  img_cfg_scale=a.get("img_cfg_scale", 1.0), timestep_shift=a.get("timestep_shift", 3.0),
                                  cfg_norm=a.get("cfg_norm", "none"), image_size=a.get("image_size"),
                                  num_steps=a.get("num_steps", 50), batch_size=a.get("n", 1), seed=a.get("seed", 0))
            group[0].result = {"images": [out[i] for i in range(out.shape[0])]}
        elif kind == "interleave":
            extra = {k: a[k] for k in ("cfg_scale", "img_cfg_scale", "timestep_shift", "cfg_norm") if a.get(k) is not None}
            if a.get("system"):
                extra["system_message"] = a["system"]
            if a.get("think"):
                extra["think_mode"] = True
            text, pics = m.interleave_gen(tok, a["prompt"], a.get("images", ()), max_rounds=a.get("max_rounds", 4),
                                          max_new_tokens=a.get("max_new_tokens", 256),
                                          image_size=(a.get("width", 512), a.get("height", 512)),
                                          num_steps=a.get("num_steps", 50), seed=a.get("seed", 0), **extra)
            group[0].result = {"text": text, "images": pics}
        elif kind == "chat":
            gc = {"max_new_tokens": a.get("max_new_tokens", 256)}
            gc.update(a.get("sampling") or {})
            extra = {}
            if a.get("history"):
                extra["history"] = list(a["history"])
            if a.get("system"):
                extra["system_message"] = a["system"]
            text = m.chat(tok, a.get("images") or None, a["prompt"], generation_config=gc, **extra)
            group[0].result = {"text": text}
        else:
            raise ValueError(f"unknown request kind {kind!r}")


def _split_messages(messages, factor, min_pixels=None, max_pixels=None):
    """OpenAI chat messages -> (prompt text of the last user turn, its decoded images, system message, history).
    ``history``: earlier (user text, assistant text) pairs; pictures of earlier turns are not replayed."""
    def text_of(c):
        if isinstance(c, str):
            return c, []
        parts, urls = [], []
        for part in c or []:
            if part.get("type") == "text":
                parts.append(part.get("text", ""))
            elif part.get("type") == "image_url":
                urls.append(part["image_url"]["url"])
        return "\n".join(parts), urls

    text, urls, system, history, pending = "", [], None, [], None
    for msg in messages:
        role = msg.get("role")
        t, u = text_of(msg.get("content"))
        if role == "system":
            system = t if system is None else system + "\n" + t
        elif role == "user":
            if pending is not None:
                history.append((pending, ""))             # a user turn without an answer
            pending, text, urls = t, t, u
        elif role == "assistant" and pending is not None:
            history.append((pending, t))
            pending = None
    if pending is None and history:                       # the conversation ends with an assistant turn: nothing to answer
        text, urls = "", []
    return text, [_decode_image(u, factor, min_pixels, max_pixels) for u in urls], system, history


# image_config of the reference's serving client (examples/serving/client.py:30-155): explicit width / height when both
# are positive, otherwise an aspect-ratio bucket scaled to a size preset
_ASPECT_BUCKETS = {"1:1": (2048, 2048), "16:9": (2752, 1536), "9:16": (1536, 2752), "3:2": (2496, 1664), "2:3": (1664, 2496),
                   "4:3": (2368, 1760), "3:4": (1760, 2368), "5:4": (2272, 1824), "4:5": (1824, 2272), "21:9": (3072, 1376),
                   "9:21": (1344, 3136)}
_SIZE_PRESETS = {"2K": 1.0, "1.5K": 0.75, "1K": 0.5, "0.5K": 0.25}


def image_size_from_config(image_config: Optional[dict], factor: int = 32, default=(1024, 1024)):
    """(width, height, seed) from an ``image_config`` object; sides are multiples of ``factor``."""
    ic = dict(image_config or {})
    seed = int(ic.get("seed", 0) or 0)
    w, h = int(ic.get("width", -1) or -1), int(ic.get("height", -1) or -1)
    if w <= 0 or h <= 0:
        ratio = str(ic.get("aspect_ratio") or "")
        if ratio in _ASPECT_BUCKETS:
            bw, bh = _ASPECT_BUCKETS[ratio]
            sc = _SIZE_PRESETS.get(str(ic.get("image_size") or "2K").upper(), 1.0)
            w, h = bw * sc, bh * sc
        else:
            w, h = default
    snap = lambda v: max(factor, int(round(v / factor)) * factor)
    return snap(w), snap(h), seed


def _interleave_extras(body: dict, system) -> dict:
    """System message, thinking switch and guidance knobs of an interleaved request."""
    out = {"system": system, "think": bool((body.get("chat_template_kwargs") or {}).get("enable_thinking", False))}
    for k in ("cfg_scale", "img_cfg_scale", "timestep_shift"):
        if body.get(k) is not None:
            out[k] = float(body[k])
    if body.get("cfg_norm") is not None:
        out["cfg_norm"] = str(body["cfg_norm"])
    if "image_config" not in body and body.get("size"):
        w, h = (int(x) for x in str(body["size"]).lower().split("x"))
        out.update(width=w, height=h)
    return out


def sampling_from_body(body: dict) -> dict:
    """Text sampling knobs of a chat-completions body: ``temperature`` (absent or 0: greedy), ``top_p``, and the
    ``top_k`` / ``repetition_penalty`` / ``seed`` extensions that OpenAI clients send through ``extra_body``."""
    extra = body.get("extra_body") or {}
    get = lambda k: body.get(k, extra.get(k))
    out = {}
    t = get("temperature")
    if t is not None and float(t) > 0:
        out.update(do_sample=True, temperature=float(t))
        if get("top_p") is not None:
            out["top_p"] = float(get("top_p"))
        if get("top_k") is not None and int(get("top_k")) > 0:
            out["top_k"] = int(get("top_k"))
        if get("seed") is not None:
            out["seed"] = int(get("seed"))
    if get("repetition_penalty") is not None and float(get("repetition_penalty")) != 1.0:
        out["repetition_penalty"] = float(get("repetition_penalty"))
    return out


def create_app(service: GenerationService, model_name: str = "sensenova-u1"):
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import StreamingResponse
    import json

    app = FastAPI(title="sensenova-u1_b200")
    factor = getattr(getattr(service.model, "cfg", None), "token_pixels", 32)

    def run(kind, **kw):
        try:
            return service.submit(kind, **kw)
        except TimeoutError as e:
            raise HTTPException(504, str(e))
        except RuntimeError as e:
            raise HTTPException(500, str(e))

    @app.get("/health")
    def health():
        return {"status": "ok", "queue": service.q.qsize(), **service.stats}

    @app.get("/v1/models")
    def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model"}]}

    @app.post("/v1/images/generations")
    def generations(body: dict):
        w, h = (int(x) for x in str(body.get("size", "1024x1024")).lower().split("x"))
        r = run("t2i", prompt=body["prompt"], width=w, height=h, n=int(body.get("n", 1)),
                num_steps=int(body.get("num_inference_steps", body.get("num_steps", 50))),
                cfg_scale=float(body.get("cfg_scale", 4.0)), timestep_shift=float(body.get("timestep_shift", 3.0)),
                cfg_norm=body.get("cfg_norm", "none"), seed=int(body.get("seed", 0)), think=bool(body.get("think", False)))
        out = {"created": int(time.time()), "data": [{"b64_json": _png_b64(i)} for i in r["images"]]}
        if r.get("think"):
            out["think"] = r["think"]
        return out

    @app.post("/v1/images/edits")
    def edits(body: dict):
        imgs = body.get("image") or body.get("images") or []
        imgs = [imgs] if isinstance(imgs, str) else imgs
        if not imgs:
            raise HTTPException(400, "edits need at least one image (base64 PNG/JPEG)")
        r = run("edit", prompt=body["prompt"], images=[_decode_image(b, factor) for b in imgs], n=int(body.get("n", 1)),
                num_steps=int(body.get("num_inference_steps", body.get("num_steps", 50))),
                cfg_scale=float(body.get("cfg_scale", 4.0)), img_cfg_scale=float(body.get("img_cfg_scale", 1.0)),
                timestep_shift=float(body.get("timestep_shift", 3.0)), cfg_norm=body.get("cfg_norm", "none"),
                seed=int(body.get("seed", 0)))
        return {"created": int(time.time()), "data": [{"b64_json": _png_b64(i)} for i in r["images"]]}

    def _images_only(body, prompt, images, rid):
        """``modalities == ["image"]`` (the reference client's t2i / it2i modes): one generated picture in
        ``message.images``; the reasoning text, if thinking was asked for, in ``message.content``."""
        w, h, seed = image_size_from_config(body.get("image_config"), factor)
        think = bool((body.get("chat_template_kwargs") or {}).get("enable_thinking", False))
        common = dict(num_steps=int(body.get("num_steps", 50)), cfg_scale=float(body.get("cfg_scale", 4.0)),
                      timestep_shift=float(body.get("timestep_shift", 3.0)), cfg_norm=body.get("cfg_norm", "none"),
                      seed=int(body.get("seed", seed)))
        if images:
            r = run("edit", prompt=prompt, images=images, n=1, img_cfg_scale=float(body.get("img_cfg_scale", 1.0)),
                    image_size=(w, h) if int((body.get("image_config") or {}).get("width", -1) or -1) > 0 else None, **common)
        else:
            r = run("t2i", prompt=prompt, width=w, height=h, n=1, think=think, **common)
        msg = {"role": "assistant", "content": r.get("think") or "",
               "images": [{"type": "image_url", "image_url": {"url": "data:image/png;base64," + _png_b64(i)}}
                          for i in r["images"]]}
        return {"id": rid, "object": "chat.completion", "created": int(time.time()), "model": model_name,
                "choices": [{"index": 0, "message": msg, "finish_reason": "stop"}]}

    @app.post("/chat/completions")
    @app.post("/v1/chat/completions")
    def chat(body: dict):
        extra = body.get("extra_body") or {}
        prompt, images, system, history = _split_messages(body.get("messages", []), factor,
                                                          body.get("min_pixels", extra.get("min_pixels")),
                                                          body.get("max_pixels", extra.get("max_pixels")))
        modalities = [str(m).lower() for m in (body.get("modalities") or [])]
        rid = "chatcmpl-" + uuid.uuid4().hex[:24]
        if modalities == ["image"]:
            return _images_only(body, prompt, images, rid)
        interleave = bool(body.get("interleave", False)) or "image" in modalities
        if interleave and body.get("stream") and "image_config" in body:
            # streamed interleaved answer in the reference client's shape: text deltas, pictures in delta.images
            w, h, seed = image_size_from_config(body.get("image_config"), factor, default=(512, 512))
            r = run("interleave", prompt=prompt, images=images, max_rounds=int(body.get("max_rounds", 4)),
                    max_new_tokens=int(body.get("max_tokens", 256)), num_steps=int(body.get("num_steps", 50)),
                    seed=int(body.get("seed", seed)), width=w, height=h, **_interleave_extras(body, system))

            def gen_parts():
                mk = lambda delta, fin=None: "data: " + json.dumps(
                    {"id": rid, "object": "chat.completion.chunk", "model": model_name,
                     "choices": [{"index": 0, "delta": delta, "finish_reason": fin}]}) + "\n\n"
                pics = list(r["images"])
                pieces = r["text"].split("[image]")
                for k, piece in enumerate(pieces):
                    if piece:
                        yield mk({"role": "assistant", "content": piece})
                    if k < len(pieces) - 1 and pics:
                        yield mk({"images": [{"type": "image_url", "image_url": {
                            "url": "data:image/png;base64," + _png_b64(pics.pop(0))}}]})
                for pic in pics:                                   # pictures the text did not mark
                    yield mk({"images": [{"type": "image_url", "image_url": {"url": "data:image/png;base64," + _png_b64(pic)}}]})
                yield mk({}, "stop")
                yield "data: [DONE]\n\n"
            return StreamingResponse(gen_parts(), media_type="text/event-stream")
        if interleave:
            r = run("interleave", prompt=prompt, images=images, max_rounds=int(body.get("max_rounds", 4)),
                    max_new_tokens=int(body.get("max_tokens", 256)), num_steps=int(body.get("num_steps", 50)),
                    seed=int(body.get("seed", 0)), **_interleave_extras(body, system))
            content: Any = [{"type": "text", "text": r["text"]}] + [
                {"type": "image_url", "image_url": {"url": "data:image/png;base64," + _png_b64(i)}} for i in r["images"]]
        else:
            r = run("chat", prompt=prompt, images=images, max_new_tokens=int(body.get("max_tokens", 256)),
                    sampling=sampling_from_body(body), system=system, history=history)
            content = r["text"]
        if body.get("stream"):
            def gen():
                chunk = {"id": rid, "object": "chat.completion.chunk", "model": model_name,
                         "choices": [{"index": 0, "delta": {"role": "assistant", "content": content}, "finish_reason": None}]}
                yield "data: " + json.dumps(chunk) + "\n\n"
                chunk["choices"][0] = {"index": 0, "delta": {}, "finish_reason": "stop"}
                yield "data: " + json.dumps(chunk) + "\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")
        return {"id": rid, "object": "chat.completion", "created": int(time.time()), "model": model_name,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": content}, "finish_reason": "stop"}]}

    return app


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_path", default=None)
    ap.add_argument("--random_init", default=None)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--max_batch", type=int, default=4)
    ap.add_argument("--layers", type=int, default=None)
    a = ap.parse_args(argv)
    import uvicorn
    from ..config import get_config
    from ..inference.api import ByteTokenizer, NEOChatModel
    if a.model_path:
        from transformers import AutoTokenizer
        model = NEOChatModel.from_pretrained(a.model_path)
        tok = AutoTokenizer.from_pretrained(a.model_path, trust_remote_code=True)
    else:
        kw = {"num_layers": a.layers} if a.layers else {}
        model = NEOChatModel.from_config(get_config(a.random_init or "8b-mot", **kw))
        tok = ByteTokenizer(model.cfg.vocab_size)
    svc = GenerationService(model, tok, max_batch=a.max_batch)
    uvicorn.run(create_app(svc), host=a.host, port=a.port, log_level="info")


if __name__ == "__main__":
    main()
