#!/usr/bin/env python
"""Client of an OpenAI-compatible server of the unified model (``python -m sensenova_u1_b200.serving.server``, or
any server that speaks the same chat-completions dialect).  Modes and flags follow the reference's client
(examples/serving/client.py:60-382): every mode posts to ``<url>/chat/completions``; pictures come back in
``message.images`` (or ``delta.images`` while streaming) as data URLs.

    python examples/serving/client.py --mode t2i --prompt "a red fox" --url http://127.0.0.1:8000/v1 --out-dir out
    python examples/serving/client.py --mode it2i --image_path in.png --prompt "make it snow"
    python examples/serving/client.py --mode interleave --prompt "a story in two pictures"
    python examples/serving/client.py --mode vqa --image_path in.png --prompt "what is shown?"
"""
import argparse
import base64
import json
import re
import sys
from datetime import datetime
from pathlib import Path

try:                      # the system prompts the released checkpoints were tuned with
    sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
    from sensenova_u1_b200.inference.prompts import SYSTEM_MESSAGE_FOR_GEN as GENERATION_SYSTEM_PROMPT
    from sensenova_u1_b200.inference.prompts import SYSTEM_MESSAGE_FOR_INTERLEAVE as INTERLEAVE_SYSTEM_PROMPT
except ImportError:       # the client alone, without this repository
    GENERATION_SYSTEM_PROMPT = "You are an image generation and editing assistant."
    INTERLEAVE_SYSTEM_PROMPT = "You are a multimodal assistant that answers with text and images."
IMAGE_CONFIG_DEFAULT = {"aspect_ratio": "1:1", "image_size": "2K", "seed": 42, "height": -1, "width": -1,
                        "dynamic_resolution": True}


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--mode", default="t2i", choices=["t2i", "it2i", "interleave", "vqa"])
    p.add_argument("--url", "--base_url", dest="url", default="http://127.0.0.1:8000/v1", help="base URL ending in /v1")
    p.add_argument("--api-key", "--api_key", dest="api_key", default="EMPTY")
    p.add_argument("--model", default="sensenova-u1")
    p.add_argument("--prompt", required=True)
    p.add_argument("--image_path", "--image", dest="image_path", default=None, help="input image (it2i, vqa, interleave)")
    p.add_argument("--out-dir", "--output_dir", dest="out_dir", default="outputs")
    p.add_argument("--temperature", type=float, default=0.8)
    p.add_argument("--top-p", "--top_p", dest="top_p", type=float, default=0.95)
    p.add_argument("--max-tokens", "--max_tokens", dest="max_tokens", type=int, default=4096)
    p.add_argument("--enable-thinking", dest="enable_thinking", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--seed", type=int, default=IMAGE_CONFIG_DEFAULT["seed"])
    p.add_argument("--aspect-ratio", "--aspect_ratio", dest="aspect_ratio", default=IMAGE_CONFIG_DEFAULT["aspect_ratio"])
    p.add_argument("--image-size", "--image_size", dest="image_size", default=IMAGE_CONFIG_DEFAULT["image_size"],
                   help="size preset (1K, 1.5K, 2K)")
    p.add_argument("--height", type=int, default=-1, help="with --width: explicit size (-1: from the aspect ratio)")
    p.add_argument("--width", type=int, default=-1)
    p.add_argument("--num_steps", type=int, default=50, help="denoising steps (this package's server)")
    p.add_argument("--cfg_scale", type=float, default=4.0)
    p.add_argument("--timeout", type=float, default=3600)
    return p.parse_args(argv)


def build_image_config(a) -> dict:
    ic = dict(IMAGE_CONFIG_DEFAULT, aspect_ratio=a.aspect_ratio, image_size=a.image_size, seed=a.seed, height=a.height,
              width=a.width)
    if a.height > 0 and a.width > 0:
        ic["dynamic_resolution"] = False
    return ic


def image_to_data_url(path: str) -> str:
    p = Path(path)
    if not p.exists():
        raise FileNotFoundError(f"image not found: {p}")
    mime = {".jpg": "image/jpeg", ".jpeg": "image/jpeg", ".png": "image/png", ".webp": "image/webp"}.get(p.suffix.lower(),
                                                                                                       "image/jpeg")
    return f"data:{mime};base64," + base64.b64encode(p.read_bytes()).decode()


def save_data_url(url: str, path: Path) -> Path:
    m = re.match(r"data:image/(?P<sub>[\w+.-]+);base64,(?P<b64>.+)", url, re.DOTALL)
    if not m:
        raise ValueError(f"not an image data URL: {url[:60]}...")
    ext = {"jpeg": "jpg", "jpg": "jpg", "webp": "webp"}.get(m.group("sub"), "png")
    path = path.with_suffix("." + ext)
    path.write_bytes(base64.b64decode(m.group("b64")))
    print(f"[saved] {path}")
    return path


def build_payload(a) -> dict:
    content = []
    if a.image_path:
        content.append({"type": "image_url", "image_url": {"url": image_to_data_url(a.image_path)}})
    content.append({"type": "text", "text": a.prompt})
    if a.mode == "vqa":
        return {"model": a.model, "messages": [{"role": "user", "content": content}], "max_tokens": a.max_tokens}
    if a.mode == "it2i" and not a.image_path:
        raise SystemExit("--mode it2i needs --image_path")
    system = INTERLEAVE_SYSTEM_PROMPT if a.mode == "interleave" else GENERATION_SYSTEM_PROMPT
    user = content if (a.image_path or a.mode == "interleave") else a.prompt
    return {"model": a.model, "messages": [{"role": "system", "content": system}, {"role": "user", "content": user}],
            "modalities": ["text", "image"] if a.mode == "interleave" else ["image"], "stream": a.mode == "interleave",
            "n": 1, "temperature": a.temperature, "top_p": a.top_p, "max_tokens": a.max_tokens,
            "chat_template_kwargs": {"enable_thinking": a.enable_thinking}, "image_config": build_image_config(a),
            "seed": a.seed, "num_steps": a.num_steps, "cfg_scale": a.cfg_scale}


def main(argv=None, session=None) -> int:
    a = parse_args(argv)
    import requests
    http = session or requests
    out = Path(a.out_dir)
    out.mkdir(parents=True, exist_ok=True)
    stamp = datetime.now().strftime("%Y%m%d_%H%M%S")
    url = a.url.rstrip("/") + "/chat/completions"
    headers = {"Authorization": f"Bearer {a.api_key}", "Content-Type": "application/json"}
    payload = build_payload(a)
    if a.mode == "interleave":
        r = http.post(url, headers=headers, json=payload, stream=True, timeout=a.timeout)
        r.raise_for_status()
        chunks, k = [], 0
        for line in r.iter_lines():
            line = line.decode() if isinstance(line, bytes) else line
            if not line or not line.startswith("data: "):
                continue
            body = line[6:]
            if body.strip() == "[DONE]":
                break
            try:
                delta = (json.loads(body).get("choices") or [{}])[0].get("delta") or {}
            except json.JSONDecodeError:
                continue
            if delta.get("content"):
                chunks.append(delta["content"])
                print(delta["content"], end="", flush=True)
            for item in delta.get("images") or []:
                save_data_url((item.get("image_url") or {}).get("url", ""), out / f"{stamp}_interleave_{k}.png")
                k += 1
        (out / f"{stamp}_interleave.txt").write_text("".join(chunks), encoding="utf-8")
        print()
        return 0
    r = http.post(url, headers=headers, json=payload, timeout=a.timeout)
    r.raise_for_status()
    data = r.json()
    msg = ((data.get("choices") or [{}])[0]).get("message") or {}
    if a.mode == "vqa":
        print(msg.get("content", ""))
        return 0
    (out / f"{stamp}_{a.mode}_response.json").write_text(json.dumps(data, ensure_ascii=False, indent=1), encoding="utf-8")
    if msg.get("content"):
        print(msg["content"])
    for i, item in enumerate(msg.get("images") or []):
        save_data_url((item.get("image_url") or {}).get("url", ""), out / f"{stamp}_{a.mode}_{i}.png")
    return 0


if __name__ == "__main__":
    sys.exit(main())
