#!/usr/bin/env python
"""Client for the OpenAI-style server (python -m sensenova_u1_b200.serving.server); same four
tasks as the reference client (examples/serving/client.py:204-356): t2i, it2i (editing),
interleave, vqa.

    python examples/serving/client.py t2i --prompt "a red fox" --size 1024x1024 --output fox.png
    python examples/serving/client.py it2i --image in.png --prompt "make it night" --output night.png
    python examples/serving/client.py interleave --prompt "a story in two pictures" --output_dir out
    python examples/serving/client.py vqa --image in.png --prompt "what is shown?"
"""
import argparse
import base64
import json
import os
import sys


def _b64_file(path):
    with open(path, "rb") as f:
        return base64.b64encode(f.read()).decode()


def _save_b64(data, path):
    with open(path, "wb") as f:
        f.write(base64.b64decode(data))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("task", choices=["t2i", "it2i", "interleave", "vqa"])
    ap.add_argument("--base_url", default="http://127.0.0.1:8000")
    ap.add_argument("--prompt", required=True)
    ap.add_argument("--image", action="append", default=[])
    ap.add_argument("--size", default="1024x1024")
    ap.add_argument("--n", type=int, default=1)
    ap.add_argument("--num_steps", type=int, default=50)
    ap.add_argument("--cfg_scale", type=float, default=4.0)
    ap.add_argument("--img_cfg_scale", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--max_tokens", type=int, default=256)
    ap.add_argument("--output", default="out.png")
    ap.add_argument("--output_dir", default="interleave_out")
    ap.add_argument("--timeout", type=float, default=3600)
    a = ap.parse_args(argv)
    import requests
    post = lambda route, body: requests.post(a.base_url + route, json=body, timeout=a.timeout)
    if a.task == "t2i":
        r = post("/v1/images/generations", {"prompt": a.prompt, "size": a.size, "n": a.n, "num_steps": a.num_steps,
                                            "cfg_scale": a.cfg_scale, "seed": a.seed})
    elif a.task == "it2i":
        r = post("/v1/images/edits", {"prompt": a.prompt, "image": [_b64_file(p) for p in a.image], "n": a.n,
                                      "num_steps": a.num_steps, "cfg_scale": a.cfg_scale,
                                      "img_cfg_scale": a.img_cfg_scale, "seed": a.seed})
    else:
        content = [{"type": "text", "text": a.prompt}] + [
            {"type": "image_url", "image_url": {"url": "data:image/png;base64," + _b64_file(p)}} for p in a.image]
        r = post("/v1/chat/completions", {"messages": [{"role": "user", "content": content}],
                                          "interleave": a.task == "interleave", "max_tokens": a.max_tokens,
                                          "num_steps": a.num_steps, "seed": a.seed})
    r.raise_for_status()
    body = r.json()
    if a.task in ("t2i", "it2i"):
        for i, d in enumerate(body["data"]):
            _save_b64(d["b64_json"], a.output if len(body["data"]) == 1 else a.output.replace(".png", f"_{i}.png"))
        print(f"saved {len(body['data'])} image(s)")
    else:
        content = body["choices"][0]["message"]["content"]
        if isinstance(content, str):
            print(content)
        else:
            os.makedirs(a.output_dir, exist_ok=True)
            k = 0
            for part in content:
                if part["type"] == "text":
                    print(part["text"])
                else:
                    _save_b64(part["image_url"]["url"].split(",", 1)[1], os.path.join(a.output_dir, f"image_{k}.png"))
                    k += 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
