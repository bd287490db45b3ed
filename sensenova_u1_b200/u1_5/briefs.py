"""Render briefs, edit instructions and captions for the U1.5 models.

* :func:`compile_render_brief`  free-text request -> structured JSON brief (subjects, scene, lighting,
  composition, style, camera, visible text, canvas) that the generator is prompted with (reference
  src/sensenova_u1_5/image_pe.py:29-167).  The canvas is always one of five fixed 2K sizes.
* :func:`enhance_edit_prompt`   (images, short instruction) -> precise edit instruction that names the region,
  the change and what must stay (reference src/sensenova_u1_5/edit/edit_pe.py:150-230).
* :func:`caption_image`         image -> JSON brief + natural-language prompt, with the target aspect ratio
  snapped to the supported set (reference src/sensenova_u1_5/caption/caption.py:64-119).

All three take a ``backend`` with ``complete(system, user, images) -> str``
(``sensenova_u1_b200.inference.prompt_enhance``: chat-completions, Anthropic or the local model); answers are
validated and the request is retried when the model returns something unusable.

    python -m sensenova_u1_b200.u1_5.briefs brief --prompt "poster for a jazz night"
    python -m sensenova_u1_b200.u1_5.briefs edit --image in.png --prompt "make it snow"
    python -m sensenova_u1_b200.u1_5.briefs caption --image in.png
"""
from __future__ import annotations

import base64
import io
import json
import re
from typing import Any, Dict, List, Optional, Sequence, Tuple

# aspect label -> (orientation, width, height): the sizes the U1.5 generator is trained at
CANVAS_ROWS: Dict[str, Tuple[str, int, int]] = {
    "1:1": ("square", 2048, 2048),
    "3:2": ("landscape", 2496, 1664),
    "2:3": ("portrait", 1664, 2496),
    "16:9": ("landscape", 2720, 1536),
    "9:16": ("portrait", 1536, 2720),
}
CAPTION_RATIOS = {"16:9": 16 / 9, "3:2": 3 / 2, "4:3": 4 / 3, "1:1": 1.0, "3:4": 3 / 4, "2:3": 2 / 3, "9:16": 9 / 16}
BRIEF_KEYS = ("subjects", "scene", "lighting", "composition", "style", "camera", "visible_copy", "image_description",
              "canvas", "negative")

BRIEF_SYSTEM = (
    "You compile an image request into ONE JSON object that fully specifies the finished picture for a "
    "text-to-image model. Output raw JSON only, with exactly these keys: "
    "subjects (list of {description, appearance_action, relationship_position, count_anatomy}), "
    "scene {setting, spatial_layers, supporting_details[]}, lighting {conditions, direction, shadow_effect}, "
    "composition {framing, hierarchy_flow, negative_space}, style {medium, art_direction, palette_materials}, "
    "camera {viewpoint, lens_focus}, visible_copy (list of {text, category, placement, appearance}), "
    "image_description (one paragraph), canvas {aspect_ratio, orientation, resolution}, negative (short). "
    "Keep every subject, count, relation, colour and quoted string of the request; decide everything left open "
    "(viewpoint, light, materials, spacing) instead of listing alternatives. visible_copy lists every string that "
    "must be readable in the picture, character for character, and nothing else; pictures that were not asked to "
    "contain text get an empty list. Never invent brands, names, prices, dates or statistics. "
    "canvas.aspect_ratio is one of 1:1, 3:2, 2:3, 16:9, 9:16: phone or story formats 9:16, posters, covers and "
    "infographics 2:3, screens and slides 16:9, landscape photography 3:2, anything else 1:1.")
EDIT_SYSTEM = (
    "You rewrite a short image-editing request into one precise instruction for an image-editing model, after "
    "looking at the attached picture(s). Name the object or region to change (by position when ambiguous), state "
    "exactly what it becomes, and state what must not change: identity and pose of people, background, framing, "
    "lighting and any text. Refer to several inputs as image 1, image 2, ... One paragraph, no preamble, in the "
    "language of the request.")
CAPTION_SYSTEM = (
    "Describe the attached picture for re-creation by a text-to-image model. Output raw JSON only: "
    "{\"json_prompt\": {subjects, scene, lighting, composition, style, camera, visible_copy}, "
    "\"nlp_prompt\": one dense paragraph}. Quote visible text exactly; do not guess identities or brands.")


class RenderBriefError(ValueError):
    pass


def extract_json(text: str) -> Dict[str, Any]:
    """The JSON object inside a model answer (plain, fenced, or surrounded by prose)."""
    t = text.strip()
    m = re.search(r"```(?:json)?\s*(.*?)```", t, flags=re.S)
    if m:
        t = m.group(1).strip()
    a, b = t.find("{"), t.rfind("}")
    if a < 0 or b < a:
        raise RenderBriefError("the answer contains no JSON object")
    try:
        out = json.loads(t[a:b + 1])
    except ValueError as e:
        raise RenderBriefError(f"the answer is not valid JSON: {e}") from e
    if not isinstance(out, dict):
        raise RenderBriefError("the answer's JSON is not an object")
    return out


def nearest_canvas(ratio, rows: Optional[Dict[str, Any]] = None) -> str:
    """The supported aspect label closest (in log ratio) to ``ratio`` (a float, ``"W:H"`` or ``"WxH"``)."""
    import math
    if isinstance(ratio, str):
        m = re.match(r"\s*(\d+(?:\.\d+)?)\s*[:xX/]\s*(\d+(?:\.\d+)?)\s*$", ratio)
        if not m or float(m.group(2)) == 0:
            raise RenderBriefError(f"not an aspect ratio: {ratio!r}")
        ratio = float(m.group(1)) / float(m.group(2))
    rows = rows if rows is not None else {k: w / h for k, (_, w, h) in CANVAS_ROWS.items()}
    return min(rows, key=lambda k: abs(math.log(rows[k]) - math.log(ratio)))


def validate_brief(brief: Dict[str, Any], request: str = "") -> Dict[str, Any]:
    """Checks the key set, snaps the canvas to a supported row and verifies that every quoted string of the
    request survived in ``visible_copy``.  Returns the (normalised) brief; raises :class:`RenderBriefError`."""
    missing = [k for k in BRIEF_KEYS if k not in brief]
    if missing:
        raise RenderBriefError(f"brief lacks {missing}")
    if not isinstance(brief["subjects"], list) or not isinstance(brief["visible_copy"], list):
        raise RenderBriefError("subjects and visible_copy must be lists")
    canvas = brief["canvas"] if isinstance(brief["canvas"], dict) else {}
    label = nearest_canvas(str(canvas.get("aspect_ratio") or "1:1"))
    orient, w, h = CANVAS_ROWS[label]
    brief["canvas"] = {"aspect_ratio": label, "orientation": orient, "resolution": f"{w} x {h}"}
    copy_texts = [str(c.get("text", "")) for c in brief["visible_copy"] if isinstance(c, dict)]
    for quoted in re.findall(r"[\"“]([^\"”]{2,})[\"”]", request):
        if not any(quoted == t or quoted in t for t in copy_texts):
            raise RenderBriefError(f"the quoted text {quoted!r} is missing from visible_copy")
    return brief


def _retry(fn, attempts: int):
    err: Optional[Exception] = None
    for _ in range(max(1, attempts)):
        try:
            return fn()
        except RenderBriefError as e:
            err = e
    raise RenderBriefError(f"no usable answer after {attempts} attempts: {err}")


def compile_render_brief(backend, request: str, attempts: int = 3) -> Dict[str, Any]:
    request = request.strip()
    if not request:
        raise RenderBriefError("the request is empty")
    return _retry(lambda: validate_brief(extract_json(backend.complete(BRIEF_SYSTEM, request)), request), attempts)


def brief_size(brief: Dict[str, Any]) -> Tuple[int, int]:
    _, w, h = CANVAS_ROWS[brief["canvas"]["aspect_ratio"]]
    return w, h


def encode_image(image, max_side: int = 2048, fmt: str = "PNG") -> str:
    """Path, bytes or PIL image -> base64 (RGB, longest side bounded)."""
    from PIL import Image
    if isinstance(image, (bytes, bytearray)):
        im = Image.open(io.BytesIO(image))
    elif isinstance(image, str) or hasattr(image, "__fspath__"):
        im = Image.open(image)
    else:
        im = image
    im = im.convert("RGB")
    if max(im.size) > max_side:
        s = max_side / max(im.size)
        im = im.resize((max(1, round(im.width * s)), max(1, round(im.height * s))), Image.LANCZOS)
    buf = io.BytesIO()
    im.save(buf, format=fmt)
    return base64.b64encode(buf.getvalue()).decode()


def enhance_edit_prompt(backend, images: Sequence, prompt: str, attempts: int = 3) -> str:
    prompt = prompt.strip()
    if not prompt:
        raise RenderBriefError("the edit request is empty")
    if not images:
        raise RenderBriefError("an edit request needs at least one image")
    enc = [encode_image(i) for i in images]
    user = (f"{len(enc)} input images. " if len(enc) > 1 else "") + "Request: " + prompt

    def once():
        out = backend.complete(EDIT_SYSTEM, user, enc).strip().strip("`").strip()
        if len(out) < len(prompt) // 2 or out.startswith("{"):
            raise RenderBriefError("the rewritten instruction is empty or not prose")
        return out
    return _retry(once, attempts)


def caption_image(backend, image, attempts: int = 3) -> Dict[str, Any]:
    """{"json_prompt": {...}, "nlp_prompt": str, "aspect_ratio": label, "size": [w, h]}"""
    from PIL import Image
    im = Image.open(image) if not hasattr(image, "size") else image
    label = nearest_canvas(im.width / im.height, CAPTION_RATIOS)
    enc = encode_image(im)

    def once():
        out = extract_json(backend.complete(CAPTION_SYSTEM, "Describe this picture.", [enc]))
        if not isinstance(out.get("json_prompt"), dict) or not str(out.get("nlp_prompt", "")).strip():
            raise RenderBriefError("caption lacks json_prompt / nlp_prompt")
        return out
    out = _retry(once, attempts)
    out["aspect_ratio"] = label
    out["size"] = [im.width, im.height]
    return out


def main(argv=None) -> int:
    import argparse
    from ..inference.prompt_enhance import backend_from_env
    ap = argparse.ArgumentParser(description="U1.5 prompt tools (endpoint from U1_ENHANCE_* environment variables)")
    ap.add_argument("task", choices=["brief", "edit", "caption"])
    ap.add_argument("--prompt", default="")
    ap.add_argument("--image", action="append", default=[])
    ap.add_argument("--attempts", type=int, default=3)
    a = ap.parse_args(argv)
    backend = backend_from_env()
    if a.task == "brief":
        out: Any = compile_render_brief(backend, a.prompt, a.attempts)
    elif a.task == "edit":
        out = enhance_edit_prompt(backend, a.image, a.prompt, a.attempts)
    else:
        out = caption_image(backend, a.image[0], a.attempts)
    print(out if isinstance(out, str) else json.dumps(out, ensure_ascii=False, separators=(",", ":")))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
