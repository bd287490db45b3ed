"""U1.5 prompt tools with a scripted back-end: JSON extraction, canvas snapping, quoted-text check, retries."""
import json

import pytest

from sensenova_u1_b200.u1_5 import (CANVAS_ROWS, RenderBriefError, caption_image, compile_render_brief,
                                    enhance_edit_prompt, extract_json, nearest_canvas)


class Scripted:
    def __init__(self, answers):
        self.answers, self.calls = list(answers), []

    def complete(self, system, user, images=()):
        self.calls.append((system, user, len(images)))
        return self.answers.pop(0)


def _brief(**kw):
    b = {"subjects": [{"description": "a saxophone"}], "scene": {}, "lighting": {}, "composition": {}, "style": {},
         "camera": {}, "visible_copy": [{"text": "JAZZ NIGHT", "category": "title"}], "image_description": "...",
         "canvas": {"aspect_ratio": "5:7"}, "negative": "garbled text"}
    b.update(kw)
    return b


def test_extract_and_canvas():
    assert extract_json('here:\n```json\n{"a": 1}\n```') == {"a": 1}
    assert extract_json('prefix {"a": {"b": 2}} suffix') == {"a": {"b": 2}}
    with pytest.raises(RenderBriefError):
        extract_json("no json here")
    assert nearest_canvas("4:3") == "3:2" and nearest_canvas("1080x1920") == "9:16" and nearest_canvas(1.0) == "1:1"
    assert nearest_canvas("21:9") == "16:9"
    with pytest.raises(RenderBriefError):
        nearest_canvas("wide")


def test_brief_is_validated_and_retried():
    req = 'poster for a jazz evening with the title "JAZZ NIGHT"'
    bad_json = "I think a poster would be nice."
    lost_text = json.dumps(_brief(visible_copy=[]))
    good = "```json\n" + json.dumps(_brief()) + "\n```"
    be = Scripted([bad_json, lost_text, good])
    out = compile_render_brief(be, req, attempts=3)
    assert len(be.calls) == 3
    assert out["canvas"] == {"aspect_ratio": "2:3", "orientation": "portrait", "resolution": "1664 x 2496"}
    assert CANVAS_ROWS[out["canvas"]["aspect_ratio"]][1:] == (1664, 2496)
    with pytest.raises(RenderBriefError):
        compile_render_brief(Scripted([bad_json, bad_json]), req, attempts=2)
    with pytest.raises(RenderBriefError):
        compile_render_brief(Scripted([]), "   ")


def test_edit_and_caption(tmp_path):
    from PIL import Image
    p = tmp_path / "in.png"
    Image.new("RGB", (1600, 900), (5, 5, 200)).save(p)
    be = Scripted(["{}", "Replace the clear sky above the roofline with falling snow; keep the house, framing and light."])
    out = enhance_edit_prompt(be, [str(p)], "make it snow")
    assert out.startswith("Replace") and be.calls[-1][2] == 1 and len(be.calls) == 2
    with pytest.raises(RenderBriefError):
        enhance_edit_prompt(be, [], "x")
    cap = caption_image(Scripted(['{"json_prompt": {"subjects": []}, "nlp_prompt": "a blue field"}']), str(p))
    assert cap["aspect_ratio"] == "16:9" and cap["size"] == [1600, 900] and cap["nlp_prompt"] == "a blue field"
