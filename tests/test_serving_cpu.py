"""HTTP front-end on CPU with a stand-in model: routes, queueing, batching of equal T2I requests,
error isolation."""
import base64
import io
import threading

import pytest
import torch


class FakeModel:
    class cfg:
        token_pixels = 32

    def __init__(self):
        self.calls = []

    def t2i_generate(self, tok, prompt, image_size=(64, 64), batch_size=1, think_mode=False, **kw):
        self.calls.append(("t2i", prompt, batch_size))
        if prompt == "boom":
            raise ValueError("bad prompt")
        img = torch.zeros(batch_size, 3, image_size[1], image_size[0])
        for i in range(batch_size):
            img[i] += i * 0.1
        return (img, "thought") if think_mode else img

    def it2i_generate(self, tok, prompt, images, image_size=None, batch_size=1, **kw):
        self.calls.append(("edit", prompt, len(images)))
        return torch.zeros(batch_size, 3, images[0].shape[1], images[0].shape[2])

    def interleave_gen(self, tok, prompt, images=(), **kw):
        return "hello [image]", [torch.zeros(3, 32, 32)]

    def chat(self, tok, images, question, generation_config=None):
        return "answer to " + question


@pytest.fixture()
def client():
    from fastapi.testclient import TestClient
    from sensenova_u1_b200.serving import GenerationService, create_app
    svc = GenerationService(FakeModel(), None, max_batch=4, batch_wait_s=0.2)
    yield TestClient(create_app(svc)), svc
    svc.close()


def _png(w=64, h=64):
    from PIL import Image
    buf = io.BytesIO()
    Image.new("RGB", (w, h), (10, 200, 30)).save(buf, format="PNG")
    return base64.b64encode(buf.getvalue()).decode()


def test_routes(client):
    c, svc = client
    assert c.get("/health").json()["status"] == "ok"
    r = c.post("/v1/images/generations", json={"prompt": "a cat", "size": "64x96", "n": 2, "num_steps": 2})
    assert r.status_code == 200 and len(r.json()["data"]) == 2
    from PIL import Image
    im = Image.open(io.BytesIO(base64.b64decode(r.json()["data"][0]["b64_json"])))
    assert im.size == (64, 96)
    r = c.post("/v1/images/edits", json={"prompt": "night", "image": _png()})
    assert r.status_code == 200 and len(r.json()["data"]) == 1
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [
        {"type": "text", "text": "what?"}, {"type": "image_url", "image_url": {"url": "data:image/png;base64," + _png()}}]}]})
    assert r.json()["choices"][0]["message"]["content"] == "answer to what?"
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "story"}], "interleave": True})
    parts = r.json()["choices"][0]["message"]["content"]
    assert parts[0]["text"].startswith("hello") and parts[1]["type"] == "image_url"
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "stream": True})
    assert "data: [DONE]" in r.text


def test_error_does_not_kill_the_worker(client):
    c, svc = client
    assert c.post("/v1/images/generations", json={"prompt": "boom", "size": "64x64"}).status_code == 500
    assert c.post("/v1/images/generations", json={"prompt": "fine", "size": "64x64"}).status_code == 200
    assert svc.stats["errors"] == 1


def test_equal_requests_are_merged_into_one_batch(client):
    c, svc = client
    # hold the worker with one request, queue three equal ones behind it
    res = []
    ts = [threading.Thread(target=lambda: res.append(svc.submit("t2i", prompt="same", width=64, height=64, n=1)))
          for _ in range(4)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert len(res) == 4 and all(len(r["images"]) == 1 for r in res)
    batched = [c_ for c_ in svc.model.calls if c_[0] == "t2i" and c_[1] == "same"]
    assert sum(b[2] for b in batched) == 4 and len(batched) < 4
