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

    def chat(self, tok, images, question, generation_config=None, **kw):
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


def test_reference_client_payloads_and_this_client(client, tmp_path):
    """The chat-completions dialect of the reference's serving client: ``modalities == ["image"]`` with an
    ``image_config`` for text-to-image and editing, streamed interleaved answers with pictures in ``delta.images``;
    and this repository's client (same modes and flags) end to end against the app."""
    import importlib.util
    import json
    import os
    from sensenova_u1_b200.serving.server import image_size_from_config
    c, svc = client
    assert image_size_from_config({"width": 100, "height": 70, "seed": 5}) == (96, 64, 5)
    assert image_size_from_config({"aspect_ratio": "16:9", "image_size": "1K", "width": -1, "height": -1})[:2] == (1376, 768)
    assert image_size_from_config(None, default=(512, 512))[:2] == (512, 512)
    body = {"model": "m", "messages": [{"role": "system", "content": "s"}, {"role": "user", "content": "a fox"}],
            "modalities": ["image"], "stream": False, "chat_template_kwargs": {"enable_thinking": True},
            "image_config": {"width": 64, "height": 96, "seed": 3}}
    r = c.post("/v1/chat/completions", json=body, headers={"Authorization": "Bearer EMPTY"})
    msg = r.json()["choices"][0]["message"]
    assert r.status_code == 200 and msg["content"] == "thought" and msg["images"][0]["image_url"]["url"].startswith("data:image/png")
    body["messages"][1]["content"] = [{"type": "image_url", "image_url": {"url": "data:image/png;base64," + _png()}},
                                      {"type": "text", "text": "night"}]
    r = c.post("/chat/completions", json=body)                       # also without the /v1 prefix
    assert r.status_code == 200 and len(r.json()["choices"][0]["message"]["images"]) == 1
    assert ("edit", "night", 1) in svc.model.calls
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "story"}], "stream": True,
                                             "modalities": ["text", "image"], "image_config": {"aspect_ratio": "1:1", "image_size": "0.5K"}})
    deltas = [json.loads(ln[6:])["choices"][0]["delta"] for ln in r.text.splitlines() if ln.startswith("data: {")]
    assert any(d.get("content", "").startswith("hello") for d in deltas) and any(d.get("images") for d in deltas)
    assert "data: [DONE]" in r.text
    # this repository's client against the same app
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("snu1_client", os.path.join(root, "examples", "serving", "client.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    class Session:                    # requests-like face of the test client
        def post(self, url, headers=None, json=None, stream=False, timeout=None):
            resp = c.post(url.replace("http://testserver", ""), json=json, headers=headers)
            resp.iter_lines = lambda: iter(resp.text.splitlines())
            return resp
    out = tmp_path / "o"
    args = ["--url", "http://testserver/v1", "--out-dir", str(out), "--prompt", "a fox"]
    assert mod.main(["--mode", "t2i", "--width", "64", "--height", "64"] + args, session=Session()) == 0
    assert len(list(out.glob("*_t2i_0.png"))) == 1 and len(list(out.glob("*_t2i_response.json"))) == 1
    img = tmp_path / "in.png"
    img.write_bytes(base64.b64decode(_png()))
    assert mod.main(["--mode", "it2i", "--image_path", str(img)] + args, session=Session()) == 0
    assert mod.main(["--mode", "interleave", "--image-size", "0.5K"] + args, session=Session()) == 0
    assert len(list(out.glob("*_interleave_0.png"))) == 1 and list(out.glob("*_interleave.txt"))[0].read_text().startswith("hello")
    assert mod.main(["--mode", "vqa", "--image_path", str(img)] + args, session=Session()) == 0


def test_balancer_spreads_requests_and_skips_dead_replicas():
    import httpx
    from fastapi.testclient import TestClient
    from sensenova_u1_b200.serving.balancer import Backends, create_balancer_app, replica_commands

    alive = {"a:1": True, "b:2": True, "c:3": False}
    hits = []

    def handler(req: httpx.Request) -> httpx.Response:
        host = f"{req.url.host}:{req.url.port}"
        if not alive[host]:
            raise httpx.ConnectError("refused", request=req)
        if req.url.path == "/health":
            return httpx.Response(200, json={"status": "ok"})
        hits.append((host, req.url.path, req.url.query.decode(), req.content))
        if req.url.path == "/v1/stream":
            return httpx.Response(200, content=b"data: one\n\ndata: [DONE]\n\n", headers={"content-type": "text/event-stream"})
        return httpx.Response(201, json={"from": host}, headers={"x-replica": host})

    client = httpx.AsyncClient(transport=httpx.MockTransport(handler))
    app = create_balancer_app(["http://a:1/", "http://b:2", "http://c:3"], health_interval=3600, startup_timeout=1.0, client=client)
    with TestClient(app) as tc:
        st = tc.get("/_lb/status").json()
        assert st["healthy"] == {"http://a:1": True, "http://b:2": True, "http://c:3": False}
        got = [tc.post("/v1/chat/completions?x=1", json={"k": i}) for i in range(4)]
        assert [r.status_code for r in got] == [201] * 4 and got[0].headers["x-replica"] in ("a:1", "b:2")
        assert sorted(h[0] for h in hits) == ["a:1", "a:1", "b:2", "b:2"]        # ties go to the replica used least recently
        assert hits[0][1:3] == ("/v1/chat/completions", "x=1") and b'"k"' in hits[0][3]
        r = tc.get("/v1/stream")
        assert r.text.endswith("data: [DONE]\n\n") and r.headers["content-type"].startswith("text/event-stream")
        assert all(v == 0 for v in tc.get("/_lb/status").json()["inflight"].values())
        alive["a:1"] = alive["b:2"] = False                                        # everything down: the error is reported
        r = tc.post("/v1/chat/completions", json={})
        assert r.status_code == 502 and "unreachable" in r.json()["error"]
    b = Backends(["http://x:1", "http://y:2"])
    b.mark("http://x:1", True), b.mark("http://y:2", True)
    b.enter("http://x:1")
    assert b.pick() == "http://y:2"                                                # fewest in flight
    cmds = replica_commands(2, 8100, ["--model_path", "CKPT"], gpus=[4, 6])
    assert cmds[1][0][-4:] == ["--port", "8101", "--model_path", "CKPT"][-4:] and cmds[1][1] == {"CUDA_VISIBLE_DEVICES": "6"}
    assert cmds[0][2] == "http://127.0.0.1:8100"


def test_chat_sampling_knobs_reach_the_generation_config(client):
    from sensenova_u1_b200.serving.server import sampling_from_body
    assert sampling_from_body({}) == {} and sampling_from_body({"temperature": 0, "top_p": 0.9}) == {}
    assert sampling_from_body({"temperature": 0.6, "top_p": 0.95, "extra_body": {"top_k": 20, "repetition_penalty": 1.05}}) == \
        {"do_sample": True, "temperature": 0.6, "top_p": 0.95, "top_k": 20, "repetition_penalty": 1.05}
    assert sampling_from_body({"repetition_penalty": 1.1}) == {"repetition_penalty": 1.1}
    tc, svc = client
    seen = {}
    orig = svc.model.chat
    svc.model.chat = lambda tok, images, prompt, generation_config=None, **kw: seen.update(generation_config) or "ok"
    try:
        r = tc.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 7,
                                                  "temperature": 0.8, "top_p": 0.9, "seed": 5})
    finally:
        svc.model.chat = orig
    assert r.status_code == 200 and r.json()["choices"][0]["message"]["content"] == "ok"
    assert seen == {"max_new_tokens": 7, "do_sample": True, "temperature": 0.8, "top_p": 0.9, "seed": 5}


def test_system_message_and_history_reach_the_model(client):
    from sensenova_u1_b200.serving.server import _split_messages
    msgs = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "one"},
            {"role": "assistant", "content": "1"}, {"role": "user", "content": [{"type": "text", "text": "two"}]}]
    assert _split_messages(msgs, 32) == ("two", [], "Be brief.", [("one", "1")])
    tc, svc = client
    seen = {}
    orig = svc.model.chat

    def chat(tok, images, prompt, generation_config=None, **kw):
        seen.update(kw, prompt=prompt)
        return "2"
    svc.model.chat = chat
    try:
        r = tc.post("/v1/chat/completions", json={"messages": msgs})
        assert r.json()["choices"][0]["message"]["content"] == "2"
        assert seen == {"history": [("one", "1")], "system_message": "Be brief.", "prompt": "two"}
        seen.clear()
        tc.post("/v1/chat/completions", json={"messages": msgs[-1:]})
        assert seen == {"prompt": "two"}                     # nothing extra for a single-turn request
    finally:
        svc.model.chat = orig


def test_interleaved_requests_carry_system_message_thinking_and_size(client):
    tc, svc = client
    seen = {}
    orig = svc.model.interleave_gen

    def gen(tok, prompt, images=(), **kw):
        seen.update(kw, prompt=prompt)
        return "t [image]", [torch.zeros(3, 32, 32)]
    svc.model.interleave_gen = gen
    try:
        r = tc.post("/v1/chat/completions", json={
            "messages": [{"role": "system", "content": "SYS"}, {"role": "user", "content": "draw"}], "interleave": True,
            "size": "640x384", "chat_template_kwargs": {"enable_thinking": True}, "cfg_scale": 3.5, "max_rounds": 2})
    finally:
        svc.model.interleave_gen = orig
    assert r.status_code == 200 and r.json()["choices"][0]["message"]["content"][0]["text"] == "t [image]"
    assert seen["system_message"] == "SYS" and seen["think_mode"] is True and seen["image_size"] == (640, 384)
    assert seen["cfg_scale"] == 3.5 and seen["max_rounds"] == 2 and seen["prompt"] == "draw"


def test_request_pixel_budget_sizes_the_input_picture(client):
    from sensenova_u1_b200.serving.server import _decode_image
    b64 = _png(320, 256)
    assert _decode_image(b64, 32).shape[1:] == (256, 320)
    small = _decode_image(b64, 32, max_pixels=128 * 128)
    assert small.shape[1] * small.shape[2] <= 128 * 128 and small.shape[1] % 32 == 0
    tc, svc = client
    seen = {}
    orig = svc.model.chat
    svc.model.chat = lambda tok, images, prompt, generation_config=None, **kw: seen.update(shape=tuple(images[0].shape)) or "ok"
    try:
        tc.post("/v1/chat/completions", json={"max_pixels": 128 * 128, "messages": [{"role": "user", "content": [
            {"type": "text", "text": "q"}, {"type": "image_url", "image_url": {"url": "data:image/png;base64," + b64}}]}]})
    finally:
        svc.model.chat = orig
    assert seen["shape"][1] * seen["shape"][2] <= 128 * 128
