"""ComfyUI extension on CPU: node protocol, example workflows against the node definitions, image
conversions, the model cache, local nodes on a stand-in model and API nodes against the real HTTP
front-end served from a thread."""
import importlib.util
import json
import sys
import threading
import time
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
APP = ROOT / "apps" / "comfyui"


@pytest.fixture(scope="module")
def ext():
    spec = importlib.util.spec_from_file_location("snu1_comfyui", APP / "__init__.py",
                                                  submodule_search_locations=[str(APP)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["snu1_comfyui"] = mod
    spec.loader.exec_module(mod)
    return mod


BUILTIN_OUTPUTS = {"LoadImage": ("IMAGE", "MASK"), "SaveImage": ()}
BUILTIN_INPUTS = {"LoadImage": {"image": "STRING"}, "SaveImage": {"images": "IMAGE", "filename_prefix": "STRING"}}


def _input_types(cls):
    spec = cls.INPUT_TYPES()
    out = {}
    for sect in ("required", "optional"):
        for name, decl in spec.get(sect, {}).items():
            out[name] = (decl[0], sect)
    return out


def test_node_protocol(ext):
    assert set(ext.NODE_CLASS_MAPPINGS) == set(ext.NODE_DISPLAY_NAME_MAPPINGS)
    for name, cls in ext.NODE_CLASS_MAPPINGS.items():
        assert callable(getattr(cls, cls.FUNCTION)), name
        assert len(cls.RETURN_TYPES) == len(cls.RETURN_NAMES), name
        for inp, (typ, _) in _input_types(cls).items():
            assert isinstance(typ, (str, list)), (name, inp)


def test_example_workflows_match_the_nodes(ext):
    files = sorted((APP / "example_workflows").glob("*.json"))
    assert len(files) >= 4
    for f in files:
        wf = json.loads(f.read_text())
        for nid, node in wf.items():
            ct = node["class_type"]
            if ct in BUILTIN_INPUTS:
                decl = {k: (v, "required") for k, v in BUILTIN_INPUTS[ct].items()}
            else:
                assert ct in ext.NODE_CLASS_MAPPINGS, (f.name, ct)
                decl = _input_types(ext.NODE_CLASS_MAPPINGS[ct])
            required = {k for k, (_, s) in decl.items() if s == "required"}
            assert required <= set(node["inputs"]), (f.name, nid, required - set(node["inputs"]))
            for k, v in node["inputs"].items():
                assert k in decl, (f.name, nid, k)
                typ = decl[k][0]
                if isinstance(v, list):              # a link [source node, output index]: types must agree
                    src = wf[v[0]]["class_type"]
                    outs = BUILTIN_OUTPUTS[src] if src in BUILTIN_OUTPUTS else ext.NODE_CLASS_MAPPINGS[src].RETURN_TYPES
                    assert outs[v[1]] == typ, (f.name, nid, k, outs[v[1]], typ)
                elif isinstance(typ, list):          # a menu: the value must be one of the options
                    assert v in typ, (f.name, nid, k, v)


def test_image_conversions(ext):
    img = sys.modules["snu1_comfyui.images"]
    x = torch.rand(2, 48, 64, 3)
    m = img.comfy_to_model(x)
    assert len(m) == 2 and m[0].shape == (3, 48, 64) and float(m[0].min()) >= -1
    back = img.model_to_comfy(torch.stack(m))
    assert torch.allclose(back, x, atol=1e-6)
    png = img.comfy_to_png_bytes(x, 1)
    again = img.bytes_to_comfy(png)
    assert again.shape == (1, 48, 64, 3) and (again - x[1:2]).abs().max() < 1 / 255 + 1e-6
    stacked = img.stack_for_comfy([torch.zeros(3, 32, 64), torch.ones(3, 64, 32)])
    assert stacked.shape == (2, 64, 64, 3)
    assert img.data_url(x).startswith("data:image/png;base64,")


class FakeModel:
    class cfg:
        token_pixels = 32

    def __init__(self):
        self.calls = []

    def t2i_generate(self, tok, prompt, image_size=(64, 64), batch_size=1, think_mode=False, **kw):
        self.calls.append(("t2i", prompt, image_size, kw))
        img = torch.zeros(batch_size, 3, image_size[1], image_size[0])
        return (img, "thought") if think_mode else img

    def it2i_generate(self, tok, prompt, images, image_size=None, batch_size=1, **kw):
        self.calls.append(("edit", prompt, [tuple(i.shape) for i in images], image_size))
        return torch.zeros(batch_size, 3, images[0].shape[1], images[0].shape[2])

    def interleave_gen(self, tok, prompt, images=(), image_size=(64, 64), **kw):
        self.calls.append(("interleave", prompt, len(images)))
        return "once [image] upon [image] a time", [torch.zeros(3, 64, 64), torch.ones(3, 32, 96)]

    def chat(self, tok, images, question, generation_config=None, **kw):
        return f"{len(images or ())} image(s): {question}"


def test_model_cache_and_local_nodes(ext):
    local = sys.modules["snu1_comfyui.local"]
    nodes = ext.NODE_CLASS_MAPPINGS
    loads = []

    def loader(path, device, vram_mode, gguf, random_init):
        loads.append(path)
        return FakeModel(), None

    local._CACHE.clear()
    a = local.load("ckpt-a", "cpu", "full", loader=loader)
    assert local.load("ckpt-a", "cpu", "full", loader=loader) is a and loads == ["ckpt-a"]
    b = local.load("ckpt-b", "cpu", "low", loader=loader)
    assert list(local._CACHE.values()) == [b] and a.model is None          # the old one was released
    with pytest.raises(ValueError):
        local.load("ckpt-b", "cpu", "tiny", loader=loader)

    imgs, thought = nodes["SNU1LocalTextToImage"]().run(b, "a cat", 100, 70, 4, 4.0, 3.0, 1, "none", 2, True)
    assert imgs.shape == (2, 64, 96, 3) and thought == "thought"           # sides snapped to multiples of 32
    (edited,) = nodes["SNU1LocalImageEdit"]().run(b, torch.rand(1, 70, 100, 3), "snow", 4, 4.0, 3.0, 1, 1.0, "none",
                                                 image_2=torch.rand(1, 64, 64, 3))
    assert edited.shape == (1, 64, 96, 3)
    assert b.model.calls[-1][2] == [(3, 64, 96), (3, 64, 64)]
    result, text, pics = nodes["SNU1LocalInterleave"]().run(b, "story", 64, 64, 4, 4.0, 3.0, 0, 3, 64)
    assert text.count("[image]") == 2 and pics.shape == (2, 64, 96, 3)
    out = nodes["SNU1InterleavePreview"]().run(result)
    assert len(out["ui"]["images"]) == 2 and out["result"][0].count("![picture") == 2
    local._CACHE.clear()


@pytest.fixture()
def served(monkeypatch):
    import socket
    import uvicorn
    from sensenova_u1_b200.serving import GenerationService, create_app
    svc = GenerationService(FakeModel(), None, max_batch=2, batch_wait_s=0.01)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    server = uvicorn.Server(uvicorn.Config(create_app(svc), host="127.0.0.1", port=port, log_level="error"))
    t = threading.Thread(target=server.run, daemon=True)
    t.start()
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.05)
    assert server.started
    monkeypatch.setenv("SENSENOVA_BASE_URL", f"http://127.0.0.1:{port}")
    monkeypatch.setenv("SENSENOVA_RETRIES", "0")
    yield svc
    server.should_exit = True
    t.join(timeout=5)
    svc.close()


def test_api_nodes_against_the_http_front_end(ext, served):
    nodes = ext.NODE_CLASS_MAPPINGS
    image, info, raw = nodes["SNU1ImageGenerate"]().run("a fox", "sensenova-u1", "512x512|1:1", 2, 4.0, 0, 60)
    assert image.shape == (1, 512, 512, 3) and "512x512" in info and "b64_json" not in raw
    text, _ = nodes["SNU1VisionImage"]().run(torch.rand(1, 64, 64, 3), "what is it?", "sensenova-u1", 32, 60)
    assert text == "1 image(s): what is it?"
    text, usage, raw = nodes["SNU1Chat"]().run("hello", "be brief", "sensenova-u1", 0.7, 1.0, 16, 60)
    assert text == "0 image(s): hello" and json.loads(raw)["object"] == "chat.completion"
    prompt, _ = nodes["SNU1PromptBuilder"]().run("jazz night", "poster", "1664x2496|2:3", "sensenova-u1", 60)
    assert prompt.endswith("jazz night")
    assert "poster style" in nodes["SNU1PromptBuilder"].system_prompt("poster", "1664x2496|2:3")
    with pytest.raises(ValueError):
        nodes["SNU1VisionURL"]().run("file:///etc/passwd", "?", "m", 8, 10)
    client = sys.modules["snu1_comfyui.client"]
    with pytest.raises(client.ApiError):
        client.ApiClient.from_env().edit_image("x", [], timeout=10)           # 400: not retried, reported
    with pytest.raises(ValueError):
        client.parse_size("500x500|1:1")


def test_config_env_file_install_and_loader_options(ext, tmp_path, monkeypatch):
    cfg_mod = sys.modules["snu1_comfyui.config"] if "snu1_comfyui.config" in sys.modules else \
        importlib.import_module("snu1_comfyui.config")
    env = tmp_path / ".env"
    env.write_text("# comment\nexport SN_API_KEY='abc'\nSN_BASE_URL=https://example.invalid/v1/\n")
    c = cfg_mod.load_config([env], environ={})
    assert c.api_key == "abc" and c.base_url == "https://example.invalid/v1"
    c = cfg_mod.load_config([env], environ={"SENSENOVA_BASE_URL": "http://127.0.0.1:9"})       # environment wins per name
    assert c.base_url in ("https://example.invalid/v1", "http://127.0.0.1:9") and c.api_key == "abc"
    with pytest.raises(RuntimeError):
        cfg_mod.load_config([], require_key=True, environ={})
    # install: link, refuse to overwrite, replace with a copy, remove
    inst = importlib.import_module("snu1_comfyui.install")
    comfy = tmp_path / "ComfyUI"
    (comfy / "custom_nodes").mkdir(parents=True)
    dst = inst.install(comfy)
    assert dst.is_symlink() and (dst / "nodes.py").is_file()
    with pytest.raises(SystemExit):
        inst.install(comfy)
    dst = inst.install(comfy, copy=True, force=True)
    assert not dst.is_symlink() and (dst / "repo_root.txt").read_text().strip() == str(ROOT)
    assert inst.uninstall(comfy) and not dst.exists()
    with pytest.raises(SystemExit):
        inst.install(tmp_path / "nowhere")
    # loader options
    local = sys.modules["snu1_comfyui.local"]
    assert local.parse_max_memory("0=20GiB, cpu=64GiB") == {0: "20GiB", "cpu": "64GiB"}
    with pytest.raises(ValueError):
        local.parse_max_memory("20GiB")
    gib = 1 << 30
    kw = local.fast_offload_kwargs("cuda", "fast", 0.5, 2.0, 4.0, 0.0, mem_info=(60 * gib, 80 * gib))
    assert kw == {"resident_budget_bytes": 36 * gib}                      # min(0.5 * 80, 60 - 2) - 4
    assert local.fast_offload_kwargs("cuda", "fast", 0.9, 2.0, 4.0, 10.0, mem_info=(1, 1)) == {"resident_budget_bytes": 6 * gib}
    assert local.fast_offload_kwargs("cuda", "balanced") is None
    spec = ext.NODE_CLASS_MAPPINGS["SNU1LocalLoader"].INPUT_TYPES()
    assert {"dtype", "max_memory", "fast_vram_budget_gib"} <= set(spec["optional"])
