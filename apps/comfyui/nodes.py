"""ComfyUI nodes for this framework: API nodes (HTTP, OpenAI-style routes) and local nodes
(in-process ``NEOChatModel``).

The node set follows the reference extension (apps/comfyui/nodes.py:217-1031: chat, image generate,
prompt builder, vision by URL / by image, local loader, local text-to-image / edit / interleave,
interleave preview).  The nodes are written against ComfyUI's plain class protocol
(``INPUT_TYPES`` / ``RETURN_TYPES`` / ``FUNCTION``), which every ComfyUI version loads and which
needs no ComfyUI import, so the module also loads (and is tested) outside ComfyUI.
"""
from __future__ import annotations

import json
import logging
import os
from pathlib import Path

import torch

try:                                    # inside ComfyUI the folder is a package
    from . import images as _img
    from . import local as _local
    from .client import IMAGE_SIZE_OPTIONS, ApiClient, parse_size
except ImportError:                     # direct import in tests
    import images as _img               # type: ignore
    import local as _local              # type: ignore
    from client import IMAGE_SIZE_OPTIONS, ApiClient, parse_size   # type: ignore

LOGGER = logging.getLogger("sensenova_u1_b200.comfyui")
CATEGORY = "SenseNova-U1 (B200)"
LOCAL_CATEGORY = CATEGORY + "/Local"
MODEL_TYPE = "SNU1_LOCAL_MODEL"
INTERLEAVE_TYPE = "SNU1_INTERLEAVE_RESULT"
VISION_SYSTEM_PROMPT = "You are a careful vision assistant. Describe only what is visible."
STYLES = ("photographic", "illustration", "infographic", "poster", "3d render", "watercolour")


def _gguf_options():
    """``""`` (no GGUF) plus every .gguf file in ComfyUI's model folders, when running inside ComfyUI."""
    found = set()
    try:
        import folder_paths               # ComfyUI module
        for folder in ("gguf", "diffusion_models"):
            try:
                found.update(f for f in folder_paths.get_filename_list(folder) if f.lower().endswith(".gguf"))
            except Exception:
                continue
    except Exception:
        pass
    return ["", *sorted(found)]


def _resolve_gguf(name: str) -> str:
    if not name:
        return ""
    try:
        import folder_paths
        for folder in ("gguf", "diffusion_models"):
            try:
                full = folder_paths.get_full_path(folder, name)
            except Exception:
                continue
            if full:
                return full
    except Exception:
        pass
    return name                           # a literal path typed into the workflow JSON


# ------------------------------------------------------------------------------------------------
# API nodes
# ------------------------------------------------------------------------------------------------
class SNU1Chat:
    CATEGORY, FUNCTION = CATEGORY, "run"
    RETURN_TYPES, RETURN_NAMES = ("STRING", "STRING", "STRING"), ("text", "usage_json", "raw_json")

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {
            "text": ("STRING", {"multiline": True, "default": ""}),
            "system_prompt": ("STRING", {"multiline": True, "default": "You are a helpful assistant."}),
            "model": ("STRING", {"default": "sensenova-u1"}),
            "temperature": ("FLOAT", {"default": 0.7, "min": 0.0, "max": 2.0, "step": 0.1}),
            "top_p": ("FLOAT", {"default": 1.0, "min": 0.0, "max": 1.0, "step": 0.05}),
            "max_tokens": ("INT", {"default": 2048, "min": 1, "max": 65536}),
            "timeout": ("INT", {"default": 120, "min": 10, "max": 3600})}}

    def run(self, text, system_prompt, model, temperature, top_p, max_tokens, timeout):
        r = ApiClient.from_env().chat(text, system_prompt, model, temperature, top_p, max_tokens, timeout)
        return r.text, json.dumps(r.usage, ensure_ascii=False), json.dumps(r.raw, ensure_ascii=False)


class SNU1ImageGenerate:
    CATEGORY, FUNCTION = CATEGORY, "run"
    RETURN_TYPES, RETURN_NAMES = ("IMAGE", "STRING", "STRING"), ("images", "image_info", "raw_json")

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {
            "prompt": ("STRING", {"multiline": True, "default": ""}),
            "model": ("STRING", {"default": "sensenova-u1"}),
            "size": (list(IMAGE_SIZE_OPTIONS), {"default": IMAGE_SIZE_OPTIONS[0]}),
            "steps": ("INT", {"default": 50, "min": 1, "max": 200}),
            "cfg_scale": ("FLOAT", {"default": 4.0, "min": 1.0, "max": 20.0, "step": 0.1}),
            "seed": ("INT", {"default": 0, "min": 0, "max": 2**31 - 1}),
            "timeout": ("INT", {"default": 300, "min": 30, "max": 3600})}}

    def run(self, prompt, model, size, steps, cfg_scale, seed, timeout):
        r = ApiClient.from_env().generate_image(prompt, model, parse_size(size), 1, timeout, num_steps=steps,
                                                cfg_scale=cfg_scale, seed=seed)
        image = torch.cat([_img.bytes_to_comfy(b) for b in r.images], 0)
        raw = {k: v for k, v in r.raw.items() if k != "data"}        # the base64 payload is not worth echoing
        return image, _img.describe(image), json.dumps(raw, ensure_ascii=False)


class SNU1PromptBuilder:
    """Expands a short idea into a full image prompt with the chat route (template in prompts/)."""
    CATEGORY, FUNCTION = CATEGORY, "run"
    RETURN_TYPES, RETURN_NAMES = ("STRING", "STRING"), ("prompt", "raw_json")

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {
            "idea": ("STRING", {"multiline": True, "default": ""}),
            "style": (list(STYLES), {"default": STYLES[0]}),
            "size": (list(IMAGE_SIZE_OPTIONS), {"default": IMAGE_SIZE_OPTIONS[0]}),
            "model": ("STRING", {"default": "sensenova-u1"}),
            "timeout": ("INT", {"default": 120, "min": 10, "max": 3600})}}

    @staticmethod
    def system_prompt(style: str, size: str) -> str:
        tpl = (Path(__file__).parent / "prompts" / "builder_prompt.txt").read_text()
        aspect = size.split("|", 1)[1] if "|" in size else size
        return tpl.format(style=style, aspect=aspect).strip()

    def run(self, idea, style, size, model, timeout):
        if not idea.strip():
            raise ValueError("the idea is empty")
        r = ApiClient.from_env().chat(idea, self.system_prompt(style, size), model, 0.7, 1.0, 1024, timeout)
        return r.text.strip(), json.dumps(r.raw, ensure_ascii=False)


class SNU1VisionURL:
    CATEGORY, FUNCTION = CATEGORY, "run"
    RETURN_TYPES, RETURN_NAMES = ("STRING", "STRING"), ("text", "raw_json")

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {
            "image_url": ("STRING", {"default": ""}),
            "question": ("STRING", {"multiline": True, "default": "Describe this image."}),
            "model": ("STRING", {"default": "sensenova-u1"}),
            "max_tokens": ("INT", {"default": 1024, "min": 1, "max": 65536}),
            "timeout": ("INT", {"default": 120, "min": 10, "max": 3600})}}

    def run(self, image_url, question, model, max_tokens, timeout):
        if not (_img.is_http_url(image_url) or image_url.startswith("data:image/")):
            raise ValueError("image_url must be an http(s) URL or a data:image/ URL")
        r = ApiClient.from_env().chat(question, VISION_SYSTEM_PROMPT, model, 0.2, 1.0, max_tokens, timeout,
                                      image_urls=[image_url])
        return r.text, json.dumps(r.raw, ensure_ascii=False)


class SNU1VisionImage:
    CATEGORY, FUNCTION = CATEGORY, "run"
    RETURN_TYPES, RETURN_NAMES = ("STRING", "STRING"), ("text", "raw_json")

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {
            "image": ("IMAGE",),
            "question": ("STRING", {"multiline": True, "default": "Describe this image."}),
            "model": ("STRING", {"default": "sensenova-u1"}),
            "max_tokens": ("INT", {"default": 1024, "min": 1, "max": 65536}),
            "timeout": ("INT", {"default": 120, "min": 10, "max": 3600})}}

    def run(self, image, question, model, max_tokens, timeout):
        urls = [_img.data_url(image, i) for i in range(image.shape[0] if image.dim() == 4 else 1)]
        r = ApiClient.from_env().chat(question, VISION_SYSTEM_PROMPT, model, 0.2, 1.0, max_tokens, timeout,
                                      image_urls=urls)
        return r.text, json.dumps(r.raw, ensure_ascii=False)


# ------------------------------------------------------------------------------------------------
# local nodes
# ------------------------------------------------------------------------------------------------
class SNU1LocalLoader:
    CATEGORY, FUNCTION = LOCAL_CATEGORY, "run"
    RETURN_TYPES, RETURN_NAMES = (MODEL_TYPE, "STRING"), ("model", "memory")

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {
            "model_path": ("STRING", {"default": "sensenova/SenseNova-U1-8B-MoT"}),
            "device": ("STRING", {"default": "cuda"}),
            "vram_mode": (list(_local.VRAM_MODES), {"default": "full"}),
            "gguf_checkpoint": (_gguf_options(), {"default": ""})},
            "optional": {
                "random_init": (["", "tiny-mot", "8b-mot", "a3b-mot"], {"default": ""}),
                "dtype": (["bfloat16", "float16", "float32"], {"default": "bfloat16"}),
                # per-device caps, e.g. "0=20GiB,cpu=64GiB": a cap below the checkpoint's size picks a streaming mode
                "max_memory": ("STRING", {"default": ""}),
                # "fast" mode: how much of the device the resident layers may take (blank = default)
                "fast_vram_fraction": ("STRING", {"default": ""}),
                "fast_vram_headroom_gib": ("STRING", {"default": ""}),
                "fast_activation_reserve_gib": ("STRING", {"default": ""}),
                "fast_vram_budget_gib": ("STRING", {"default": ""})}}

    def run(self, model_path, device, vram_mode, gguf_checkpoint, random_init="", dtype="bfloat16", max_memory="",
            fast_vram_fraction="", fast_vram_headroom_gib="", fast_activation_reserve_gib="", fast_vram_budget_gib=""):
        num = lambda text, default: float(text) if str(text).strip() else default
        okw = _local.fast_offload_kwargs(device, vram_mode, num(fast_vram_fraction, 0.9), num(fast_vram_headroom_gib, 2.0),
                                         num(fast_activation_reserve_gib, 4.0), num(fast_vram_budget_gib, 0.0))
        lm = _local.load(model_path, device, vram_mode, _resolve_gguf(gguf_checkpoint), random_init, dtype=dtype,
                         max_memory=max_memory, offload_kwargs=okw)
        return lm, _local.memory_report()


_SAMPLING = {
    "steps": ("INT", {"default": 50, "min": 1, "max": 200}),
    "cfg_scale": ("FLOAT", {"default": 4.0, "min": 1.0, "max": 20.0, "step": 0.1}),
    "timestep_shift": ("FLOAT", {"default": 3.0, "min": 0.1, "max": 10.0, "step": 0.1}),
    "seed": ("INT", {"default": 0, "min": 0, "max": 2**31 - 1}),
}


class SNU1LocalTextToImage:
    CATEGORY, FUNCTION = LOCAL_CATEGORY, "run"
    RETURN_TYPES, RETURN_NAMES = ("IMAGE", "STRING"), ("images", "think_text")

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {
            "model": (MODEL_TYPE,),
            "prompt": ("STRING", {"multiline": True, "default": ""}),
            "width": ("INT", {"default": 2048, "min": 64, "max": 4096, "step": 32}),
            "height": ("INT", {"default": 2048, "min": 64, "max": 4096, "step": 32}),
            **_SAMPLING,
            "cfg_norm": (list(_local.CFG_NORMS), {"default": "none"}),
            "batch_size": ("INT", {"default": 1, "min": 1, "max": 16}),
            "think": ("BOOLEAN", {"default": False})}}

    def run(self, model, prompt, width, height, steps, cfg_scale, timestep_shift, seed, cfg_norm, batch_size, think):
        imgs, thought = model.text_to_image(prompt, width, height, steps, cfg_scale, timestep_shift, cfg_norm, seed,
                                            batch_size, think)
        return _img.model_to_comfy(imgs), thought


class SNU1LocalImageEdit:
    CATEGORY, FUNCTION = LOCAL_CATEGORY, "run"
    RETURN_TYPES, RETURN_NAMES = ("IMAGE",), ("images",)

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {
            "model": (MODEL_TYPE,),
            "image": ("IMAGE",),
            "prompt": ("STRING", {"multiline": True, "default": ""}),
            **_SAMPLING,
            "img_cfg_scale": ("FLOAT", {"default": 1.0, "min": 0.0, "max": 10.0, "step": 0.1}),
            "cfg_norm": (list(_local.CFG_NORMS), {"default": "none"})},
            "optional": {"image_2": ("IMAGE",), "image_3": ("IMAGE",),
                         "width": ("INT", {"default": 0, "min": 0, "max": 4096, "step": 32}),
                         "height": ("INT", {"default": 0, "min": 0, "max": 4096, "step": 32})}}

    def run(self, model, image, prompt, steps, cfg_scale, timestep_shift, seed, img_cfg_scale, cfg_norm,
            image_2=None, image_3=None, width=0, height=0):
        sources = []
        for im in (image, image_2, image_3):
            if im is not None:
                sources += _img.comfy_to_model(im)
        out = model.edit_image(prompt, sources, steps, cfg_scale, img_cfg_scale, timestep_shift, cfg_norm, seed,
                               width, height)
        return (_img.model_to_comfy(out),)


class SNU1LocalInterleave:
    CATEGORY, FUNCTION = LOCAL_CATEGORY, "run"
    RETURN_TYPES, RETURN_NAMES = (INTERLEAVE_TYPE, "STRING", "IMAGE"), ("result", "text", "images")

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {
            "model": (MODEL_TYPE,),
            "prompt": ("STRING", {"multiline": True, "default": ""}),
            "width": ("INT", {"default": 1024, "min": 64, "max": 4096, "step": 32}),
            "height": ("INT", {"default": 1024, "min": 64, "max": 4096, "step": 32}),
            **_SAMPLING,
            "max_rounds": ("INT", {"default": 4, "min": 1, "max": 16}),
            "max_new_tokens": ("INT", {"default": 512, "min": 16, "max": 8192})},
            "optional": {"image": ("IMAGE",)}}

    def run(self, model, prompt, width, height, steps, cfg_scale, timestep_shift, seed, max_rounds, max_new_tokens,
            image=None):
        sources = _img.comfy_to_model(image) if image is not None else []
        text, imgs = model.interleave(prompt, sources, width, height, steps, cfg_scale, timestep_shift, seed,
                                      max_rounds, max_new_tokens)
        return {"text": text, "images": imgs}, text, _img.stack_for_comfy(imgs)


class SNU1InterleavePreview:
    """Shows an interleaved answer: the text with its pictures saved to ComfyUI's temp folder."""
    CATEGORY, FUNCTION, OUTPUT_NODE = LOCAL_CATEGORY, "run", True
    RETURN_TYPES, RETURN_NAMES = ("STRING",), ("markdown",)

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"result": (INTERLEAVE_TYPE,)}}

    @staticmethod
    def _save(images):
        try:
            import folder_paths
            out_dir = folder_paths.get_temp_directory()
        except Exception:
            import tempfile
            out_dir = tempfile.mkdtemp(prefix="snu1_interleave_")
        os.makedirs(out_dir, exist_ok=True)
        saved = []
        for i, im in enumerate(images):
            name = f"snu1_interleave_{os.getpid()}_{i:02d}.png"
            with open(os.path.join(out_dir, name), "wb") as f:
                f.write(_img.comfy_to_png_bytes(_img.model_to_comfy(im)))
            saved.append({"filename": name, "subfolder": "", "type": "temp"})
        return saved

    def run(self, result):
        saved = self._save(result["images"])
        parts = result["text"].split("[image]")
        md = parts[0]
        for i, rest in enumerate(parts[1:]):
            md += (f"\n\n![picture {i + 1}]({saved[i]['filename']})\n\n" if i < len(saved) else "\n\n[image]\n\n") + rest
        return {"ui": {"images": saved, "text": [md]}, "result": (md,)}


NODE_CLASS_MAPPINGS = {
    "SNU1Chat": SNU1Chat, "SNU1ImageGenerate": SNU1ImageGenerate, "SNU1PromptBuilder": SNU1PromptBuilder,
    "SNU1VisionURL": SNU1VisionURL, "SNU1VisionImage": SNU1VisionImage, "SNU1LocalLoader": SNU1LocalLoader,
    "SNU1LocalTextToImage": SNU1LocalTextToImage, "SNU1LocalImageEdit": SNU1LocalImageEdit,
    "SNU1LocalInterleave": SNU1LocalInterleave, "SNU1InterleavePreview": SNU1InterleavePreview,
}
NODE_DISPLAY_NAME_MAPPINGS = {
    "SNU1Chat": "SenseNova-U1 Chat (API)", "SNU1ImageGenerate": "SenseNova-U1 Image Generate (API)",
    "SNU1PromptBuilder": "SenseNova-U1 Prompt Builder (API)", "SNU1VisionURL": "SenseNova-U1 Vision by URL (API)",
    "SNU1VisionImage": "SenseNova-U1 Vision by Image (API)", "SNU1LocalLoader": "SenseNova-U1 Local Loader",
    "SNU1LocalTextToImage": "SenseNova-U1 Local Text to Image", "SNU1LocalImageEdit": "SenseNova-U1 Local Image Edit",
    "SNU1LocalInterleave": "SenseNova-U1 Local Interleave", "SNU1InterleavePreview": "SenseNova-U1 Interleave Preview",
}
