"""Public inference API with the reference's names and call signatures
(src/sensenova_u1/__init__.py:1-81; NEOChatModel methods: modeling_neo_chat.py:663, 1003, 1369,
1691, 1862, 1916), served by the sm_100a inference engine of this package.

``tokenizer`` is anything with ``__call__(text)`` returning a dict with ``input_ids`` (a HF
tokenizer works) or with ``encode(text) -> list[int]`` and ``decode(list[int]) -> str``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import List, Optional, Sequence, Tuple

import torch

from ..config import ModelConfig
from ..models.params import ParamStore
from . import prompts
from .images import load_image_native, smart_resize  # noqa: F401  (re-exported: the reference's utils expose them next to the model)

__version__ = "0.1.0"
_ATTN_BACKEND = "sm100"


def set_attn_backend(name: str) -> None:
    """Kept for API compatibility: the only backend is this package's tcgen05 kernel."""
    global _ATTN_BACKEND
    if name not in ("sm100", "auto", "flash", "sdpa"):
        raise ValueError(f"unknown attention backend {name!r}")
    _ATTN_BACKEND = "sm100"


def get_attn_backend() -> str:
    return _ATTN_BACKEND


def effective_attn_backend() -> str:
    return "sm100"


def has_flash_attn() -> bool:
    return False


def check_checkpoint_compatibility(config: dict) -> None:
    """Raises when the checkpoint asks for a newer package (``sensenova_u1_min_version``)."""
    need = str(config.get("sensenova_u1_min_version", "0.0.0"))
    key = lambda v: tuple(int(p) for p in v.split(".")[:3])
    if key(need) > key(__version__):
        raise RuntimeError(f"checkpoint requires sensenova_u1 >= {need}, this is {__version__}")


@dataclass
class NEOVisionConfig:
    patch_size: int = 16
    hidden_size: int = 1024
    downsample_ratio: float = 0.5
    rope_theta_vision: float = 10000.0
    min_pixels: int = 65536
    max_pixels: int = 4194304


@dataclass
class NEOLLMConfig:
    hidden_size: int = 4096
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 12288
    num_hidden_layers: int = 42
    vocab_size: int = 151936
    rope_theta: float = 5e6
    rope_theta_hw: float = 10000.0
    max_position_embeddings_hw: int = 10000


@dataclass
class NEOMoELLMConfig(NEOLLMConfig):
    num_experts: int = 128
    num_experts_per_tok: int = 8
    gen_num_experts: int = 32
    gen_num_experts_per_tok: int = 8
    moe_intermediate_size: int = 768
    gen_moe_intermediate_size: int = 768


@dataclass
class NEOChatConfig:
    llm_config: NEOLLMConfig = field(default_factory=NEOLLMConfig)
    vision_config: NEOVisionConfig = field(default_factory=NEOVisionConfig)
    template: str = "sensenovalm2-chat-v3"

    def to_model_config(self, **kw) -> ModelConfig:
        l, v = self.llm_config, self.vision_config
        d = dict(hidden_size=l.hidden_size, num_heads=l.num_attention_heads, num_kv_heads=l.num_key_value_heads,
                 head_dim=l.head_dim, ffn_size=l.intermediate_size, num_layers=l.num_hidden_layers,
                 vocab_size=l.vocab_size, rope_base=l.rope_theta, rope_base_hw=l.rope_theta_hw,
                 patch_size=v.patch_size, vision_hidden=v.hidden_size, merge_size=int(round(1 / v.downsample_ratio)))
        if isinstance(l, NEOMoELLMConfig):
            d.update(num_experts=l.num_experts, num_experts_per_tok=l.num_experts_per_tok,
                     gen_num_experts=l.gen_num_experts, gen_num_experts_per_tok=l.gen_num_experts_per_tok,
                     moe_intermediate_size=l.moe_intermediate_size)
        d.update(kw)
        return ModelConfig(**d)


def _encode(tokenizer, text: str) -> torch.Tensor:
    if hasattr(tokenizer, "encode") and not hasattr(tokenizer, "__call__"):
        return torch.tensor(tokenizer.encode(text), dtype=torch.long)
    try:
        out = tokenizer(text)
        ids = out["input_ids"] if isinstance(out, dict) or hasattr(out, "keys") else out
    except TypeError:
        ids = tokenizer.encode(text)
    ids = torch.as_tensor(ids, dtype=torch.long)
    return ids.reshape(-1)


class NEOVisionModel:
    """Pixel front-end of one branch (patch GEMM + GELU + 2-D RoPE + 2x2 merge GEMM)."""

    def __init__(self, engine, branch: str = "und"):
        self.engine, self.branch = engine, branch

    def __call__(self, patches, px, py):
        return self.engine.vision_embed(self.branch, patches, px, py)


class NEOChatModel:
    def __init__(self, cfg: ModelConfig, store: ParamStore, vram_mode: str = "full", device=None,
                 offload_kwargs: Optional[dict] = None):
        """``vram_mode`` "full": every weight on the device.  "fast" / "balanced" / "low": ``store`` lives in
        host memory, the decoder layers are streamed to ``device`` through a few slots (utils/offload.py)
        and only embeddings, pixel front-ends and heads stay resident."""
        from .engine import InferenceEngine
        self.cfg, self.store = cfg, store
        if vram_mode == "full":
            self.engine = InferenceEngine(cfg, store)
        else:
            from ..utils.offload import LayerOffloader
            device = torch.device(device if device is not None else "cuda")
            head = ParamStore(cfg.replace(num_layers=0), device=device, dtype=store.dtype, with_grads=False)
            for name, t in head.p.items():
                t.copy_(store.p[name])
            self.engine = InferenceEngine(cfg, head, offload=LayerOffloader(store, device, vram_mode, **(offload_kwargs or {})))
        # set to a process group with one rank per guidance branch to sample guidance-parallel
        self.cfg_group = None
        # all ranks of a guidance-parallel x sequence-parallel run (enable_sequence_parallel)
        self.par_group = None
        self.vision_model = NEOVisionModel(self.engine, "und")
        self.system_message = None
        self.last_think_content = ""
        self.img_context_token_id = None

    def enable_sequence_parallel(self, sp_group, par_group=None) -> None:
        """Sequence-parallel image sampling: the ranks of ``sp_group`` split every image's tokens (keys /
        values and predictions exchanged through peer memory).  With ``cfg_group`` also set, ``par_group``
        is the group of all branches x slices (default: the world group)."""
        self.engine.enable_sequence_parallel(sp_group)
        self.par_group = par_group

    # ---- construction ---------------------------------------------------------
    @classmethod
    def from_pretrained(cls, path: str, device="cuda", dtype=torch.bfloat16, vram_mode: str = "full",
                        offload_kwargs: Optional[dict] = None, **cfg_overrides) -> "NEOChatModel":
        from ..train.checkpoint import import_hf
        check_checkpoint_compatibility(json.loads((Path(path) / "config.json").read_text()))
        store = import_hf(path, device=device if vram_mode == "full" else "cpu", dtype=dtype, with_grads=False,
                          **cfg_overrides)
        return cls(store.cfg, store, vram_mode=vram_mode, device=device, offload_kwargs=offload_kwargs)

    @classmethod
    def from_config(cls, cfg: ModelConfig, device="cuda", seed: int = 0, vram_mode: str = "full",
                    offload_kwargs: Optional[dict] = None) -> "NEOChatModel":
        store = ParamStore(cfg, device=device if vram_mode == "full" else "cpu", with_grads=False)
        store.init_weights(seed)
        return cls(cfg, store, vram_mode=vram_mode, device=device, offload_kwargs=offload_kwargs)

    # ---- text-to-image ----------------------------------------------------------
    @torch.no_grad()
    def t2i_generate(self, tokenizer, prompt, cfg_scale=1, timestep_shift=1, enable_timestep_shift=True,
                     cfg_norm="none", image_size=(256, 256), num_steps=30, IMG_START_TOKEN="<img>",
                     IMG_END_TOKEN="</img>", IMG_CONTEXT_TOKEN="<IMG_CONTEXT>", method="euler", cfg_interval=(0, 1),
                     batch_size=1, t_eps=0.02, think_mode=False, seed=0):
        if method != "euler":
            raise ValueError("only the Euler sampler exists")
        if cfg_norm not in ("cfg_zero_star", "global", "none", "channel"):
            raise ValueError(f"unknown cfg_norm {cfg_norm}")
        cond_q, uncond_q = prompts.t2i_queries(prompt, think_mode)
        cond = _encode(tokenizer, cond_q)
        uncond = _encode(tokenizer, uncond_q) if cfg_scale > 1 else None
        think_text = ""
        if think_mode:
            stop = int(_encode(tokenizer, IMG_START_TOKEN)[-1])
            lay, h = self.engine.prefill([cond], reserve_image_tokens=1024)
            new = self.engine.decode_greedy(lay, h, 1024, stop_ids=(stop,))[0]
            think_text = tokenizer.decode(new) if hasattr(tokenizer, "decode") else ""
            cond = torch.cat([cond, torch.tensor(new, dtype=torch.long)])
            if not new or new[-1] != stop:
                cond = torch.cat([cond, torch.tensor([stop])])
        img = self.engine.t2i(cond, uncond, image_size=tuple(image_size), num_steps=num_steps, cfg_scale=cfg_scale,
                              timestep_shift=timestep_shift if enable_timestep_shift else 1.0, cfg_norm=cfg_norm,
                              cfg_interval=cfg_interval, t_eps=t_eps, seed=seed, batch_size=batch_size,
                              cfg_group=getattr(self, "cfg_group", None), par_group=getattr(self, "par_group", None))
        self.last_think_content = think_text
        return (img, think_text) if think_mode else img

    # ---- editing / interleaved ---------------------------------------------------
    @torch.no_grad()
    def it2i_generate(self, tokenizer, prompt, images, cfg_scale=4.0, img_cfg_scale=1.0, timestep_shift=3.0,
                      cfg_norm="none", image_size=None, num_steps=50, batch_size=1, t_eps=0.02, seed=0,
                      cfg_interval=(0, 1)):
        """Image editing: ``images`` are [3,H,W] tensors (ImageNet-normalised, sizes multiples of the token
        size).  Three guidance branches: text + images, images only, nothing
        (modeling_neo_chat.py:1369-1688)."""
        images = list(images)
        if image_size is None:
            image_size = (images[0].shape[2], images[0].shape[1])
        tags = "<image>\n" * len(images)
        tail = f"{prompts.THINK_START}\n\n{prompts.THINK_END}\n\n{prompts.IMG_START_TOKEN}"
        full = self._embed_prompt(tokenizer, tags + prompt, images, system=prompts.SYSTEM_MESSAGE_FOR_GEN, tail=tail)
        img_only = self._embed_prompt(tokenizer, tags, images, system=prompts.SYSTEM_MESSAGE_FOR_GEN, tail=tail)
        un_ids = _encode(tokenizer, prompts.render_chat([("user", ""), ("assistant", None)]) + prompts.IMG_START_TOKEN)
        sample = [full, (un_ids, None, None), img_only]
        return self.engine.denoise([sample] * batch_size, tuple(image_size), num_steps, cfg_scale, img_cfg_scale,
                                   timestep_shift, cfg_norm, cfg_interval, t_eps, seed)

    @torch.no_grad()
    def interleave_gen(self, tokenizer, prompt, images=(), max_rounds=4, max_new_tokens=256, image_size=(512, 512),
                       cfg_scale=4.0, img_cfg_scale=1.0, timestep_shift=3.0, num_steps=50, seed=0, t_eps=0.02,
                       cfg_norm="none", cfg_interval=(0, 1), system_message=None, think_mode=False,
                       generation_config=None, max_images=None):
        """Interleaved text + image generation: greedy text until ``<img>`` (generate an image conditioned on
        everything so far, append it to the context as an understanding image) or end of turn
        (modeling_neo_chat.py:1003-1366).  Without ``think_mode`` the assistant turn opens with an empty think block,
        as in the reference (:1078-1079); ``max_images`` / ``generation_config["max_new_tokens"]`` are the reference's
        names for ``max_rounds`` / ``max_new_tokens``; ``generation_config`` may also carry the text sampling knobs of
        ``chat`` (``do_sample``, ``temperature``, ``top_p``, ``top_k``, ``repetition_penalty``, ``seed``).
        Returns (text, [images])."""
        if max_images is not None:
            max_rounds = int(max_images)
        if generation_config:
            max_new_tokens = int(generation_config.get("max_new_tokens", max_new_tokens))
        system = prompts.SYSTEM_MESSAGE_FOR_GEN if system_message is None else system_message
        sampling = self._sampling(dict(generation_config or {}))       # None: greedy text (the default)
        tags = "<image>\n" * len(images)
        context_images = list(images)
        question = tags + prompt
        opening = "" if think_mode else f"{prompts.THINK_START}\n\n{prompts.THINK_END}\n\n"
        answer, out_images = opening, []
        img_start = int(_encode(tokenizer, prompts.IMG_START_TOKEN)[-1])
        eos = int(_encode(tokenizer, prompts.IM_END)[-1])
        for rnd in range(max_rounds):
            ids, x, pos3 = self._embed_prompt(tokenizer, question, context_images, system=system, tail=answer)
            lay, h = self.engine.prefill([ids], reserve_image_tokens=max_new_tokens, docs_embeds=[x], docs_pos3=[pos3])
            new = self.engine.decode(lay, h, max_new_tokens, stop_ids=(img_start, eos), sampling=sampling,
                                     prompt_ids=[ids] if sampling else None)[0]
            text = tokenizer.decode(new) if hasattr(tokenizer, "decode") else ""
            answer += text
            if not new or new[-1] != img_start:
                break
            full = self._embed_prompt(tokenizer, question, context_images, system=system, tail=answer)
            un_ids = _encode(tokenizer, prompts.render_chat([("user", ""), ("assistant", None)]) + prompts.IMG_START_TOKEN)
            img = self.engine.denoise([[full, (un_ids, None, None)]], tuple(image_size), num_steps, cfg_scale, 0.0,
                                      timestep_shift, cfg_norm, tuple(cfg_interval), t_eps, seed + rnd)
            out_images.append(img[0])
            # the generated picture re-enters the context through the understanding branch
            mean = torch.tensor([0.485, 0.456, 0.406], device=img.device).view(3, 1, 1)
            std = torch.tensor([0.229, 0.224, 0.225], device=img.device).view(3, 1, 1)
            context_images.append((((img[0] * 0.5 + 0.5).clamp(0, 1) - mean) / std).cpu())
            answer = answer[: -len(prompts.IMG_START_TOKEN)] if answer.endswith(prompts.IMG_START_TOKEN) else answer
            answer += "<image>"
        return answer[len(opening):].replace("<image>", "[image]"), out_images

    def interleave_gen_image_only(self, tokenizer, prompt, images=(), **kw):
        return self.interleave_gen(tokenizer, prompt, images, **kw)[1]

    # ---- understanding ------------------------------------------------------------
    def _embed_prompt(self, tokenizer, question: str, images: Sequence[torch.Tensor], system=None, tail: str = "",
                      history: Sequence[Tuple[str, str]] = ()):
        """Token ids, embeddings and (t,h,w) indexes of a prompt with ``<image>`` placeholders
        (also inside ``tail``, the already generated part of the assistant turn)."""
        from ..data.batch import patchify_block_major
        cfg, eng = self.cfg, self.engine
        tp = cfg.token_pixels
        counts = [(im.shape[1] // tp) * (im.shape[2] // tp) for im in images]
        history, text, tail = prompts.expand_conversation(list(history), question, tail, counts)
        query = prompts.render_chat(list(history) + [("user", text), ("assistant", None)], system or self.system_message) + tail
        ids = _encode(tokenizer, query)
        ctx_id = int(_encode(tokenizer, prompts.IMG_CONTEXT_TOKEN)[-1])
        self.img_context_token_id = ctx_id
        dev = self.store.device
        x = self.store.p["embed_tokens"].index_select(0, ids.to(dev))
        is_ctx = (ids == ctx_id)
        pos3 = self.get_thw_indexes(ids, [(im.shape[1] // tp, im.shape[2] // tp) for im in images], ctx_id)
        if images:
            embs = []
            for im in images:
                p16, px, py, _, _ = patchify_block_major(im.float(), cfg.patch_size, cfg.merge_size)
                embs.append(eng.vision_embed("und", p16.to(dev, torch.bfloat16), px.to(dev), py.to(dev)))
            x = x.clone()
            x[is_ctx.to(dev)] = torch.cat(embs)
        return ids, x, pos3

    def extract_feature(self, pixel_values, gen_model: bool = False, grid_hw=None) -> torch.Tensor:
        """Image-token embeddings of flattened 16 x 16 patches ``[sum(gh * gw), 3 * 16 * 16]`` (the patches of one
        merged token adjacent, as the reference's ``preprocess_pixel_values`` emits them) with ``grid_hw`` = patch
        grid per image: the understanding front-end, or the generation branch's copy with ``gen_model``
        (modeling_neo_chat.py:337-347).  Returns ``[sum(gh * gw) / merge^2, hidden]``."""
        from ..data.batch import patch_grid_positions
        if grid_hw is None:
            raise ValueError("extract_feature needs grid_hw (patch grid of every image)")
        dev, m = self.store.device, self.cfg.merge_size
        embs, off = [], 0
        for gh, gw in torch.as_tensor(grid_hw).tolist():
            n = int(gh) * int(gw)
            px, py = patch_grid_positions(int(gh), int(gw), m)
            embs.append(self.engine.vision_embed("gen" if gen_model else "und", pixel_values[off:off + n].to(dev, torch.bfloat16),
                                                 px.to(dev), py.to(dev)))
            off += n
        return torch.cat(embs)

    @staticmethod
    def patchify(images: torch.Tensor, patch_size: int, channel_first: bool = False) -> torch.Tensor:
        """``[N,3,H,W]`` -> ``[N, (H/p)(W/p), p*p*3]``; pixel order inside a patch (row, column, channel), or
        (channel, row, column) with ``channel_first`` (modeling_neo_chat.py:399-413)."""
        N, C, H, W = images.shape
        h, w = H // patch_size, W // patch_size
        x = images.reshape(N, C, h, patch_size, w, patch_size)
        x = x.permute(0, 2, 4, 1, 3, 5) if channel_first else x.permute(0, 2, 4, 3, 5, 1)
        return x.reshape(N, h * w, patch_size * patch_size * C)

    @staticmethod
    def unpatchify(x: torch.Tensor, patch_size: int, h: Optional[int] = None, w: Optional[int] = None) -> torch.Tensor:
        """Inverse of :meth:`patchify` (row, column, channel order); ``h`` / ``w`` are the image's pixel sizes
        (a square image is assumed without them)."""
        N, L, _ = x.shape
        gh, gw = (int(round(L ** 0.5)),) * 2 if h is None or w is None else (h // patch_size, w // patch_size)
        x = x.reshape(N, gh, gw, patch_size, patch_size, 3).permute(0, 5, 1, 3, 2, 4)
        return x.reshape(N, 3, gh * patch_size, gw * patch_size)

    def batch_chat(self, tokenizer, pixel_values, questions, generation_config=None, **kw):
        """Several independent questions: answered one after the other (the reference declares the method and raises
        ``NotImplementedError``, modeling_neo_chat.py:349-352)."""
        pv = pixel_values if isinstance(pixel_values, (list, tuple)) else [pixel_values] * len(questions)
        return [self.chat(tokenizer, p, q, generation_config) for p, q in zip(pv, questions)]

    @property
    def lm_head(self) -> torch.Tensor:
        """The output projection ``[vocab, hidden]`` (the reference returns the module that holds it)."""
        return self.store.p["lm_head"]

    @staticmethod
    def get_thw_indexes(ids: torch.Tensor, grids: Sequence[Tuple[int, int]], ctx_id: int) -> torch.Tensor:
        """(t,h,w) per token: text advances t by one; all tokens of an image share the next t and
        carry their grid row / column (modeling_neo_chat.py:1977-1992)."""
        n = ids.numel()
        t = torch.zeros(n, dtype=torch.int32)
        h = torch.zeros(n, dtype=torch.int32)
        w = torch.zeros(n, dtype=torch.int32)
        cur, i, g = 0, 0, 0
        flags = (ids == ctx_id).tolist()
        while i < n:
            if not flags[i]:
                t[i] = cur; cur += 1; i += 1
                continue
            gh, gw = grids[g]; g += 1
            cnt = gh * gw
            t[i:i + cnt] = cur
            idx = torch.arange(cnt)
            h[i:i + cnt] = (idx // gw).int(); w[i:i + cnt] = (idx % gw).int()
            cur += 1; i += cnt
        return torch.stack([t, h, w])

    @staticmethod
    def _sampling(gc: dict) -> Optional[dict]:
        """Sampling knobs of a generation config (``do_sample / temperature / top_p / top_k / repetition_penalty /
        seed``); None for plain greedy decoding."""
        rp = float(gc.get("repetition_penalty", 1.0) or 1.0)
        if not gc.get("do_sample", False) and rp == 1.0:
            return None
        return {"do_sample": bool(gc.get("do_sample", False)), "temperature": gc.get("temperature", 1.0) or 1.0,
                "top_p": gc.get("top_p", 1.0) or 1.0, "top_k": gc.get("top_k", 0) or 0, "repetition_penalty": rp,
                "seed": gc.get("seed")}

    @torch.no_grad()
    def chat(self, tokenizer, pixel_values, question, generation_config=None, history=None, return_history=False,
             system_message=None, **kw):
        """Answer to ``question`` about ``pixel_values`` (None, one [3,H,W] tensor, or a list): greedy, or sampled
        when ``generation_config`` has ``do_sample`` (with ``temperature``, ``top_p``, ``top_k``, ``seed``), as the
        reference's ``chat`` forwards them to ``generate`` (modeling_neo_chat.py:1862-1914)."""
        gc = dict(generation_config or {})
        gc.update({k: v for k, v in kw.items() if k in ("do_sample", "temperature", "top_p", "top_k", "repetition_penalty",
                                                       "seed", "max_new_tokens")})
        images = [] if pixel_values is None else (list(pixel_values) if isinstance(pixel_values, (list, tuple)) else [pixel_values])
        n_marked = question.count("<image>") + sum(q.count("<image>") + (a or "").count("<image>") for q, a in (history or []))
        if images and n_marked == 0:
            question = "<image>\n" * len(images) + question
        turns = []
        for q, a in (history or []):
            turns += [("user", q), ("assistant", a)]
        ids, x, pos3 = self._embed_prompt(tokenizer, question, images, system=system_message, history=turns)
        eos = int(_encode(tokenizer, prompts.IM_END)[-1])
        out = self._generate_ids(ids, x, pos3, int(gc.get("max_new_tokens", 256)), (eos,), self._sampling(gc))
        if out and out[-1] == eos:
            out = out[:-1]
        text = tokenizer.decode(out) if hasattr(tokenizer, "decode") else out
        if return_history:
            return text, (history or []) + [(question, text)]
        return text

    def _generate_ids(self, ids, x, pos3, max_new_tokens, stop_ids, sampling):
        lay, h = self.engine.prefill([ids], reserve_image_tokens=max_new_tokens, docs_embeds=[x], docs_pos3=[pos3])
        return self.engine.decode(lay, h, max_new_tokens, stop_ids=stop_ids, sampling=sampling, prompt_ids=[ids])[0]

    @torch.no_grad()
    def generate(self, pixel_values=None, input_ids=None, grid_hw=None, attention_mask=None, visual_features=None,
                 generation_config=None, output_hidden_states=None, **generate_kwargs) -> torch.Tensor:
        """Token-level generation with the reference's signature (modeling_neo_chat.py:1916-1975): ``input_ids``
        [1, N] already holds the ``<IMG_CONTEXT>`` runs; ``pixel_values`` are the flattened 16x16 patches of all
        images in block-major order with ``grid_hw`` [n_images, 2] patch grids (or ``visual_features`` = their
        embeddings).  Returns the new token ids [1, n_new].  Knobs: ``max_new_tokens``, ``eos_token_id``,
        ``do_sample``, ``temperature``, ``top_p``, ``top_k``, ``seed`` (in ``generation_config`` or as keywords)."""
        if input_ids is None or input_ids.shape[0] != 1:
            raise ValueError("generate takes one sequence: input_ids of shape [1, N]")
        if self.img_context_token_id is None:
            raise ValueError("set img_context_token_id (chat() does it from the tokenizer) before generate()")
        gc = {}
        if generation_config is not None:
            gc.update(generation_config if isinstance(generation_config, dict) else generation_config.to_dict())
        gc.update(generate_kwargs)
        cfg, dev = self.cfg, self.store.device
        ids = input_ids[0].cpu()
        m = cfg.merge_size
        grids = [] if grid_hw is None else [(int(h) // m, int(w) // m) for h, w in torch.as_tensor(grid_hw).tolist()]
        pos3 = self.get_thw_indexes(ids, grids, self.img_context_token_id)
        x = self.store.p["embed_tokens"].index_select(0, ids.to(dev))
        if pixel_values is not None or visual_features is not None:
            if visual_features is None:
                visual_features = self.extract_feature(pixel_values, grid_hw=grid_hw)
            x = x.clone()
            x[(ids == self.img_context_token_id).to(dev)] = visual_features.reshape(-1, x.shape[1]).to(x.dtype)
        eos = gc.get("eos_token_id")
        stops = tuple(eos) if isinstance(eos, (list, tuple)) else ((int(eos),) if eos is not None else ())
        out = self._generate_ids(ids, x, pos3, int(gc.get("max_new_tokens", 256) or 256), stops, self._sampling(gc))
        return torch.tensor([out], dtype=torch.long)


class ByteTokenizer:
    """Stand-in tokenizer for tests and synthetic benchmarks (UTF-8 bytes + a few special ids);
    real checkpoints use the Qwen3 tokenizer files through ``transformers.AutoTokenizer``."""

    def __init__(self, vocab_size: int = 1024):
        self.specials = {s: 256 + i for i, s in enumerate(prompts.SPECIAL_TOKENS + [prompts.IM_START, prompts.IM_END])}
        self.inv = {v: k for k, v in self.specials.items()}
        if vocab_size < 256 + len(self.specials):
            raise ValueError("vocabulary too small")

    def encode(self, text: str) -> List[int]:
        out, i = [], 0
        while i < len(text):
            for s, t in self.specials.items():
                if text.startswith(s, i):
                    out.append(t); i += len(s)
                    break
            else:
                out += list(text[i].encode("utf-8")); i += 1
        return out

    def __call__(self, text, **kw):
        return {"input_ids": self.encode(text)}

    def decode(self, ids) -> str:
        b, out = bytearray(), ""
        for t in ids:
            if t in self.inv:
                out += b.decode("utf-8", "replace") + self.inv[t]; b = bytearray()
            elif t < 256:
                b.append(t)
        return out + b.decode("utf-8", "replace")
