"""Supervised multimodal dataset: annotation records -> ``Sample`` (text / understanding-image /
generation-image segments) for the packer.

Covers what the reference's ``LazySupervisedDataset`` does before tokens reach the packer
(training/sensenovavl/data/multimodal_dataset.py:62-206 construction, :364-560 generation-task
preparation, :681-910 sample assembly), re-expressed as small pure functions over plain dicts so
that every policy is testable without images or a tokenizer:

* task types: ``mm_t2i`` (text -> image), ``mm_it2i`` (editing), ``mm_interleave_gen``
  (interleaved text + images), understanding (image/video QA), pure text;
* classifier-free-guidance condition dropping: with the configured probabilities the text
  condition, the image condition or both are removed from a generation sample, the thinking text
  before the generated picture is removed with the text, and the generation system prompt is only
  added when nothing was dropped (:378-540);
* the clean copy of a generated image that re-enters the context through the understanding branch
  for interleaved data (``duplicate_for_und``);
* native-resolution resize (``smart_resize`` budget per image) and the token budget per sample;
* several datasets mixed by ``repeat_time`` weights, sharded over data-parallel ranks, with a
  resumable position (``state_dict``).
"""
from __future__ import annotations

import copy
import json
import random
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from ..inference import prompts
from .batch import Sample, Segment

TASKS = {"mm_t2i": 3, "mm_it2i": 4, "mm_interleave_gen": 5}


@dataclass
class CfgDrop:
    """Condition-dropping probabilities (config keys ``cfg_txt_uncond_drop_prob`` etc.)."""
    txt: float = 0.0
    img: float = 0.0
    txtimg: float = 0.0
    independent: bool = True


@dataclass
class ChatOptions:
    """Text-side preparation switches the reference reads as loose config globals (dataset.py:539-632):

    * ``thinking_method``: ``"tag"`` (the shipped configs): the sentence that asks for reasoning is removed from system
      messages and every assistant turn that does not open with ``<think>`` gets an empty think block in front of it
      (part of the prompt, no loss) unless the text condition was dropped; ``"sys"``: samples that contain reasoning
      get the sentence added to their system message instead, and only those get the empty block on their other turns;
    * ``st_prompt_ratio``: probability of adding the default identity sentence to a sample without a system message;
    * ``rm_all_think_token``: strip all reasoning from the targets;
    * ``image_token_position_random``: ``"none"``, ``"end"`` or ``"random"``: with probability 1/2 a single leading
      ``<image>`` of a turn moves to the end of / a random place in its text."""
    thinking_method: str = "tag"
    st_prompt_ratio: float = 0.0
    rm_all_think_token: bool = False
    image_token_position_random: str = "none"


ROLES = {"human": "user", "user": "user", "system": "system", "knowledge": "knowledge", "gpt": "assistant",
         "assistant": "assistant", "plugin": "system name=<|plugin|>", "plugin-return": "environment name=<|plugin|>",
         "interpreter": "system name=<|interpreter|>", "interpreter-return": "environment name=<|interpreter|>"}


def apply_chat_options(conv: List[dict], opts: ChatOptions, rng: random.Random) -> Tuple[List[dict], bool]:
    """Returns (conversation, has_reasoning) after the rewrites above; the input list is not modified."""
    import re
    conv = [dict(t) for t in conv]
    if opts.image_token_position_random in ("end", "random"):
        for t in conv:
            v = t["value"]
            if v.count("<image>") == 1 and v.startswith("<image>\n") and rng.random() < 0.5:
                text = v.replace("<image>\n", "")
                if opts.image_token_position_random == "end":
                    t["value"] = text + "\n<image>"
                else:
                    pos = rng.randint(0, len(text))
                    t["value"] = text[:pos] + "\n<image>\n" + text[pos:]
    reason = prompts.REASON_PROMPT
    strip_reason = lambda s: re.sub(r"(\n?)(" + re.escape(reason) + ")", "", s)
    thinking = any((t["from"] == "system" and reason in t["value"]) or
                   (t["from"] in ("gpt", "assistant") and t["value"].startswith(prompts.THINK_START)) for t in conv)
    if opts.thinking_method == "tag" and conv and conv[0]["from"] == "system":
        conv[0]["value"] = strip_reason(conv[0]["value"])
        if conv[0]["value"] == "":
            conv.pop(0)
    if opts.thinking_method == "sys" and thinking:
        if conv and conv[0]["from"] == "system":
            if reason not in conv[0]["value"]:
                conv[0]["value"] = (reason + "\n" + conv[0]["value"]) if rng.random() < 0.5 else (conv[0]["value"] + "\n" + reason)
        else:
            conv.insert(0, {"from": "system", "value": reason})
    if opts.st_prompt_ratio > 0 and rng.random() < opts.st_prompt_ratio and (not conv or conv[0]["from"] != "system"):
        conv.insert(0, {"from": "system", "value": prompts.DEFAULT_IDENTITY_PROMPT})
    if opts.rm_all_think_token:
        kept = []
        for t in conv:
            if t["from"] == "system":
                t["value"] = strip_reason(t["value"])
            elif t["from"] in ("gpt", "assistant"):
                t["value"] = t["value"].replace(f"{prompts.THINK_START}\n", "").replace(f"\n{prompts.THINK_END}", "")
            if t["value"] != "":
                kept.append(t)
        conv = kept
    return conv, thinking


def _human_index(conv: List[dict]) -> int:
    for i, t in enumerate(conv):
        if t["from"] in ("human", "user"):
            return i
    return 0


def prepare_generation_record(rec: dict, task: str, drop: CfgDrop, rng: random.Random) -> Tuple[dict, dict]:
    """Applies condition dropping to one annotation record of a generation task.

    Returns (record, info): ``info["gen_flags"]`` marks which images are generation targets,
    ``info["dup_for_und"]`` which of them are followed by a clean understanding copy,
    ``info["dropped_text"]`` whether the text condition was removed (such samples carry no
    text loss)."""
    rec = copy.deepcopy(rec)
    conv = rec["conversations"]
    images = list(rec.get("images") or ([rec["image"]] if rec.get("image") else []))
    h = _human_index(conv)
    system = {"from": "system", "value": prompts.SYSTEM_MESSAGE_FOR_GEN}
    dropped_text = False
    if task == "mm_t2i":
        if len(images) != 1:
            raise ValueError("a text-to-image record has exactly one (target) image")
        if rng.random() < drop.txt:
            conv[h]["value"] = ""
            conv[-1]["value"] = "<image>"            # also removes thinking text before the picture
            dropped_text = True
        else:
            conv.insert(0, system)
        gen_flags, dup = [1], [0]
    elif task == "mm_it2i":
        if len(images) < 2:
            raise ValueError("an editing record has at least one source image and one target image")
        n_src = len(images) - 1
        strip = lambda s: s.replace("<image>\n", "").replace("<image>", "")
        if drop.independent:
            case_txt = rng.random() < drop.txt
            case_img = rng.random() < drop.img
        else:
            case_txt = case_img = False
            total = drop.txt + drop.img + drop.txtimg
            if rng.random() < total:
                c = rng.choices(["txt", "img", "txtimg"], weights=[drop.txt, drop.img, drop.txtimg], k=1)[0]
                case_txt, case_img = c in ("txt", "txtimg"), c in ("img", "txtimg")
        if case_txt:
            conv[h]["value"] = "<image>" * n_src
            conv[-1]["value"] = "<image>"
            dropped_text = True
        if case_img:
            conv[h]["value"] = strip(conv[h]["value"])
            images = images[-1:]
        if not case_txt and not case_img:
            conv.insert(0, system)
        gen_flags = [0] * (len(images) - 1) + [1]
        dup = [0] * len(images)
    elif task == "mm_interleave_gen":
        # every picture in an assistant turn is a target; each one is followed by its clean copy so
        # that later text and pictures condition on it through the understanding branch
        gen_flags, dup = [], []
        for t in conv:
            k = t["value"].count("<image>")
            is_answer = t["from"] in ("gpt", "assistant")
            gen_flags += [1 if is_answer else 0] * k
            dup += [1 if is_answer else 0] * k
        if gen_flags and gen_flags[-1] == 1 and conv[-1]["value"].rstrip().endswith("<image>"):
            dup[-1] = 0                              # nothing follows the last picture
        if rng.random() < drop.txt:
            conv[h]["value"] = "<image>" * conv[h]["value"].count("<image>")
            dropped_text = True
        else:
            conv.insert(0, system)
    else:
        raise ValueError(f"not a generation task: {task}")
    rec["images"] = images
    rec.pop("image", None)
    return rec, {"gen_flags": gen_flags, "dup_for_und": dup, "dropped_text": dropped_text}


def record_to_sample(rec: dict, task: str, tokenize: Callable[[str], List[int]],
                     load_image: Callable[[str, bool], torch.Tensor], info: Optional[dict] = None,
                     root: Path = Path("."), und_loss: bool = True, max_text_tokens: int = 1 << 30,
                     chat: Optional[ChatOptions] = None, rng: Optional[random.Random] = None) -> Sample:
    """Builds the segment list of one record.  ``load_image(path, for_generation)`` returns a float
    tensor [3,H,W] (ImageNet-normalised for understanding inputs, [-1,1] for generation targets).  With ``chat`` the
    conversation is first rewritten by :func:`apply_chat_options`; assistant turns flagged ``"is_input": true`` are
    context without loss; turns of unknown roles are skipped (dataset.py:634-672)."""
    images = list(rec.get("images") or ([rec["image"]] if rec.get("image") else []))
    thinking = False
    if chat is not None:
        conv, thinking = apply_chat_options(rec["conversations"], chat, rng or random.Random(0))
        rec = dict(rec, conversations=conv)
    n_img = sum(t["value"].count("<image>") for t in rec["conversations"])
    if n_img != len(images):
        raise ValueError(f"{n_img} <image> placeholders but {len(images)} images")
    gen_flags = (info or {}).get("gen_flags") or [0] * len(images)
    dup = (info or {}).get("dup_for_und") or [0] * len(images)
    text_loss = und_loss and not (info or {}).get("dropped_text", False)
    segs: List[Segment] = []
    k = 0
    dropped = bool((info or {}).get("dropped_text", False))
    for turn in rec["conversations"]:
        if chat is not None and turn["from"] not in ROLES:
            continue
        role = ROLES.get(turn["from"], turn["from"])
        is_answer = role == "assistant" and not turn.get("is_input", False)
        parts = turn["value"].split("<image>")
        head = f"{prompts.IM_START}{role}\n"
        if chat is not None and is_answer and (chat.thinking_method == "tag" or thinking) and not dropped \
                and not turn["value"].startswith(prompts.THINK_START):
            head += prompts.EMPTY_THINK                 # "no reasoning for this answer": part of the prompt, no loss
        segs.append(Segment("text", ids=torch.tensor(tokenize(head), dtype=torch.long), loss=False))
        for i, txt in enumerate(parts):
            if i > 0:
                as_gen = bool(gen_flags[k])
                try:                 # loaders that share the pixel budget between the images of a sample take their count
                    px = load_image(str(root / images[k]), as_gen, len(images))
                except TypeError:
                    px = load_image(str(root / images[k]), as_gen)
                # the packer brackets the picture with <img> ... </img>; in an assistant turn the
                # opening token is a prediction target (the model decides when to draw)
                segs.append(Segment("gen_image" if as_gen else "und_image", pixels=px,
                                    loss=is_answer and as_gen and text_loss,
                                    duplicate_for_und=bool(dup[k]) and as_gen))
                k += 1
            if txt:
                ids = tokenize(txt)[:max_text_tokens]
                segs.append(Segment("text", ids=torch.tensor(ids, dtype=torch.long), loss=is_answer and text_loss))
        segs.append(Segment("text", ids=torch.tensor(tokenize(f"{prompts.IM_END}\n"), dtype=torch.long),
                            loss=is_answer and text_loss))
    return Sample(segs, TASKS.get(task, 0))


def plain_pair_to_sample(rec: dict, tokenize: Callable[[str], List[int]], load_image, root: Path = Path("."),
                         max_text_tokens: int = 1 << 30, eos: str = prompts.IM_END) -> Sample:
    """Caption pairs in the "plain" style of the reference's pre-training data (``dataset_type`` ``cc`` / ``plain_pair``,
    template ``sensenovalm2-plain``: multimodal_dataset.py:1452-1523): no chat markup, the pictures first, then the
    caption, every caption token a prediction target.  Records: ``{"image": path, "caption": text}`` or a conversation
    whose last turn is the caption."""
    images = list(rec.get("images") or ([rec["image"]] if rec.get("image") else []))
    if not images:
        raise ValueError("a caption pair needs an image")
    text = rec.get("caption")
    if text is None:
        text = rec["conversations"][-1]["value"]
    text = text.replace("<image>\n", "").replace("<image>", "").strip()
    segs: List[Segment] = []
    for im in images:
        try:
            px = load_image(str(root / im), False, len(images))
        except TypeError:
            px = load_image(str(root / im), False)
        segs.append(Segment("und_image", pixels=px))
    ids = tokenize(text + eos)[:max_text_tokens]
    segs.append(Segment("text", ids=torch.tensor(ids, dtype=torch.long), loss=True))
    return Sample(segs, 0)


class ConversationDataset:
    """Iterates samples of several annotation files mixed by weight.

    ``meta``: ``{name: {"annotation": jsonl path, "root": image dir, "data_type": task,
    "repeat_time": weight}}`` (the reference's meta JSON, training/README.md:193-229).  Records
    are dealt to data-parallel ranks round-robin (record i goes to rank i mod world); the position
    in every file and the RNG are part of ``state_dict`` so a resumed run continues the stream."""

    def __init__(self, meta, tokenize, load_image, drop: CfgDrop = CfgDrop(), rank: int = 0, world: int = 1,
                 seed: int = 0, und_loss: bool = True, repeat: bool = True, max_text_tokens: int = 1 << 30,
                 min_length: int = 0, weights: Optional[Sequence[float]] = None, max_epochs: int = -1,
                 min_num_frame: int = 4, max_num_frame: int = 24, frame_max_pixels: int = 448 * 448,
                 chat: Optional[ChatOptions] = None):
        self.meta = json.loads(Path(meta).read_text()) if isinstance(meta, (str, Path)) else dict(meta)
        self.tokenize, self.load_image, self.drop = tokenize, load_image, drop
        self.rank, self.world, self.repeat = rank, world, repeat
        self.und_loss, self.max_text_tokens = und_loss, max_text_tokens
        self.rng = random.Random(seed * 1000003 + rank)
        self.names = sorted(self.meta)
        # sampling weight per file: the meta file's repeat_time, or explicit weights (dataset mixing by kind)
        self.weights = [float(w) for w in weights] if weights is not None else \
            [float(self.meta[n].get("repeat_time", 1.0)) for n in self.names]
        if len(self.weights) != len(self.names):
            raise ValueError("one sampling weight per annotation file")
        self.min_num_frame, self.max_num_frame, self.frame_max_pixels = int(min_num_frame), int(max_num_frame), int(frame_max_pixels)
        self.chat = chat                           # None: conversations are used as written
        self.min_length = int(min_length)          # samples with fewer tokens are dropped (data.min_length)
        self.max_epochs = int(max_epochs)          # passes over every file before it is exhausted (-1: endless)
        self.short = 0
        self.cursor: Dict[str, int] = {n: 0 for n in self.names}     # records consumed per file (all ranks)
        self.skipped = 0
        self._lines: Dict[str, List[str]] = {}

    def _file(self, name: str) -> List[str]:
        if name not in self._lines:
            with open(self.meta[name]["annotation"]) as f:
                self._lines[name] = [ln for ln in f if ln.strip()]
        return self._lines[name]

    def _next_record(self, name: str) -> Optional[dict]:
        lines = self._file(name)
        if not lines:
            return None
        c = self.cursor[name]
        # my next record at or after the cursor: index = rank (mod world)
        idx = c + ((self.rank - c) % self.world)
        if not self.repeat and idx >= len(lines):
            return None
        if self.max_epochs > 0 and idx >= self.max_epochs * len(lines):
            return None
        self.cursor[name] = idx + 1
        try:
            return json.loads(lines[idx % len(lines)])
        except ValueError:
            self.skipped += 1
            return {}

    def __iter__(self) -> Iterator[Sample]:
        live = [i for i in range(len(self.names)) if self.weights[i] > 0]      # a weight of zero switches a file off
        while live:
            i = self.rng.choices(live, weights=[self.weights[j] for j in live], k=1)[0]
            name = self.names[i]
            rec = self._next_record(name)
            if rec is None:
                live.remove(i)
                continue
            if not rec:
                continue
            ds = self.meta[name]
            task = ds.get("data_type", "")
            try:
                info = None
                root = Path(ds.get("root", "."))
                if rec.get("video"):
                    # video QA: sampled frames become "FrameN: <image>" understanding pictures (data/video.py)
                    from .video import video_record_to_sample
                    sample = video_record_to_sample(rec, self.tokenize, self._prepare_frame, root=root, rng=self.rng,
                                                    min_num_frame=self.min_num_frame, max_num_frame=self.max_num_frame,
                                                    und_loss=self.und_loss)
                elif ds.get("dataset_type") in ("cc", "plain_pair") or ds.get("template") == "plain":
                    sample = plain_pair_to_sample(rec, self.tokenize, self.load_image, root, self.max_text_tokens)
                else:
                    if task in TASKS:
                        rec, info = prepare_generation_record(rec, task, self.drop, self.rng)
                    sample = record_to_sample(rec, task, self.tokenize, self.load_image, info, root,
                                              self.und_loss, self.max_text_tokens, chat=self.chat, rng=self.rng)
                if self.min_length > 0:
                    n = sum(int(sg.ids.numel()) if sg.kind == "text"
                            else (sg.pixels.shape[1] // 32) * (sg.pixels.shape[2] // 32) + 2 for sg in sample.segments)
                    if n < self.min_length:
                        self.short += 1
                        continue
                yield sample
            except Exception:
                self.skipped += 1          # a broken record must not end the run
                continue

    def _prepare_frame(self, frame: torch.Tensor) -> torch.Tensor:
        """uint8 ``[3, H, W]`` video frame -> understanding picture inside the per-frame pixel budget."""
        from PIL import Image
        from ..inference.images import load_image_native
        im = Image.fromarray(frame.permute(1, 2, 0).contiguous().numpy())
        return load_image_native(im, factor=32, min_pixels=min(65536, self.frame_max_pixels), max_pixels=self.frame_max_pixels,
                                 normalize="imagenet")

    def state_dict(self):
        return {"cursor": dict(self.cursor), "rng": self.rng.getstate(), "skipped": self.skipped}

    def load_state_dict(self, sd):
        self.cursor.update(sd["cursor"])
        st = sd["rng"]
        self.rng.setstate((st[0], tuple(st[1]), st[2]) if isinstance(st, (list, tuple)) else st)
        self.skipped = sd.get("skipped", 0)


def default_image_loader(token_pixels: int = 32, min_pixels: int = 65536, max_pixels: int = 4194304):
    """``load_image(path, for_generation)`` with native-resolution resize (``smart_resize``)."""
    from ..inference.images import load_image_native

    def load(path: str, for_generation: bool) -> torch.Tensor:
        return load_image_native(path, factor=token_pixels, min_pixels=min_pixels, max_pixels=max_pixels,
                                 normalize="pm1" if for_generation else "imagenet")
    return load
