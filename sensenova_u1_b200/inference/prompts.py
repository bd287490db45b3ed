"""Chat template, special tokens and the generation system prompt.

These strings are data the released checkpoints were trained with, so they are kept verbatim
(template: training/sensenovavl/data/dataset.py:510-679 and
src/sensenova_u1/models/neo_unify/conversation.py; special tokens:
training/sensenovavl/data/constants.py:1-17; system prompt:
src/sensenova_u1/models/neo_unify/utils.py:9)."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

IMG_CONTEXT_TOKEN = "<IMG_CONTEXT>"
IMG_START_TOKEN = "<img>"
IMG_END_TOKEN = "</img>"
THINK_START, THINK_END = "<think>", "</think>"
SPECIAL_TOKENS = [IMG_CONTEXT_TOKEN, IMG_START_TOKEN, IMG_END_TOKEN, THINK_START, THINK_END]
IM_START, IM_END = "<|im_start|>", "<|im_end|>"

SYSTEM_MESSAGE_FOR_GEN = (
    "You are an image generation and editing assistant that accurately understands and executes "
    "user intent.\n\nYou support two modes:\n\n1. Think Mode:\nIf the task requires reasoning, you "
    "MUST start with a <think></think> block. Put all reasoning inside the block using plain text. "
    "DO NOT include any image tags. Keep it reasonable and directly useful for producing the final "
    "image.\n\n2. Non-Think Mode:\nIf no reasoning is needed, directly produce the final image.\n\n"
    "Task Types:\n\nA. Text-to-Image Generation:\n"
    "- Generate a high-quality image based on the user's description.\n"
    "- Ensure visual clarity, semantic consistency, and completeness.\n"
    "- DO NOT introduce elements that contradict or override the user's intent.\n\n"
    "B. Image Editing:\n"
    "- Use the provided image(s) as input or reference for modification or transformation.\n"
    "- The result can be an edited image or a new image based on the reference(s).\n"
    "- Preserve all unspecified attributes unless explicitly changed.\n\n"
    "General Rules:\n"
    "- For any visible text in the image, follow the language specified for the rendered text in "
    "the user's description, not the language of the prompt. If no language is specified, use the "
    "user's input language."
)


# system prompt the released checkpoints were tuned with for interleaved text + image answers (the reference's
# examples/interleave/inference.py:67 passes it as ``system_message``)
SYSTEM_MESSAGE_FOR_INTERLEAVE = (
    "You are a multimodal assistant capable of reasoning with both text and images. You support two modes:\n\n"
    "Think Mode: When reasoning is needed, you MUST start with a <think></think> block and place all reasoning inside "
    "it. You MUST interleave text with generated images using tags like <image1>, <image2>. Images can ONLY be "
    "generated between <think> and </think>, and may be referenced in the final answer.\n\n"
    "Non-Think Mode: When no reasoning is needed, directly provide the answer without reasoning. Do not use tags like "
    "<image1>, <image2>; present any images naturally alongside the text.\n\n"
    "After the think block, always provide a concise, user-facing final answer. The answer may include text, images, "
    "or both. Match the user's language in both reasoning and the final answer."
)


# Strings the training data of the released checkpoints was prepared with (training/sensenovavl/data/dataset.py:584-585):
# the system sentence that asks for a think block, and the default identity sentence added to samples without a system
# message with probability ``st_prompt_ratio``.  They are data, kept verbatim.
REASON_PROMPT = ("Reason step by step and place the thought process within the <think></think> tags, and provide the final "
                 "conclusion at the end.")
DEFAULT_IDENTITY_PROMPT = "你是商汤科技开发的日日新融合模态大模型，中文名叫商量，英文名叫SenseNova，是一个有用无害的人工智能助手。"
EMPTY_THINK = f"{THINK_START}\n\n{THINK_END}\n\n"


def render_chat(messages: Sequence[Tuple[str, Optional[str]]], system: Optional[str] = None) -> str:
    """``<|im_start|>{role}\\n{content}<|im_end|>\\n`` per turn; a turn whose content is None is left
    open (the model continues it)."""
    out: List[str] = []
    if system:
        out.append(f"{IM_START}system\n{system}{IM_END}\n")
    for role, content in messages:
        if content is None:
            out.append(f"{IM_START}{role}\n")
        else:
            out.append(f"{IM_START}{role}\n{content}{IM_END}\n")
    return "".join(out)


def t2i_queries(prompt: str, think_mode: bool = False, system: str = SYSTEM_MESSAGE_FOR_GEN):
    """Conditional and unconditional prompts of text-to-image generation
    (src/sensenova_u1/models/neo_unify/modeling_neo_chat.py:1700-1708)."""
    tail = f"{THINK_START}\n" if think_mode else f"{THINK_START}\n\n{THINK_END}\n\n{IMG_START_TOKEN}"
    cond = render_chat([("user", prompt), ("assistant", None)], system) + tail
    uncond = render_chat([("user", ""), ("assistant", None)]) + IMG_START_TOKEN
    return cond, uncond


def expand_image_placeholders(text: str, token_counts: Sequence[int]) -> str:
    """Each ``<image>`` becomes ``<img>`` + n x ``<IMG_CONTEXT>`` + ``</img>``."""
    parts = text.split("<image>")
    if len(parts) - 1 != len(token_counts):
        raise ValueError(f"{len(parts) - 1} <image> placeholders but {len(token_counts)} images")
    out = parts[0]
    for n, rest in zip(token_counts, parts[1:]):
        out += IMG_START_TOKEN + IMG_CONTEXT_TOKEN * n + IMG_END_TOKEN + rest
    return out


def expand_conversation(history: Sequence[Tuple[str, Optional[str]]], question: str, tail: str,
                        token_counts: Sequence[int]) -> Tuple[list, str, str]:
    """Expands the ``<image>`` placeholders of a whole conversation in reading order: earlier turns first, then the
    question, then the part of the answer that exists already (``tail``).  The pictures are given in the same order
    (the reference replaces placeholders one by one over the rendered query, history included:
    modeling_neo_chat.py:1879-1891).  Returns (history, question, tail) with the placeholders replaced."""
    counts = list(token_counts)
    total = sum((c or "").count("<image>") for _, c in history) + question.count("<image>") + tail.count("<image>")
    if total != len(counts):
        raise ValueError(f"{total} <image> placeholders but {len(counts)} images")

    def take(text):
        n = text.count("<image>")
        out = expand_image_placeholders(text, counts[:n]) if n else text
        del counts[:n]
        return out
    new_hist = [(role, take(c) if c is not None else None) for role, c in history]
    q = take(question)
    return new_hist, q, take(tail)
