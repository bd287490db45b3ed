#!/usr/bin/env python
"""Visual question answering CLI (reference: examples/vqa/inference.py:29-112)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_path", default=None)
    ap.add_argument("--random_init", default=None)
    ap.add_argument("--image", default=None)
    ap.add_argument("--question", default="Describe the image.")
    ap.add_argument("--max_new_tokens", type=int, default=256)
    ap.add_argument("--max_pixels", type=int, default=4194304)
    ap.add_argument("--min_pixels", type=int, default=65536)
    a = ap.parse_args(argv)
    from sensenova_u1_b200.config import get_config
    from sensenova_u1_b200.inference.api import ByteTokenizer, NEOChatModel
    from sensenova_u1_b200.inference.images import load_image_native
    if a.model_path:
        from transformers import AutoTokenizer
        model = NEOChatModel.from_pretrained(a.model_path)
        tok = AutoTokenizer.from_pretrained(a.model_path, trust_remote_code=True)
    else:
        model = NEOChatModel.from_config(get_config(a.random_init or "tiny-mot", head_dim=128, patch_size=16))
        tok = ByteTokenizer(model.cfg.vocab_size)
    px = load_image_native(a.image, model.cfg.token_pixels, a.min_pixels, a.max_pixels) if a.image else None
    print(model.chat(tok, px, a.question, dict(max_new_tokens=a.max_new_tokens)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
