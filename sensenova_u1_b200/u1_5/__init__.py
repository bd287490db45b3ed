"""Prompt tooling of the U1.5 generation: render-brief compiler for text-to-image requests, edit-instruction
rewriter and image captioner, all over an OpenAI-style chat endpoint (or the loaded model itself).
Role of the reference's src/sensenova_u1_5/{image_pe.py, edit/edit_pe.py, caption/caption.py}."""
from .briefs import (CANVAS_ROWS, RenderBriefError, caption_image, compile_render_brief, enhance_edit_prompt,  # noqa: F401
                     extract_json, nearest_canvas, validate_brief)
