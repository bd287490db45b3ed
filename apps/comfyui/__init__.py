"""ComfyUI custom-node package of sensenova-u1_b200 (drop or link this folder into
``ComfyUI/custom_nodes/``; the repository root must be importable, e.g. ``pip install -e`` or
``PYTHONPATH``)."""
from .nodes import NODE_CLASS_MAPPINGS, NODE_DISPLAY_NAME_MAPPINGS

__all__ = ["NODE_CLASS_MAPPINGS", "NODE_DISPLAY_NAME_MAPPINGS"]
