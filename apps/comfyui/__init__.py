"""ComfyUI custom-node package of sensenova-u1_b200.  ``python apps/comfyui/install.py --comfyui <checkout>`` links
(or copies) this folder into ``ComfyUI/custom_nodes/``; the repository root that holds ``sensenova_u1_b200`` is
found through the link, or through ``repo_root.txt`` of a copied install, and put on ``sys.path``."""
import sys
from pathlib import Path

_here = Path(__file__).resolve().parent
_marker = _here / "repo_root.txt"
_root = Path(_marker.read_text(encoding="utf-8").strip()) if _marker.is_file() else _here.parents[1]
if (_root / "sensenova_u1_b200").is_dir() and str(_root) not in sys.path:
    sys.path.insert(0, str(_root))

from .nodes import NODE_CLASS_MAPPINGS, NODE_DISPLAY_NAME_MAPPINGS  # noqa: E402

__all__ = ["NODE_CLASS_MAPPINGS", "NODE_DISPLAY_NAME_MAPPINGS"]
