#!/usr/bin/env python
"""Puts this extension into a ComfyUI checkout (role of the reference's apps/comfyui/install.py:1-135).

    python apps/comfyui/install.py --comfyui /path/to/ComfyUI            # directory link (default)
    python apps/comfyui/install.py --comfyui /path/to/ComfyUI --copy     # plain copy
    python apps/comfyui/install.py --comfyui /path/to/ComfyUI --uninstall

The link keeps the extension inside this repository, so the nodes import ``sensenova_u1_b200`` from the checkout
they came with (a ``.pth``-free install: the extension's ``__init__`` adds the repository root to ``sys.path``); a
copy records that root in ``repo_root.txt`` instead."""
from __future__ import annotations

import argparse
import shutil
import sys
from pathlib import Path

DEFAULT_NAME = "ComfyUI-SenseNova-U1-B200"
SKIP = shutil.ignore_patterns("__pycache__", "*.pyc", ".env")


def install(comfyui: Path, name: str = DEFAULT_NAME, copy: bool = False, force: bool = False) -> Path:
    nodes_dir = comfyui / "custom_nodes"
    if not nodes_dir.is_dir():
        raise SystemExit(f"{comfyui} has no custom_nodes directory: not a ComfyUI checkout")
    src = Path(__file__).resolve().parent
    dst = nodes_dir / name
    if dst.is_symlink() or dst.exists():
        if not force:
            raise SystemExit(f"{dst} exists; pass --force to replace it")
        uninstall(comfyui, name)
    if copy:
        shutil.copytree(src, dst, ignore=SKIP)
        (dst / "repo_root.txt").write_text(str(src.parents[1]) + "\n", encoding="utf-8")
    else:
        dst.symlink_to(src, target_is_directory=True)
    return dst


def uninstall(comfyui: Path, name: str = DEFAULT_NAME) -> bool:
    dst = comfyui / "custom_nodes" / name
    if dst.is_symlink():
        dst.unlink()
        return True
    if dst.is_dir():
        shutil.rmtree(dst)
        return True
    return False


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Install the SenseNova-U1 (B200) ComfyUI extension.")
    ap.add_argument("--comfyui", required=True, help="ComfyUI checkout (the directory that holds custom_nodes)")
    ap.add_argument("--name", default=DEFAULT_NAME, help="directory name under custom_nodes")
    ap.add_argument("--copy", action="store_true", help="copy the files instead of linking the directory")
    ap.add_argument("--force", action="store_true", help="replace an existing installation")
    ap.add_argument("--uninstall", action="store_true")
    a = ap.parse_args(argv)
    root = Path(a.comfyui).expanduser().resolve()
    if a.uninstall:
        print("removed" if uninstall(root, a.name) else "nothing to remove")
        return 0
    dst = install(root, a.name, a.copy, a.force)
    print(f"{'copied to' if a.copy else 'linked at'} {dst}; restart ComfyUI to load the nodes")
    return 0


if __name__ == "__main__":
    sys.exit(main())
