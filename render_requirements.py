#!/usr/bin/env python
"""Writes ``requirements.txt`` (and ``requirements-<extra>.txt`` per optional group) from ``pyproject.toml``, so pip users
and the packaging metadata cannot drift; ``--check`` fails when a written file is stale (for CI).  Role of the
reference's scripts/render_requirements.py:1-93.  The serving balancer needs ``httpx`` next to ``fastapi`` / ``uvicorn``;
it is listed in the ``serving`` group."""
import argparse
import sys
from pathlib import Path

try:
    import tomllib
except ModuleNotFoundError:                      # Python 3.10
    import tomli as tomllib

ROOT = Path(__file__).resolve().parent
HEADER = ("# generated from pyproject.toml by render_requirements.py: edit pyproject.toml, then run it again\n"
          "# source: {src}\n"
          "# building the native library needs the CUDA 12.8+ toolchain (nvcc): python -m sensenova_u1_b200.build\n")


def outputs(pyproject: Path):
    """{file name: text} for the base dependencies and every optional group."""
    proj = tomllib.loads(pyproject.read_text())["project"]
    out = {"requirements.txt": HEADER.format(src="[project].dependencies") + "\n".join(proj.get("dependencies", [])) + "\n"}
    for extra, deps in sorted((proj.get("optional-dependencies") or {}).items()):
        out[f"requirements-{extra}.txt"] = (HEADER.format(src=f"[project.optional-dependencies].{extra}") + "-r requirements.txt\n"
                                            + "\n".join(deps) + "\n")
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--check", action="store_true", help="do not write; exit 1 if a file differs from what would be written")
    ap.add_argument("--root", default=str(ROOT))
    a = ap.parse_args(argv)
    root = Path(a.root)
    stale = []
    for name, text in outputs(root / "pyproject.toml").items():
        f = root / name
        if a.check:
            if not f.is_file() or f.read_text() != text:
                stale.append(name)
        else:
            f.write_text(text)
    if stale:
        print("stale: " + ", ".join(stale) + " (run render_requirements.py)", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
