"""Connection settings of the API nodes (role of the reference's apps/comfyui/config.py:1-31).

The key and the endpoint come from the environment, optionally seeded from a ``.env`` file beside this package or in
the working directory (``KEY=value`` lines; the process environment wins).  Both spellings are read: the
reference's ``SN_API_KEY`` / ``SN_BASE_URL`` and this package's ``SENSENOVA_API_KEY`` / ``SENSENOVA_BASE_URL``.
A local server needs no key, so a missing key is an error only when ``require_key`` is set."""
from __future__ import annotations

import os
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, Optional

DEFAULT_BASE_URL = "http://127.0.0.1:8000"
KEY_ENVS = ("SN_API_KEY", "SENSENOVA_API_KEY")
URL_ENVS = ("SN_BASE_URL", "SENSENOVA_BASE_URL")


@dataclass(frozen=True)
class ApiConfig:
    api_key: str = ""
    base_url: str = DEFAULT_BASE_URL
    retries: int = 2


def read_env_file(path: Path) -> Dict[str, str]:
    """``KEY=value`` lines; ``#`` comments, blank lines and an ``export`` prefix are skipped, quotes stripped."""
    out: Dict[str, str] = {}
    try:
        text = path.read_text(encoding="utf-8")
    except OSError:
        return out
    for line in text.splitlines():
        line = line.strip()
        if not line or line.startswith("#") or "=" not in line:
            continue
        if line.startswith("export "):
            line = line[7:].lstrip()
        k, v = line.split("=", 1)
        v = v.strip()
        if len(v) >= 2 and v[0] == v[-1] and v[0] in "'\"":
            v = v[1:-1]
        out[k.strip()] = v
    return out


def load_config(env_files: Optional[Iterable[Path]] = None, require_key: bool = False, environ=None) -> ApiConfig:
    environ = os.environ if environ is None else environ
    files = list(env_files) if env_files is not None else [Path(__file__).resolve().parent / ".env", Path.cwd() / ".env"]
    merged: Dict[str, str] = {}
    for f in files:
        merged.update(read_env_file(Path(f)))
    merged.update({k: v for k, v in environ.items() if v != ""})
    first = lambda names: next((merged[n].strip() for n in names if merged.get(n, "").strip()), "")
    key = first(KEY_ENVS)
    if require_key and not key:
        raise RuntimeError(f"missing API key: set {' or '.join(KEY_ENVS)} in the environment or in a .env file")
    url = (first(URL_ENVS) or DEFAULT_BASE_URL).rstrip("/")
    return ApiConfig(key, url, int(merged.get("SENSENOVA_RETRIES", "2") or 2))
