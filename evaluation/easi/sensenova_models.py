"""Model entries for VLMEvalKit / EASI (spatial-intelligence suite): the served model as an OpenAI-style endpoint.

VLMEvalKit reads its model table from ``vlmeval/config.py``; copy this file next to it as
``vlmeval/sensenova_models.py`` and add two lines there::

    from .sensenova_models import entries as _sensenova_entries
    supported_VLM.update(_sensenova_entries)

(the reference ships the same hook as evaluation/easi/config/sensenova_models.py plus a patch file).  The endpoint is
this framework's server, or the balancer in front of several replicas
(``python -m sensenova_u1_b200.serving.balancer --replicas 8 --model_path CKPT --port 9000``); set ``U1_API_BASE`` to
point elsewhere.  Thinking answers are long: keep ``max_tokens`` generous."""
import os
from functools import partial

_BASE = os.environ.get("U1_API_BASE", "http://127.0.0.1:9000/v1/chat/completions")


def _entries():
    from vlmeval.api.gpt import GPT4V          # resolves inside VLMEvalKit only
    common = dict(api_base=_BASE, key=os.environ.get("U1_API_KEY", "dummy"), temperature=0, retry=10, verbose=False)
    return {"SenseNova-U1-8B-MoT-Local": partial(GPT4V, model="sensenova-u1-8b-mot", max_tokens=8192, **common),
            "SenseNova-U1-A3B-MoT-Local": partial(GPT4V, model="sensenova-u1-a3b-mot", max_tokens=8192, **common)}


try:
    entries = _entries()
except ImportError:                                # imported outside VLMEvalKit (documentation, tests)
    entries = {}
