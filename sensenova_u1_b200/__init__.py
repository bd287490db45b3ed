"""B200-native NEO-unify (SenseNova-U1) training and inference framework.

The inference names of the reference package are re-exported here
(src/sensenova_u1/__init__.py:1-81): ``NEOChatModel`` and the configuration classes are the
``transformers``-integrated ones of ``inference/hf.py`` (registered with ``AutoConfig`` / ``AutoModel`` on first
use), the attention-backend helpers those of ``inference/api.py``."""
__version__ = "0.1.0"

_HF = ("NEOChatModel", "NEOChatConfig", "NEOLLMConfig", "NEOMoELLMConfig", "NEOVisionConfig",
       "load_model_and_tokenizer", "resolve_checkpoint_path")
_API = ("NEOVisionModel", "set_attn_backend", "get_attn_backend", "effective_attn_backend", "has_flash_attn",
        "check_checkpoint_compatibility", "ByteTokenizer")
__all__ = list(_HF + _API) + ["__version__", "main"]
_registered = False


def _register():
    """Registers ``neo_chat`` / ``neo_vision`` with the Auto classes (reference: models/neo_unify/__init__.py:36-55)."""
    global _registered
    if not _registered:
        from .inference import hf
        hf.register()
        _registered = True


def __getattr__(name):
    if name in _HF:
        from .inference import hf
        _register()
        return getattr(hf, name)
    if name in _API:
        from .inference import api
        return getattr(api, name)
    raise AttributeError(name)


def main() -> None:
    """Console entry point: prints the package version (reference: src/sensenova_u1/__init__.py:80-81)."""
    print(f"sensenova-u1_b200 v{__version__}")
