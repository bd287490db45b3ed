"""B200-native NEO-unify (SenseNova-U1) training and inference framework.

The inference names of the reference package are re-exported here
(src/sensenova_u1/__init__.py:1-81)."""
__version__ = "0.1.0"

_API = ("NEOChatModel", "NEOChatConfig", "NEOLLMConfig", "NEOMoELLMConfig", "NEOVisionConfig", "NEOVisionModel",
        "set_attn_backend", "get_attn_backend", "effective_attn_backend", "has_flash_attn",
        "check_checkpoint_compatibility")
__all__ = list(_API)


def __getattr__(name):
    if name in _API:
        from .inference import api
        return getattr(api, name)
    raise AttributeError(name)
