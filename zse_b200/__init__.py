"""zse_b200 — a Blackwell (sm_100a) LLM inference engine that serves ``.zse`` models."""
__version__ = "0.1.0"

_LAZY = {"ZSEEngine": "engine", "ZStreamerEngine": "engine", "GenerateConfig": "engine", "EngineConfig": "config",
         "ZSEServer": "server.app"}


def __getattr__(name):
    """The main classes are reachable as ``zse_b200.ZSEEngine`` etc. without making ``import zse_b200`` load torch."""
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module 'zse_b200' has no attribute '{name}'")
    import importlib
    return getattr(importlib.import_module(f"{__name__}.{mod}"), name)


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
