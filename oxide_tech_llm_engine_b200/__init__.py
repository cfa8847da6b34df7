"""B200-native LLM inference engine with the capabilities of Oxide-Tech-LLM-Engine.

PyTorch is the framework layer; every hot op is a hand-written sm_100a kernel in ``csrc/``
(``oxb_cuda``), the serving runtime (paged-KV block manager, radix prefix cache, continuous
batching scheduler) is C++ (``oxb_host``).
"""
__version__ = "0.1.0"

from . import _build  # noqa: F401


def __getattr__(name):  # lazy: importing the package must not import torch-heavy modules
    if name in ("Engine", "EngineBuilder"):
        from . import facade

        return getattr(facade, name)
    raise AttributeError(name)
