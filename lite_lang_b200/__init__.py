"""lite_lang_b200: a small, whole inference engine for one GPU (B200, sm_100a).

Public surface::

    from lite_lang_b200 import Engine, EngineConfig, SamplingParams
    engine = Engine("/path/to/model", EngineConfig(dtype="bfloat16"))
    new_tokens = engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_new_tokens=16))

Importing the package needs no GPU; building an ``Engine`` does.
"""

from . import models as _models  # noqa: F401  (registers the architectures)
from .config import EngineConfig, load_config, register_architecture
from .sampling import SamplingParams

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "generate"):
        from .engine import engine as _engine
        return getattr(_engine, name)
    raise AttributeError(name)


__all__ = ["Engine", "EngineConfig", "SamplingParams", "generate", "load_config", "register_architecture"]
