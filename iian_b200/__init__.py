"""iian_b200: a small, whole LLM inference engine for one NVIDIA B200 and one architecture
(Qwen3 dense), from a request's token ids to its next token.

    from iian_b200 import Engine, EngineConfig, SamplingParams
    engine = Engine("/path/to/model_dir", EngineConfig(dtype="bfloat16"))
    outputs = engine.generate([[1, 2, 3]], max_tokens=16, temperature=0.0)
"""
__version__ = "0.1.0"

from .config.engine import EngineConfig, SchedulerConfig  # noqa: E402,F401
from .sampling.params import SamplingParams  # noqa: E402,F401


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name == "Model":
        from .engine.model import Model
        return Model
    raise AttributeError(name)
