"""gollmgo_b200: a single-GPU inference engine for the Llama dense decoder on B200
(sm_100a): configuration, weights, parts, paged cache, one step function, a
continuous-batching scheduler, sampling, trace replay."""
from . import architectures  # noqa: F401  registers "LlamaForCausalLM"

__version__ = "0.1.0"

from .config import EngineConfig  # noqa: E402
from .sampling import SamplingParams  # noqa: E402


def __getattr__(name):
    if name in ("Engine", "RequestOutput", "TokenResult"):
        from .engine import llm_engine
        return getattr(llm_engine, name)
    raise AttributeError(name)


__all__ = ["Engine", "EngineConfig", "SamplingParams", "RequestOutput", "TokenResult"]
