"""A single-GPU inference engine for the Qwen2 dense decoder on NVIDIA B200 (sm_100a):
typed configuration and registry, safetensors weights, layers put together from parts, a
paged cache manager, one step function, a scheduler, sampling, and hand-written CUDA."""
from .config import Qwen2Config, load_config, get_architecture, register_architecture, preset
from .sampling.config import GenerationConfig, SamplingParams

__version__ = "0.1.0"


def __getattr__(name):          # heavier pieces load on first use, as the reference's package does
    if name == "LLM":           # (python/microllm/__init__.py:21-31)
        from .engine.llm import LLM
        return LLM
    if name in ("Engine", "StepEntry"):
        from .engine import step
        return getattr(step, name)
    if name in ("load_engine", "random_engine"):
        from .engine import loading
        return getattr(loading, name)
    raise AttributeError(name)
