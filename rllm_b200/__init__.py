"""rllm_b200: a small, whole inference engine for Qwen3 dense on one B200 (sm_100a)."""
from .config import load_config, register_architecture
from .sampling.params import SamplingParams

__all__ = ["LLM", "generate", "load_config", "register_architecture", "SamplingParams"]


def __getattr__(name):
    if name in ("LLM", "generate"):
        from . import llm
        return getattr(llm, name)
    raise AttributeError(name)
