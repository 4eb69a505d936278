"""yalis_b200: a one-GPU inference engine for the Llama 3 dense decoder on NVIDIA B200 (sm_100a).

Public names follow axonn-ai/yalis (yalis/__init__.py): ``ModelConfig``,
``InferenceConfig`` and ``LLMEngine``; ``generate`` is the token-ids-in,
token-ids-out shortcut.  Importing the package touches neither CUDA nor the
compiler; the native libraries are built at first use.
"""

from yalis_b200.config.engine_config import EngineConfig
from yalis_b200.config.runtime import InferenceConfig, ModelConfig

__all__ = ["ModelConfig", "InferenceConfig", "EngineConfig", "LLMEngine", "generate", "Generation", "Engine",
           "SamplingParams"]


def __getattr__(name):
    if name == "SamplingParams":
        from yalis_b200.sampling.sampler import SamplingParams
        return SamplingParams
    if name in ("LLMEngine", "generate", "Generation"):
        from yalis_b200.engine import llm_engine
        return getattr(llm_engine, name)
    if name == "Engine":
        from yalis_b200.engine.engine import Engine
        return Engine
    raise AttributeError(name)
