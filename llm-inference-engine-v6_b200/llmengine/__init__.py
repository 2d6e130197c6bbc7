"""llmengine: a small, whole inference engine for the Llama dense GQA decoder on one B200.

    import llmengine
    eng = llmengine.Engine(model_dir, "bf16")          # or "fp32": everything in true 32-bit
    tokens, reason = eng.generate([1, 2, 3], 16)

Names follow the reference's Python package (python/llmengine/__init__.py:6-26).
"""
from .cache.host import host_module as _host_module
from .config import ConfigError, LlamaConfig, register_architecture
from .engine import BlockManager, CapacityError, ContinuousBatchScheduler, Engine
from .ops import KernelError
from .weights import WeightError, write_random_model

ModelConfig = LlamaConfig


def __getattr__(name):
    if name == "SequenceResult":
        return _host_module().SequenceResult
    raise AttributeError(name)


__all__ = ["BlockManager", "CapacityError", "ConfigError", "ContinuousBatchScheduler", "Engine", "KernelError", "LlamaConfig",
           "ModelConfig", "SequenceResult", "WeightError", "register_architecture", "write_random_model"]
