"""blackwellllm_b200: a single-GPU inference engine for the Llama/Qwen2 dense decoder on B200."""
from . import config as _config  # noqa: F401  (registers the architectures)
from .engine.engine import Engine, EngineError, EngineOptions
from .engine.batch import StepEntry
from .engine.llm import FROM_LAST, LLM, BlackwellEngine, DecodeRequest, GenerationResult, InferenceConfig, PendingTokens
from .sampling.params import SamplingParams

__version__ = "0.1.0"
__all__ = ["Engine", "EngineError", "EngineOptions", "StepEntry", "LLM", "BlackwellEngine", "DecodeRequest",
           "GenerationResult", "InferenceConfig", "SamplingParams", "FROM_LAST", "PendingTokens"]
