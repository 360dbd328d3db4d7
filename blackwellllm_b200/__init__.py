"""blackwellllm_b200: a single-GPU inference engine for the Llama/Qwen2 dense decoder on B200."""
from . import config as _config  # noqa: F401  (registers the architectures)

__version__ = "0.1.0"
