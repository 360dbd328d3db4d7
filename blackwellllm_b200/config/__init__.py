"""Typed configuration and the architecture registry."""
from .registry import ConfigError, load_config, parse_config, register_architecture, registered_architectures
from .specs import (AttentionSpec, LayerSpec, Llama3RopeScaling, ModelConfig, NoPositionSpec, RMSNormSpec,
                    RopeSpec, ScheduleEntry, SwiGLUSpec)
from ..models import dense_decoder as _dense_decoder  # noqa: F401  (registers Llama and Qwen2)
