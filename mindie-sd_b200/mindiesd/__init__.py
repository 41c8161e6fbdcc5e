"""B200-native attention hot path behind the MindIE-SD layer API."""
from .cache_agent import CacheAgent, CacheConfig
from .layers import (attention_forward, attention_forward_varlen, attention_forward_host, sparse_attention,
                     rotary_position_embedding)
from .parallel import ulysses_attention
from .quantization import FP8RotateQuantFA
from .utils import ParametersInvalid, ConfigError, ModelInitError, ModelExecError

__all__ = ["CacheAgent", "CacheConfig", "attention_forward", "attention_forward_varlen", "attention_forward_host", "sparse_attention", "rotary_position_embedding", "ulysses_attention", "FP8RotateQuantFA",
           "ParametersInvalid", "ConfigError", "ModelInitError", "ModelExecError"]
