"""B200-native attention hot path behind the MindIE-SD layer API."""
from .layers import attention_forward, sparse_attention
from .parallel import ulysses_attention
from .quantization import FP8RotateQuantFA
from .utils import ParametersInvalid, ConfigError, ModelInitError, ModelExecError

__all__ = ["attention_forward", "sparse_attention", "ulysses_attention", "FP8RotateQuantFA",
           "ParametersInvalid", "ConfigError", "ModelInitError", "ModelExecError"]
