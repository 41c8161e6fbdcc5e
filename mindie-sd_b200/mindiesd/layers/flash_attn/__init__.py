from .attention_forward import attention_forward
from .attention_forward_varlen import attention_forward_varlen
from .host_io import attention_forward_host
from .sparse_flash_attn import sparse_attention

__all__ = ["attention_forward", "attention_forward_varlen", "attention_forward_host", "sparse_attention"]
