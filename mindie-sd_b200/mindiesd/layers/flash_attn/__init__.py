from .attention_forward import attention_forward
from .sparse_flash_attn import sparse_attention

__all__ = ["attention_forward", "sparse_attention"]
