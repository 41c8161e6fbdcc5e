from .flash_attn import attention_forward, sparse_attention

__all__ = ["attention_forward", "sparse_attention"]
