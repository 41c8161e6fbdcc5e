from .flash_attn import attention_forward, attention_forward_varlen, attention_forward_host, sparse_attention

__all__ = ["attention_forward", "attention_forward_varlen", "attention_forward_host", "sparse_attention"]
