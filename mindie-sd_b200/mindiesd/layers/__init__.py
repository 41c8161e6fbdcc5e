from .flash_attn import attention_forward, attention_forward_varlen, attention_forward_host, sparse_attention
from .rope import rotary_position_embedding

__all__ = ["attention_forward", "attention_forward_varlen", "attention_forward_host", "sparse_attention",
           "rotary_position_embedding"]
