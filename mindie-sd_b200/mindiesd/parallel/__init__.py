from .ulysses import ulysses_attention, default_head_chunks

__all__ = ["ulysses_attention", "default_head_chunks"]
