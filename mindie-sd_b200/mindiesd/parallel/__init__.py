from .ulysses import ulysses_attention

__all__ = ["ulysses_attention"]
