from .ulysses import (ulysses_attention, ulysses_attention_host, default_head_chunks, default_head_pieces,
                      release_buffers)

__all__ = ["ulysses_attention", "ulysses_attention_host", "default_head_chunks", "default_head_pieces",
           "release_buffers"]
