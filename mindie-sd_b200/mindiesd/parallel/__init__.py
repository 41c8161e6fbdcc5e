from .ulysses import (ulysses_attention, ulysses_attention_host, default_head_chunks, default_head_pieces,
                      default_transport, release_buffers)

__all__ = ["ulysses_attention", "ulysses_attention_host", "default_head_chunks", "default_head_pieces",
           "default_transport", "release_buffers"]
