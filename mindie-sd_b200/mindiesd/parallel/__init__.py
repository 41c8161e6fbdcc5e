from .ulysses import ulysses_attention, default_head_chunks, default_head_pieces, release_buffers

__all__ = ["ulysses_attention", "default_head_chunks", "default_head_pieces", "release_buffers"]
