from .block_quant import fa_block_quant_preprocess, fa_channel_quant_preprocess

__all__ = ["fa_block_quant_preprocess", "fa_channel_quant_preprocess"]
