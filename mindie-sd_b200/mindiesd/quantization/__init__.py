from .layer import FP8RotateQuantFA, add_fa_quant

__all__ = ["FP8RotateQuantFA", "add_fa_quant"]
