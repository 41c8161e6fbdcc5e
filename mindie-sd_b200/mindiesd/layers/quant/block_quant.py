"""`fa_block_quant_preprocess` (mindiesd/layers/quant/block_quant.py:19-48 of MindIE-SD): dynamic
quantisation of an attention operand to e4m3, one scale per (block_size tokens x 128 channels)."""
import torch

from ...utils.exception import ParametersInvalid


def fa_block_quant_preprocess(input_tensor, block_size=128, dst_type=torch.float8_e4m3fn, **kwargs):
    """Returns (e4m3 [B, N, S, D], fp32 scales [B, N, ceil(S/block_size), 1]); real = stored * scale.
    `layout` ('BNSD' default, or 'BSND') names the input layout; the output is always BNSD.
    `rotate=True` first rotates every token by the 128-point Hadamard matrix / sqrt(128) inside the
    same kernel (use it on q and k together: q k^T is unchanged, outlier channels are spread).
    `rot=` a [128, 128] matrix: the tokens are multiplied by it on the tensor cores inside the
    quantisation kernel (the product is never written out)."""
    if len(input_tensor.shape) != 4:
        raise ParametersInvalid(f"fa block quant preprocess only support qkv quant, dim = 4, "
                                f"but got {len(input_tensor.shape)}.")
    if dst_type != torch.float8_e4m3fn:
        raise ParametersInvalid(f"fa block quant preprocess only supports float8_e4m3fn, but got {dst_type}.")
    if block_size not in (128, 256, 512):
        raise ParametersInvalid(f"block_size must be 128, 256 or 512, but got {block_size}.")
    layout = kwargs.get("layout", "BNSD")
    if layout not in ("BNSD", "BSND"):
        raise ParametersInvalid(f"Unsupported layout: {layout}, expected 'BNSD' or 'BSND'.")
    rot = kwargs.get("rot")
    if rot is not None:
        if kwargs.get("rotate", False):
            raise ParametersInvalid("give either rotate=True (fixed Hadamard rotation) or rot= (a matrix), not both.")
        quant, scale = torch.ops.mindiesd.fa_rotate_quant(input_tensor, rot, int(block_size), layout == "BNSD")
    else:
        quant, scale = torch.ops.mindiesd.fa_block_quant(input_tensor, int(block_size), layout == "BNSD", False,
                                                         bool(kwargs.get("rotate", False)))
    return quant, scale.unsqueeze(-1)


def fa_channel_quant_preprocess(input_tensor, **kwargs):
    """One scale per channel over the whole sequence (for V): returns (e4m3 [B, N, S, D], fp32 [B, N, D])."""
    layout = kwargs.get("layout", "BNSD")
    return torch.ops.mindiesd.fa_block_quant(input_tensor, 128, layout == "BNSD", True, False)
