"""`FP8RotateQuantFA`: the FP8 attention hook a quantised model calls instead of attention_forward
(mindiesd/quantization/layer.py:274-324 of MindIE-SD)."""
import math

import torch
from torch import nn

from ..layers.quant.block_quant import fa_block_quant_preprocess, fa_channel_quant_preprocess
from ..utils.exception import ParametersInvalid
from ..utils.status import checked


def get_quant_weight(weights, name):
    if weights is None or name not in weights:
        return None
    w = weights[name]
    return w if isinstance(w, torch.Tensor) else torch.as_tensor(w)


class FP8RotateQuantFA(nn.Module):
    """forward(query, key, value, layout=): rotate q and k by the learned 128x128 matrices (fused into
    the quantisation kernel), quantise
    q (128-token blocks), k and v (256-token blocks) to e4m3, run FP8 attention, return the input
    dtype and layout.  Without learned matrices q and k are rotated by the fixed Hadamard matrix
    inside the quantisation kernel.  `v_per_channel=True` quantises v with one scale per channel."""

    def __init__(self, prefix=None, weights=None, v_per_channel=False):
        super().__init__()
        self.register_buffer("q_rot", get_quant_weight(weights, f"{prefix}.q_rot"), persistent=False)
        self.register_buffer("k_rot", get_quant_weight(weights, f"{prefix}.k_rot"), persistent=False)
        self.v_per_channel = v_per_channel
        if (self.q_rot is None) != (self.k_rot is None):
            # q k^T is only preserved when both operands are rotated by matching matrices; the
            # reference fails in its first matmul when one of them is missing (layer.py:284-285).
            missing = "k_rot" if self.k_rot is None else "q_rot"
            raise ParametersInvalid(f"FP8RotateQuantFA needs both {prefix}.q_rot and {prefix}.k_rot, or neither "
                                    f"(fixed Hadamard rotation); {prefix}.{missing} is missing.")

    def forward(self, query, key, value, **kwargs):
        layout = kwargs.get("layout", "BNSD")
        if layout not in ("BNSD", "BSND"):
            raise ValueError(f"Unsupported layout: {layout}, expected 'BNSD' or 'BSND'.")
        d = query.shape[-1]
        fixed = self.q_rot is None and self.k_rot is None
        # A learned rotation runs on the tensor cores inside the quantisation kernel; without learned
        # matrices both operands get the fixed Hadamard rotation, also inside that kernel.
        q, q_scale = fa_block_quant_preprocess(query, block_size=128, layout=layout, rotate=fixed, rot=self.q_rot)
        k, k_scale = fa_block_quant_preprocess(key, block_size=256, layout=layout, rotate=fixed, rot=self.k_rot)
        if self.v_per_channel:
            v, v_scale = fa_channel_quant_preprocess(value, layout=layout)
            v_block = 0
        else:
            v, v_scale = fa_block_quant_preprocess(value, block_size=256, layout=layout)
            v_block = 256
        out = torch.ops.mindiesd.fp8_attention(q, k, v, q_scale, k_scale, v_scale, 1.0 / math.sqrt(d), 256, v_block,
                                               query.dtype)
        return checked(out.transpose(1, 2) if layout == "BSND" else out, "FP8RotateQuantFA")


def add_fa_quant(module, prefix=None, weights=None):
    """Attaches the hook as `module.fa_quant` (mindiesd/quantization/quantize.py:158-161)."""
    module.fa_quant = FP8RotateQuantFA(prefix, weights)
    return module
