"""Dynamic Tanh in the place of a normalisation: y = tanh(alpha x) w + b with a learned scalar
alpha, a weight and a bias per feature.  It computes no mean and no variance, so nothing crosses a
row and there is no epsilon; 32-bit arithmetic.  The residual sum that the parts before it left
(one addend or a stack of partial sums) is added on the way, as in the RMS norm's kernel.

Tensor names: the weight is `weight_name` (default "weight"); bias and alpha are
`bias_name` / `alpha_name` (defaults "bias", "alpha").
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Norm, PreparedRows, register_part


class DynamicTanh(Norm):
    adds_partial_sums = True            # delta may be a stack [S, rows, width] of float32 partial sums
    prepares_complete_rows = True       # prepared_by() leaves finished rows: any reader takes them

    def __init__(self, width: int, weight_name: str = "weight", bias_name: str = "bias", alpha_name: str = "alpha"):
        self.width = int(width)
        self.names = (str(weight_name), str(bias_name), str(alpha_name))
        self.weight = self.bias = self.alpha = None

    def param_specs(self):
        w, b, a = self.names
        return {w: ParamSpec((self.width,), init="norm"),
                b: ParamSpec((self.width,), std=0.05),
                a: ParamSpec((), init="norm")}

    def bind(self, tensors):
        w, b, a = (tensors[n] for n in self.names)
        if not (w.dtype == b.dtype == a.dtype):
            w, b, a = w.float(), b.float(), a.float()
        self.weight, self.bias, self.alpha = w.contiguous(), b.contiguous(), a.reshape(1).contiguous()

    def prepared_by(self, ctx, a, w, residual):
        """residual += a w^T by a product whose cluster also makes this norm's rows of the new residual (a decode step's
        few rows, bfloat16, widths in tiles of 128): PreparedRows for forward(delta=that), or None where that form does
        not apply and nothing was done."""
        if self.weight is None or ctx.dtype != torch.bfloat16 or not ops.DEFER_SUMS or residual.shape[1] != self.width:
            return None
        made = ops.gemm_bf16_residual_norm(a, w, residual, self.weight, dyt=(self.bias, self.alpha))
        return None if made is None else PreparedRows(self, made[0], None)

    def forward(self, ctx, x, out=None, delta=None, row_idx=None):
        if isinstance(delta, PreparedRows):
            if delta.norm is not self or out is not None or row_idx is not None:
                raise ValueError("dyt: rows prepared by a product are for the norm they were made for")
            return delta.rows
        if delta is not None and delta.dtype != torch.float32:
            ops.residual_add(x, delta)
            delta = None
        rows = x.shape[0] if row_idx is None else row_idx.numel()
        if out is None:
            out = torch.empty((rows, self.width), dtype=ctx.dtype, device=x.device)
        ops.dyt(x, delta, self.weight, self.bias, self.alpha, out, row_idx)
        return out


register_part("norm", "dyt", DynamicTanh)
