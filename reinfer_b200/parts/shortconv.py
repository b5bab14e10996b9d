"""A short causal convolution over time on each channel of a projection (a few taps, no bias,
the last tap on the present token, zeros before a request's first token).  It is a piece of a
mixer, not a part of its own: the mixer declares `state_spec()` for it and hands over the
request slots' rows, which hold every request's last taps-1 inputs between steps.

Several tensors `[channels_i, taps]` (one per projection that the mixer convolves) are kept as
one `[sum channels_i, taps]` float32 table, in the order of the mixer's fused projection.
"""
from __future__ import annotations

from typing import Sequence, Tuple

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import SlotStateSpec


class ShortConv:
    def __init__(self, names: Sequence[str], channels: Sequence[int], taps: int):
        self.names = tuple(names)                   # local tensor names, in the order of the channels
        self.channels = tuple(int(c) for c in channels)
        self.taps = int(taps)
        if self.taps < 1:
            raise ValueError(f"short convolution with {self.taps} taps")
        self.total = sum(self.channels)
        self.weight = None

    def param_specs(self):
        return {n: ParamSpec((c, self.taps), std=0.5) for n, c in zip(self.names, self.channels)}

    def bind(self, tensors) -> None:
        self.weight = torch.cat([tensors[n].float() for n in self.names], dim=0).contiguous()

    def state_spec(self) -> SlotStateSpec:
        return SlotStateSpec((max(self.taps - 1, 0), self.total), "float32")

    def forward(self, ctx, u: torch.Tensor, state: torch.Tensor, silu: bool) -> torch.Tensor:
        """u [T, total] (a view of the fused projection; rows may be strided) -> y [T, total], and the slots' rows
        move on.  Reads the step's entries from the device tables only."""
        y = torch.empty((u.shape[0], self.total), dtype=u.dtype, device=u.device)
        ops.shortconv(u, self.weight, state, y, ctx.cu_q, ctx.entry_slot, ctx.n_entries, max(1, ctx.max_q_len), silu)
        return y
