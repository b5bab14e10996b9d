"""Softmax attention inside chunks, without a rotation: position i sees the keys j <= i of its own
chunk of `chunk` positions (chunks counted from position 0 of the request, wherever a prompt was
cut).  q, k and v pass a short causal convolution over time directly behind their projection; q and
k are then divided by their root mean square per head (no weight).  Positions enter through a
penalty on distance only:  score = q.k * scale - r1[h] ln(1 + r2[h] (i - j)).  Query heads are
grouped over fewer key/value heads; the value heads may have a size of their own.

Keys and values live in the paged cache; pages of chunks that are over go back to the pool
(`PagedKVSpec.chunk`).  The convolution's last taps-1 inputs live in the request's slot.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Mixer, PagedKVSpec, register_part
from .linear import matmul, matmul_into_residual
from .shortconv import ShortConv


class ChunkAttention(Mixer):
    steps_from_device_tables = True

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, chunk: int, scale: float,
                 eps: float, out_scale: float = 1.0):
        self.hidden, self.QH, self.KH, self.dk, self.dv = int(hidden), int(heads), int(kv_heads), int(dim), int(vdim)
        if self.KH <= 0 or self.QH % self.KH:
            raise ValueError(f"chunk attention: {self.QH} query heads over {self.KH} key/value heads")
        self.chunk, self.scale, self.eps, self.out_scale = int(chunk), float(scale), float(eps), float(out_scale)
        if self.chunk < 1:
            raise ValueError("chunk attention: the chunk holds at least one position")
        self.conv = ShortConv(("q.conv", "k.conv", "v.conv"), (self.QH * self.dk, self.KH * self.dk, self.KH * self.dv), conv)

    def param_specs(self):
        h = self.hidden
        out = {"q": ParamSpec((self.QH * self.dk, h)), "k": ParamSpec((self.KH * self.dk, h)),
               "v": ParamSpec((self.KH * self.dv, h)), "o": ParamSpec((h, self.QH * self.dv)),
               "r1": ParamSpec((self.QH,), init="norm"), "r2": ParamSpec((self.QH,), init="norm")}
        out.update(self.conv.param_specs())
        return out

    def cache_spec(self):
        return PagedKVSpec(self.KH, self.dk, None, None if self.dv == self.dk else self.dv, self.chunk)

    def state_spec(self):
        return {"conv": self.conv.state_spec()}

    def bind(self, t):
        q, k, v = t["q"], t["k"], t["v"]
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = q.float(), k.float(), v.float()
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        self.w_o = t["o"]
        self.conv.bind(t)
        self.r1, self.r2 = t["r1"].float().contiguous(), t["r2"].float().contiguous()

    def forward(self, ctx, xn, residual, cache):
        T, QH, KH, dk, dv = xn.shape[0], self.QH, self.KH, self.dk, self.dv
        g = cache.group
        proj = matmul(ctx, xn, self.w_qkv)
        y = self.conv.forward(ctx, proj, cache.state["conv"], silu=False)
        q = torch.empty((T, QH, dk), dtype=y.dtype, device=y.device)
        ops.unit_heads_append(y, g.kv_slot if cache.write else None, q, cache.kv, QH, KH, dk, dv, g.page_size, self.eps)
        attn = torch.empty((T, QH, dv), dtype=y.dtype, device=y.device)
        ops.chunk_attention(ctx, q, cache.kv, g, attn, QH, KH, dk, dv, self.chunk, self.scale, (self.r1, self.r2),
                            self.out_scale)
        return matmul_into_residual(ctx, attn.view(T, QH * dv), self.w_o, residual)


register_part("mixer", "chunk_attention", ChunkAttention)
