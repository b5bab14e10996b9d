"""Softmax attention without a rotation, whose scores get a learned bias by distance:

    score(i, j) = q_i . k_j * scale + rel[bucket(i - j), head]

over the keys j <= i, or over the last `window` of them (i - j < window).  The table `rel` has B rows:
the first B // 2 stand for one distance each, the others are spread evenly over the logarithm of the
distance up to `bias_max`, and the last row takes every greater distance:

    bucket(n) = n                                                                   for n < B // 2
              = min(B - 1, B // 2 + floor(ln(n / (B // 2)) / ln(bias_max / (B // 2)) * (B - B // 2)))   otherwise

At load the table is unrolled over the distances 0..bias_max (every distance from bias_max on reads the last
row), and turned head-major, so that the kernels index a head's row by min(i - j, bias_max) and know nothing of buckets.

Queries and keys pass an RMS norm with a plain weight: per head with one weight [dim] for all heads
(`qk_norm="head"`), or over the whole projection at once with a weight of that size (`"whole"`).  The queries may
be warmed up with position: q *= 1 + coef * ln(floor((p + 1) / every) + 1)  (`q_temp=(coef, every)`).  Query heads
are grouped over fewer key/value heads; the value heads have a size of their own; the values are a projection of
their own or (`values="keys"`) the keys as projected, before their norm.  With `own_kv=False` the layer has no key
and value tensors: it reads the pages of another layer (the layer's `cache_from`) with its own queries.

Normalised keys and the values live in the paged cache; with a window, pages that no later token can see go
back to the pool.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Mixer, PagedKVSpec, register_part
from .linear import matmul, matmul_into_residual


def distance_rows(rows: int, far: int):
    """For every distance 0..far the row of a table of `rows` rows that serves it (the module's bucket function,
    evaluated in double precision); every distance beyond `far` is served by the last entry's row, rows - 1."""
    half = rows // 2
    if rows < 2 or far <= half:
        raise ValueError(f"distance bias: {rows} rows need a greatest distance beyond {half}, got {far}")
    out = []
    for n in range(far + 1):
        if n < half:
            out.append(n)
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    out[far] = rows - 1
    return out


class BiasedAttention(Mixer):
    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, eps: float,
                 bias_rows: int, bias_max: int, window: Optional[int] = None, qk_norm: str = "head",
                 values: str = "projection", q_temp=None, own_kv: bool = True):
        self.hidden, self.QH, self.KH, self.dk, self.dv = int(hidden), int(heads), int(kv_heads), int(dim), int(vdim)
        if self.KH <= 0 or self.QH % self.KH:
            raise ValueError(f"biased attention: {self.QH} query heads over {self.KH} key/value heads")
        if qk_norm not in ("head", "whole") or values not in ("projection", "keys"):
            raise ValueError(f"biased attention: qk_norm {qk_norm!r}, values {values!r}")
        if values == "keys" and self.dv != self.dk:
            raise ValueError("biased attention: values that are the keys have the keys' size")
        self.scale, self.eps = float(scale), float(eps)
        self.bias_rows, self.bias_max = int(bias_rows), int(bias_max)
        self.row_of_distance = distance_rows(self.bias_rows, self.bias_max)
        self.window = int(window) if window else None
        self.whole, self.values_are_keys, self.own_kv = qk_norm == "whole", values == "keys", bool(own_kv)
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp else None
        if self.q_temp is not None and self.q_temp[1] < 1:
            raise ValueError("biased attention: the queries' warm-up counts positions in steps of at least one")
        self.w_in = self.w_o = self.qw = self.kw = self.bias = None

    def param_specs(self):
        h, QH, KH, dk, dv = self.hidden, self.QH, self.KH, self.dk, self.dv
        out = {"q": ParamSpec((QH * dk, h)), "q.norm": ParamSpec((QH * dk if self.whole else dk,), init="norm"),
               "rel": ParamSpec((self.bias_rows, QH), std=0.5), "o": ParamSpec((h, QH * dv))}
        if self.own_kv:
            out["k"] = ParamSpec((KH * dk, h))
            out["k.norm"] = ParamSpec((KH * dk if self.whole else dk,), init="norm")
            if not self.values_are_keys:
                out["v"] = ParamSpec((KH * dv, h))
        return out

    def cache_spec(self):
        return PagedKVSpec(self.KH, self.dk, self.window, None if self.dv == self.dk else self.dv)

    def bind(self, t):
        mats = [t["q"]]
        if self.own_kv:
            mats.append(t["k"])
            if not self.values_are_keys:
                mats.append(t["v"])
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        self.w_o = t["o"]
        self.qw = t["q.norm"]
        self.kw = t["k.norm"].to(self.qw.dtype) if self.own_kv else None
        rel = t["rel"].float()
        idx = torch.tensor(self.row_of_distance, dtype=torch.long, device=rel.device)
        self.bias = rel.index_select(0, idx).t().contiguous()          # [QH, bias_max + 1] float32: a head's distances side by side

    def forward(self, ctx, xn, residual, cache):
        T, QH, KH, dk, dv = xn.shape[0], self.QH, self.KH, self.dk, self.dv
        g = cache.group
        store = self.own_kv and cache.write
        proj = matmul(ctx, xn, self.w_in)                                # [T, q | k | v]
        q = torch.empty((T, QH, dk), dtype=proj.dtype, device=proj.device)
        ops.norm_heads_append(proj, self.qw, self.kw, ctx.positions, g.kv_slot if store else None, q, cache.kv, QH, KH, dk, dv,
                              QH * dk if self.whole else dk, KH * dk if self.whole else dk, self.values_are_keys,
                              g.page_size, self.eps, temp=self.q_temp)
        attn = torch.empty((T, QH, dv), dtype=proj.dtype, device=proj.device)
        ops.biased_attention(ctx, q, cache.kv, g, attn, QH, KH, dk, dv, self.window or 0, self.scale, self.bias)
        return matmul_into_residual(ctx, attn.view(T, QH * dv), self.w_o, residual)


register_part("mixer", "biased_attention", BiasedAttention)
