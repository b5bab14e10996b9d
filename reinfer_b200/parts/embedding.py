"""Token embedding (a row gather into the float32 residual stream) and the output
head (final norm on the wanted rows only, then the vocabulary product in float32,
never rounded: crates/cuda/src/engine.rs:4337-4347).  The reference computes the
head for every prompt row and keeps the last (engine.rs:5685-5720); here only the
rows whose logits are asked for are normalised and multiplied."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Part, register_part
from .linear import matmul


class Embedding(Part):
    """`positions` > 0: a table of that many learned position vectors (tensor `positions_name`) whose row for the
    token's position is added to the token's row, unscaled, in the same kernel.  `table_name`: the local name of
    the token table (a tied output head takes the table under this name)."""

    def __init__(self, vocab: int, hidden: int, positions: int = 0, table_name: str = "weight",
                 positions_name: str = "positions.weight", scale: float = 1.0, rounded_copy: bool = False):
        """scale: a factor on the rows.  rounded_copy: in bfloat16 the gather also leaves the rows rounded, as
        `ctx.rounded_stream`, for a first block whose sublayers read the stream itself."""
        self.vocab, self.hidden, self.positions = int(vocab), int(hidden), int(positions)
        self.scale, self.rounded_copy = float(scale), bool(rounded_copy)
        self.table_name, self.positions_name = str(table_name), str(positions_name)
        self.weight = None
        self.pos_weight = None

    def param_specs(self):
        out = {self.table_name: ParamSpec((self.vocab, self.hidden), init="table")}
        if self.positions:
            out[self.positions_name] = ParamSpec((self.positions, self.hidden), init="table")
        return out

    def bind(self, tensors):
        self.weight = tensors[self.table_name]
        if self.positions:
            self.pos_weight = tensors[self.positions_name]
            if self.pos_weight.dtype != self.weight.dtype:
                self.pos_weight = self.pos_weight.to(self.weight.dtype)

    @property
    def max_positions(self):
        """The longest request the embedding can place (None: no limit of its own)."""
        return self.positions or None

    def forward(self, ctx) -> torch.Tensor:
        x = torch.empty((ctx.n_tokens, self.hidden), dtype=torch.float32, device=ctx.device)
        rounded = None
        if self.rounded_copy and ctx.dtype == torch.bfloat16:
            rounded = torch.empty((ctx.n_tokens, self.hidden), dtype=torch.bfloat16, device=ctx.device)
        ops.embed_gather(self.weight, ctx.token_ids, x, ctx.slot_token, ctx.entry_slot, ctx.tok_entry,
                         pos_table=self.pos_weight, positions=ctx.positions, scale=self.scale, rounded=rounded)
        ctx.rounded_stream = rounded
        return x


class LMHead(Part):
    """`tied`: the embedding table is the output matrix; the model hands it over in bind()
    under the local name 'weight' either way."""

    def __init__(self, vocab: int, hidden: int, tied: bool = False, fallback: str = "", softcap: float = 0.0,
                 weight_name: str = "weight"):
        """weight_name: the local name of an untied output matrix ("" where the part's prefix is the whole name)."""
        self.vocab, self.hidden, self.tied, self.fallback = int(vocab), int(hidden), bool(tied), fallback
        self.weight_name = str(weight_name)
        self.softcap = float(softcap or 0.0)        # > 0: logits <- cap * tanh(logits / cap)
        self.weight = None

    def param_specs(self):
        if self.tied:
            return {}
        return {self.weight_name: ParamSpec((self.vocab, self.hidden), optional=bool(self.fallback), fallback=self.fallback)}

    def bind(self, tensors):
        self.weight = tensors["weight" if self.tied else self.weight_name]

    def forward(self, ctx, xn_rows: torch.Tensor) -> torch.Tensor:
        logits = matmul(ctx, xn_rows, self.weight, out_dtype=torch.float32)
        if self.softcap > 0.0:
            ops.softcap(logits, self.softcap)
        return logits


register_part("embedding", "embedding", Embedding)
register_part("lm_head", "linear", LMHead)
