"""Token embedding, learned positions and output head.

Embedding: row t of the table, upcast to the float32 residual stream, no scaling
(crates/model/src/weights.rs:29-51) unless a `scale` is given; a table of learned position
vectors, when the model has one, is added by the same kernel (unscaled).  Output head: logits = W_out x on the wanted rows only;
W_out is its own matrix or, when the file has none, the embedding table
(crates/model/src/llama.rs:28-40,103-111).
"""
from __future__ import annotations

import torch

from ..ops import lib as ops
from .base import ParamSpec, Part, PositionEncoding
from .linear import STORE_F32, linear


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, n_vocab, width, scale=1.0, positions: "LearnedPositions" = None, copies=1, copy_dtype=None):
        """positions: a `LearnedPositions` part whose vector for a token's position is added to the
        (scaled) embedding; the model lists it as its position encoding, which owns the table.
        copies > 1: the residual rows are [tokens, copies * width], every copy the embedded token (a
        model whose blocks keep several residual streams).  copy_dtype (a 16-bit type): the rows are also left
        in that type in the step's buffer `residual_copy`, for blocks whose sublayers read the residual row
        itself (`PostNormBlock`, which keeps the copy up to date)."""
        self.n_vocab, self.width, self.scale, self.positions = n_vocab, width, float(scale), positions
        self.copies = int(copies)
        self.copy_dtype = copy_dtype if copy_dtype not in (None, torch.float32) else None
        self.w_weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.n_vocab, self.width))}

    def forward(self, ctx):
        h = ctx.buf("hidden", (ctx.token_capacity, self.copies * self.width), torch.float32)
        pos = self.positions.w_weight if self.positions is not None else None
        ops.embedding(self.w_weight, ctx.token_ids, h, ctx.err, scale=self.scale, pos_table=pos,
                      positions=ctx.positions if pos is not None else None, copies=self.copies)
        if self.copy_dtype is not None:
            ops.post_norm_add(h, ctx.n_tokens, xc=ctx.buf("residual_copy", (ctx.token_capacity, h.shape[1]), self.copy_dtype))
        return h


class LearnedPositions(PositionEncoding):
    """One learned vector per position, added to the embedded token.  The sum happens inside the
    embedding kernel (`TokenEmbedding(positions=...)`); a position past the table raises the step's
    error flag."""
    graph_safe = True

    def __init__(self, n_positions, width):
        self.n_positions, self.width = int(n_positions), width
        self.w_weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.n_positions, self.width))}


class OutputHead(Part):
    graph_safe = True

    def __init__(self, n_vocab, width, tied_to: TokenEmbedding = None, tied="auto", softcap=0.0):
        """tied: True (no matrix of its own), False (must have one), "auto" (use the file's
        matrix when present, else the embedding: the reference's rule).  softcap c > 0: the logits
        leave as c * tanh(logits / c)."""
        self.n_vocab, self.width, self.tied_to, self.tied = n_vocab, width, tied_to, tied
        self.softcap = float(softcap or 0.0)
        self.w_weight = None

    def param_specs(self):
        if self.tied is True:
            return {}
        return {"weight": ParamSpec((self.n_vocab, self.width), optional=self.tied == "auto")}

    def finalize(self):
        if self.w_weight is None:
            if self.tied_to is None:
                raise ValueError("output head has neither a matrix nor an embedding to share")
            self.w_weight = self.tied_to.w_weight

    def forward(self, x, ctx, n_rows):
        logits = ctx.buf("logits", (ctx.want_capacity, self.n_vocab), torch.float32)
        linear(x, self.w_weight, logits, STORE_F32, ctx, M=n_rows)
        if self.softcap > 0.0:
            ops.softcap(logits, n_rows, self.softcap)
        return logits
