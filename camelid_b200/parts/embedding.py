"""Token embedding (a row gather into the float32 residual stream, no scaling:
src/tensor/mod.rs:2253-2283) and the output projection, which is the embedding matrix
itself when the model ties them (src/model.rs:772-775, src/inference.rs:314-316)."""
from __future__ import annotations

import torch

from ..csrc import ops
from . import linear
from .base import Part, TensorSpec, register_part, to_device


@register_part("embedding", "embedding")
class TokenEmbedding(Part):
    """x = scale * E[token] (+ P[position]). ``scale`` (default 1) multiplies the embedding row; ``position_tensor``
    names a table of learned position rows [``positions``, hidden] that are added unscaled (positions count from 0 in
    every sequence; the plan's ``max_position`` keeps sequences inside the table)."""
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.tensor = params.get("tensor") or self.prefix + "weight"      # the table's full name
        self.scale = float(params["scale"]) if params.get("scale") is not None else 1.0
        self.position_tensor = params.get("position_tensor")
        self.positions = int(params["positions"]) if self.position_tensor else 0
        self.weight = None
        self.position_rows = None

    def tensor_specs(self):
        specs = {self.tensor: TensorSpec((self.vocab_size, self.hidden_size), "embedding")}
        if self.position_tensor:
            specs[self.position_tensor] = TensorSpec((self.positions, self.hidden_size), "embedding")
        return specs

    def load(self, tensors, device, dtype):
        self.weight = to_device(tensors[self.tensor], device, dtype)
        if self.position_tensor:
            self.position_rows = to_device(tensors[self.position_tensor], device, dtype)

    def forward(self, ctx, tokens, out, err):
        if self.scale == 1.0 and self.position_rows is None:
            ops.embed_gather(self.weight, tokens, out, err)
            return
        # the same rows in the compute type too: a first layer that reads the stream as it is needs no pass of its own
        x = ctx.buffer("stream_rows", out.shape) if ctx.dtype != torch.float32 and self.weight.dtype == ctx.dtype else None
        ops.embed_positions(self.weight, tokens, self.scale, self.position_rows, ctx.row_pos, out, err, x)
        ctx.rows_copy = (out, x) if x is not None else None


@register_part("embedding", "bigram_embedding")
class BigramEmbedding(Part):
    """Token embedding plus a row of a second table picked by a hash of the previous and the
    current token: row (previous * mul_prev + current * mul_cur) mod buckets, and row ``buckets``
    (the table's last) for a sequence's first token. The previous token is per-sequence state:
    the step's last token is kept for the next step. Without ``bigram_tensor`` it is a plain
    embedding whose table has the name ``tensor``."""
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.tensor = params.get("tensor") or self.prefix + "weight"
        self.bigram_tensor = params.get("bigram_tensor")
        self.buckets = int(params["buckets"]) if self.bigram_tensor else 0
        self.mul_prev = int(params["mul_prev"]) if self.bigram_tensor else 0
        self.mul_cur = int(params["mul_cur"]) if self.bigram_tensor else 0
        self.weight = None
        self.bigram = None

    def tensor_specs(self):
        specs = {self.tensor: TensorSpec((self.vocab_size, self.hidden_size), "embedding")}
        if self.bigram_tensor:
            specs[self.bigram_tensor] = TensorSpec((self.buckets + 1, self.hidden_size), "embedding")
        return specs

    def load(self, tensors, device, dtype):
        self.weight = to_device(tensors[self.tensor], device, dtype)
        if self.bigram_tensor:
            self.bigram = to_device(tensors[self.bigram_tensor], device, dtype)

    def cache_spec(self):
        from ..cache.book import StateSpec
        return StateSpec((1,), "int32", "previous_token") if self.bigram_tensor else None

    def forward(self, ctx, tokens, out, err):
        prev = ctx.state("previous_token").view(-1) if self.bigram_tensor else None
        ops.bigram_embed(self.weight, self.bigram, tokens, ctx.row_seq, ctx.row_pos, ctx.seq_row0, ctx.seq_new, ctx.seq_slot,
                         prev, out, ctx.n_seqs, self.buckets, self.mul_prev, self.mul_cur, err)


@register_part("head", "lm_head")
class OutputProjection(Part):
    """logits = x W^T in float32, without bias or scale (src/inference.rs:4284-4290); with
    ``softcap`` c the logits become c tanh(logits / c); with ``scale`` they are multiplied by it (before a cap). ``tensor``
    names the matrix in full."""
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.tied_to = params.get("tied_to")
        self.tensor = params.get("tensor") or self.prefix + "weight"
        self.softcap = float(params["softcap"]) if params.get("softcap") else None
        self.scale = float(params["scale"]) if params.get("scale") is not None else 1.0
        self.weight = None

    def tensor_specs(self):
        if self.tied_to:
            return {}
        return {self.tensor: TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors, device, dtype, tied_weight: torch.Tensor | None = None):
        if self.tied_to:
            self.weight = tied_weight
        else:
            self.weight = to_device(tensors[self.tensor], device, dtype)

    def forward(self, ctx, x, out):
        linear.linear(ctx, x, self.weight, out, linear.STORE_F32)
        if self.scale != 1.0:
            ops.scale_(out, self.scale)
        if self.softcap is not None:
            ops.softcap_(out, self.softcap)
