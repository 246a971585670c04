"""A per-layer token input: at the end of a layer the stream takes a contribution that depends on the token itself.

    e = T[token, layer * dim : (layer + 1) * dim]          (the layer's own columns of a second embedding table)
    y = Wp (gelu_tanh(Wg x) * e)                            (Wg [dim, hidden], Wp [hidden, dim])
    x <- x + y / sqrt(mean(y^2) + eps) * w

Tensors: the table (``table``, shared by all layers: [vocab, layers * dim], every layer keeps its own columns), and under the
prefix ``gate``, ``proj``, ``norm``. The two small products run on the library's product kernels (split sums for steps of few
rows); the GELU, the table look-up and the norm with the add are float32.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from . import linear
from .base import Part, TensorSpec, register_part, to_device


@register_part("layer_input", "token_side")
class TokenSideInput(Part):
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.vocab_size = int(params["vocab_size"])
        self.dim = int(params["dim"])
        self.layer = int(params["layer"])
        self.layers = int(params["layers"])
        self.eps = float(params.get("eps", 1e-6))
        self.table_name = params.get("table") or "side.embed"
        self.table = self.w_gate = self.w_proj = self.norm_w = None

    def tensor_specs(self):
        p = self.prefix
        return {self.table_name: TensorSpec((self.vocab_size, self.layers * self.dim), "embedding"),
                p + "gate": TensorSpec((self.dim, self.hidden_size)), p + "proj": TensorSpec((self.hidden_size, self.dim)),
                p + "norm": TensorSpec((self.hidden_size,), "norm")}

    def load(self, tensors, device, dtype):
        p = self.prefix
        cols = tensors[self.table_name][:, self.layer * self.dim:(self.layer + 1) * self.dim]
        self.table = to_device(cols, device, dtype)
        self.w_gate = to_device(tensors[p + "gate"], device, dtype)
        self.w_proj = to_device(tensors[p + "proj"], device, dtype)
        w = tensors[p + "norm"]
        self.norm_w = to_device(w, device, None if w.dtype == torch.float32 else dtype)

    def forward(self, ctx, x, h):
        """``x``: the stream's rows in the compute type; ``h``: the float32 stream, added into in place. Leaves the new
        rows in the compute type on the context."""
        rows = h.shape[0]
        z = linear.product_f32(ctx, x, self.w_gate, "side_gate")
        g = ctx.buffer("side_gated", (rows, self.dim))
        ops.gelu_mul_lookup(z, self.table, 0, ctx.tokens, g)
        y = linear.product_f32(ctx, g, self.w_proj, "side_out")
        x_out = ctx.buffer("stream_rows", h.shape) if ctx.dtype != torch.float32 else None
        ops.post_norm_add(y, None, self.norm_w, self.eps, 1.0, h, None, 0.0, x_out)
        ctx.rows_copy = (h, x_out) if x_out is not None else None
        return x_out
