"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w in float32 (src/tensor/mod.rs:2086-2096;
device twins rms_norm_f32 and rms_norm_batched at src/cuda_resident.rs:89, :1925). The
input is the float32 residual stream; the output has the compute type."""
from __future__ import annotations

import torch

from ..csrc import ops
from . import linear
from .base import Part, TensorSpec, register_part, to_device


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    graph_safe = True
    graph_safe_any_step = True
    handles_pending = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.tensor = params.get("tensor") or self.prefix + "weight"      # the weight's full name
        self.weight = None

    def tensor_specs(self):
        return {self.tensor: TensorSpec((self.hidden_size,), "norm")}

    def load(self, tensors, device, dtype):
        w = tensors[self.tensor]
        # a weight stored in 32-bit stays so; a 16-bit one becomes float32 only on the float32 path
        keep = None if w.dtype == torch.float32 else dtype
        self.weight = to_device(w, device, keep)

    def forward(self, ctx, h, rows_index=None, n_rows=None, name="normed", allow_row_scale=False):
        """The normalised rows of ``h``. With ``allow_row_scale`` the caller promises that whoever
        reads the result takes ``ctx.take_row_scale()`` and applies it: then a product into ``h``
        that is still deferred runs here together with the residual add and the weight half of
        this norm, and only the rows' scale is left to the reader."""
        rows = h.shape[0] if n_rows is None else n_rows
        out = ctx.buffer(name, (rows, self.hidden_size))
        if ctx.deferred is not None:
            if allow_row_scale and rows_index is None and linear.product_add_norm(ctx, h, self.weight, self.eps, out):
                return out
            linear.run_deferred(ctx)
        pending, ctx.pending = ctx.pending, None            # split sums still to be added to h: added here
        ops.rmsnorm(h, self.weight, self.eps, out, rows_index, pending)
        return out

    def sum_normed(self, ctx, y, residual, alpha: float = 1.0, bias=None):
        """residual = rmsnorm(alpha * residual + y + bias) * w in place: this norm *after* a residual sum, where the
        stream itself is normed. ``y``: a sublayer's output as float32 rows or split sums. Returns the new rows in the
        compute type (the stream itself on the float32 path) for the parts that read the stream as it is."""
        x = ctx.buffer("stream_rows", residual.shape) if ctx.dtype != torch.float32 else None
        ops.sum_norm(y, bias, self.weight, self.eps, alpha, residual, x)
        ctx.rows_copy = (residual, x) if x is not None else None
        return x if x is not None else residual

    def add_normed(self, ctx, y, residual, scale: float = 1.0, bias=None, then=None, name="normed"):
        """residual += scale * rmsnorm(y + bias) * w: this norm on a sublayer's output rows ``y`` (float32
        [rows, hidden], or split sums [splits, rows, hidden] that are added first), added into the stream.
        ``then``: the norm part that reads the stream next; if it is one of this kind, its rows come out of the
        same pass and are returned (else None: the caller runs that norm itself)."""
        fuse = (isinstance(then, RMSNorm) and then.weight is not None and then.weight.dtype == self.weight.dtype
                and then.hidden_size == self.hidden_size)
        x = ctx.buffer(name, (residual.shape[0], self.hidden_size)) if fuse else None
        ops.post_norm_add(y, bias, self.weight, self.eps, scale, residual, then.weight if fuse else None,
                          then.eps if fuse else 0.0, x)
        return x
