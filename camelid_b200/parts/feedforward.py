"""Feed-forwards. SwiGLU: g = x Wg^T, u = x Wu^T, act = (g / (1 + exp(-g))) * u,
d = act Wd^T, added into the residual stream (src/inference.rs:9657-9664, :6654-6706;
device twin silu_mul at src/cuda_resident.rs:1769). Gate and up are one packed matrix so
that one product makes both and the activation happens in its epilogue."""
from __future__ import annotations

from ..csrc import ops
from . import linear
from .base import Part, TensorSpec, register_part, to_device


@register_part("ffn", "swiglu")
class SwiGLU(Part):
    graph_safe = True
    graph_safe_any_step = True
    handles_pending = True
    accepts_row_scale = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.group = linear.swiglu_group(self.intermediate_size)
        # the three matrices' names under the prefix (``names``: gate, up, down; default the Llama checkpoints' names)
        self.names = tuple(params.get("names") or ("gate_proj.weight", "up_proj.weight", "down_proj.weight"))
        # the gated activation (alpha, limit, shift): min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, +-limit) + shift);
        # absent: SiLU gating, silu(g) * u
        self.act = ops.GateAct(*params["gate_act"]) if params.get("gate_act") else None
        self.w_gate_up = None
        self.w_down = None

    def tensor_specs(self):
        p, (gate, up, down) = self.prefix, self.names
        return {
            p + gate: TensorSpec((self.intermediate_size, self.hidden_size)),
            p + up: TensorSpec((self.intermediate_size, self.hidden_size)),
            p + down: TensorSpec((self.hidden_size, self.intermediate_size)),
        }

    def load(self, tensors, device, dtype):
        p, (gate, up, down) = self.prefix, self.names
        gate = to_device(tensors[p + gate], device, dtype)
        up = to_device(tensors[p + up], device, dtype)
        self.w_gate_up = linear.pack_gate_up(gate, up, self.group)
        self.w_down = to_device(tensors[p + down], device, dtype)

    def _activations(self, ctx, x, name="ffn_act"):
        act = ctx.buffer(name, (x.shape[0], self.intermediate_size))
        linear.linear(ctx, x, self.w_gate_up, act, linear.SWIGLU, self.group, row_scale=ctx.take_row_scale(), act=self.act)
        return act

    def forward(self, ctx, x, residual):
        linear.add_into_residual(ctx, self._activations(ctx, x), self.w_down, residual, "down_partial")

    def output(self, ctx, x, name: str):
        """(y, None): the feed-forward's output as float32 rows or split sums in a buffer of its own, for a
        block that norms it before it is added."""
        return linear.product_f32(ctx, self._activations(ctx, x, name + "_act"), self.w_down, name), None


@register_part("ffn", "dense")
class DenseFeedForward(Part):
    """d = act(x Wu^T + bu) Wd^T + bd. ``activation``: "gelu_tanh" (the tanh form of GELU), "gelu_erf" (the exact one,
    0.5 z (1 + erf(z / sqrt 2))) or "relu_squared" (max(z, 0)^2); ``bias``: whether the two projections have biases (``up.b``, ``down.b``). Tensors ``up``
    [intermediate, hidden] and ``down`` [hidden, intermediate] under the prefix."""
    graph_safe = True
    graph_safe_any_step = True
    handles_pending = True
    default_activation = "gelu_tanh"

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.activation = params.get("activation") or self.default_activation
        if self.activation not in ("gelu_tanh", "gelu_erf", "relu_squared"):
            from ..errors import ConfigError
            raise ConfigError("activation", f"unknown activation {self.activation!r}; known: gelu_tanh, gelu_erf, relu_squared")
        self.act = ops.ACTIVATIONS[self.activation]
        self.bias = bool(params.get("bias", False))
        self.w_up = self.w_down = self.b_up = self.b_down = None

    def tensor_specs(self):
        p = self.prefix
        specs = {p + "up": TensorSpec((self.intermediate_size, self.hidden_size)),
                 p + "down": TensorSpec((self.hidden_size, self.intermediate_size))}
        if self.bias:
            specs[p + "up.b"] = TensorSpec((self.intermediate_size,), "input_bias")
            specs[p + "down.b"] = TensorSpec((self.hidden_size,), "input_bias")
        return specs

    def load(self, tensors, device, dtype):
        import torch
        self.w_up = to_device(tensors[self.prefix + "up"], device, dtype)
        self.w_down = to_device(tensors[self.prefix + "down"], device, dtype)
        if self.bias:
            self.b_up = tensors[self.prefix + "up.b"].to(device=device, dtype=torch.float32).contiguous()
            self.b_down = tensors[self.prefix + "down.b"].to(device=device, dtype=torch.float32).contiguous()

    def _activations(self, ctx, x, name="ffn_act"):
        act = ctx.buffer(name, (x.shape[0], self.intermediate_size))
        linear.product_act(ctx, x, self.w_up, act, "up_partial", act=self.act, bias=self.b_up)
        return act

    def forward(self, ctx, x, residual):
        act = self._activations(ctx, x)
        if self.b_down is not None:
            ctx.settle(residual)
            ops.add_rows_vec(residual, None, self.b_down)
        linear.add_into_residual(ctx, act, self.w_down, residual, "down_partial")

    def output(self, ctx, x, name: str):
        """(y, bias): the output without its last bias as float32 rows or split sums in a buffer of its own, and
        that bias (None without), for a block that norms the sum before it is added."""
        return linear.product_f32(ctx, self._activations(ctx, x, name + "_act"), self.w_down, name), self.b_down


@register_part("ffn", "dense_gelu")
class DenseGelu(DenseFeedForward):
    """d = gelu(x Wu^T) Wd^T with the tanh form of GELU, added into the residual stream."""
